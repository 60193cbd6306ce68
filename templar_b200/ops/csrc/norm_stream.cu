// Backward of the fused residual-add + RMSNorm as a bulk-copy-fed streaming kernel (sm_100a).
//
// The warp-per-row kernel in elementwise.cu keeps a row's x, dy and the weight-gradient partials in registers
// (240 per thread at D = 2048): one CTA of eight warps per SM, and nothing is in flight while a warp reduces and
// writes, so it reaches about a third of the copy bandwidth inside a training step.  Here one producer thread per
// CTA streams tiles of eight whole rows of dy, x and dres into shared memory with cp.async.bulk (rows are contiguous,
// so a tile of one tensor is ONE copy of 8 * D * 2 bytes) two tiles ahead of the eight consumer warps, which read
// their row from shared memory twice (dot product, then output) and keep only the weight-gradient partials in
// registers.  96 KB are in flight per SM all the time.
//
//   dx = dres + rstd * (dy * w - xhat * mean(dy * w * xhat)),  xhat = x * rstd;   dw += sum_rows dy * xhat
//
// Same arithmetic, in the same order per row, as add_rmsnorm_bwd_warp_kernel.  Every wait is bounded; on expiry the
// status word gets TPLR_ST_WAIT_TIMEOUT and all roles return after the copies in flight have landed.
#include "tcgen05.cuh"
#include <stdlib.h>

namespace {
using namespace tplr_tc;
typedef __nv_bfloat16 bf16;
struct alignas(16) bf16x8 { __nv_bfloat162 v[4]; };

__device__ __forceinline__ void unpack8(const bf16x8& p, float* f) {
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(p.v[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ bf16x8 pack8(const float* f) {
  bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

constexpr int NS_ROWS = 8;          // rows per tile = consumer warps
constexpr int NS_STAGES = 2;
constexpr int NS_THREADS = 288;     // 8 consumer warps + 1 producer warp

template <int VPL>
__global__ void __launch_bounds__(NS_THREADS, 1)
add_rmsnorm_bwd_stream_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ w,
                              const float* __restrict__ rstd, const bf16* __restrict__ dres, bf16* __restrict__ dx,
                              float* __restrict__ dw, long long T, int D, unsigned int* status) {
  extern __shared__ uint8_t ns_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(ns_smem_raw) + 127) & ~(uintptr_t)127);
  __shared__ __align__(8) uint64_t bar_full[NS_STAGES], bar_empty[NS_STAGES];
  __shared__ int s_abort;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nv = D / 8;
  const uint32_t row_bytes = (uint32_t)D * 2u, arr_bytes = NS_ROWS * row_bytes, stage_bytes = 3u * arr_bytes;
  uint8_t* w_sm = smem + NS_STAGES * stage_bytes;
  const long long n_tiles = (T + NS_ROWS - 1) / NS_ROWS;
  volatile int* abort_flag = &s_abort;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < NS_STAGES; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), NS_ROWS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  for (int i = threadIdx.x; i < nv; i += NS_THREADS)
    reinterpret_cast<bf16x8*>(w_sm)[i] = reinterpret_cast<const bf16x8*>(w)[i];
  __syncthreads();

  if (warp == NS_ROWS) {
    // ------------------------------ producer ------------------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++it) {
        const uint32_t s = it % NS_STAGES, ph = (it / NS_STAGES) & 1u;
        if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, abort_flag)) break;
        const long long r0 = tile * NS_ROWS;
        const uint32_t rows = (uint32_t)((T - r0) < NS_ROWS ? (T - r0) : NS_ROWS);
        const uint32_t bytes = rows * row_bytes;
        const uint32_t fb = smem_u32(&bar_full[s]);
        const uint32_t base = smem_u32(smem) + s * stage_bytes;
        mbar_expect_tx(fb, bytes * (dres ? 3u : 2u));
        bulk_g2s(base, dy + r0 * D, bytes, fb);
        bulk_g2s(base + arr_bytes, x + r0 * D, bytes, fb);
        if (dres) bulk_g2s(base + 2u * arr_bytes, dres + r0 * D, bytes, fb);
      }
      // every copy that was issued has landed before this CTA may retire (the consumers may have given up)
      for (uint32_t back = 0; back < NS_STAGES && back < it; ++back) {
        const uint32_t j = it - 1u - back;
        mbar_wait(smem_u32(&bar_full[j % NS_STAGES]), (j / NS_STAGES) & 1u, abort_flag);
      }
    }
  } else {
    // ------------------------------ consumers: warp r of the CTA owns row r of every tile ----------
    float dwv[VPL][8];
#pragma unroll
    for (int v = 0; v < VPL; ++v)
#pragma unroll
      for (int e = 0; e < 8; ++e) dwv[v][e] = 0.f;
    const bf16x8* wv_sm = reinterpret_cast<const bf16x8*>(w_sm);
    uint32_t it = 0;
    for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++it) {
      const uint32_t s = it % NS_STAGES, ph = (it / NS_STAGES) & 1u;
      bool ok = mbar_wait(smem_u32(&bar_full[s]), ph, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const long long row = tile * NS_ROWS + warp;
      if (row < T) {
        const uint8_t* st = smem + s * stage_bytes + (uint32_t)warp * row_bytes;
        const bf16x8* gr = reinterpret_cast<const bf16x8*>(st);
        const bf16x8* xr = reinterpret_cast<const bf16x8*>(st + arr_bytes);
        const bf16x8* ar = reinterpret_cast<const bf16x8*>(st + 2u * arr_bytes);
        const float r = rstd[row];
        float dot = 0.f;
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
          const int i = lane + 32 * v;
          if (i < nv) {
            float xv[8], dv[8], wv[8];
            unpack8(xr[i], xv); unpack8(gr[i], dv); unpack8(wv_sm[i], wv);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const float xh = xv[e] * r;
              dwv[v][e] = fmaf(dv[e], xh, dwv[v][e]);
              dot = fmaf(dv[e] * wv[e], xh, dot);
            }
          }
        }
        dot = warp_sum_f(dot) / (float)D;
        bf16x8* outr = reinterpret_cast<bf16x8*>(dx + row * D);
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
          const int i = lane + 32 * v;
          if (i < nv) {
            float xv[8], dv[8], wv[8], o[8];
            unpack8(xr[i], xv); unpack8(gr[i], dv); unpack8(wv_sm[i], wv);
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = r * (dv[e] * wv[e] - xv[e] * r * dot);
            if (dres) {
              float a[8]; unpack8(ar[i], a);
#pragma unroll
              for (int e = 0; e < 8; ++e) o[e] += a[e];
            }
            outr[i] = pack8(o);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_empty[s]));
    }
    // the eight warps' partial dw through the (now unused) first stage, one slab of 32 vectors at a time
    if (dw) {
      float* s_dw = reinterpret_cast<float*>(smem);          // [8][256 + 1]
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        asm volatile("bar.sync 1, 256;" ::: "memory");
#pragma unroll
        for (int e = 0; e < 8; ++e) s_dw[warp * 257 + lane * 8 + e] = dwv[v][e];
        asm volatile("bar.sync 1, 256;" ::: "memory");
        const int col = threadIdx.x;                         // 256 columns of this slab
        const int i = (col >> 3) + 32 * v;
        if (i < nv) {
          float acc = 0.f;
#pragma unroll
          for (int k = 0; k < 8; ++k) acc += s_dw[k * 257 + col];
          atomicAdd(dw + (long long)i * 8 + (col & 7), acc);
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && s_abort && status) atomicOr(status, TPLR_ST_WAIT_TIMEOUT);
}

}  // namespace

extern "C" int tplr_add_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                                    void* dx, float* dw, long long T, int D, void* stream);

// tplr_add_rmsnorm_bwd with a status word: rows of 1032..2048 elements (multiples of 8) on 16-byte aligned tensors go
// through the streaming kernel above, everything else through the warp-per-row kernel.  dres and dw may be null.
TPLR_API int tplr_add_rmsnorm_bwd_v2(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                                     void* dx, float* dw, long long T, int D, unsigned int* status, void* stream) {
  TPLR_ENTER();
  if (D % 8 || D > 2048) return (int)cudaErrorInvalidValue;
  if (T <= 0) return 0;
  static const bool off = [] { const char* e = getenv("TPLR_NORM_BWD"); return e && e[0] == 'w'; }();   // "warp": old kernel
  const bool aligned = !(((uintptr_t)dy | (uintptr_t)x | (uintptr_t)w | (uintptr_t)dx | (uintptr_t)dres) & 15);
  if (off || !aligned || D <= 1024 || T < 8 * NS_ROWS)
    return tplr_add_rmsnorm_bwd(dy, x, w, rstd, dres, dx, dw, T, D, stream);
  const int smem_bytes = NS_STAGES * 3 * NS_ROWS * D * 2 + D * 2 + 128;
  auto kern = add_rmsnorm_bwd_stream_kernel<8>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (e != cudaSuccess) return (int)e;
  long long grid = tplr_sm_count();
  const long long n_tiles = (T + NS_ROWS - 1) / NS_ROWS;
  if (grid > n_tiles) grid = n_tiles;
  kern<<<(unsigned)grid, NS_THREADS, smem_bytes, (cudaStream_t)stream>>>(
      (const bf16*)dy, (const bf16*)x, (const bf16*)w, rstd, (const bf16*)dres, (bf16*)dx, dw, T, D, status);
  return (int)cudaGetLastError();
}
