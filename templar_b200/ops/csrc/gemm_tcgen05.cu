// bf16 GEMM on the 5th-generation tensor cores (sm_100a): TMA-fed shared-memory pipeline,
// tcgen05.mma issued by one elected thread with fp32 accumulators in tensor memory (TMEM),
// double-buffered accumulators so the epilogue of tile i overlaps the main loop of tile i+1.
//
//   C[M,N] (+)= op(A) * op(B)        A: [M,K] K-contiguous or [K,M] M-contiguous
//                                     B: [N,K] K-contiguous or [K,N] N-contiguous
// covers the three GEMMs of a linear layer without any transposed copy:
//   forward   Y  = X  W^T   (A = X  K-major,  B = W  K-major)
//   dgrad     dX = dY W     (A = dY K-major,  B = W  MN-major)
//   wgrad     dW += dY^T X  (A = dY MN-major, B = X  MN-major, fp32 accumulate epilogue)
//
// CTA = 6 warps: warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2-5 epilogue
// (one per TMEM lane quadrant). Tile 128 x 256 x 64, 4 smem stages (192 KB), persistent
// over tiles. No cluster multicast is used anywhere. Every mbarrier wait is bounded; on
// expiry the CTA records TPLR_ST_WAIT_TIMEOUT in *status, all roles leave their loops, TMEM
// is freed and the kernel returns.
//
// Replaces the cuBLAS GEMMs behind the reference's nn.Linear layers
// (torchtitan models/llama3/model/model.py:140-147, :236-237, :351).
#include "tcgen05.cuh"

namespace {
using namespace tplr_tc;

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;   // 16 KB
constexpr int B_STAGE_BYTES = BN * BK * 2;   // 32 KB
constexpr int SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 1024 /*align slack*/;
constexpr int NUM_THREADS = 192;

// EPI: 0 store bf16, 1 fp32 accumulate (C += acc), 2 store fp32
template <bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 void* __restrict__ Cptr, int M, int N, int K, long long ldc, unsigned int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t bar_full[STAGES], bar_empty[STAGES], bar_tfull[2], bar_tempty[2];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = (K + BK - 1) / BK;
  volatile int* abort_flag = &s_abort;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < STAGES; ++s) { mbar_init(smem_u32(&bar_full[s]), 1); mbar_init(smem_u32(&bar_empty[s]), 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(smem_u32(&bar_tfull[s]), 1); mbar_init(smem_u32(&bar_tempty[s]), 4); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&s_tmem_base)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  const uint32_t sA = smem_u32(smem), sB = sA + STAGES * A_STAGE_BYTES;

  if (warp == 0) {
    // ----------------------------- TMA producer ------------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int m0 = (t % tiles_m) * BM, n0 = (t / tiles_m) * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!(ok = mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1, abort_flag))) break;
          const uint32_t fb = smem_u32(&bar_full[s]);
          mbar_expect_tx(fb, A_STAGE_BYTES + B_STAGE_BYTES);
          const uint32_t a_dst = sA + s * A_STAGE_BYTES, b_dst = sB + s * B_STAGE_BYTES;
          const int k0 = kb * BK;
          if (!A_MN) {
            tma_load_2d(a_dst, &tmA, fb, k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(a_dst + j * (BK * 128), &tmA, fb, m0 + 64 * j, k0);
          }
          if (!B_MN) {
            tma_load_2d(b_dst, &tmB, fb, k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * (BK * 128), &tmB, fb, n0 + 64 * j, k0);
          }
        }
      }
      // drain: every armed stage must have landed before the CTA may retire
      for (uint32_t back = 0; back < STAGES && back < it; ++back) {
        const uint32_t j = it - 1 - back;
        mbar_wait(smem_u32(&bar_full[j % STAGES]), (j / STAGES) & 1, abort_flag);
      }
    }
  } else if (warp == 1) {
    // ----------------------------- MMA issuer --------------------------------------
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) |
                             ((B_MN ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      uint32_t it = 0, tile_i = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_i) {
        const uint32_t acc = tile_i & 1, acc_ph = (tile_i >> 1) & 1;
        if (!(ok = mbar_wait(smem_u32(&bar_tempty[acc]), acc_ph ^ 1, abort_flag))) break;
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!(ok = mbar_wait(smem_u32(&bar_full[s]), ph, abort_flag))) break;
          tcgen05_fence_after();
          const uint32_t a_base = sA + s * A_STAGE_BYTES, b_base = sB + s * B_STAGE_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t da = A_MN ? make_desc(a_base + kk * (UMMA_K * 128), BK * 128, 1024)
                                     : make_desc(a_base + kk * (UMMA_K * 2), 16, 1024);
            const uint64_t db = B_MN ? make_desc(b_base + kk * (UMMA_K * 128), BK * 128, 1024)
                                     : make_desc(b_base + kk * (UMMA_K * 2), 16, 1024);
            umma_bf16(d_tmem, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(smem_u32(&bar_empty[s]));
        }
        if (ok) umma_commit(smem_u32(&bar_tfull[acc]));
      }
    }
  } else {
    // ----------------------------- epilogue (warps 2..5) ---------------------------
    const int quad = warp & 3;   // TMEM lane quadrant this warp may access
    uint32_t tile_i = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_i) {
      const int m0 = (t % tiles_m) * BM, n0 = (t / tiles_m) * BN;
      const uint32_t acc = tile_i & 1, acc_ph = (tile_i >> 1) & 1;
      ok = mbar_wait(smem_u32(&bar_tfull[acc]), acc_ph, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const int row = m0 + quad * 32 + lane;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_base + acc * BN + c * 32 + ((uint32_t)(quad * 32) << 16), r);
        const int col0 = n0 + c * 32;
        if (row < M && col0 < N) {
          if (EPI == 0) {
            __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(Cptr) + (long long)row * ldc + col0;
            if (col0 + 32 <= N && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0)) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint4 pk;
                uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[8 * v + 2 * e]), __uint_as_float(r[8 * v + 2 * e + 1]));
                  pw[e] = *reinterpret_cast<uint32_t*>(&h);
                }
                reinterpret_cast<uint4*>(crow)[v] = pk;
              }
            } else {
              for (int e = 0; e < 32 && col0 + e < N; ++e) crow[e] = __float2bfloat16(__uint_as_float(r[e]));
            }
          } else {
            float* crow = reinterpret_cast<float*>(Cptr) + (long long)row * ldc + col0;
            if (col0 + 32 <= N && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0)) {
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                float4 o = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                       __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
                if (EPI == 1) {
                  const float4 old = reinterpret_cast<const float4*>(crow)[v];
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                reinterpret_cast<float4*>(crow)[v] = o;
              }
            } else {
              for (int e = 0; e < 32 && col0 + e < N; ++e) {
                const float o = __uint_as_float(r[e]);
                crow[e] = (EPI == 1) ? crow[e] + o : o;
              }
            }
          }
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_tempty[acc]));
    }
  }
  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
  }
  if (threadIdx.x == 0 && s_abort && status) atomicOr(status, TPLR_ST_WAIT_TIMEOUT);
}

template <bool A_MN, bool B_MN, int EPI>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, void* C, int M, int N, int K, long long ldc,
           unsigned int* status, int max_ctas, cudaStream_t st) {
  auto kern = gemm_bf16_kernel<A_MN, B_MN, EPI>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return (int)e;
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int grid = tplr_sm_count();
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  if (grid > tiles) grid = tiles;
  kern<<<grid, NUM_THREADS, SMEM_BYTES, st>>>(ta, tb, C, M, N, K, ldc, status);
  return (int)cudaGetLastError();
}

}  // namespace

// a_mn = 0: A is [M,K] row-major with leading dimension lda (elements); a_mn = 1: A is [K,M] row-major.
// b_mn = 0: B is [N,K] row-major with leading dimension ldb;            b_mn = 1: B is [K,N] row-major.
// epi: 0 C bf16 = acc, 1 C fp32 += acc, 2 C fp32 = acc.  All base pointers 16-byte aligned and
// leading dimensions multiples of 8 elements (TMA stride rule).  max_ctas <= 0: one CTA per SM.
TPLR_API int tplr_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                            long long ldb, long long ldc, int a_mn, int b_mn, int epi, unsigned int* status,
                            int max_ctas, void* stream) {
  TPLR_ENTER();
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  // negative return codes are this library's own argument errors (CUDA errors are positive)
  if ((lda % 8) || (ldb % 8) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return -101;
  CUtensorMap ta, tb;
  if (!(a_mn ? make_map(&ta, A, M, K, lda, 64, BK) : make_map(&ta, A, K, M, lda, BK, BM))) return -102;
  if (!(b_mn ? make_map(&tb, B, N, K, ldb, 64, BK) : make_map(&tb, B, K, N, ldb, BK, BN))) return -103;
  cudaStream_t st = (cudaStream_t)stream;
#define TPLR_GEMM_CASE(AM, BMJ, E) \
  if (a_mn == AM && b_mn == BMJ && epi == E) return launch<AM != 0, BMJ != 0, E>(ta, tb, C, M, N, K, ldc, status, max_ctas, st);
  TPLR_GEMM_CASE(0, 0, 0) TPLR_GEMM_CASE(0, 0, 1) TPLR_GEMM_CASE(0, 0, 2)
  TPLR_GEMM_CASE(0, 1, 0) TPLR_GEMM_CASE(0, 1, 1) TPLR_GEMM_CASE(0, 1, 2)
  TPLR_GEMM_CASE(1, 1, 0) TPLR_GEMM_CASE(1, 1, 1) TPLR_GEMM_CASE(1, 1, 2)
  TPLR_GEMM_CASE(1, 0, 0) TPLR_GEMM_CASE(1, 0, 1) TPLR_GEMM_CASE(1, 0, 2)
#undef TPLR_GEMM_CASE
  return -104;
}
