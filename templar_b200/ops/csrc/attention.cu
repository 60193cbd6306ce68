// Causal flash attention on tcgen05 (sm_100a): S = Q K^T and O += P V run on the 5th-generation
// tensor cores with the accumulators in tensor memory; the softmax reads its row of S straight
// from TMEM (lane = query row, so row max / row sum need no shuffles), writes P back into the
// same TMEM columns as packed bf16 and the second MMA takes P from TMEM as its A operand.
//
// Operands come from the packed projection output [B*S, (H + 2 KV) * 128] (q heads, k heads,
// v heads; RoPE already applied in place), loaded by TMA with 128-byte swizzle; no copy splits
// q, k and v.  Head dimension 128, sequence length a multiple of 128, grouped-query heads.
//
// CTA = one 128-row query block of one head: warp 0 TMA producer, warp 1 MMA issuer + TMEM
// owner, warps 2-5 softmax / correction / epilogue.  256 TMEM columns and 97 KB of shared
// memory per CTA, so two CTAs share an SM and one's softmax overlaps the other's MMAs.
// The running maximum is only raised when it grows by more than 2^8 (any consistent reference
// value gives the same result), which keeps the O-rescale off the common path.
// Every mbarrier wait is bounded; on expiry TPLR_ST_WAIT_TIMEOUT is set and all roles return.
//
// Replaces F.scaled_dot_product_attention(is_causal=True) of the reference model
// (torchtitan models/llama3/model/model.py:203-206, :244-262).
#include "tcgen05.cuh"
#include <cuda/std/type_traits>
#include <stdlib.h>

namespace {
using namespace tplr_tc;

constexpr int BQ = 128, BKV = 128, DH = 128;
constexpr int TILE_BYTES = 128 * DH * 2;                 // 32 KB: one 128 x 128 bf16 tile
constexpr int FWD_SMEM = 3 * TILE_BYTES + 1024;          // Q, K, V
constexpr int FWD_THREADS = 192;
constexpr float RESCALE_THRESHOLD = 8.0f;                // log2 units

struct AttnFwdParams {
  CUtensorMap tmQKV;      // [B*S, C] bf16, box 64 x 128, 128-byte swizzle
  CUtensorMap tmO;        // [B*S, H*128] bf16, box 64 x 32, 128-byte swizzle
  float* lse;             // [B, H, S] natural-log sum-exp of the scaled scores
  int B, S, H, KV;
  float scale_log2;       // softmax scale * log2(e)
  unsigned int* status;
};

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(src), "r"(x), "r"(y) : "memory");
}

// instruction descriptor: fp32 accumulate, bf16 A and B, M = 128, N = 128; b_mn selects an N-contiguous B
__device__ __forceinline__ uint32_t idesc_128x128(bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(128 >> 3) << 17) |
         ((uint32_t)(128 >> 4) << 24);
}

// Softmax passes over one row of S (128 fp32 columns in tensor memory, lane = query row).  DIAG = the block
// on the diagonal (columns above the row are masked); the other blocks run the variant without the per-element
// compare and select, which is a third of the instructions of the issue-bound softmax warps.
// packed fp32 pairs (sm_100): one instruction for two lanes of fma / add, and the three-input max
__device__ __forceinline__ unsigned long long pack_f32x2(uint32_t lo, uint32_t hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma_f32x2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ unsigned long long add_f32x2(unsigned long long a, unsigned long long b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

template <bool DIAG>
__device__ __forceinline__ float attn_row_max(uint32_t ts_lane, int r) {
  float mx = -INFINITY;
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {
    uint32_t v[32];
    tmem_ld32(ts_lane + c * 32, v);
    if (DIAG) {
#pragma unroll
      for (int e = 0; e < 32; ++e) mx = fmaxf(mx, (c * 32 + e > r) ? -INFINITY : __uint_as_float(v[e]));
    } else {
#pragma unroll
      for (int e = 0; e < 16; ++e) mx = max3(mx, __uint_as_float(v[2 * e]), __uint_as_float(v[2 * e + 1]));
    }
  }
  return mx;
}
// P = exp2(S * scale - m) written as packed bf16 over the first 64 columns of S; returns the row sum of P.
template <bool DIAG>
__device__ __forceinline__ float attn_row_exp(uint32_t ts_lane, int r, float sl2, float m_used) {
  const unsigned long long sl2x2 = pack_f32x2(__float_as_uint(sl2), __float_as_uint(sl2));
  const unsigned long long negm = pack_f32x2(__float_as_uint(-m_used), __float_as_uint(-m_used));
  unsigned long long sum = 0ull;                         // (0.f, 0.f)
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {
    uint32_t v[32], pk[16];
    tmem_ld32(ts_lane + c * 32, v);
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      float a0, a1;
      unpack_f32x2(fma_f32x2(pack_f32x2(v[2 * e], v[2 * e + 1]), sl2x2, negm), a0, a1);
      float p0 = exp2f(a0), p1 = exp2f(a1);
      if (DIAG) {
        if (c * 32 + 2 * e > r) p0 = 0.f;
        if (c * 32 + 2 * e + 1 > r) p1 = 0.f;
      }
      sum = add_f32x2(sum, pack_f32x2(__float_as_uint(p0), __float_as_uint(p1)));
      __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
      pk[e] = *reinterpret_cast<uint32_t*>(&hh);
    }
    tmem_st16(ts_lane + c * 16, pk);
  }
  float s0, s1;
  unpack_f32x2(sum, s0, s1);
  return s0 + s1;
}

__global__ void __launch_bounds__(FWD_THREADS, 2)
attn_fwd_kernel(const __grid_constant__ AttnFwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t bar_q, bar_k_full, bar_k_empty, bar_v_full, bar_v_empty, bar_s_full, bar_p_full, bar_o_full;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nQ = p.S / BQ;
  // heavy (late) query blocks first
  const int hb = p.H * p.B;
  const int qi = nQ - 1 - (int)(blockIdx.x / hb);
  const int h = (int)(blockIdx.x % hb) % p.H, b = (int)(blockIdx.x % hb) / p.H;
  const int g = h / (p.H / p.KV);
  const int nb = qi + 1;                                   // causal: kv blocks 0..qi
  const int row0 = b * p.S + qi * BQ;
  const int qcol = h * DH, kcol = (p.H + g) * DH, vcol = (p.H + p.KV + g) * DH;
  volatile int* abort_flag = &s_abort;

  if (threadIdx.x == 0) {
    s_abort = 0;
    mbar_init(smem_u32(&bar_q), 1);
    mbar_init(smem_u32(&bar_k_full), 1); mbar_init(smem_u32(&bar_k_empty), 1);
    mbar_init(smem_u32(&bar_v_full), 1); mbar_init(smem_u32(&bar_v_empty), 1);
    mbar_init(smem_u32(&bar_s_full), 1); mbar_init(smem_u32(&bar_p_full), 4);
    mbar_init(smem_u32(&bar_o_full), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 256;" ::"r"(smem_u32(&s_tmem_base)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  const uint32_t tS = tmem_base, tO = tmem_base + 128;     // S / P columns 0..127, O columns 128..255
  const uint32_t sQ = smem_u32(smem), sK = sQ + TILE_BYTES, sV = sK + TILE_BYTES;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(smem_u32(&bar_q), TILE_BYTES);
      tma_load_2d(sQ, &p.tmQKV, smem_u32(&bar_q), qcol, row0);
      tma_load_2d(sQ + TILE_BYTES / 2, &p.tmQKV, smem_u32(&bar_q), qcol + 64, row0);
      bool ok = true;
      for (int j = 0; j < nb && ok; ++j) {
        const uint32_t ph = j & 1;
        const int krow = b * p.S + j * BKV;
        if (!(ok = mbar_wait(smem_u32(&bar_k_empty), ph ^ 1, abort_flag))) break;
        mbar_expect_tx(smem_u32(&bar_k_full), TILE_BYTES);
        tma_load_2d(sK, &p.tmQKV, smem_u32(&bar_k_full), kcol, krow);
        tma_load_2d(sK + TILE_BYTES / 2, &p.tmQKV, smem_u32(&bar_k_full), kcol + 64, krow);
        if (!(ok = mbar_wait(smem_u32(&bar_v_empty), ph ^ 1, abort_flag))) break;
        mbar_expect_tx(smem_u32(&bar_v_full), TILE_BYTES);
        tma_load_2d(sV, &p.tmQKV, smem_u32(&bar_v_full), vcol, krow);
        tma_load_2d(sV + TILE_BYTES / 2, &p.tmQKV, smem_u32(&bar_v_full), vcol + 64, krow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t id_qk = idesc_128x128(false), id_pv = idesc_128x128(true);
      const DescBase bQ = desc_base(sQ, 16, 1024), bK = desc_base(sK, 16, 1024), bV = desc_base(sV, TILE_BYTES / 2, 1024);
      bool ok = mbar_wait(smem_u32(&bar_q), 0, abort_flag);
      for (int j = 0; j < nb && ok; ++j) {
        const uint32_t ph = j & 1;
        if (!(ok = mbar_wait(smem_u32(&bar_k_full), ph, abort_flag))) break;
        tcgen05_fence_after();
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
          const uint32_t off = (uint32_t)(kk >> 2) * (TILE_BYTES / 32) + (uint32_t)(kk & 3) * 2u;    // 16-byte units
          umma_bf16_b(tS, bQ, off, bK, off, id_qk, kk > 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(&bar_s_full));
        umma_commit(smem_u32(&bar_k_empty));
        if (!(ok = mbar_wait(smem_u32(&bar_p_full), ph, abort_flag))) break;
        if (!(ok = mbar_wait(smem_u32(&bar_v_full), ph, abort_flag))) break;
        tcgen05_fence_after();
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk)
          umma_ts_bf16_b(tO, tS + 8 * kk, bV, (uint32_t)kk * 128u, id_pv, (j > 0 || kk > 0) ? 1u : 0u);
        umma_commit(smem_u32(&bar_v_empty));
        if (j == nb - 1) umma_commit(smem_u32(&bar_o_full));
      }
    }
  } else {
    const int quad = warp & 3;
    const int r = quad * 32 + lane;                        // query row inside the block = TMEM lane
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nb && ok; ++j) {
      ok = mbar_wait(smem_u32(&bar_s_full), j & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const bool diag = j == qi;
      // pass 1: row maximum of the scores
      const float mx = diag ? attn_row_max<true>(tS + lane_off, r) : attn_row_max<false>(tS + lane_off, r);
      const float m_new = fmaxf(m_used, mx * p.scale_log2);
      const bool need = m_new > m_used + RESCALE_THRESHOLD;       // true for the first block (m_used = -inf)
      if (__any_sync(0xffffffffu, need)) {
        const float alpha = need ? exp2f(m_used - m_new) : 1.f;   // 0 for the first block
        if (need) { m_used = m_new; l *= alpha; }
        if (j > 0) {
          // S of block j is complete, so every earlier MMA, PV of block j-1 included, has finished with O
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t v[32];
            tmem_ld32(tO + c * 32 + lane_off, v);
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * alpha);
            tmem_st32(tO + c * 32 + lane_off, v);
          }
        }
      }
      // pass 2: P as packed bf16 over the first 64 columns of S
      l += diag ? attn_row_exp<true>(tS + lane_off, r, p.scale_log2, m_used)
                : attn_row_exp<false>(tS + lane_off, r, p.scale_log2, m_used);
      tmem_wait_st();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_p_full));
    }
    // epilogue: O / l -> bf16 -> swizzled staging (the Q tile is no longer read) -> TMA store
    if (ok) ok = mbar_wait(smem_u32(&bar_o_full), 0, abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tcgen05_fence_after();
      const float inv_l = 1.f / l;
      const uint32_t stage = sQ + (uint32_t)quad * 8192u;
      const uint32_t sw = (uint32_t)(lane & 7);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(tO + c * 32 + lane_off, v);
        const uint32_t rowaddr = stage + (uint32_t)(c >> 1) * 4096u + (uint32_t)lane * 128u;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint32_t pw[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(v[8 * q4 + 2 * e]) * inv_l,
                                                      __uint_as_float(v[8 * q4 + 2 * e + 1]) * inv_l);
            pw[e] = *reinterpret_cast<uint32_t*>(&hh);
          }
          const uint32_t jj = (uint32_t)((c & 1) * 4 + q4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + ((jj ^ sw) << 4)), "r"(pw[0]), "r"(pw[1]),
                       "r"(pw[2]), "r"(pw[3]) : "memory");
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(&p.tmO, stage, qcol, row0 + quad * 32);
        tma_store_2d(&p.tmO, stage + 4096u, qcol + 64, row0 + quad * 32);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      }
      if (p.lse) p.lse[((long long)b * p.H + h) * p.S + qi * BQ + r] = (m_used + log2f(l)) * 0.6931471805599453f;
    }
  }
  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;" ::"r"(tmem_base) : "memory");
  }
  if (threadIdx.x == 0 && s_abort && p.status) atomicOr(p.status, TPLR_ST_WAIT_TIMEOUT);
}

}  // namespace

// qkv: packed [B*S, (H + 2*KV) * 128] bf16 (row stride ld_qkv elements); out: [B*S, H*128] bf16 (row stride ld_o);
// lse: [B, H, S] fp32 or null.  S must be a multiple of 128 and H a multiple of KV.
TPLR_API int tplr_attention_fwd(const void* qkv, void* out, float* lse, int B, int S, int H, int KV, long long ld_qkv,
                                long long ld_o, float scale, unsigned int* status, void* stream) {
  TPLR_ENTER();
  if (B <= 0 || S <= 0) return 0;
  if (S % BQ || H % KV || (ld_qkv % 8) || (ld_o % 8) || ((uintptr_t)qkv & 15) || ((uintptr_t)out & 15)) return -201;
  AttnFwdParams p = {};
  if (!make_map(&p.tmQKV, qkv, (long long)(H + 2 * KV) * DH, (long long)B * S, ld_qkv, 64, 128)) return -202;
  if (!make_map(&p.tmO, out, (long long)H * DH, (long long)B * S, ld_o, 64, 32)) return -203;
  p.lse = lse; p.B = B; p.S = S; p.H = H; p.KV = KV;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM);
  if (e != cudaSuccess) return (int)e;
  const unsigned grid = (unsigned)((S / BQ) * H * B);
  attn_fwd_kernel<<<grid, FWD_THREADS, FWD_SMEM, (cudaStream_t)stream>>>(p);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------ //
// Backward.  CTA = one 128-row key/value block of one kv head; it walks the query heads of the
// group and the query blocks at or below the diagonal.  Per step:
//   S = Q K^T, dP = dO V^T            (tensor cores -> TMEM)
//   P = exp2(S*scale - lse), dS = P * (dP - delta) * scale   (softmax warps, one query row per thread;
//                                      P and dS go to shared memory as bf16 in 128-byte-swizzled tiles)
//   dV += P^T dO, dK += dS^T Q        (accumulated in TMEM over the whole walk)
//   dQ_partial = dS K                 (into the S columns, then TMA reduce-add into the fp32 dQ buffer)
// The same swizzled tile serves as a K-major operand of one MMA and an MN-major operand of another,
// so Q, dO, P and dS are each stored once.  K and V stay resident in shared memory.
// ------------------------------------------------------------------------------------------ //
namespace {

constexpr int BWD_SMEM = 6 * TILE_BYTES + 1024;
constexpr int BWD_THREADS = 320;                        // TMA warp, MMA warp, 8 softmax warps (2 per TMEM lane quadrant)

struct AttnBwdParams {
  CUtensorMap tmQKV;    // [B*S, C] bf16, box 64 x 128
  CUtensorMap tmDO;     // [B*S, H*128] bf16, box 64 x 128
  CUtensorMap tmDQ;     // [B*S, H*128] fp32, box 32 x 32 (reduce-add target)
  CUtensorMap tmDQKV;   // [B*S, C] bf16, box 64 x 32 (dK and dV stores)
  const float* lse;
  const float* delta;
  int B, S, H, KV;
  float scale, scale_log2;
  unsigned int* status;
  // not null: q and k were rotated (rotary embedding, interleaved pairs, tables [S, 64] fp32) by the producer of qkv and
  // the gradient is wanted with respect to the un-rotated projection: dK is rotated back in the epilogue
  const float* rope_cos;
  const float* rope_sin;
};

__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(src), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ uint32_t idesc_bwd(bool a_mn, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ AttnBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t bar_kv, bar_q_full, bar_q_empty, bar_do_full, bar_do_empty, bar_sp_full, bar_pds_full, bar_dq_full, bar_s_free;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nQ = p.S / BQ;
  const int gb = p.KV * p.B;
  const int j = (int)(blockIdx.x / gb);                    // kv block; small j (long walks) first
  const int g = (int)(blockIdx.x % gb) % p.KV, b = (int)(blockIdx.x % gb) / p.KV;
  const int group = p.H / p.KV;
  const int n_i = nQ - j;                                  // query blocks j..nQ-1
  const int n_it = group * n_i;
  const int kvrow0 = b * p.S + j * BKV;
  const int kcol = (p.H + g) * DH, vcol = (p.H + p.KV + g) * DH;
  volatile int* abort_flag = &s_abort;

  if (threadIdx.x == 0) {
    s_abort = 0;
    mbar_init(smem_u32(&bar_kv), 1);
    mbar_init(smem_u32(&bar_q_full), 1); mbar_init(smem_u32(&bar_q_empty), 1);
    mbar_init(smem_u32(&bar_do_full), 1); mbar_init(smem_u32(&bar_do_empty), 1);
    mbar_init(smem_u32(&bar_sp_full), 1); mbar_init(smem_u32(&bar_pds_full), 8);
    mbar_init(smem_u32(&bar_dq_full), 1); mbar_init(smem_u32(&bar_s_free), 8);
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
  const uint32_t tS = tmem_base, tdP = tmem_base + 128, tdV = tmem_base + 256, tdK = tmem_base + 384;
  const uint32_t sK = smem_u32(smem), sV = sK + TILE_BYTES, sQ = sV + TILE_BYTES, sdO = sQ + TILE_BYTES,
                 sP = sdO + TILE_BYTES, sdS = sP + TILE_BYTES;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(smem_u32(&bar_kv), 2 * TILE_BYTES);
      tma_load_2d(sK, &p.tmQKV, smem_u32(&bar_kv), kcol, kvrow0);
      tma_load_2d(sK + TILE_BYTES / 2, &p.tmQKV, smem_u32(&bar_kv), kcol + 64, kvrow0);
      tma_load_2d(sV, &p.tmQKV, smem_u32(&bar_kv), vcol, kvrow0);
      tma_load_2d(sV + TILE_BYTES / 2, &p.tmQKV, smem_u32(&bar_kv), vcol + 64, kvrow0);
      bool ok = true;
      for (int t = 0; t < n_it && ok; ++t) {
        const int h = g * group + t / n_i, i = j + t % n_i;
        const int qrow0 = b * p.S + i * BQ, qcol = h * DH;
        // Q is released by the dK MMAs and dO by the dV MMAs of the previous step, both before its dQ MMAs and the
        // dQ drain: the next tiles are in flight while those run
        if (!(ok = mbar_wait(smem_u32(&bar_q_empty), (uint32_t)((t & 1) ^ 1), abort_flag))) break;
        const uint32_t fq = smem_u32(&bar_q_full);
        mbar_expect_tx(fq, TILE_BYTES);
        tma_load_2d(sQ, &p.tmQKV, fq, qcol, qrow0);
        tma_load_2d(sQ + TILE_BYTES / 2, &p.tmQKV, fq, qcol + 64, qrow0);
        if (!(ok = mbar_wait(smem_u32(&bar_do_empty), (uint32_t)((t & 1) ^ 1), abort_flag))) break;
        const uint32_t fd = smem_u32(&bar_do_full);
        mbar_expect_tx(fd, TILE_BYTES);
        tma_load_2d(sdO, &p.tmDO, fd, qcol, qrow0);
        tma_load_2d(sdO + TILE_BYTES / 2, &p.tmDO, fd, qcol + 64, qrow0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t id_kk = idesc_bwd(false, false), id_mm = idesc_bwd(true, true), id_km = idesc_bwd(false, true);
      // descriptor bases: "k" = contraction along the 128-byte rows, "m" = contraction along the tile rows
      const DescBase kQ = desc_base(sQ, 16, 1024), kK = desc_base(sK, 16, 1024), kdO = desc_base(sdO, 16, 1024),
                     kV = desc_base(sV, 16, 1024), kdS = desc_base(sdS, 16, 1024);
      const DescBase mP = desc_base(sP, TILE_BYTES / 2, 1024), mdO = desc_base(sdO, TILE_BYTES / 2, 1024),
                     mdS = desc_base(sdS, TILE_BYTES / 2, 1024), mQ = desc_base(sQ, TILE_BYTES / 2, 1024),
                     mK = desc_base(sK, TILE_BYTES / 2, 1024);
#define TPLR_KOFF(kk) ((uint32_t)((kk) >> 2) * (TILE_BYTES / 32) + (uint32_t)((kk) & 3) * 2u)
#define TPLR_MOFF(kk) ((uint32_t)(kk) * 128u)
      bool ok = mbar_wait(smem_u32(&bar_kv), 0, abort_flag);
      for (int t = 0; t < n_it && ok; ++t) {
        const uint32_t ph = t & 1;
        if (!(ok = mbar_wait(smem_u32(&bar_q_full), ph, abort_flag))) break;
        if (t > 0 && !(ok = mbar_wait(smem_u32(&bar_s_free), ph ^ 1, abort_flag))) break;
        tcgen05_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) umma_bf16_b(tS, kQ, TPLR_KOFF(kk), kK, TPLR_KOFF(kk), id_kk, kk > 0 ? 1u : 0u);
        if (!(ok = mbar_wait(smem_u32(&bar_do_full), ph, abort_flag))) break;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) umma_bf16_b(tdP, kdO, TPLR_KOFF(kk), kV, TPLR_KOFF(kk), id_kk, kk > 0 ? 1u : 0u);
        umma_commit(smem_u32(&bar_sp_full));
        if (!(ok = mbar_wait(smem_u32(&bar_pds_full), ph, abort_flag))) break;
        tcgen05_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)      // dK[kv, d] += dS^T[kv, q] Q[q, d]   (first: Q is what the next step needs first)
          umma_bf16_b(tdK, mdS, TPLR_MOFF(kk), mQ, TPLR_MOFF(kk), id_mm, (t > 0 || kk > 0) ? 1u : 0u);
        umma_commit(smem_u32(&bar_q_empty));
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)      // dV[kv, d] += P^T[kv, q] dO[q, d]
          umma_bf16_b(tdV, mP, TPLR_MOFF(kk), mdO, TPLR_MOFF(kk), id_mm, (t > 0 || kk > 0) ? 1u : 0u);
        umma_commit(smem_u32(&bar_do_empty));
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)      // dQ[q, d] = dS[q, kv] K[kv, d]
          umma_bf16_b(tS, kdS, TPLR_KOFF(kk), mK, TPLR_MOFF(kk), id_km, kk > 0 ? 1u : 0u);
        umma_commit(smem_u32(&bar_dq_full));
      }
    }
  } else {
    const int quad = warp & 3;                 // TMEM lane quadrant this warp may access
    const int ch = (warp - 2) >> 2;            // column half (64 columns) this warp works on
    const int r = quad * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const uint32_t sw = (uint32_t)(lane & 7);
    // two private 4 KB staging buffers: the bytes of this warp's own rows and column half in the P and dS tiles
    const uint32_t stg0 = sP + (uint32_t)ch * (TILE_BYTES / 2) + (uint32_t)quad * 4096u;
    const uint32_t stg1 = sdS + (uint32_t)ch * (TILE_BYTES / 2) + (uint32_t)quad * 4096u;
    bool ok = true;
    for (int t = 0; t < n_it && ok; ++t) {
      const int h = g * group + t / n_i, i = j + t % n_i;
      const long long stat = ((long long)b * p.H + h) * p.S + i * BQ + r;
      const float lse2 = p.lse[stat] * 1.4426950408889634f;
      const float dl = p.delta[stat];
      ok = mbar_wait(smem_u32(&bar_sp_full), t & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      // P and dS of this warp's two 32-column chunks; the diagonal block runs the variant with the causal mask,
      // the others the one without the per-element compare (the softmax warps are issue-bound).  dS carries the
      // softmax scale: d = p * (dp - delta) * scale = p * fma(dp, scale, -delta * scale).
      const float dls = dl * p.scale;
      auto chunk_pair = [&](auto DIAG) {
        constexpr bool kDiag = decltype(DIAG)::value;
#pragma unroll 1
        for (int c = 2 * ch; c < 2 * ch + 2; ++c) {
          uint32_t sv[32], dv[32];
          tmem_ld32(tS + c * 32 + lane_off, sv);
          tmem_ld32(tdP + c * 32 + lane_off, dv);
          const uint32_t prow = sP + (uint32_t)(c >> 1) * (TILE_BYTES / 2) + (uint32_t)r * 128u;
          const uint32_t drow = sdS + (uint32_t)(c >> 1) * (TILE_BYTES / 2) + (uint32_t)r * 128u;
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint32_t pw[4], dw[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float p0 = exp2f(fmaf(__uint_as_float(sv[q4 * 8 + 2 * e]), p.scale_log2, -lse2));
              float p1 = exp2f(fmaf(__uint_as_float(sv[q4 * 8 + 2 * e + 1]), p.scale_log2, -lse2));
              if (kDiag) {
                const int col = c * 32 + q4 * 8 + 2 * e;
                if (col > r) p0 = 0.f;
                if (col + 1 > r) p1 = 0.f;
              }
              const float d0 = p0 * fmaf(__uint_as_float(dv[q4 * 8 + 2 * e]), p.scale, -dls);
              const float d1 = p1 * fmaf(__uint_as_float(dv[q4 * 8 + 2 * e + 1]), p.scale, -dls);
              __nv_bfloat162 hp = __floats2bfloat162_rn(p0, p1), hd = __floats2bfloat162_rn(d0, d1);
              pw[e] = *reinterpret_cast<uint32_t*>(&hp);
              dw[e] = *reinterpret_cast<uint32_t*>(&hd);
            }
            const uint32_t off = (((uint32_t)((c & 1) * 4 + q4)) ^ sw) << 4;
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(prow + off), "r"(pw[0]), "r"(pw[1]), "r"(pw[2]), "r"(pw[3]) : "memory");
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(drow + off), "r"(dw[0]), "r"(dw[1]), "r"(dw[2]), "r"(dw[3]) : "memory");
          }
        }
      };
      if (i == j) chunk_pair(cuda::std::true_type{}); else chunk_pair(cuda::std::false_type{});
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_pds_full));
      // drain dQ_partial (fp32, in the S columns) into the global fp32 dQ with TMA reduce-add
      ok = mbar_wait(smem_u32(&bar_dq_full), t & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const int qrow0 = b * p.S + i * BQ + quad * 32;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = 2 * ch + cc;
        uint32_t v[32];
        tmem_ld32(tS + c * 32 + lane_off, v);
        const uint32_t buf = cc ? stg1 : stg0;
        const uint32_t rowaddr = buf + (uint32_t)lane * 128u;
#pragma unroll
        for (int q8 = 0; q8 < 8; ++q8)
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + (((uint32_t)q8 ^ sw) << 4)), "r"(v[4 * q8]),
                       "r"(v[4 * q8 + 1]), "r"(v[4 * q8 + 2]), "r"(v[4 * q8 + 3]) : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          tma_reduce_add_2d(&p.tmDQ, buf, h * DH + c * 32, qrow0);
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
      if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // P rows may be rewritten
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_s_free));
    }
    // dV and dK of this kv block: TMEM -> bf16 -> staging -> TMA store into the packed gradient
    if (ok) {
      tcgen05_fence_after();
      const int orow0 = kvrow0 + quad * 32;
#pragma unroll
      for (int acc = 0; acc < 2; ++acc) {      // 0 = dV, 1 = dK; this warp stores its 64-column half of each
        const uint32_t tacc = acc ? tdK : tdV;
        const uint32_t buf = acc ? stg1 : stg0;
        const uint32_t rowaddr = buf + (uint32_t)lane * 128u;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          uint32_t v[32];
          tmem_ld32(tacc + ch * 64 + hf * 32 + lane_off, v);
          if (acc == 1 && p.rope_cos) {          // dK back through the rotation of this key row: the opposite angle
            const long long tb = (long long)((orow0 + lane) % p.S) * (DH / 2) + (ch * 64 + hf * 32) / 2;
            const float4* cp = reinterpret_cast<const float4*>(p.rope_cos + tb);
            const float4* sp = reinterpret_cast<const float4*>(p.rope_sin + tb);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float4 cv = cp[q], sv = sp[q];
              const float cc[4] = {cv.x, cv.y, cv.z, cv.w}, ss[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float a = __uint_as_float(v[8 * q + 2 * e]), b = __uint_as_float(v[8 * q + 2 * e + 1]);
                v[8 * q + 2 * e] = __float_as_uint(a * cc[e] + b * ss[e]);
                v[8 * q + 2 * e + 1] = __float_as_uint(b * cc[e] - a * ss[e]);
              }
            }
          }
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint32_t pw[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(v[8 * q4 + 2 * e]), __uint_as_float(v[8 * q4 + 2 * e + 1]));
              pw[e] = *reinterpret_cast<uint32_t*>(&hh);
            }
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + ((((uint32_t)(hf * 4 + q4)) ^ sw) << 4)),
                         "r"(pw[0]), "r"(pw[1]), "r"(pw[2]), "r"(pw[3]) : "memory");
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&p.tmDQKV, buf, (acc ? kcol : vcol) + ch * 64, orow0);
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }
  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
  }
  if (threadIdx.x == 0 && s_abort && p.status) atomicOr(p.status, TPLR_ST_WAIT_TIMEOUT);
}

// delta[b, h, s] = sum_d dO * O : one warp per (token, head), 4 elements per lane
__global__ void __launch_bounds__(256) attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                                         float* __restrict__ delta, long long tokens, int S, int H,
                                                         long long ld_o) {
  const long long w = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (w >= tokens * H) return;
  const int lane = threadIdx.x & 31;
  const long long tok = w / H;
  const int h = (int)(w % H);
  const uint2 a = *reinterpret_cast<const uint2*>(o + tok * ld_o + h * DH + lane * 4);
  const uint2 d = *reinterpret_cast<const uint2*>(dout + tok * (long long)H * DH + h * DH + lane * 4);
  const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.x));
  const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.y));
  const float2 d0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&d.x));
  const float2 d1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&d.y));
  float s = a0.x * d0.x + a0.y * d0.y + a1.x * d1.x + a1.y * d1.y;
  s = warp_sum(s);
  if (lane == 0) delta[((tok / S) * H + h) * S + tok % S] = s;
}

// dq32 [tokens, H*128] fp32 -> first H*128 columns of the packed bf16 gradient
// cosb / sinb not null: the two pairs are rotated back by the angles of (token % S, pair index in the head) on the way
__global__ void __launch_bounds__(256) attn_dq_cast_kernel(const float* __restrict__ dq32, __nv_bfloat16* __restrict__ dqkv,
                                                           long long tokens, int width, long long ld,
                                                           const float* __restrict__ cosb, const float* __restrict__ sinb, int S) {
  const long long n4 = tokens * (width / 4);
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < n4; v += (long long)gridDim.x * blockDim.x) {
    const long long tok = v / (width / 4);
    const int c4 = (int)(v % (width / 4));
    float4 f = reinterpret_cast<const float4*>(dq32)[v];
    if (cosb) {
      const long long tb = (tok % S) * (DH / 2) + ((c4 * 4) % DH) / 2;
      const float2 c = *reinterpret_cast<const float2*>(cosb + tb), sn = *reinterpret_cast<const float2*>(sinb + tb);
      f = make_float4(f.x * c.x + f.y * sn.x, f.y * c.x - f.x * sn.x, f.z * c.y + f.w * sn.y, f.w * c.y - f.z * sn.y);
    }
    __nv_bfloat162 lo = __floats2bfloat162_rn(f.x, f.y), hi = __floats2bfloat162_rn(f.z, f.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&lo); o.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dqkv + tok * ld + c4 * 4) = o;
  }
}

}  // namespace

// ------------------------------------------------------------------------------------------ //
// Pipelined backward.  Same work split as above (CTA = one 128-row key/value block of one kv head), but a
// step covers 64 query rows and everything is computed transposed, with the key/value row as the TMEM lane:
//   S^T = K Q^T, dP^T = V dO^T          (128 x 64 accumulators)
//   P^T, dS^T                            written back over S^T / dP^T as packed bf16 and fed to the next MMAs
//                                        straight from tensor memory (no shared-memory round trip for P)
//   dV += P^T dO, dK += dS^T Q           (A operand from TMEM)
//   dQ^T = K^T dS^T                      (dS^T also stored once in shared memory as the N-contiguous B operand)
// S^T is double buffered and Q / dO / dS^T are two-stage, so the softmax warps work on step t+1 while the
// tensor cores run dV, dK, dQ^T of step t; dQ^T of step t-1 is drained (TMA reduce-add into a [B,H,128,S] fp32
// scratch) between the P and the dS half of step t.  A last kernel transposes that scratch into the packed gradient.
// ------------------------------------------------------------------------------------------ //
namespace {

constexpr int B2_BQ = 64;
constexpr int B2_QTILE = B2_BQ * DH * 2;                // 16 KB: 64 x 128 bf16 (two blocks of 64 rows x 128 B)
constexpr int B2_DS_TILE = BKV * B2_BQ * 2;             // 16 KB: 128 kv rows x 64 q
constexpr int B2_STAGE = 8 * 4096;                      // dQ^T drain staging, one 32 x 32 fp32 box per warp
constexpr int B2_SMEM = 2 * TILE_BYTES + 4 * B2_QTILE + 2 * B2_DS_TILE + B2_STAGE + 1024 + 1024;
constexpr int B2_THREADS = 320;

struct AttnBwd2Params {
  CUtensorMap tmKV;     // [B*S, C] bf16, box 64 x 128 (K and V tiles)
  CUtensorMap tmQ;      // [B*S, C] bf16, box 64 x 64  (Q tiles)
  CUtensorMap tmDO;     // [B*S, H*128] bf16, box 64 x 64
  CUtensorMap tmDQT;    // [B*H*128, S] fp32, box 32 x 32 (reduce-add target, transposed dQ)
  CUtensorMap tmDQKV;   // [B*S, C] bf16, box 64 x 32 (dK and dV stores)
  const float* lse;
  const float* delta;
  int B, S, H, KV;
  float scale, scale_log2;
  unsigned int* status;
};

__device__ __forceinline__ uint32_t idesc_mn(int n, bool a_mn, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__global__ void __launch_bounds__(B2_THREADS, 1)
attn_bwd2_kernel(const __grid_constant__ AttnBwd2Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t bar_kv, bar_q_full[2], bar_q_empty[2], bar_s_full[2], bar_dp_full, bar_p_ready,
      bar_ds_ready, bar_dq_full, bar_dq_free;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nQ = p.S / B2_BQ;
  const int gb = p.KV * p.B;
  const int j = (int)(blockIdx.x / gb);
  const int g = (int)(blockIdx.x % gb) % p.KV, b = (int)(blockIdx.x % gb) / p.KV;
  const int group = p.H / p.KV;
  const int iq0 = 2 * j, n_i = nQ - iq0, n_it = group * n_i;
  const int kvrow0 = b * p.S + j * BKV;
  const int kcol = (p.H + g) * DH, vcol = (p.H + p.KV + g) * DH;
  volatile int* abort_flag = &s_abort;

  if (threadIdx.x == 0) {
    s_abort = 0;
    mbar_init(smem_u32(&bar_kv), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&bar_q_full[s]), 1); mbar_init(smem_u32(&bar_q_empty[s]), 9);
      mbar_init(smem_u32(&bar_s_full[s]), 1);
    }
    mbar_init(smem_u32(&bar_dp_full), 1); mbar_init(smem_u32(&bar_p_ready), 8); mbar_init(smem_u32(&bar_ds_ready), 8);
    mbar_init(smem_u32(&bar_dq_full), 1); mbar_init(smem_u32(&bar_dq_free), 8);
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
  const uint32_t tS0 = tmem_base, tdP = tmem_base + 128, tdQ = tmem_base + 192, tdV = tmem_base + 256, tdK = tmem_base + 384;
  const uint32_t sK = smem_u32(smem), sV = sK + TILE_BYTES, sQ0 = sV + TILE_BYTES, sdO0 = sQ0 + 2 * B2_QTILE,
                 sdS0 = sdO0 + 2 * B2_QTILE, sStage = sdS0 + 2 * B2_DS_TILE, sStat = sStage + B2_STAGE;
  const float* stat = reinterpret_cast<const float*>(smem + (sStat - sK));     // [2][lse 64 | delta 64]

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(smem_u32(&bar_kv), 2 * TILE_BYTES);
      tma_load_2d(sK, &p.tmKV, smem_u32(&bar_kv), kcol, kvrow0);
      tma_load_2d(sK + TILE_BYTES / 2, &p.tmKV, smem_u32(&bar_kv), kcol + 64, kvrow0);
      tma_load_2d(sV, &p.tmKV, smem_u32(&bar_kv), vcol, kvrow0);
      tma_load_2d(sV + TILE_BYTES / 2, &p.tmKV, smem_u32(&bar_kv), vcol + 64, kvrow0);
      bool ok = true;
      for (int t = 0; t < n_it && ok; ++t) {
        const int s = t & 1, k = t >> 1;
        const int h = g * group + t / n_i, iq = iq0 + t % n_i;
        const int qrow0 = b * p.S + iq * B2_BQ, qcol = h * DH;
        if (!(ok = mbar_wait(smem_u32(&bar_q_empty[s]), (uint32_t)((k & 1) ^ 1), abort_flag))) break;
        const uint32_t fb = smem_u32(&bar_q_full[s]);
        mbar_expect_tx(fb, 2 * B2_QTILE + 512);
        const uint32_t q_dst = sQ0 + s * B2_QTILE, do_dst = sdO0 + s * B2_QTILE;
        tma_load_2d(q_dst, &p.tmQ, fb, qcol, qrow0);
        tma_load_2d(q_dst + 8192, &p.tmQ, fb, qcol + 64, qrow0);
        tma_load_2d(do_dst, &p.tmDO, fb, qcol, qrow0);
        tma_load_2d(do_dst + 8192, &p.tmDO, fb, qcol + 64, qrow0);
        const long long so = ((long long)b * p.H + h) * p.S + (long long)iq * B2_BQ;
        bulk_load_1d(sStat + s * 512, p.lse + so, 256, fb);
        bulk_load_1d(sStat + s * 512 + 256, p.delta + so, 256, fb);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t id_st = idesc_mn(64, false, false);     // S^T, dP^T : K-major A and B, N = 64
      const uint32_t id_dv = idesc_mn(128, false, true);     // dV, dK   : A from TMEM, B N-contiguous, N = 128
      const uint32_t id_dq = idesc_mn(64, true, true);       // dQ^T     : A M-contiguous (K^T), B N-contiguous
      // descriptor bases, built once ("k": contraction along the 128-byte rows, "m": along the tile rows)
      const DescBase kK = desc_base(sK, 16, 1024), kV = desc_base(sV, 16, 1024), mK = desc_base(sK, TILE_BYTES / 2, 1024);
      DescBase kQ[2], kdO[2], mQ[2], mdO[2], mdS[2];
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        kQ[s] = desc_base(sQ0 + s * B2_QTILE, 16, 1024);    kdO[s] = desc_base(sdO0 + s * B2_QTILE, 16, 1024);
        mQ[s] = desc_base(sQ0 + s * B2_QTILE, 8192, 1024);  mdO[s] = desc_base(sdO0 + s * B2_QTILE, 8192, 1024);
        mdS[s] = desc_base(sdS0 + s * B2_DS_TILE, 8192, 1024);
      }
#define TPLR_K128(kk) ((uint32_t)((kk) >> 2) * (TILE_BYTES / 32) + (uint32_t)((kk) & 3) * 2u)   /* 128-row tile, 16-byte units */
#define TPLR_K64(kk) ((uint32_t)((kk) >> 2) * 512u + (uint32_t)((kk) & 3) * 2u)                /* 64-row tile */
#define TPLR_M(kk) ((uint32_t)(kk) * 128u)
      auto issue_st = [&](int t) {                            // S^T(t) = K Q^T into S buffer t & 1
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_bf16_b(tS0 + (t & 1) * 64, kK, TPLR_K128(kk), kQ[t & 1], TPLR_K64(kk), id_st, kk > 0 ? 1u : 0u);
        umma_commit(smem_u32(&bar_s_full[t & 1]));
      };
      auto issue_dp = [&](int t) {                            // dP^T(t) = V dO^T
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) umma_bf16_b(tdP, kV, TPLR_K128(kk), kdO[t & 1], TPLR_K64(kk), id_st, kk > 0 ? 1u : 0u);
        umma_commit(smem_u32(&bar_dp_full));
      };
      bool ok = mbar_wait(smem_u32(&bar_kv), 0, abort_flag);
      if (ok) ok = mbar_wait(smem_u32(&bar_q_full[0]), 0, abort_flag);
      if (ok) {
        tcgen05_fence_after();
        issue_st(0);
        issue_dp(0);
      }
      if (ok && n_it > 1) {
        ok = mbar_wait(smem_u32(&bar_q_full[1]), 0, abort_flag);
        if (ok) { tcgen05_fence_after(); issue_st(1); }
      }
      for (int t = 0; t < n_it && ok; ++t) {
        const int s = t & 1;
        const uint32_t ph = t & 1;
        if (!(ok = mbar_wait(smem_u32(&bar_p_ready), ph, abort_flag))) break;
        tcgen05_fence_after();
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)          // dV += P^T dO ; P^T packed at columns 0-15 and 32-47 of the S buffer
          umma_ts_bf16_b(tdV, tS0 + s * 64 + (kk >> 1) * 32 + (kk & 1) * 8, mdO[s], TPLR_M(kk), id_dv, (t > 0 || kk > 0) ? 1u : 0u);
        if (!(ok = mbar_wait(smem_u32(&bar_ds_ready), ph, abort_flag))) break;
        tcgen05_fence_after();
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)          // dK += dS^T Q
          umma_ts_bf16_b(tdK, tdP + (kk >> 1) * 32 + (kk & 1) * 8, mQ[s], TPLR_M(kk), id_dv, (t > 0 || kk > 0) ? 1u : 0u);
        if (t > 0 && !(ok = mbar_wait(smem_u32(&bar_dq_free), (uint32_t)((t - 1) & 1), abort_flag))) break;
        tcgen05_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)          // dQ^T = K^T dS^T
          umma_bf16_b(tdQ, mK, TPLR_M(kk), mdS[s], TPLR_M(kk), id_dq, kk > 0 ? 1u : 0u);
        umma_commit(smem_u32(&bar_dq_full));
        umma_commit(smem_u32(&bar_q_empty[s]));
        if (t + 1 < n_it) issue_dp(t + 1);
        if (t + 2 < n_it) {
          if (!(ok = mbar_wait(smem_u32(&bar_q_full[s]), (uint32_t)(((t + 2) >> 1) & 1), abort_flag))) break;
          tcgen05_fence_after();
          issue_st(t + 2);
        }
      }
    }
  } else {
    const int quad = warp & 3, ch = (warp - 2) >> 2;
    const int r = quad * 32 + lane;                       // kv row of the block = TMEM lane
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const uint32_t sw = (uint32_t)(lane & 7);
    const uint32_t stg = sStage + (uint32_t)(warp - 2) * 4096u;
    bool ok = true;
    // drain of dQ^T(tt): this warp's 32 d-rows x 32 q-columns box, reduce-added into the transposed scratch
    auto drain = [&](int tt) -> bool {
      bool o = mbar_wait(smem_u32(&bar_dq_full), (uint32_t)(tt & 1), abort_flag);
      o = __all_sync(0xffffffffu, o);
      if (!o) return false;
      tcgen05_fence_after();
      uint32_t v[32];
      tmem_ld32(tdQ + ch * 32 + lane_off, v);
      tcgen05_fence_before();
      if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_dq_free));
      const uint32_t rowaddr = stg + (uint32_t)lane * 128u;
#pragma unroll
      for (int q8 = 0; q8 < 8; ++q8)
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + (((uint32_t)q8 ^ sw) << 4)), "r"(v[4 * q8]),
                     "r"(v[4 * q8 + 1]), "r"(v[4 * q8 + 2]), "r"(v[4 * q8 + 3]) : "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        const int hh = g * group + tt / n_i, iq = iq0 + tt % n_i;
        tma_reduce_add_2d(&p.tmDQT, stg, iq * B2_BQ + ch * 32, (b * p.H + hh) * DH + quad * 32);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      }
      return true;
    };
    for (int t = 0; t < n_it && ok; ++t) {
      const int s = t & 1;
      const int iq = iq0 + t % n_i;
      const int moff = (iq - iq0) * B2_BQ;                // query column offset of this block relative to the kv block
      const bool diag = iq - iq0 < 2;
      ok = mbar_wait(smem_u32(&bar_q_full[s]), (uint32_t)((t >> 1) & 1), abort_flag);     // lse / delta of this step
      if (ok) ok = mbar_wait(smem_u32(&bar_s_full[s]), (uint32_t)((t >> 1) & 1), abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const float* st = stat + s * 128 + ch * 32;
      float pv[32];
      {
        uint32_t sv[32], pk[16];
        tmem_ld32(tS0 + s * 64 + ch * 32 + lane_off, sv);
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          float x = exp2f(fmaf(__uint_as_float(sv[e]), p.scale_log2, -st[e] * 1.4426950408889634f));
          if (diag && r > ch * 32 + e + moff) x = 0.f;
          pv[e] = x;
        }
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          __nv_bfloat162 hh = __floats2bfloat162_rn(pv[2 * e], pv[2 * e + 1]);
          pk[e] = *reinterpret_cast<uint32_t*>(&hh);
        }
        tmem_st16(tS0 + s * 64 + ch * 32 + lane_off, pk);   // P^T over this warp's own S^T columns
      }
      tmem_wait_st();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_p_ready));
      if (t > 0 && !(ok = drain(t - 1))) break;
      ok = mbar_wait(smem_u32(&bar_dp_full), (uint32_t)(t & 1), abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      {
        uint32_t dv[32], pk[16];
        tmem_ld32(tdP + ch * 32 + lane_off, dv);
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float d0 = pv[2 * e] * (__uint_as_float(dv[2 * e]) - st[64 + 2 * e]) * p.scale;
          const float d1 = pv[2 * e + 1] * (__uint_as_float(dv[2 * e + 1]) - st[64 + 2 * e + 1]) * p.scale;
          __nv_bfloat162 hh = __floats2bfloat162_rn(d0, d1);
          pk[e] = *reinterpret_cast<uint32_t*>(&hh);
        }
        tmem_st16(tdP + ch * 32 + lane_off, pk);             // dS^T for the dK MMA
        const uint32_t rowaddr = sdS0 + s * B2_DS_TILE + (uint32_t)r * 128u;      // and as B operand of dQ^T
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4)
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + ((((uint32_t)(ch * 4 + q4)) ^ sw) << 4)),
                       "r"(pk[4 * q4]), "r"(pk[4 * q4 + 1]), "r"(pk[4 * q4 + 2]), "r"(pk[4 * q4 + 3]) : "memory");
      }
      tmem_wait_st();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) { mbar_arrive(smem_u32(&bar_ds_ready)); mbar_arrive(smem_u32(&bar_q_empty[s])); }
    }
    if (ok && n_it > 0) ok = drain(n_it - 1);
    // dV and dK of this kv block: every MMA has completed (the last dQ^T commit covers them)
    if (ok) {
      const int orow0 = kvrow0 + quad * 32;
#pragma unroll
      for (int acc = 0; acc < 2; ++acc) {
        const uint32_t tacc = acc ? tdK : tdV;
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
        const uint32_t rowaddr = stg + (uint32_t)lane * 128u;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          uint32_t v[32];
          tmem_ld32(tacc + ch * 64 + hf * 32 + lane_off, v);
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint32_t pw[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(v[8 * q4 + 2 * e]), __uint_as_float(v[8 * q4 + 2 * e + 1]));
              pw[e] = *reinterpret_cast<uint32_t*>(&hh);
            }
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + ((((uint32_t)(hf * 4 + q4)) ^ sw) << 4)),
                         "r"(pw[0]), "r"(pw[1]), "r"(pw[2]), "r"(pw[3]) : "memory");
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&p.tmDQKV, stg, (acc ? kcol : vcol) + ch * 64, orow0);
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }
  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
  }
  if (threadIdx.x == 0 && s_abort && p.status) atomicOr(p.status, TPLR_ST_WAIT_TIMEOUT);
}

// dqT [B*H*128, S] fp32 (row = (b, h, d)) -> dqkv[(b*S + s), h*128 + d] bf16, 32 x 32 tiles through shared memory
__global__ void __launch_bounds__(256) attn_dq_transpose_kernel(const float* __restrict__ dqT, __nv_bfloat16* __restrict__ dqkv,
                                                                int S, int H, long long ld) {
  __shared__ float tile[32][33];
  const int s0 = blockIdx.x * 32, row0 = blockIdx.y * 32;      // row0 indexes (b, h, d)
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;      // 32 x 8
#pragma unroll
  for (int i = 0; i < 4; ++i) tile[ty + 8 * i][tx] = dqT[(long long)(row0 + ty + 8 * i) * S + s0 + tx];
  __syncthreads();
  const int bh = row0 / DH, d0 = row0 % DH;
  const int bb = bh / H, hh = bh % H;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int sl = ty + 8 * i;                                  // s within the tile
    dqkv[((long long)bb * S + s0 + sl) * ld + hh * DH + d0 + tx] = __float2bfloat16(tile[tx][sl]);
  }
}

}  // namespace

// Backward variant: 1 = one 128-row query block per step, P / dS through shared memory (default: measured
// 0.72 ms against 0.76 ms for B8 S2048 H16 KV8); 2 = pipelined transposed form, 64 query rows per step.
static int g_bwd_variant = [] { const char* e = getenv("TPLR_ATTN_BWD"); return (e && atoi(e) == 2) ? 2 : 1; }();
TPLR_API int tplr_attention_set_bwd_variant(int v) {
  if (v != 1 && v != 2) return -1;
  g_bwd_variant = v;
  return 0;
}

// Gradient of tplr_attention_fwd.  qkv / dqkv: packed [B*S, C] bf16 with row stride ld_qkv; out: the forward's
// output (row stride ld_o); dout: contiguous [B*S, H*128]; lse from the forward; delta: [B,H,S] fp32 scratch;
// dq32: [B*S, H*128] fp32 scratch that the caller has zeroed.  dqkv receives dq | dk | dv.
extern "C" int tplr_rope(void* buf, const float* cosb, const float* sinb, long long tokens, int S, int n_heads, int Dh,
                         long long row_stride, int inverse, void* stream);

static int attention_bwd_impl(const void* qkv, const void* out, const void* dout, const float* lse, float* delta,
                              float* dq32, void* dqkv, int B, int S, int H, int KV, long long ld_qkv, long long ld_o,
                              float scale, const float* cosb, const float* sinb, unsigned int* status, void* stream,
                              bool delta_ready = false) {
  if (B <= 0 || S <= 0) return 0;
  if (S % BQ || H % KV || (ld_qkv % 8) || (ld_o % 8) || ((uintptr_t)qkv & 15) || ((uintptr_t)dqkv & 15) ||
      ((uintptr_t)dout & 15) || ((uintptr_t)out & 7) || ((uintptr_t)dq32 & 15))
    return -201;
  cudaStream_t st = (cudaStream_t)stream;
  const long long tokens = (long long)B * S;
  const int C = (H + 2 * KV) * DH;
  if (!delta_ready)
    attn_delta_kernel<<<(unsigned)((tokens * H + 7) / 8), 256, 0, st>>>((const __nv_bfloat16*)out, (const __nv_bfloat16*)dout,
                                                                         delta, tokens, S, H, ld_o);
  if (g_bwd_variant == 2) {
    // pipelined kernel: dq32 is used as the transposed scratch [B*H*128, S]
    AttnBwd2Params p = {};
    if (!make_map(&p.tmKV, qkv, C, tokens, ld_qkv, 64, 128)) return -202;
    if (!make_map(&p.tmQ, qkv, C, tokens, ld_qkv, 64, 64)) return -202;
    if (!make_map(&p.tmDO, dout, (long long)H * DH, tokens, (long long)H * DH, 64, 64)) return -203;
    if (!make_map(&p.tmDQT, dq32, S, (long long)B * H * DH, S, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B, true)) return -204;
    if (!make_map(&p.tmDQKV, dqkv, C, tokens, ld_qkv, 64, 32)) return -205;
    p.lse = lse; p.delta = delta; p.B = B; p.S = S; p.H = H; p.KV = KV;
    p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
    cudaError_t e = cudaFuncSetAttribute(attn_bwd2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, B2_SMEM);
    if (e != cudaSuccess) return (int)e;
    attn_bwd2_kernel<<<(unsigned)((S / BKV) * KV * B), B2_THREADS, B2_SMEM, st>>>(p);
    attn_dq_transpose_kernel<<<dim3((unsigned)(S / 32), (unsigned)(B * H * DH / 32)), 256, 0, st>>>(
        dq32, (__nv_bfloat16*)dqkv, S, H, ld_qkv);
    if (cosb) return tplr_rope(dqkv, cosb, sinb, tokens, S, H + KV, DH, ld_qkv, 1, stream);   // this variant rotates back in a pass of its own
    return (int)cudaGetLastError();
  }
  AttnBwdParams p = {};
  if (!make_map(&p.tmQKV, qkv, C, tokens, ld_qkv, 64, 128)) return -202;
  if (!make_map(&p.tmDO, dout, (long long)H * DH, tokens, (long long)H * DH, 64, 128)) return -203;
  if (!make_map(&p.tmDQ, dq32, (long long)H * DH, tokens, (long long)H * DH, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B, true)) return -204;
  if (!make_map(&p.tmDQKV, dqkv, C, tokens, ld_qkv, 64, 32)) return -205;
  p.lse = lse; p.delta = delta; p.B = B; p.S = S; p.H = H; p.KV = KV;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
  p.rope_cos = cosb; p.rope_sin = sinb;
  cudaError_t e = cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM);
  if (e != cudaSuccess) return (int)e;
  attn_bwd_kernel<<<(unsigned)((S / BKV) * KV * B), BWD_THREADS, BWD_SMEM, st>>>(p);
  attn_dq_cast_kernel<<<tplr_sm_count() * 8, 256, 0, st>>>(dq32, (__nv_bfloat16*)dqkv, tokens, H * DH, ld_qkv, cosb, sinb, S);
  return (int)cudaGetLastError();
}

TPLR_API int tplr_attention_bwd(const void* qkv, const void* out, const void* dout, const float* lse, float* delta,
                                float* dq32, void* dqkv, int B, int S, int H, int KV, long long ld_qkv, long long ld_o,
                                float scale, unsigned int* status, void* stream) {
  TPLR_ENTER();
  return attention_bwd_impl(qkv, out, dout, lse, delta, dq32, dqkv, B, S, H, KV, ld_qkv, ld_o, scale, nullptr, nullptr, status, stream);
}

// tplr_attention_bwd for a qkv whose q and k heads were rotated by the producer (tplr_gemm2_rope): dq and dk are
// returned with respect to the un-rotated projection, i.e. rotated back by the opposite angles where they are written
// (dq in the fp32 -> bf16 pass, dk in the kernel's epilogue), so that no separate pass over the gradient is needed.
// cosb / sinb: [S, 64] fp32, 16-byte aligned.
TPLR_API int tplr_attention_bwd_unrope(const void* qkv, const void* out, const void* dout, const float* lse, float* delta,
                                       float* dq32, void* dqkv, int B, int S, int H, int KV, long long ld_qkv, long long ld_o,
                                       float scale, const float* cosb, const float* sinb, unsigned int* status, void* stream) {
  TPLR_ENTER();
  if (!cosb || !sinb || ((uintptr_t)cosb & 15) || ((uintptr_t)sinb & 15)) return -201;
  return attention_bwd_impl(qkv, out, dout, lse, delta, dq32, dqkv, B, S, H, KV, ld_qkv, ld_o, scale, cosb, sinb, status, stream);
}

// tplr_attention_bwd_unrope for a caller that has already filled `delta` ([B, H, S] fp32, delta[b, h, s] = sum over the
// head's 128 columns of dout * out): the producer of `dout` (tplr_gemm2_attn_dout, the output projection's data
// gradient) forms it in its epilogue, where a row of dout is in registers anyway.
TPLR_API int tplr_attention_bwd_unrope_delta(const void* qkv, const void* out, const void* dout, const float* lse,
                                             float* delta, float* dq32, void* dqkv, int B, int S, int H, int KV,
                                             long long ld_qkv, long long ld_o, float scale, const float* cosb,
                                             const float* sinb, unsigned int* status, void* stream) {
  TPLR_ENTER();
  if (!cosb || !sinb || ((uintptr_t)cosb & 15) || ((uintptr_t)sinb & 15)) return -201;
  return attention_bwd_impl(qkv, out, dout, lse, delta, dq32, dqkv, B, S, H, KV, ld_qkv, ld_o, scale, cosb, sinb, status, stream,
                            true);
}

