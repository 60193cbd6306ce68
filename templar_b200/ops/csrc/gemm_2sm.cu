// bf16 GEMM on CTA pairs (tcgen05 cta_group::2), optionally fused with a tensor-parallel collective.
//
//   C[M,N] (+)= op(A) * op(B)     same operand layouts as tplr_gemm_bf16 (K-major or MN-major)
//
// A cluster of two CTAs computes one 256 x 256 tile: each CTA stages its own 128 rows of A and
// its own 128 rows of B (so every shared-memory byte feeds two SMs' tensor cores), the even CTA
// issues tcgen05.mma.cta_group::2, and each CTA drains its 128 x 256 half of the accumulator
// from its own tensor memory.  6 smem stages of 32 KB per CTA, two accumulator buffers.
//
// Fused collectives (one process per GPU, peers mapped through the symmetric heap):
//   gather  (all-gather -> GEMM): trailing "comm" CTAs of the same launch pull the peers' row
//           shards of one operand into this GPU's full buffer with bulk copies, 128 rows at a
//           time, and release one flag per 128 rows; the TMA producer of a compute CTA waits
//           (bounded) for the flags of the rows it is about to load.  Every remote byte crosses
//           NVLink once and the tiles of the local shard start at once.
//   scatter (GEMM -> reduce-scatter): the epilogue of every tile reduce-adds its 32 x 128-byte boxes
//           (bf16 or fp32) with TMA straight into the buffer of the rank that owns those rows, over
//           NVLink for a peer and in the local L2 for itself; tile rows are visited so that all
//           owners receive traffic all the time.  No staging buffer, no second pass.
// No load in this file carries a cluster-multicast qualifier; only tcgen05.commit does.
// Every wait is bounded by wall time; on expiry TPLR_ST_WAIT_TIMEOUT is set and all roles return.
//
// Replaces cuBLAS + NCCL behind the reference's tensor-parallel plan: colwise q/k/v/w1/w3,
// rowwise wo/w2 with sequence-sharded activations (torchtitan models/llama3/infra/parallelize.py:151-219).
#include "tcgen05.cuh"
#include <stdlib.h>

namespace {
using namespace tplr_tc;

constexpr int TILE_M = 256, CTA_M = 128, TILE_N = 256, CTA_N = 128, BK = 64, STAGES = 6, UMMA_K = 16;
constexpr int A_STAGE = CTA_M * BK * 2;            // 16 KB
constexpr int B_STAGE = CTA_N * BK * 2;            // 16 KB
constexpr int STAGE_BYTES = A_STAGE + B_STAGE;     // 32 KB
constexpr int EPI_STAGE_BYTES = 4 * 2 * 4096;      // 4 epilogue warps x 2 buffers x (32 rows x 128 B)
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_STAGE_BYTES + 1024;
constexpr int NUM_THREADS = 192;
constexpr int MAX_RANKS = 8;
constexpr int CHUNK_ROWS = 128;                    // gather / scatter flag granularity (rows)

struct Gemm2Params {
  CUtensorMap tmA, tmB;
  CUtensorMap tmC;                   // output: box 64 x 32 bf16 or 32 x 32 fp32, 128-byte swizzle
  int c_tma;                         // 1: epilogue through TMA, 0: direct stores (unaligned C)
  CUtensorMap tmCr[MAX_RANKS];       // scatter: rank o's owned rows [rows_per_rank, N], same box as tmC
  void* C;
  long long ldc;
  int M, N, K;
  unsigned int* status;
  int n_compute_pairs;               // CTA pairs [0, n_compute_pairs) compute, the rest are comm CTAs
  int group_m;                       // tile order: bands of group_m tile rows, tile row fastest inside a band
  int m_rot;                         // rotation of the tile-row order (in 256-row tiles)
  int n_rot;                         // rotation of the tile-column order (in 256-column tiles)
  int m_inter;                       // > 1: logical tile row l is row (l % m_inter) * (tiles_m / m_inter) + l / m_inter
  int k_splits;                      // > 1 (reduce-add epilogues only): a tile's K range is cut into this many work units
  int tri;                           // 1: C is symmetric (B is A): only tiles on or above the diagonal are computed
  int swiglu_f;                      // > 0 (EPI 3): B is the packed [w1; w3] weight of 2 * swiglu_f rows.  Tile column j pairs
                                     // gate rows [128 j, 128 j + 128) (staged by the even CTA) with up rows swiglu_f + the same
                                     // (odd CTA), so every accumulator row holds g and u of the same 128 features; the epilogue
                                     // stores both into C [M, 2 * swiglu_f] and silu(g) * u into tmCr[0]'s tensor [M, swiglu_f]
  // backward of the SwiGLU in the epilogue of the down projection's data gradient (EPI 5): the accumulator tile is
  // dh[M, swiglu_f] = dY W2; gu is the forward's packed [M, 2 * swiglu_f] projection (gate | up), leading dimension ld_gu;
  // the epilogue stores dg | du (bf16) through tmC, a map over the [M, 2 * swiglu_f] gradient of that projection
  const __nv_bfloat16* gu;
  long long ld_gu;
  // data gradient of the attention output projection (EPI 6): C = dO [M, heads * 128] stored as bf16, and for every row
  // and head delta = sum over the head's 128 columns of dO * O, with O = gu (leading dimension ld_gu), written to
  // attn_delta[(row / attn_s * heads + head) * attn_s + row % attn_s]
  float* attn_delta;
  int attn_s, attn_heads;
  // rotary embedding in the epilogue (EPI 4): the first rope_cols columns of C are heads of rope_dh columns whose
  // interleaved pairs (2i, 2i + 1) are rotated by the angle of (row % rope_s, i); tables [rope_s, rope_dh / 2] fp32
  const float* rope_cos;
  const float* rope_sin;
  int rope_s, rope_cols, rope_dh;
  int world, rank;
  unsigned int epoch;
  // gather
  int ag_operand;                    // 0 none, 1 A, 2 B
  int ag_rows_per_rank;              // rows (outer dimension) of the gathered operand per rank
  long long ag_row_bytes;            // bytes of one dense row
  const uint8_t* ag_src[MAX_RANKS];  // base of every rank's full buffer (own entry unused)
  uint8_t* ag_dst;                   // base of this rank's full buffer
  unsigned int* ag_flags;            // one per CHUNK_ROWS rows of the full buffer (local memory)
  // scatter
  int rs_on;
  int rs_bound[MAX_RANKS + 1];       // owner o holds rows [rs_bound[o], rs_bound[o + 1]) of C; multiples of 32
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `saddr` (a shared::cta address of this CTA) inside CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load of a CTA pair: data lands in this CTA, completion bytes go to `bar` which may live in the peer CTA.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar_cluster), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// The same with descriptors given as (low word, high word): the low word carries the start address (bytes >> 4), so the
// issuing thread advances an operand by one 32-bit add instead of rebuilding a 64-bit descriptor per instruction.
__device__ __forceinline__ void umma_bf16_pair_lohi(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                                    uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n\t}"
      ::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned int* p, unsigned int v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded wait for *flag == want (flags carry the call's epoch).  SYS selects the scope of the acquire.
template <bool SYS>
__device__ __forceinline__ bool flag_wait(const unsigned int* flag, unsigned int want, volatile int* abort_flag) {
  unsigned long long t0 = 0;
  for (uint32_t i = 0;; ++i) {
    const unsigned int v = SYS ? ld_acquire_sys(flag) : ld_acquire_gpu(flag);
    if (v == want) return true;
    if ((i & 7u) == 7u) {
      if (*abort_flag) return false;
      const unsigned long long now = gtimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > WAIT_LIMIT_NS) break;
    }
  }
  *abort_flag = 1;
  return false;
}

// The work units of one CTA pair, walked identically by its producer, MMA and epilogue roles: units pair, pair + P,
// ... of the (tile, k split) list, k split fastest.  (A stream-K cut of the flattened (tile, k block) space, every pair
// an equal contiguous run, was measured on the weight-gradient shapes and lost 20-25 % to this static order: pairs
// that share operand tiles stop running in step, and the L2 reuse between them goes.)
struct Work {
  int t;                             // unit index
  int tile, kb0, nkb;                // current unit: tile index, first k block, k blocks
};
__device__ __forceinline__ void work_init(const Gemm2Params& p, Work& w, int pair) { w.t = pair; }
__device__ __forceinline__ bool work_get(const Gemm2Params& p, Work& w, int tiles, int k_blocks_all, int k_per) {
  if (w.t >= tiles * p.k_splits) return false;
  w.tile = w.t / p.k_splits;
  w.kb0 = (w.t % p.k_splits) * k_per;
  w.nkb = min(k_per, k_blocks_all - w.kb0);
  return true;
}
__device__ __forceinline__ void work_next(const Gemm2Params& p, Work& w) { w.t += p.n_compute_pairs; }

// tile index -> (tile row, tile column) under the launch's order
__device__ __forceinline__ void tile_coords(const Gemm2Params& p, int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  if (p.tri) {                       // t-th tile of the upper triangle, row by row: row i holds tiles_n - i tiles
    int i = 0, left = t;
    while (left >= tiles_n - i) { left -= tiles_n - i; ++i; }
    tm = i;
    tn = i + left;
    return;
  }
  const int band = p.group_m * tiles_n;
  const int g = t / band, first = g * p.group_m;
  const int rows = p.group_m < tiles_m - first ? p.group_m : tiles_m - first;
  const int in = t - g * band;
  int tml = first + in % rows;
  tn = in / rows;
  if (p.m_inter > 1) tml = (tml % p.m_inter) * (tiles_m / p.m_inter) + tml / p.m_inter;
  tm = tml + p.m_rot;
  if (tm >= tiles_m) tm -= tiles_m;
  tn += p.n_rot;
  if (tn >= tiles_n) tn -= tiles_n;
}

// Epilogue without TMA (C not 16-byte aligned or odd leading dimension): each lane stores its own row.
template <int EPI>
__device__ __forceinline__ void epilogue_direct(const Gemm2Params& p, uint32_t tmem_acc, int quad, int lane, int m0, int n0) {
  const int row = m0 + quad * 32 + lane;
#pragma unroll 1
  for (int c = 0; c < TILE_N / 32; ++c) {
    uint32_t r[32];
    tmem_ld32(tmem_acc + c * 32 + ((uint32_t)(quad * 32) << 16), r);
    const int col0 = n0 + c * 32;
    if (row < p.M && col0 < p.N) {
      if (EPI == 0 || EPI >= 3) {      // (the epilogue modes 3-5 never take this path: their entries require TMA stores)
        __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col0;
        for (int e = 0; e < 32 && col0 + e < p.N; ++e) crow[e] = __float2bfloat16(__uint_as_float(r[e]));
      } else {
        float* crow = reinterpret_cast<float*>(p.C) + (long long)row * p.ldc + col0;
        for (int e = 0; e < 32 && col0 + e < p.N; ++e) {
          const float o = __uint_as_float(r[e]);
          crow[e] = (EPI == 1) ? crow[e] + o : o;
        }
      }
    }
  }
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(src), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(src), "r"(x), "r"(y) : "memory");
}

// Epilogue through shared memory and TMA: a warp stages 32 rows x 128 bytes (64 bf16 or 32 fp32
// columns) in 128-byte-swizzled order, then one lane stores (EPI 0, 2) or reduce-adds (EPI 1) the
// box.  Two staging buffers per warp; `n_boxes` counts the boxes this warp has issued so far.
template <int EPI>
__device__ __forceinline__ void epilogue_tma(const Gemm2Params& p, uint32_t tmem_acc, int quad, int lane, int m0, int n0,
                                             uint32_t stage_base, uint32_t& n_boxes) {
  constexpr bool BF16_OUT = EPI == 0 || EPI == 4;
  constexpr int COLS = BF16_OUT ? 64 : 32;
  const int row0 = m0 + quad * 32;
  const uint32_t sw = (uint32_t)(lane & 7);
  const CUtensorMap* map = &p.tmC;
  int y = row0;
  if (p.rs_on && row0 < p.M) {                       // the 32 rows of a warp have one owner (32 | every bound)
    int owner = 0;
    while (owner + 1 < p.world && row0 >= p.rs_bound[owner + 1]) ++owner;
    map = &p.tmCr[owner];
    y = row0 - p.rs_bound[owner];
  }
#pragma unroll 1
  for (int c = 0; c < TILE_N / COLS; ++c) {
    const int col0 = n0 + c * COLS;
    if (row0 >= p.M || col0 >= p.N) break;          // warp-uniform: nothing of this box is inside C
    const uint32_t buf = stage_base + (n_boxes & 1u) * 4096u;
    if (n_boxes >= 2) {                              // the box issued two steps ago has left this buffer
      if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      __syncwarp();
    }
    const uint32_t rowaddr = buf + (uint32_t)lane * 128u;
    if (BF16_OUT) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t r[32];
        tmem_ld32(tmem_acc + c * 64 + h * 32 + ((uint32_t)(quad * 32) << 16), r);
        if (EPI == 4 && col0 + h * 32 < p.rope_cols) {
          // rotary pairs of this lane's token: 16 angles starting at pair ((col % head) / 2) of position row % S
          const int row = min(row0 + lane, p.M - 1);
          const long long tb = (long long)(row % p.rope_s) * (p.rope_dh / 2) + ((col0 + h * 32) % p.rope_dh) / 2;
          const float4* cp = reinterpret_cast<const float4*>(p.rope_cos + tb);
          const float4* sp = reinterpret_cast<const float4*>(p.rope_sin + tb);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float4 cv = cp[q], sv = sp[q];
            const float cc[4] = {cv.x, cv.y, cv.z, cv.w}, ss[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float a = __uint_as_float(r[8 * q + 2 * e]), b = __uint_as_float(r[8 * q + 2 * e + 1]);
              r[8 * q + 2 * e] = __float_as_uint(a * cc[e] - b * ss[e]);
              r[8 * q + 2 * e + 1] = __float_as_uint(a * ss[e] + b * cc[e]);
            }
          }
        }
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint32_t pw[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(r[8 * v + 2 * e]), __uint_as_float(r[8 * v + 2 * e + 1]));
            pw[e] = *reinterpret_cast<uint32_t*>(&hh);
          }
          const uint32_t j = (uint32_t)(h * 4 + v);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + ((j ^ sw) << 4)), "r"(pw[0]), "r"(pw[1]),
                       "r"(pw[2]), "r"(pw[3]) : "memory");
        }
      }
    } else {
      uint32_t r[32];
      tmem_ld32(tmem_acc + c * 32 + ((uint32_t)(quad * 32) << 16), r);
#pragma unroll
      for (int v = 0; v < 8; ++v)
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + (((uint32_t)v ^ sw) << 4)), "r"(r[4 * v]),
                     "r"(r[4 * v + 1]), "r"(r[4 * v + 2]), "r"(r[4 * v + 3]) : "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (lane == 0) {
      if (EPI == 1 || p.rs_on) tma_reduce_add_2d(map, buf, col0, y);
      else                     tma_store_2d(map, buf, col0, y);
      bulk_commit();
    }
    ++n_boxes;
  }
}

// Staging of one 32 x 64 bf16 box in two halves of 32 columns (same double-buffer protocol as epilogue_tma):
// box_begin waits until the buffer is free, box_half writes this lane's 32 values of half `hh`, box_store issues the store.
__device__ __forceinline__ uint32_t box_begin(int lane, uint32_t stage_base, uint32_t n_boxes) {
  if (n_boxes >= 2) {
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
    __syncwarp();
  }
  return stage_base + (n_boxes & 1u) * 4096u;
}
__device__ __forceinline__ void box_half(uint32_t buf, int lane, int hh, const float* v) {
  const uint32_t rowaddr = buf + (uint32_t)lane * 128u, sw = (uint32_t)(lane & 7);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t pw[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      __nv_bfloat162 b2 = __floats2bfloat162_rn(v[8 * j + 2 * e], v[8 * j + 2 * e + 1]);
      pw[e] = *reinterpret_cast<uint32_t*>(&b2);
    }
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + (((uint32_t)(hh * 4 + j) ^ sw) << 4)), "r"(pw[0]),
                 "r"(pw[1]), "r"(pw[2]), "r"(pw[3]) : "memory");
  }
}
__device__ __forceinline__ void box_store(const CUtensorMap* map, uint32_t buf, int lane, uint32_t& n_boxes, int col0, int row0) {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncwarp();
  if (lane == 0) {
    tma_store_2d(map, buf, col0, row0);
    bulk_commit();
  }
  ++n_boxes;
}

// Epilogue of the fused [w1; w3] projection (EPI 3): accumulator columns 0..127 of a row are the gate values g of features
// [128 tn, 128 tn + 128), columns 128..255 the up values u of the same features.  Per 64 features: g and u go to C (bf16,
// columns 128 tn + .. and swiglu_f + 128 tn + ..: what the backward pass reads) and h = silu(g) * u, computed from the fp32
// accumulators, goes to the [M, swiglu_f] tensor behind tmCr[0].  Replaces a separate pass that re-reads g and u
// (the reference's F.silu(w1(x)) * w3(x), torchtitan models/llama3/model/model.py FeedForward.forward).
// The accumulators are read twice (once for the g / u boxes, once for h): tensor-memory loads are cheap and 32 values
// at a time keep the register count of the epilogue warps where it was.
__device__ __forceinline__ void epilogue_swiglu(const Gemm2Params& p, uint32_t tmem_acc, int quad, int lane, int m0, int tn,
                                                uint32_t stage_base, uint32_t& n_boxes) {
  const int row0 = m0 + quad * 32;
  if (row0 >= p.M) return;                           // warp-uniform
  const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
#pragma unroll 1
  for (int c = 0; c < 2; ++c) {
    const int f0 = tn * CTA_N + c * 64;              // first feature of this box
    if (f0 >= p.swiglu_f) break;
#pragma unroll 1
    for (int part = 0; part < 2; ++part) {           // 0: g box, 1: u box
      const uint32_t buf = box_begin(lane, stage_base, n_boxes);
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t r[32];
        float v[32];
        tmem_ld32(tmem_acc + part * CTA_N + c * 64 + hh * 32 + lane_sel, r);
#pragma unroll
        for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(r[e]);
        box_half(buf, lane, hh, v);
      }
      box_store(&p.tmC, buf, lane, n_boxes, part * p.swiglu_f + f0, row0);
    }
    const uint32_t buf = box_begin(lane, stage_base, n_boxes);
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      uint32_t rg[32], ru[32];
      float v[32];
      tmem_ld32(tmem_acc + c * 64 + hh * 32 + lane_sel, rg);
      tmem_ld32(tmem_acc + CTA_N + c * 64 + hh * 32 + lane_sel, ru);
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const float g = __uint_as_float(rg[e]);
        v[e] = __fdividef(g, 1.f + __expf(-g)) * __uint_as_float(ru[e]);            // silu(g) * u
      }
      box_half(buf, lane, hh, v);
    }
    box_store(&p.tmCr[0], buf, lane, n_boxes, f0, row0);
  }
}

// Epilogue of the down projection's data gradient fused with the backward of the SwiGLU (EPI 5).  The accumulator row
// holds dh for 256 features; with g and u of the same row and features read from the forward's packed projection,
//   s = sigmoid(g),  du = dh * g * s,  dg = dh * u * s * (1 + g * (1 - s)),
// and dg / du are stored (bf16) at columns f and swiglu_f + f of the packed gradient.  This replaces a pass that writes
// dh, reads it back with g and u and writes dg | du (the backward of the reference's F.silu(w1(x)) * w3(x)).
// Both staging buffers of the warp are in use at once (one box of dg, one of du), so a step waits until the two stores
// of the previous step have read them.
__device__ __forceinline__ void epilogue_swiglu_bwd(const Gemm2Params& p, uint32_t tmem_acc, int quad, int lane, int m0, int n0,
                                                    uint32_t stage_base, uint32_t& n_boxes) {
  const int row0 = m0 + quad * 32;
  if (row0 >= p.M) return;                           // warp-uniform
  const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
  const int row = min(row0 + lane, p.M - 1);
  const __nv_bfloat16* grow = p.gu + (long long)row * p.ld_gu;
  const uint32_t buf_g = stage_base, buf_u = stage_base + 4096u;
  // g and u of this lane's row for one step of 32 features: 64 bytes each (row base and feature offset are multiples
  // of 8 elements).  The loads of step i + 1 are issued before step i is computed: a step's loads come from L2 or
  // DRAM, and eight such latencies in a row would make the epilogue as long as the tile's main loop.
  uint4 gq[4], uq[4], gn[4], un[4];
  auto fetch = [&](int step, uint4* g4, uint4* u4) {
    const int f = n0 + step * 32;
    if (f < p.swiglu_f) {
      const uint4* gp = reinterpret_cast<const uint4*>(grow + f);
      const uint4* up = reinterpret_cast<const uint4*>(grow + p.swiglu_f + f);
#pragma unroll
      for (int q = 0; q < 4; ++q) { g4[q] = gp[q]; u4[q] = up[q]; }
    }
  };
  fetch(0, gq, uq);
#pragma unroll
  for (int step = 0; step < TILE_N / 32; ++step) {
    const int c = step >> 1, hh = step & 1;
    const int f0 = n0 + c * 64;
    if (f0 >= p.swiglu_f) break;                     // warp-uniform (swiglu_f is a multiple of 64)
    if (step + 1 < TILE_N / 32) fetch(step + 1, gn, un);
    if (hh == 0 && n_boxes > 0) {                    // both buffers free: the previous step's stores have read them
      if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      __syncwarp();
    }
    uint32_t r[32];
    tmem_ld32(tmem_acc + c * 64 + hh * 32 + lane_sel, r);
    float dg[32], du[32];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint32_t gw[4] = {gq[q].x, gq[q].y, gq[q].z, gq[q].w}, uw[4] = {uq[q].x, uq[q].y, uq[q].z, uq[q].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 g2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw[e]));
        const float2 u2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uw[e]));
        const float gg[2] = {g2.x, g2.y}, uu[2] = {u2.x, u2.y};
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const float dh = __uint_as_float(r[8 * q + 2 * e + k]);
          const float sg = __fdividef(1.f, 1.f + __expf(-gg[k]));
          const float silu = gg[k] * sg;
          du[8 * q + 2 * e + k] = dh * silu;
          dg[8 * q + 2 * e + k] = dh * uu[k] * (sg + silu * (1.f - sg));
        }
      }
    }
    box_half(buf_g, lane, hh, dg);
    box_half(buf_u, lane, hh, du);
    if (hh == 1) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(&p.tmC, buf_g, f0, row0);
        tma_store_2d(&p.tmC, buf_u, p.swiglu_f + f0, row0);
        bulk_commit();
      }
      n_boxes += 2;
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) { gq[q] = gn[q]; uq[q] = un[q]; }
  }
}

// Epilogue of the attention output projection's data gradient (EPI 6): the accumulator row is dO for two heads (256
// columns).  dO is stored as bf16 like a plain epilogue; on the way every lane multiplies its (bf16-rounded) values
// with the forward's attention output O of the same row and sums per head, which is the `delta` term of the attention
// backward (the row sum of dO * O): no separate pass over dO and O.  O is fetched one step of 32 columns ahead.
__device__ __forceinline__ void epilogue_attn_dout(const Gemm2Params& p, uint32_t tmem_acc, int quad, int lane, int m0, int n0,
                                                   uint32_t stage_base, uint32_t& n_boxes) {
  const int row0 = m0 + quad * 32;
  if (row0 >= p.M) return;                           // warp-uniform
  const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
  const int row = min(row0 + lane, p.M - 1);
  const bool live = row0 + lane < p.M;
  const __nv_bfloat16* orow = p.gu + (long long)row * p.ld_gu;
  const long long drow = (long long)(row / p.attn_s) * p.attn_heads * p.attn_s + row % p.attn_s;
  uint4 oq[4], on[4];
  auto fetch = [&](int step, uint4* o4) {
    const int f = n0 + step * 32;
    if (f < p.N) {
      const uint4* op = reinterpret_cast<const uint4*>(orow + f);
#pragma unroll
      for (int q = 0; q < 4; ++q) o4[q] = op[q];
    }
  };
  fetch(0, oq);
  float acc = 0.f;
#pragma unroll
  for (int step = 0; step < TILE_N / 32; ++step) {
    const int c = step >> 1, hh = step & 1;
    const int f0 = n0 + c * 64;
    if (f0 >= p.N) break;                            // warp-uniform (N is a multiple of 128)
    if (step + 1 < TILE_N / 32) fetch(step + 1, on);
    uint32_t buf = 0;
    if (hh == 0) buf = box_begin(lane, stage_base, n_boxes); else buf = stage_base + (n_boxes & 1u) * 4096u;
    uint32_t r[32];
    tmem_ld32(tmem_acc + c * 64 + hh * 32 + lane_sel, r);
    float v[32];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint32_t ow[4] = {oq[q].x, oq[q].y, oq[q].z, oq[q].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 o2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ow[e]));
        // the attention kernels read dO as bf16: the sum is taken over the values they will see
        const __nv_bfloat162 d2 = __floats2bfloat162_rn(__uint_as_float(r[8 * q + 2 * e]), __uint_as_float(r[8 * q + 2 * e + 1]));
        const float2 df = __bfloat1622float2(d2);
        v[8 * q + 2 * e] = df.x; v[8 * q + 2 * e + 1] = df.y;
        acc = fmaf(df.x, o2.x, acc);
        acc = fmaf(df.y, o2.y, acc);
      }
    }
    box_half(buf, lane, hh, v);
    if (hh == 1) box_store(&p.tmC, buf, lane, n_boxes, f0, row0);
    if ((step & 3) == 3) {                           // a head (128 columns) is complete
      const int head = (n0 + step * 32) / 128;
      if (live) p.attn_delta[drow + (long long)head * p.attn_s] = acc;
      acc = 0.f;
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) oq[q] = on[q];
  }
}

// EPI: 0 store bf16, 1 fp32 accumulate (C += acc), 2 store fp32, 3 fused SwiGLU of a packed [w1; w3] projection,
// 4 store bf16 with the rotary embedding applied to the leading columns, 5 backward of the SwiGLU on the data gradient
// of the down projection, 6 data gradient of the attention output projection with the attention backward's delta term
template <bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm2_kernel(const __grid_constant__ Gemm2Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t bar_full[STAGES], bar_empty[STAGES], bar_tfull[2], bar_tempty[2];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ uint32_t s_ready[32];   // gather: bit c set once chunk c was seen ready (1024 chunks)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cr = cluster_ctarank();
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const bool is_compute = pair < p.n_compute_pairs;
  const int tiles_m = (p.M + TILE_M - 1) / TILE_M, tiles_n = (p.N + TILE_N - 1) / TILE_N;
  const int k_blocks_all = (p.K + BK - 1) / BK;
  const int k_per = (k_blocks_all + p.k_splits - 1) / p.k_splits;   // k blocks per work unit (static mode)
  const int num_tiles = p.tri ? tiles_m * (tiles_m + 1) / 2 : tiles_m * tiles_n;
  volatile int* abort_flag = &s_abort;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int s = 0; s < 2; ++s) { mbar_init(smem_u32(&bar_tfull[s]), 1); mbar_init(smem_u32(&bar_tempty[s]), 8); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (threadIdx.x < 32) s_ready[threadIdx.x] = 0;
  if (warp == 1 && is_compute) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&s_tmem_base)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();   // the peer's barriers are initialised before any remote arrive or TMA completion
  tcgen05_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sA = sbase, sB = sbase + STAGES * A_STAGE, sEpi = sbase + STAGES * STAGE_BYTES;

  if (is_compute) {
    if (warp == 0) {
      // ----------------------------- TMA producer (both CTAs of the pair) ------------
      if (lane == 0) {
        const int chunks_per_rank = p.ag_operand ? p.ag_rows_per_rank / CHUNK_ROWS : 1;
        // bounded wait until rows [r0, r0 + nrows) of the gathered operand are in local memory
        auto rows_ready = [&](int r0, int nrows) -> bool {
          const int c0 = r0 / CHUNK_ROWS, c1 = (r0 + nrows - 1) / CHUNK_ROWS;
          for (int c = c0; c <= c1; ++c) {
            if (c / chunks_per_rank == p.rank || c >= p.world * chunks_per_rank) continue;
            if (s_ready[(c >> 5) & 31] & (1u << (c & 31))) continue;
            if (!flag_wait<false>(p.ag_flags + c, p.epoch, abort_flag)) return false;
            fence_proxy_async();
            s_ready[(c >> 5) & 31] |= 1u << (c & 31);
          }
          return true;
        };
        uint32_t it = 0;
        bool ok = true;
        Work w;
        work_init(p, w, pair);
        for (; ok && work_get(p, w, num_tiles, k_blocks_all, k_per); work_next(p, w)) {
          int tm, tn;
          tile_coords(p, w.tile, tiles_m, tiles_n, tm, tn);
          const int kb0 = w.kb0;
          const int k_blocks = w.nkb;
          const int m0 = tm * TILE_M + (int)cr * CTA_M;
          const int n0 = EPI == 3 ? tn * CTA_N + (int)cr * p.swiglu_f : tn * TILE_N + (int)cr * CTA_N;
          if (p.ag_operand == 1 && !A_MN) ok = rows_ready(m0, CTA_M);
          if (p.ag_operand == 2 && !B_MN) ok = ok && rows_ready(n0, CTA_N);
          for (int kb = 0; kb < k_blocks && ok; ++kb, ++it) {
            // k order rotated so that the rows of the local shard come first when k is the gathered dimension
            int kbr = kb0 + kb;
            if ((p.ag_operand == 1 && A_MN) || (p.ag_operand == 2 && B_MN)) {
              kbr = kb + p.rank * (p.ag_rows_per_rank / BK);       // gathered k: never split (host side)
              if (kbr >= k_blocks) kbr -= k_blocks;
              if (!(ok = rows_ready(kbr * BK, BK))) break;
            }
            const int s = it % STAGES;
            const uint32_t ph = (it / STAGES) & 1;
            if (!(ok = mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1, abort_flag))) break;
            const uint32_t fb_local = smem_u32(&bar_full[s]);
            const uint32_t fb = mapa(fb_local, 0);
            if (cr == 0) mbar_expect_tx(fb_local, 2 * STAGE_BYTES);
            const uint32_t a_dst = sA + s * A_STAGE, b_dst = sB + s * B_STAGE;
            const int k0 = kbr * BK;
            if (!A_MN) {
              tma_load_2d_pair(a_dst, &p.tmA, fb, k0, m0);
            } else {
#pragma unroll
              for (int j = 0; j < CTA_M / 64; ++j) tma_load_2d_pair(a_dst + j * (BK * 128), &p.tmA, fb, m0 + 64 * j, k0);
            }
            if (!B_MN) {
              tma_load_2d_pair(b_dst, &p.tmB, fb, k0, n0);
            } else {
#pragma unroll
              for (int j = 0; j < CTA_N / 64; ++j) tma_load_2d_pair(b_dst + j * (BK * 128), &p.tmB, fb, n0 + 64 * j, k0);
            }
          }
        }
        // drain (leader): every armed stage has landed in both CTAs before the pair may retire
        if (cr == 0) {
          for (uint32_t back = 0; back < STAGES && back < it; ++back) {
            const uint32_t j = it - 1 - back;
            mbar_wait(smem_u32(&bar_full[j % STAGES]), (j / STAGES) & 1, abort_flag);
          }
        }
      }
    } else if (warp == 1) {
      // ----------------------------- MMA issuer (even CTA only) ----------------------
      if (lane == 0 && cr == 0) {
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) |
                               ((B_MN ? 1u : 0u) << 16) | ((uint32_t)(TILE_N >> 3) << 17) | ((uint32_t)(TILE_M >> 4) << 24);
        uint32_t it = 0, tile_i = 0;
        bool ok = true;
        Work w;
        work_init(p, w, pair);
        // descriptors of stage 0, built once: a stage or a k step only moves the start address (bytes >> 4 in the low
        // word; the whole ring lies below 256 KB, so the additions never carry out of the 14-bit address field).
        // The issuing thread is one lane: every instruction it does not execute per MMA is tensor-pipe time.
        const DescBase dA0 = A_MN ? desc_base(sA, BK * 128, 1024) : desc_base(sA, 16, 1024);
        const DescBase dB0 = B_MN ? desc_base(sB, BK * 128, 1024) : desc_base(sB, 16, 1024);
        constexpr uint32_t A_KSTEP = (A_MN ? UMMA_K * 128 : UMMA_K * 2) >> 4, B_KSTEP = (B_MN ? UMMA_K * 128 : UMMA_K * 2) >> 4;
        uint32_t s = 0, ph = 0;                          // ring position of `it` (no division in the loop)
        for (; ok && work_get(p, w, num_tiles, k_blocks_all, k_per); work_next(p, w), ++tile_i) {
          const int k_blocks = w.nkb;
          const uint32_t acc = tile_i & 1, acc_ph = (tile_i >> 1) & 1;
          if (!(ok = mbar_wait(smem_u32(&bar_tempty[acc]), acc_ph ^ 1, abort_flag))) break;
          tcgen05_fence_after();
          const uint32_t d_tmem = tmem_base + acc * TILE_N;
          for (int kb = 0; kb < k_blocks; ++kb, ++it) {
            if (!(ok = mbar_wait(smem_u32(&bar_full[s]), ph, abort_flag))) break;
            tcgen05_fence_after();
            const uint32_t a_lo = dA0.lo + s * (A_STAGE >> 4), b_lo = dB0.lo + s * (B_STAGE >> 4);
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; ++kk)
              umma_bf16_pair_lohi(d_tmem, a_lo + kk * A_KSTEP, dA0.hi, b_lo + kk * B_KSTEP, dB0.hi, idesc,
                                  (kb > 0 || kk > 0) ? 1u : 0u);
            umma_commit_pair(smem_u32(&bar_empty[s]));
            if (++s == STAGES) { s = 0; ph ^= 1u; }
          }
          if (ok) umma_commit_pair(smem_u32(&bar_tfull[acc]));
        }
      }
    } else {
      // ----------------------------- epilogue (warps 2..5 of both CTAs) --------------
      const int quad = warp & 3;
      uint32_t tile_i = 0, n_boxes = 0;
      bool ok = true;
      Work w;
      work_init(p, w, pair);
      for (; ok && work_get(p, w, num_tiles, k_blocks_all, k_per); work_next(p, w), ++tile_i) {
        int tm, tn;
        tile_coords(p, w.tile, tiles_m, tiles_n, tm, tn);
        const int m0 = tm * TILE_M + (int)cr * CTA_M, n0 = tn * TILE_N;
        const uint32_t acc = tile_i & 1, acc_ph = (tile_i >> 1) & 1;
        ok = mbar_wait(smem_u32(&bar_tfull[acc]), acc_ph, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t tmem_acc = tmem_base + acc * TILE_N;
        if (EPI == 3)      epilogue_swiglu(p, tmem_acc, quad, lane, m0, tn, sEpi + (uint32_t)quad * 8192u, n_boxes);
        else if (EPI == 5) epilogue_swiglu_bwd(p, tmem_acc, quad, lane, m0, n0, sEpi + (uint32_t)quad * 8192u, n_boxes);
        else if (EPI == 6) epilogue_attn_dout(p, tmem_acc, quad, lane, m0, n0, sEpi + (uint32_t)quad * 8192u, n_boxes);
        else if (p.c_tma)  epilogue_tma<EPI>(p, tmem_acc, quad, lane, m0, n0, sEpi + (uint32_t)quad * 8192u, n_boxes);
        else               epilogue_direct<EPI>(p, tmem_acc, quad, lane, m0, n0);
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa(smem_u32(&bar_tempty[acc]), 0));
      }
      if (lane == 0) {
        bulk_wait0();                // staging buffers are read out and the stores / reductions are performed
        if (p.rs_on) __threadfence_system();
      }
    }
  } else if (p.ag_operand) {
    // ----------------------------- comm CTA: pull the peers' row shards -----------------
    if (warp == 0 && lane == 0) {
      const int ci = (pair - p.n_compute_pairs) * 2 + (int)cr, n_comm = (n_pairs - p.n_compute_pairs) * 2;
      const int chunks_per_rank = p.ag_rows_per_rank / CHUNK_ROWS;
      const long long chunk_bytes = (long long)CHUNK_ROWS * p.ag_row_bytes;
      const int spc = (int)((chunk_bytes + STAGE_BYTES - 1) / STAGE_BYTES);   // steps per chunk
      const int peer_chunks = (p.world - 1) * chunks_per_rank;
      const int my_chunks = ci < peer_chunks ? (peer_chunks - ci + n_comm - 1) / n_comm : 0;
      const long long total = (long long)my_chunks * spc;
      auto locate = [&](long long g, long long& off, uint32_t& bytes, int& chunk, int& src, bool& last) {
        const int q = ci + (int)(g / spc) * n_comm;          // q-th peer chunk in ring order
        const int piece = (int)(g % spc);
        src = (p.rank + 1 + q / chunks_per_rank) % p.world;
        chunk = src * chunks_per_rank + q % chunks_per_rank;
        off = (long long)chunk * chunk_bytes + (long long)piece * STAGE_BYTES;
        const long long left = chunk_bytes - (long long)piece * STAGE_BYTES;
        bytes = (uint32_t)(left < STAGE_BYTES ? left : STAGE_BYTES);
        last = piece == spc - 1;
      };
      long long issued = 0, stored = 0;
      bool ok = true;
      while (stored < total && ok) {
        // a stage is reused by load g only after the store of step g - STAGES finished reading it
        asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        while (issued < total && issued < stored + STAGES - 1) {
          long long off; uint32_t bytes; int chunk, src; bool last;
          locate(issued, off, bytes, chunk, src, last);
          const int s = (int)(issued % STAGES);
          const uint32_t fb = smem_u32(&bar_full[s]);
          mbar_expect_tx(fb, bytes);
          bulk_g2s(sbase + s * STAGE_BYTES, p.ag_src[src] + off, bytes, fb);
          ++issued;
        }
        long long off; uint32_t bytes; int chunk, src; bool last;
        locate(stored, off, bytes, chunk, src, last);
        const int s = (int)(stored % STAGES);
        if (!(ok = mbar_wait(smem_u32(&bar_full[s]), (uint32_t)((stored / STAGES) & 1), abort_flag))) break;
        bulk_s2g(p.ag_dst + off, sbase + s * STAGE_BYTES, bytes);
        bulk_commit();
        ++stored;
        if (last) {
          bulk_wait0();            // the whole chunk is written
          fence_proxy_async();
          __threadfence();
          st_release_gpu(p.ag_flags + chunk, p.epoch);
        }
      }
      bulk_wait0();
      // loads that were issued but never stored (abort path) must land before the CTA retires
      for (long long g = stored; g < issued; ++g)
        mbar_wait(smem_u32(&bar_full[g % STAGES]), (uint32_t)((g / STAGES) & 1), abort_flag);
    }
  }
  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();   // no CTA retires while its peer may still signal its barriers or read its smem
  if (warp == 1 && is_compute) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
  }
  if (threadIdx.x == 0 && s_abort && p.status) atomicOr(p.status, TPLR_ST_WAIT_TIMEOUT);
}

// ------------------------------ host side ----------------------------------------------
template <bool A_MN, bool B_MN, int EPI>
int launch2(Gemm2Params& p, int n_comm_pairs, int max_pairs, cudaStream_t st) {
  auto kern = gemm2_kernel<A_MN, B_MN, EPI>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return (int)e;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = st;
  cfg.attrs = attr; cfg.numAttrs = 1;
  // all CTAs must be resident at once: compute CTAs wait for comm CTAs of the same launch
  static int max_clusters[2][2][7] = {};
  int& mc = max_clusters[A_MN][B_MN][EPI];
  if (mc == 0) {
    cfg.gridDim = dim3(2 * (tplr_sm_count() / 2));
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
    if (e != cudaSuccess) return (int)e;
    mc = n > 0 ? n : -1;
  }
  if (mc < 1) return -105;
  int pairs = mc < tplr_sm_count() / 2 ? mc : tplr_sm_count() / 2;
  if (max_pairs > 0 && pairs > max_pairs) pairs = max_pairs;
  if (n_comm_pairs >= pairs) return -106;
  const int tiles_m_h = (p.M + TILE_M - 1) / TILE_M;
  const int tiles = p.tri ? tiles_m_h * (tiles_m_h + 1) / 2 : tiles_m_h * ((p.N + TILE_N - 1) / TILE_N);
  int compute = pairs - n_comm_pairs;
  if (compute > tiles * p.k_splits) compute = tiles * p.k_splits;
  p.n_compute_pairs = compute;
  cfg.gridDim = dim3(2 * (compute + n_comm_pairs));
  return (int)cudaLaunchKernelEx(&cfg, kern, p);
}

int dispatch2(Gemm2Params& p, int a_mn, int b_mn, int epi, int n_comm_pairs, int max_pairs, cudaStream_t st) {
#define TPLR_GEMM2_CASE(AM, BMJ, E) \
  if (a_mn == AM && b_mn == BMJ && epi == E) return launch2<AM != 0, BMJ != 0, E>(p, n_comm_pairs, max_pairs, st);
  TPLR_GEMM2_CASE(0, 0, 0) TPLR_GEMM2_CASE(0, 0, 1) TPLR_GEMM2_CASE(0, 0, 2)
  TPLR_GEMM2_CASE(0, 1, 0) TPLR_GEMM2_CASE(0, 1, 1) TPLR_GEMM2_CASE(0, 1, 2)
  TPLR_GEMM2_CASE(1, 1, 0) TPLR_GEMM2_CASE(1, 1, 1) TPLR_GEMM2_CASE(1, 1, 2)
  TPLR_GEMM2_CASE(1, 0, 0) TPLR_GEMM2_CASE(1, 0, 1) TPLR_GEMM2_CASE(1, 0, 2)
  TPLR_GEMM2_CASE(0, 0, 3) TPLR_GEMM2_CASE(0, 0, 4) TPLR_GEMM2_CASE(0, 1, 5) TPLR_GEMM2_CASE(0, 1, 6)
#undef TPLR_GEMM2_CASE
  return -104;
}

// Accumulating GEMMs (C += ...) reduce-add their tiles, so K may be cut in two to fill the last wave.
// Every split costs another M*N*4 bytes of L2 reductions (measured: 4 and 8 splits lose more than the
// fuller waves win), so K is halved only when that lifts the wave efficiency by more than 10 points.
int pick_k_splits(int M, int N, int K, int max_pairs) {
  static const int forced = [] { const char* e = getenv("TPLR_GEMM_KSPLITS"); return e ? atoi(e) : 0; }();
  if (forced > 0) return (K + BK - 1) / BK / forced >= 1 ? forced : 1;   // tuning override
  int pairs = tplr_sm_count() / 2;
  if (max_pairs > 0 && pairs > max_pairs) pairs = max_pairs;
  const long long tiles = (long long)((M + TILE_M - 1) / TILE_M) * ((N + TILE_N - 1) / TILE_N);
  if ((K + BK - 1) / BK < 128) return 1;
  auto eff = [&](long long units) { return (double)units / (double)(((units + pairs - 1) / pairs) * pairs); };
  return eff(2 * tiles) > eff(tiles) + 0.10 ? 2 : 1;
}

// Fills the operand maps and the plain fields; returns 0 or a negative argument error.
int fill_common(Gemm2Params& p, const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                long long ldb, long long ldc, int a_mn, int b_mn, int epi, unsigned int* status) {
  if ((lda % 8) || (ldb % 8) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return -101;
  if (!(a_mn ? make_map(&p.tmA, A, M, K, lda, 64, BK) : make_map(&p.tmA, A, K, M, lda, BK, CTA_M))) return -102;
  if (!(b_mn ? make_map(&p.tmB, B, N, K, ldb, 64, BK) : make_map(&p.tmB, B, K, N, ldb, BK, CTA_N))) return -103;
  p.C = C; p.ldc = ldc; p.M = M; p.N = N; p.K = K; p.status = status;
  static const int group_m = [] { const char* e = getenv("TPLR_GEMM_GROUP_M"); const int v = e ? atoi(e) : 0; return v > 0 ? v : 8; }();
  p.world = 1; p.rank = 0; p.epoch = 0; p.group_m = group_m; p.m_rot = 0; p.n_rot = 0; p.m_inter = 1; p.k_splits = 1;
  p.tri = 0;
  p.ag_operand = 0; p.rs_on = 0;
  const bool f32 = epi != 0;
  p.c_tma = !((uintptr_t)C & 15) && (ldc * (f32 ? 4 : 2)) % 16 == 0;
  if (p.c_tma && !make_map(&p.tmC, C, N, M, ldc, f32 ? 32 : 64, 32, CU_TENSOR_MAP_SWIZZLE_128B, f32)) return -110;
  return 0;
}

}  // namespace

// Symmetric rank-k product for Newton-Schulz: the 256 x 256 tiles of C = A A^T (A: [M, K] bf16, K-major; C bf16) that
// lie on or above the diagonal.  Tiles below the diagonal are NOT written: tplr_sym_axpby mirrors them.  Half the
// tensor-core work of the full product, as the reference's Triton kernels ns_line_1 / ns_line_2 do with one triangle
// and a mirrored store (src/tplr/muon/newton_schulz_triton.py:62-131, :173-258).
TPLR_API int tplr_gemm2_syrk(const void* A, void* C, int M, int K, long long lda, long long ldc, unsigned int* status,
                             void* stream) {
  TPLR_ENTER();
  if (M <= 0 || K <= 0) return 0;
  Gemm2Params p = {};
  if (int r = fill_common(p, A, A, C, M, M, K, lda, lda, ldc, 0, 0, 0, status)) return r;
  p.tri = 1;
  return dispatch2(p, 0, 0, 0, 0, 0, (cudaStream_t)stream);
}

// Same contract as tplr_gemm_bf16; max_pairs <= 0 uses every SM pair.
TPLR_API int tplr_gemm2_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                             long long ldb, long long ldc, int a_mn, int b_mn, int epi, unsigned int* status,
                             int max_pairs, void* stream) {
  TPLR_ENTER();
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  Gemm2Params p = {};
  if (int r = fill_common(p, A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, epi, status)) return r;
  if (epi == 1 && p.c_tma) p.k_splits = pick_k_splits(M, N, K, max_pairs);
  return dispatch2(p, a_mn, b_mn, epi, 0, max_pairs, (cudaStream_t)stream);
}

// GU[M, 2F] = X W^T for the packed weight W = [w1; w3] ([2F, K] bf16, K-major) and H[M, F] = silu(GU[:, :F]) * GU[:, F:]
// in one launch (see Gemm2Params::swiglu_f).  F a multiple of 128; X, W, GU, H 16-byte aligned with leading dimensions
// that are multiples of 8 elements.  -111: shapes or alignment that this entry does not take (the caller runs the
// projection and the activation as two launches instead).
TPLR_API int tplr_gemm2_swiglu(const void* X, const void* W, void* GU, void* H, int M, int F, int K, long long ldx,
                               long long ldw, long long ldgu, long long ldh, unsigned int* status, void* stream) {
  TPLR_ENTER();
  if (M <= 0 || F <= 0 || K <= 0) return 0;
  if (F % CTA_N || ((uintptr_t)GU & 15) || ((uintptr_t)H & 15) || (ldgu % 8) || (ldh % 8)) return -111;
  Gemm2Params p = {};
  if (int r = fill_common(p, X, W, GU, M, 2 * F, K, ldx, ldw, ldgu, 0, 0, 0, status)) return r;
  if (!p.c_tma) return -111;
  if (!make_map(&p.tmCr[0], H, F, M, ldh, 64, 32, CU_TENSOR_MAP_SWIZZLE_128B, false)) return -110;
  p.swiglu_f = F;
  return dispatch2(p, 0, 0, 3, 0, 0, (cudaStream_t)stream);
}

// dGU[M, 2F] = backward of the SwiGLU applied to dH = dY W2 (dY [M, K] bf16 K-major, W2 [K, F] bf16 with F contiguous:
// the down projection's weight as stored), with GU [M, 2F] the forward's packed gate | up projection: one launch instead
// of the data-gradient GEMM followed by an element-wise pass (see epilogue_swiglu_bwd).  F a multiple of 64, all tensors
// 16-byte aligned with leading dimensions that are multiples of 8; -111 when this entry does not take the arguments.
TPLR_API int tplr_gemm2_swiglu_bwd(const void* dY, const void* W2, const void* GU, void* dGU, int M, int F, int K,
                                   long long lddy, long long ldw2, long long ldgu, long long lddgu, unsigned int* status,
                                   void* stream) {
  TPLR_ENTER();
  if (M <= 0 || F <= 0 || K <= 0) return 0;
  if (F % 64 || ((uintptr_t)GU & 15) || ((uintptr_t)dGU & 15) || (ldgu % 8) || (lddgu % 8)) return -111;
  Gemm2Params p = {};
  // operands and tile grid of the [M, F] product; the output map then covers the [M, 2F] packed gradient
  if (int r = fill_common(p, dY, W2, dGU, M, F, K, lddy, ldw2, lddgu, 0, 1, 0, status)) return r;
  if (!p.c_tma) return -111;
  if (!make_map(&p.tmC, dGU, 2LL * F, M, lddgu, 64, 32, CU_TENSOR_MAP_SWIZZLE_128B, false)) return -110;
  p.swiglu_f = F;
  p.gu = (const __nv_bfloat16*)GU; p.ld_gu = ldgu;
  return dispatch2(p, 0, 1, 5, 0, 0, (cudaStream_t)stream);
}

// dO[M, N] = dY Wo (dY [M, K] bf16 K-major, Wo [K, N] bf16 with N contiguous: the attention output projection's weight
// as stored; N = heads * 128), and delta[b, h, s] = sum over head h's 128 columns of dO * O for row b * S + s, with O
// [M, N] the forward's attention output (see epilogue_attn_dout).  -111 when this entry does not take the arguments.
TPLR_API int tplr_gemm2_attn_dout(const void* dY, const void* Wo, const void* O, void* dO, float* delta, int M, int N, int K,
                                  int S, long long lddy, long long ldwo, long long ldo, long long lddo, unsigned int* status,
                                  void* stream) {
  TPLR_ENTER();
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (N % 128 || S <= 0 || M % S || ((uintptr_t)O & 15) || ((uintptr_t)dO & 15) || (ldo % 8) || (lddo % 8) || !delta) return -111;
  Gemm2Params p = {};
  if (int r = fill_common(p, dY, Wo, dO, M, N, K, lddy, ldwo, lddo, 0, 1, 0, status)) return r;
  if (!p.c_tma) return -111;
  p.gu = (const __nv_bfloat16*)O; p.ld_gu = ldo;
  p.attn_delta = delta; p.attn_s = S; p.attn_heads = N / 128;
  return dispatch2(p, 0, 1, 6, 0, 0, (cudaStream_t)stream);
}

// QKV[M, N] = X W^T (bf16, W K-major) with the rotary embedding applied to the first rope_cols columns in the epilogue:
// heads of `head_dim` columns, interleaved pairs, angle tables cos / sin [S, head_dim / 2] fp32, position = row % S
// (the reference's apply_rotary_emb on xq and xk, torchtitan models/llama3/model/model.py, after the wq / wk projections).
// rope_cols and head_dim multiples of 32 and 16-byte aligned tables; -111 when this entry does not take the arguments.
TPLR_API int tplr_gemm2_rope(const void* X, const void* W, void* QKV, int M, int N, int K, long long ldx, long long ldw,
                             long long ldc, const float* cosb, const float* sinb, int S, int rope_cols, int head_dim,
                             unsigned int* status, void* stream) {
  TPLR_ENTER();
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (S <= 0 || head_dim % 32 || rope_cols % 32 || rope_cols > N || ((uintptr_t)cosb & 15) || ((uintptr_t)sinb & 15)) return -111;
  Gemm2Params p = {};
  if (int r = fill_common(p, X, W, QKV, M, N, K, ldx, ldw, ldc, 0, 0, 0, status)) return r;
  if (!p.c_tma) return -111;
  p.rope_cos = cosb; p.rope_sin = sinb; p.rope_s = S; p.rope_cols = rope_cols; p.rope_dh = head_dim;
  return dispatch2(p, 0, 0, 4, 0, 0, (cudaStream_t)stream);
}

// All-gather fused into the GEMM.  Operand `ag_operand` (1 = A, 2 = B) is the local FULL buffer
// whose rows (its outer dimension: m or n when K-major, k when MN-major) are sharded over `world`
// ranks, `rows_per_rank` (multiple of 128) each; rank r's rows are valid in rank r's buffer when the
// kernel starts (the caller runs a barrier first) and are copied from `peer_bases[r]` into the local
// buffer by `n_comm_pairs` CTA pairs while the other pairs compute.  `flags` holds one zero-initialised
// word per 128 rows of the full buffer; `epoch` must differ from every earlier call's on these flags.
TPLR_API int tplr_gemm2_gather(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                               long long ldb, long long ldc, int a_mn, int b_mn, int epi, int ag_operand,
                               int world, int rank, int rows_per_rank, const void* const* peer_bases,
                               unsigned int* flags, unsigned int epoch, int n_comm_pairs, unsigned int* status,
                               void* stream) {
  TPLR_ENTER();
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || (ag_operand != 1 && ag_operand != 2)) return -107;
  if (rows_per_rank % CHUNK_ROWS || (long long)world * rows_per_rank / CHUNK_ROWS > 1024 || n_comm_pairs < 1) return -107;
  const bool mn = ag_operand == 1 ? a_mn != 0 : b_mn != 0;
  const long long outer = mn ? K : (ag_operand == 1 ? M : N);
  if (outer != (long long)world * rows_per_rank) return -108;
  Gemm2Params p = {};
  if (int r = fill_common(p, A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, epi, status)) return r;
  p.world = world; p.rank = rank; p.epoch = epoch;
  p.ag_operand = ag_operand; p.ag_rows_per_rank = rows_per_rank;
  p.ag_row_bytes = (ag_operand == 1 ? lda : ldb) * 2;
  for (int r = 0; r < world; ++r) p.ag_src[r] = static_cast<const uint8_t*>(peer_bases[r]);
  p.ag_dst = static_cast<uint8_t*>(const_cast<void*>(ag_operand == 1 ? A : B));
  p.ag_flags = flags;
  if (!mn && ag_operand == 1) {           // tiles of the local row shard first, then the peers in ring order
    p.group_m = 1;
    p.m_rot = (int)(((long long)rank * rows_per_rank) / TILE_M);
  }
  if (!mn && ag_operand == 2) {           // gathered weight rows (FSDP shards): all tile rows of the local columns first
    p.group_m = (M + TILE_M - 1) / TILE_M;
    p.n_rot = (int)(((long long)rank * rows_per_rank) / TILE_N);
  }
  return dispatch2(p, a_mn, b_mn, epi, world > 1 ? n_comm_pairs : 0, 0, (cudaStream_t)stream);
}

// GEMM fused with a reduce-scatter over the rows of C.  Every rank computes its partial
// [M,N] = op(A) op(B) over its own K shard; rank o owns rows [o*rows_per_rank, (o+1)*rows_per_rank)
// and `peer_out[o]` is its [rows_per_rank, N] result buffer (leading dimension ld_out, bf16 or fp32
// by `out_fp32`) as mapped in this process.  The partial tiles are reduce-added into those buffers by
// the epilogue, so every buffer must be zero and all ranks past a barrier when the kernel starts,
// and the sums are complete once all ranks' kernels have finished (a barrier after it).
TPLR_API int tplr_gemm2_scatter(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb,
                                int a_mn, int b_mn, int world, int rank, int rows_per_rank,
                                void* const* peer_out, long long ld_out, int out_fp32, unsigned int* status,
                                void* stream) {
  TPLR_ENTER();
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return -107;
  const int esz = out_fp32 ? 4 : 2;
  if (rows_per_rank % CHUNK_ROWS || M != world * rows_per_rank || (ld_out * esz) % 16) return -108;
  Gemm2Params p = {};
  const int epi = out_fp32 ? 1 : 0;
  if (int r = fill_common(p, A, B, peer_out[rank], rows_per_rank, N, K, lda, ldb, ld_out, a_mn, b_mn, epi, status)) return r;
  if (!p.c_tma) return -108;
  p.M = M;                                 // fill_common built tmC over the owned rows only
  if (!(a_mn ? make_map(&p.tmA, A, M, K, lda, 64, BK) : make_map(&p.tmA, A, K, M, lda, BK, CTA_M))) return -102;
  p.world = world; p.rank = rank;
  p.rs_on = 1;
  for (int r = 0; r <= world; ++r) p.rs_bound[r] = r * rows_per_rank;
  for (int r = 0; r < world; ++r) {
    if ((uintptr_t)peer_out[r] & 15) return -108;
    if (!make_map(&p.tmCr[r], peer_out[r], N, rows_per_rank, ld_out, out_fp32 ? 32 : 64, 32, CU_TENSOR_MAP_SWIZZLE_128B,
                  out_fp32 != 0)) return -109;
  }
  // every band of tile rows touches every owner, so all links carry traffic throughout the GEMM
  const int tiles_m = (M + TILE_M - 1) / TILE_M;
  if (world > 1 && tiles_m % world == 0) p.m_inter = world;
  return dispatch2(p, a_mn, b_mn, epi, 0, 0, (cudaStream_t)stream);
}

// GEMM fused with a reduce-scatter over the rows of C whose owners hold UNEQUAL row ranges: owner o holds rows
// [bounds[o], bounds[o + 1]) (multiples of 32, bounds[0] = 0, bounds[world] = M; an owner may hold none) in
// `peer_out[o]`, a dense fp32 [rows_o, N] array as mapped in this process (its own, for o == rank).  This is the
// weight-gradient GEMM of sharded data parallelism: every rank multiplies its own tokens (the whole K range) and
// the epilogue reduce-adds each tile into the shard of the rank that owns those rows, over NVLink for a peer
// and in the local L2 for itself, so the fp32 gradient exists only as shards and the reduce-scatter ends with
// the backward pass.  Nothing is zeroed here: the shards accumulate over micro-batches; the caller zeroes them
// between inner steps and separates that from the next backward pass with a barrier.
// Replaces FSDP2's per-block fp32 reduce-scatter (src/tplr/model_factory.py:153,183).
TPLR_API int tplr_gemm2_scatter_v(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb,
                                  int a_mn, int b_mn, int world, int rank, const int* bounds,
                                  void* const* peer_out, unsigned int* status, void* stream) {
  TPLR_ENTER();
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return -107;
  if (bounds[0] != 0 || bounds[world] != M || (N * 4) % 16) return -108;
  for (int r = 0; r < world; ++r)
    if (bounds[r + 1] < bounds[r] || (bounds[r + 1] % 32)) return -108;
  int first = 0;
  while (first < world && bounds[first + 1] == bounds[first]) ++first;      // first owner that holds rows
  Gemm2Params p = {};
  if (int r = fill_common(p, A, B, peer_out[first], bounds[first + 1] - bounds[first], N, K, lda, ldb, N, a_mn, b_mn, 1,
                          status)) return r;
  if (!p.c_tma) return -108;
  p.M = M;
  if (!(a_mn ? make_map(&p.tmA, A, M, K, lda, 64, BK) : make_map(&p.tmA, A, K, M, lda, BK, CTA_M))) return -102;
  p.world = world; p.rank = rank;
  p.rs_on = 1;
  for (int r = 0; r <= world; ++r) p.rs_bound[r] = bounds[r];
  for (int r = 0; r < world; ++r) {
    const int rows = bounds[r + 1] - bounds[r];
    if (rows == 0) continue;
    if ((uintptr_t)peer_out[r] & 15) return -108;
    if (!make_map(&p.tmCr[r], peer_out[r], N, rows, N, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B, true)) return -109;
  }
  // ranks start on different owners and consecutive tile rows go to different owners where the tile rows
  // divide evenly, so that every owner's link receives traffic throughout the GEMM
  const int tiles_m = (M + TILE_M - 1) / TILE_M;
  if (world > 1 && tiles_m % world == 0) p.m_inter = world;
  if (world > 1) p.m_rot = (int)(((long long)rank * tiles_m) / world);
  p.k_splits = pick_k_splits(M, N, K, 0);
  return dispatch2(p, a_mn, b_mn, 1, 0, 0, (cudaStream_t)stream);
}
