// Per-window compression and aggregation kernels (sm_100a).
//
//   tplr_compress_chunks   error-feedback update  e <- gamma*e + delta,  2-D chunk DCT,
//                          per-chunk magnitude top-k, 12-bit index packing, value
//                          write-out, and the error-feedback residual
//                          e <- e - iDCT(selected), all in ONE pass over the dense tensors
//                          (reads theta0/theta/e once, writes e once).
//   tplr_peer_sumsq / tplr_clip_factors
//                          per-(peer, tensor) L2 norms of the received values and the
//                          median-norm clip factors, without any host round trip.
//   tplr_aggregate_apply   for every chunk: pull each peer's packed (index, value)
//                          lists (the pointers may be peer-GPU memory mapped over
//                          NVLink), unpack, scale by the clip factor, mean over the
//                          contributors of each coefficient, inverse chunk DCT and the
//                          outer update theta <- theta0 - lr * g (or its sign form),
//                          writing the fp32 master and the bf16 compute copy.
//
// One CTA owns one chunk at a time (persistent grid-stride loop); a launch covers
// every tensor of the model through a descriptor table, so a window costs a handful
// of launches instead of dozens per tensor.
//
// Semantics follow the reference's src/tplr/compress.py:225-292 (chunking + DCT),
// :385-481 (top-k, scatter-mean over contributors), :526-556 (median-norm clip) and
// src/tplr/neurons.py:138-173 (error feedback), :342-450 (outer step).
#include "tcgen05.cuh"

#include <atomic>

// Switches of the tensor-core compress / aggregate kernels, for comparison runs (tplr_compress_set_variant):
// bit 0 candidate threshold search instead of the radix select, bit 1 L2 prefetch of the next chunk pair in the
// compress kernel, bit 2 payload entries fetched one pair ahead in the aggregate kernel.  Default: all on.
static std::atomic<int> g_tc_variant{7};

#define NT 256
#define LD 64

// acc[a][b] = sum_k At[k][4*ty+a] * B[k][4*tx+b]   (ty = tid/16, tx = tid%16)
static __device__ __forceinline__ void mm_tile(const float* __restrict__ At,
                                               const float* __restrict__ B, int K,
                                               float acc[4][4]) {
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  const float4* a4 = reinterpret_cast<const float4*>(At) + ty;
  const float4* b4 = reinterpret_cast<const float4*>(B) + tx;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
#pragma unroll 8
  for (int k = 0; k < K; ++k) {
    const float4 a = a4[k * (LD / 4)];
    const float4 b = b4[k * (LD / 4)];
    const float av[4] = {a.x, a.y, a.z, a.w};
    const float bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
  }
}

static __device__ __forceinline__ void store_tile(float* __restrict__ C, const float acc[4][4]) {
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    reinterpret_cast<float4*>(C + (4 * ty + i) * LD)[tx] =
        make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
}

static __device__ __forceinline__ int find_desc(const TplrParamDesc* __restrict__ descs, int n, int c) {
  int lo = 0, hi = n - 1;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (__ldg(&descs[mid].chunk_begin) <= c) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// Loads the n x n DCT matrix F (row-major, ld = n) zero-padded into F[64][64] and its
// transpose into Ft[64][64].
static __device__ __forceinline__ void load_basis(const float* __restrict__ g, int n,
                                                  float* F, float* Ft) {
  for (int i = threadIdx.x; i < TPLR_TILE_ELEMS; i += NT) {
    int r = i >> 6, c = i & 63;
    float v = (r < n && c < n) ? __ldg(g + r * n + c) : 0.f;
    F[i] = v;
    Ft[c * LD + r] = v;
  }
}

struct CompressArgs {
  const TplrParamDesc* descs;
  const float* basis;
  float* ef;
  const float* theta0;
  const float* theta;
  uint8_t* idx_out;
  float* val_out;
  unsigned int* status;
  int n_desc, total_chunks;
  float gamma;
  int use_dct, delta_mode, null_round, write_residual, distinct;
  int variant;              // tensor-core kernel: bit 0 candidate threshold search, bit 1 L2 prefetch of the next pair
};

__global__ void __launch_bounds__(NT, 2) compress_kernel(const CompressArgs a) {
  extern __shared__ __align__(16) float smem[];
  float* X = smem;
  float* Y = X + TPLR_TILE_ELEMS;
  float* U = Y + TPLR_TILE_ELEMS;
  float* Fh = U + TPLR_TILE_ELEMS;
  float* Fht = Fh + TPLR_TILE_ELEMS;
  float* Fw = a.distinct ? Fht + TPLR_TILE_ELEMS : Fh;
  float* Fwt = a.distinct ? Fw + TPLR_TILE_ELEMS : Fht;
  __shared__ int s_hist[256];
  __shared__ int s_wsum[8];
  __shared__ int s_bin, s_krem;
  __shared__ int s_sel_idx[TPLR_TILE];
  __shared__ float s_sel_val[TPLR_TILE];

  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int ty = tid >> 4, tx = tid & 15;
  int cur_fh = -1, cur_fw = -1;

  for (int c = blockIdx.x; c < a.total_chunks; c += gridDim.x) {
    const TplrParamDesc d = a.descs[find_desc(a.descs, a.n_desc, c)];
    const int h = d.h, w = d.w, n = h * w, k = d.k;
    const int cl = c - d.chunk_begin;
    const int cy = d.chunk_row0 + cl / d.chunks_x, cx = cl % d.chunks_x;
    const long long base = d.elem_off + (long long)cy * h * d.cols + (long long)cx * w;
    __syncthreads();  // previous chunk's smem fully consumed
    if (a.use_dct && (d.fh_off != cur_fh || d.fw_off != cur_fw)) {
      load_basis(a.basis + d.fh_off, h, Fh, Fht);
      if (a.distinct) load_basis(a.basis + d.fw_off, w, Fw, Fwt);
      cur_fh = d.fh_off;
      cur_fw = d.fw_off;
    }
    // ---- X = gamma*e + delta, zero padded to 64x64 -------------------------------
    const bool vec = (w == 64) && ((d.cols & 3) == 0) && ((base & 3) == 0);
    if (vec) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = ty + 16 * i;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < h && !a.null_round) {
          const long long g = base + (long long)r * d.cols + 4 * tx;
          const float4 e = *reinterpret_cast<const float4*>(a.ef + g);
          float4 dl = *reinterpret_cast<const float4*>(a.theta0 + g);
          if (a.delta_mode) {
            const float4 t = *reinterpret_cast<const float4*>(a.theta + g);
            dl.x -= t.x; dl.y -= t.y; dl.z -= t.z; dl.w -= t.w;
          }
          x.x = fmaf(a.gamma, e.x, dl.x); x.y = fmaf(a.gamma, e.y, dl.y);
          x.z = fmaf(a.gamma, e.z, dl.z); x.w = fmaf(a.gamma, e.w, dl.w);
        }
        reinterpret_cast<float4*>(X + r * LD)[tx] = x;
      }
    } else {
      for (int i = tid; i < TPLR_TILE_ELEMS; i += NT) {
        const int r = i >> 6, cc = i & 63;
        float x = 0.f;
        if (r < h && cc < w && !a.null_round) {
          const long long g = base + (long long)r * d.cols + cc;
          float dl = a.theta0[g];
          if (a.delta_mode) dl -= a.theta[g];
          x = fmaf(a.gamma, a.ef[g], dl);
        }
        X[i] = x;
      }
    }
    __syncthreads();
    // ---- Y = F_h X F_w^T ------------------------------------------------------------
    const float* Ysel = X;
    if (a.use_dct) {
      float acc[4][4];
      mm_tile(X, Fht, h, acc);   // U[c][b] = sum_r X[r][c] F_h[b][r]
      store_tile(U, acc);
      __syncthreads();
      mm_tile(U, Fwt, w, acc);   // Y[b][d] = sum_c U[c][b] F_w[d][c]
      store_tile(Y, acc);
      __syncthreads();
      Ysel = Y;
    }
    // ---- radix select of the k largest |Y| over the n valid coefficients -----------
    unsigned int key[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int e = i * NT + tid;
      key[i] = 0u;
      if (e < n) key[i] = __float_as_uint(Ysel[(e / w) * LD + (e % w)]) & 0x7fffffffu;
    }
    unsigned int prefix = 0u, mask = 0u;
    int krem = k;
#pragma unroll 1
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      s_hist[tid] = 0;
      __syncthreads();
#pragma unroll
      for (int i = 0; i < 16; ++i)
        if (i * NT + tid < n && (key[i] & mask) == prefix) atomicAdd(&s_hist[(key[i] >> shift) & 255u], 1);
      __syncthreads();
      if (wid == 0) {
        const int hi = 255 - 8 * lane;
        int s = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) s += s_hist[hi - j];
        int incl = s;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          int t = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += t;
        }
        const int excl = incl - s;
        if (excl < krem && krem <= incl) {
          int run = excl;
          for (int j = 0; j < 8; ++j) {
            const int cnt = s_hist[hi - j];
            if (run + cnt >= krem) { s_bin = hi - j; s_krem = krem - run; break; }
            run += cnt;
          }
        }
      }
      __syncthreads();
      prefix |= ((unsigned int)s_bin) << shift;
      mask |= 255u << shift;
      krem = s_krem;
      __syncthreads();
    }
    // ---- ordered compaction (thread-major order): all keys above the threshold, then the
    //      first krem keys equal to it; deterministic for a given input ------------------
    int g = 0, q = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (i * NT + tid < n) { g += key[i] > prefix; q += key[i] == prefix; }
    int packed = g | (q << 16);
    int incl = packed;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) s_wsum[wid] = incl;
    __syncthreads();
    int woff = 0;
    for (int j = 0; j < wid; ++j) woff += s_wsum[j];
    int excl = incl - packed + woff;
    int gb = excl & 0xffff, qb = excl >> 16;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int e = i * NT + tid;
      if (e < n) {
        int pos = -1;
        if (key[i] > prefix) { pos = gb + min(qb, krem); ++gb; }
        else if (key[i] == prefix) { if (qb < krem) pos = gb + qb; ++qb; }
        if (pos >= 0 && pos < TPLR_TILE) {
          s_sel_idx[pos] = e;
          s_sel_val[pos] = Ysel[(e / w) * LD + (e % w)];
        }
      }
    }
    __syncthreads();
    // ---- payload: 3 bytes per index pair, fp32 values ------------------------------
    {
      uint8_t* ip = a.idx_out + d.idx_off + (long long)cl * (k / 2) * 3;
      float* vp = a.val_out + d.val_off + (long long)cl * k;
      if (tid < k / 2) {
        const int i0 = s_sel_idx[2 * tid], i1 = s_sel_idx[2 * tid + 1];
        ip[3 * tid + 0] = (uint8_t)(i0 & 0xff);
        ip[3 * tid + 1] = (uint8_t)(((i0 >> 8) & 0xf) | ((i1 & 0xf) << 4));
        ip[3 * tid + 2] = (uint8_t)((i1 >> 4) & 0xff);
      }
      if (tid >= 64 && tid < 64 + k) vp[tid - 64] = s_sel_val[tid - 64];
    }
    // ---- error feedback residual -----------------------------------------------------
    float acc[4][4];
    if (a.write_residual && a.use_dct) {
      // transmit = F_h^T S F_w with S the k selected coefficients:
      //   Y[j][r] <- F_h[b_j][r],  U[j][l] <- v_j F_w[d_j][l],  out = Y^T U over j < k
      for (int i = tid; i < k * LD; i += NT) {
        const int j = i >> 6, r = i & 63;
        const int e = s_sel_idx[j];
        Y[i] = Fh[(e / w) * LD + r];
        U[i] = s_sel_val[j] * Fw[(e % w) * LD + r];
      }
      __syncthreads();
      mm_tile(Y, U, k, acc);
    } else {
      if (a.write_residual) {
        if (tid < k) { const int e = s_sel_idx[tid]; X[(e / w) * LD + (e % w)] = 0.f; }
        __syncthreads();
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = 4 * ty + i;
      if (r >= h) continue;
      const float4 x = reinterpret_cast<const float4*>(X + r * LD)[tx];
      const float o[4] = {x.x - acc[i][0], x.y - acc[i][1], x.z - acc[i][2], x.w - acc[i][3]};
      const long long g0 = base + (long long)r * d.cols + 4 * tx;
      if (vec) {
        *reinterpret_cast<float4*>(a.ef + g0) = make_float4(o[0], o[1], o[2], o[3]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (4 * tx + j < w) a.ef[g0 + j] = o[j];
      }
    }
  }
}

TPLR_API int tplr_compress_chunks(const void* descs, int n_desc, int total_chunks, const float* basis,
                                  float* ef, const float* theta0, const float* theta,
                                  uint8_t* idx_out, float* val_out, unsigned int* status,
                                  float gamma, int use_dct, int delta_mode, int null_round,
                                  int write_residual, int distinct, void* stream) {
  TPLR_ENTER();
  if (total_chunks <= 0) return 0;
  CompressArgs a;
  a.descs = (const TplrParamDesc*)descs; a.basis = basis; a.ef = ef; a.theta0 = theta0; a.theta = theta;
  a.idx_out = idx_out; a.val_out = val_out; a.status = status; a.n_desc = n_desc;
  a.total_chunks = total_chunks; a.gamma = gamma; a.use_dct = use_dct; a.delta_mode = delta_mode;
  a.null_round = null_round; a.write_residual = write_residual; a.distinct = distinct; a.variant = 0;
  const int smem = (distinct ? 7 : 5) * TPLR_TILE_ELEMS * (int)sizeof(float);
  cudaError_t err = cudaFuncSetAttribute(compress_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (err != cudaSuccess) return (int)err;
  int grid = tplr_sm_count() * (distinct ? 1 : 2);
  if (grid > total_chunks) grid = total_chunks;
  compress_kernel<<<grid, NT, smem, (cudaStream_t)stream>>>(a);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------- //
// received-payload norms and clip factors
// ------------------------------------------------------------------------------------- //
struct PeerPtrs {
  const uint8_t* idx[TPLR_MAX_PEERS];
  const void* val[TPLR_MAX_PEERS];
};

// val_dtype: 0 fp32, 1 bf16, 2 uint8 codes with a per-(peer, tensor) table of
// n_bins lookup entries followed by the shift.
static __device__ __forceinline__ float load_val(const void* p, long long i, int val_dtype,
                                                 const float* qt, int n_bins) {
  if (val_dtype == 0) return reinterpret_cast<const float*>(p)[i];
  if (val_dtype == 1) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  const int code = reinterpret_cast<const uint8_t*>(p)[i];
  return qt[min(code, n_bins - 1)] + qt[n_bins];
}

#define SUMSQ_SPLIT 8
__global__ void __launch_bounds__(256) peer_sumsq_kernel(const TplrParamDesc* __restrict__ descs,
                                                         PeerPtrs pp, int n_params, int val_dtype,
                                                         const float* __restrict__ qtable, int n_bins,
                                                         float* __restrict__ partial) {
  __shared__ float red[32];
  const TplrParamDesc d = descs[blockIdx.x];
  const int peer = blockIdx.y, split = blockIdx.z;
  const long long n = (long long)d.n_chunks * d.k;
  const long long per = (n + SUMSQ_SPLIT - 1) / SUMSQ_SPLIT;
  const long long lo = per * split, hi = min(n, lo + per);
  const float* qt = qtable ? qtable + ((long long)peer * n_params + d.param_id) * (n_bins + 1) : nullptr;
  float s = 0.f;
  for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = load_val(pp.val[peer], d.val_off + i, val_dtype, qt, n_bins);
    s = fmaf(v, v, s);
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) partial[((long long)peer * n_params + d.param_id) * SUMSQ_SPLIT + split] = s;
}

TPLR_API int tplr_peer_sumsq(const void* descs, int n_desc, int n_params, int n_peers,
                             const void* const* val_ptrs, int val_dtype, const float* qtable,
                             int n_bins, float* partial, void* stream) {
  TPLR_ENTER();
  if (n_peers > TPLR_MAX_PEERS || n_peers <= 0) return (int)cudaErrorInvalidValue;
  PeerPtrs pp;
  for (int i = 0; i < n_peers; ++i) { pp.val[i] = val_ptrs[i]; pp.idx[i] = nullptr; }
  dim3 grid(n_desc, n_peers, SUMSQ_SPLIT);
  peer_sumsq_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const TplrParamDesc*)descs, pp, n_params,
                                                             val_dtype, qtable, n_bins, partial);
  return (int)cudaGetLastError();
}

// One thread per tensor: norms, lower median over peers, clip = min(1, med / (norm + 1e-8)).
// A tensor with a non-finite norm from any peer is marked skipped (its update would be
// non-finite and is dropped as a whole).
__global__ void clip_factors_kernel(const float* __restrict__ partial, int n_params, int n_peers,
                                    float* __restrict__ norms, float* __restrict__ clip,
                                    float* __restrict__ median, int* __restrict__ skip,
                                    unsigned int* status) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= n_params) return;
  float nv[TPLR_MAX_PEERS];
  bool bad = false;
  for (int i = 0; i < n_peers; ++i) {
    float s = 0.f;
    const float* q = partial + ((long long)i * n_params + p) * SUMSQ_SPLIT;
    for (int j = 0; j < SUMSQ_SPLIT; ++j) s += q[j];
    const float nrm = sqrtf(s);
    norms[(long long)i * n_params + p] = nrm;
    nv[i] = nrm;
    bad |= !isfinite(nrm);
  }
  for (int i = 1; i < n_peers; ++i) {  // insertion sort, n_peers <= 32
    const float x = nv[i];
    int j = i - 1;
    while (j >= 0 && nv[j] > x) { nv[j + 1] = nv[j]; --j; }
    nv[j + 1] = x;
  }
  const float med = nv[(n_peers - 1) / 2];
  median[p] = med;
  skip[p] = bad ? 1 : 0;
  if (bad && status) atomicOr(status, TPLR_ST_NONFINITE);
  for (int i = 0; i < n_peers; ++i) {
    const float nrm = norms[(long long)i * n_params + p];
    clip[(long long)i * n_params + p] = bad ? 0.f : fminf(1.f, med / (nrm + 1e-8f));
  }
}

TPLR_API int tplr_clip_factors(const float* partial, int n_params, int n_peers, float* norms,
                               float* clip, float* median, int* skip, unsigned int* status,
                               void* stream) {
  TPLR_ENTER();
  if (n_peers > TPLR_MAX_PEERS || n_peers <= 0) return (int)cudaErrorInvalidValue;
  clip_factors_kernel<<<(n_params + 127) / 128, 128, 0, (cudaStream_t)stream>>>(
      partial, n_params, n_peers, norms, clip, median, skip, status);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------- //
// aggregate + inverse DCT + outer update
// ------------------------------------------------------------------------------------- //
struct AggArgs {
  const TplrParamDesc* descs;
  const float* basis;
  const float* clip;        // [n_peers][n_params] or null
  const int* skip;          // [n_params] or null
  const float* qtable;      // see load_val
  const float* theta0;
  float* theta;
  __nv_bfloat16* theta_bf16;
  float* grad_out;
  unsigned int* status;
  int n_desc, total_chunks, n_peers, n_params, n_bins;
  float lr, weight_decay;
  int use_dct, update_mode, val_dtype, distinct;
  int variant;              // tensor-core kernel: bit 2 payload entries of the next pair fetched one pair ahead
  PeerPtrs pp;
};

__global__ void __launch_bounds__(NT, 2) aggregate_kernel(const AggArgs a) {
  extern __shared__ __align__(16) float smem[];
  float* S = smem;
  float* V = S + TPLR_TILE_ELEMS;
  int* Cnt = reinterpret_cast<int*>(V + TPLR_TILE_ELEMS);
  float* Fh = reinterpret_cast<float*>(Cnt + TPLR_TILE_ELEMS);
  float* Fw = a.distinct ? Fh + TPLR_TILE_ELEMS : Fh;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  int cur_fh = -1, cur_fw = -1;

  for (int c = blockIdx.x; c < a.total_chunks; c += gridDim.x) {
    const TplrParamDesc d = a.descs[find_desc(a.descs, a.n_desc, c)];
    const bool skipped = a.skip && a.skip[d.param_id];   // uniform per block
    const int h = d.h, w = d.w, n = h * w, k = d.k;
    const int cl = c - d.chunk_begin;
    const int cy = d.chunk_row0 + cl / d.chunks_x, cx = cl % d.chunks_x;
    const long long base = d.elem_off + (long long)cy * h * d.cols + (long long)cx * w;
    __syncthreads();
    if (a.use_dct && (d.fh_off != cur_fh || d.fw_off != cur_fw)) {
      for (int i = tid; i < TPLR_TILE_ELEMS; i += NT) {
        const int r = i >> 6, cc = i & 63;
        Fh[i] = (r < h && cc < h) ? __ldg(a.basis + d.fh_off + r * h + cc) : 0.f;
        if (a.distinct) Fw[i] = (r < w && cc < w) ? __ldg(a.basis + d.fw_off + r * w + cc) : 0.f;
      }
      cur_fh = d.fh_off;
      cur_fw = d.fw_off;
    }
    for (int i = tid; i < TPLR_TILE_ELEMS; i += NT) { S[i] = 0.f; Cnt[i] = 0; }
    __syncthreads();
    // ---- pull + unpack + scale + scatter-add -----------------------------------------
    const int pairs = k / 2;
    for (int t = tid; t < (skipped ? 0 : a.n_peers * pairs); t += NT) {
      const int peer = t / pairs, pr = t - peer * pairs;
      const uint8_t* ip = a.pp.idx[peer] + d.idx_off + ((long long)cl * pairs + pr) * 3;
      const unsigned b0 = ip[0], b1 = ip[1], b2 = ip[2];
      const int i0 = (int)(b0 | ((b1 & 0xfu) << 8));
      const int i1 = (int)(((b1 >> 4) & 0xfu) | (b2 << 4));
      const long long vo = d.val_off + (long long)cl * k + 2 * pr;
      const float* qt = a.qtable ? a.qtable + ((long long)peer * a.n_params + d.param_id) * (a.n_bins + 1) : nullptr;
      const float sc = a.clip ? a.clip[(long long)peer * a.n_params + d.param_id] : 1.f;
      const float v0 = load_val(a.pp.val[peer], vo, a.val_dtype, qt, a.n_bins) * sc;
      const float v1 = load_val(a.pp.val[peer], vo + 1, a.val_dtype, qt, a.n_bins) * sc;
      if (i0 < n) { const int p = (i0 / w) * LD + (i0 % w); atomicAdd(&S[p], v0); atomicAdd(&Cnt[p], 1); }
      else atomicOr(a.status, TPLR_ST_BAD_INDEX);
      if (i1 < n) { const int p = (i1 / w) * LD + (i1 % w); atomicAdd(&S[p], v1); atomicAdd(&Cnt[p], 1); }
      else atomicOr(a.status, TPLR_ST_BAD_INDEX);
    }
    __syncthreads();
    for (int i = tid; i < TPLR_TILE_ELEMS; i += NT) {
      const int cnt = Cnt[i];
      if (cnt > 1) S[i] = S[i] / (float)cnt;
    }
    __syncthreads();
    // ---- g = F_h^T S F_w -------------------------------------------------------------
    float acc[4][4];
    if (a.use_dct) {
      mm_tile(S, Fh, h, acc);    // V[d][r] = sum_b S[b][d] F_h[b][r]
      store_tile(V, acc);
      __syncthreads();
      mm_tile(V, Fw, w, acc);    // g[r][c] = sum_d V[d][r] F_w[d][c]
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 s = reinterpret_cast<const float4*>(S + (4 * ty + i) * LD)[tx];
        acc[i][0] = s.x; acc[i][1] = s.y; acc[i][2] = s.z; acc[i][3] = s.w;
      }
    }
    // ---- outer update ----------------------------------------------------------------
    const bool vec = (w == 64) && ((d.cols & 3) == 0) && ((base & 3) == 0);
    const float lr = skipped ? 0.f : a.lr;
    const float decay = skipped ? 1.f : (1.f - a.lr * a.weight_decay);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = 4 * ty + i;
      if (r >= h) continue;
      const long long g0 = base + (long long)r * d.cols + 4 * tx;
      float gv[4] = {acc[i][0], acc[i][1], acc[i][2], acc[i][3]};
      if (skipped) { gv[0] = gv[1] = gv[2] = gv[3] = 0.f; }
      if (vec) {
        if (a.grad_out) *reinterpret_cast<float4*>(a.grad_out + g0) = make_float4(gv[0], gv[1], gv[2], gv[3]);
        if (a.update_mode != 2) {
          const float4 t0 = *reinterpret_cast<const float4*>(a.theta0 + g0);
          const float tv[4] = {t0.x, t0.y, t0.z, t0.w};
          float o[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float step = (a.update_mode == 1) ? (gv[j] > 0.f ? 1.f : (gv[j] < 0.f ? -1.f : 0.f)) : gv[j];
            o[j] = tv[j] * decay - lr * step;
          }
          *reinterpret_cast<float4*>(a.theta + g0) = make_float4(o[0], o[1], o[2], o[3]);
          if (a.theta_bf16) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]), hi = __floats2bfloat162_rn(o[2], o[3]);
            uint2 pk;
            pk.x = *reinterpret_cast<unsigned int*>(&lo);
            pk.y = *reinterpret_cast<unsigned int*>(&hi);
            *reinterpret_cast<uint2*>(a.theta_bf16 + g0) = pk;
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (4 * tx + j >= w) continue;
          const float g = gv[j];
          if (a.grad_out) a.grad_out[g0 + j] = g;
          if (a.update_mode != 2) {
            const float step = (a.update_mode == 1) ? (g > 0.f ? 1.f : (g < 0.f ? -1.f : 0.f)) : g;
            const float t = a.theta0[g0 + j] * decay - lr * step;
            a.theta[g0 + j] = t;
            if (a.theta_bf16) a.theta_bf16[g0 + j] = __float2bfloat16(t);
          }
        }
      }
    }
  }
}

TPLR_API int tplr_aggregate_apply(const void* descs, int n_desc, int total_chunks, const float* basis,
                                  int n_peers, const void* const* idx_ptrs, const void* const* val_ptrs,
                                  int val_dtype, const float* qtable, int n_bins, int n_params,
                                  const float* clip, const int* skip, const float* theta0, float* theta,
                                  void* theta_bf16, float* grad_out, float lr, float weight_decay,
                                  int use_dct, int update_mode, int distinct, unsigned int* status,
                                  void* stream) {
  TPLR_ENTER();
  if (total_chunks <= 0) return 0;
  if (n_peers > TPLR_MAX_PEERS || n_peers <= 0) return (int)cudaErrorInvalidValue;
  AggArgs a;
  a.descs = (const TplrParamDesc*)descs; a.basis = basis; a.clip = clip; a.skip = skip; a.qtable = qtable;
  a.theta0 = theta0; a.theta = theta; a.theta_bf16 = (__nv_bfloat16*)theta_bf16; a.grad_out = grad_out;
  a.status = status; a.n_desc = n_desc; a.total_chunks = total_chunks; a.n_peers = n_peers;
  a.n_params = n_params; a.n_bins = n_bins; a.lr = lr; a.weight_decay = weight_decay; a.use_dct = use_dct;
  a.update_mode = update_mode; a.val_dtype = val_dtype; a.distinct = distinct; a.variant = 0;
  for (int i = 0; i < n_peers; ++i) { a.pp.idx[i] = (const uint8_t*)idx_ptrs[i]; a.pp.val[i] = val_ptrs[i]; }
  const int smem = (distinct ? 5 : 4) * TPLR_TILE_ELEMS * (int)sizeof(float);
  cudaError_t err = cudaFuncSetAttribute(aggregate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (err != cudaSuccess) return (int)err;
  int grid = tplr_sm_count() * 2;
  if (grid > total_chunks) grid = total_chunks;
  aggregate_kernel<<<grid, NT, smem, (cudaStream_t)stream>>>(a);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------- //
// Tensor-core path of the inverse chunk DCT (all chunks 64 x 64, one shared basis F).
//
// g = F^T S F for two chunks at a time as two tcgen05 GEMMs of shape 128 x 64 x 64 against the basis:
//   Z[(c,j)][r]   = sum_n S_c[n][j] F[n][r]     A = S^T rows (K-major),        B = F read N-contiguous
//   g[(c,r)][col] = sum_j Z_c[j][r] F[j][col]   A = Z read M-contiguous (no transpose pass), B = F again
// fp32 operands are split into three bf16 terms (x = b1 + b2 + b3, 24 mantissa bits) and the six
// products whose weight is above 2^-24 are accumulated in fp32 in tensor memory, so the result has
// fp32-grade accuracy.  The 128-byte-swizzled tile that holds Z is written once and read by the second
// GEMM through an M-major descriptor; the basis tile is shared by both GEMMs.
// ------------------------------------------------------------------------------------- //
namespace {
using namespace tplr_tc;

constexpr int TC_A_TILE = 128 * 128;          // bytes: 128 rows x 64 bf16
constexpr int TC_B_TILE = 64 * 128;           // bytes: 64 rows x 64 bf16
constexpr int TC_ACC_BYTES = 2 * 4096 * 8;    // two chunks: fp32 sums + int counts = 64 KB
constexpr int TC_SMEM_AGG = TC_ACC_BYTES + 3 * TC_B_TILE + 1024;

__device__ __forceinline__ void split3(float x, __nv_bfloat16& b1, __nv_bfloat16& b2, __nv_bfloat16& b3) {
  b1 = __float2bfloat16_rn(x);
  const float r1 = x - __bfloat162float(b1);
  b2 = __float2bfloat16_rn(r1);
  b3 = __float2bfloat16_rn(r1 - __bfloat162float(b2));
}

// Writes 32 consecutive fp32 values of one tile row (columns 32*hf .. 32*hf+31) as three bf16 split tiles.
// row: 128-byte row index inside the tile whose three term copies start at base, base + stride, base + 2*stride.
__device__ __forceinline__ void store_split_row(uint32_t base, uint32_t stride, int row, int hf, const float* v) {
  const uint32_t rowaddr = base + (uint32_t)row * 128u;
  const uint32_t sw = (uint32_t)(row & 7);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint32_t w1[4], w2[4], w3[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      __nv_bfloat16 a1, a2, a3, c1, c2, c3;
      split3(v[8 * q + 2 * e], a1, a2, a3);
      split3(v[8 * q + 2 * e + 1], c1, c2, c3);
      __nv_bfloat162 h1 = __halves2bfloat162(a1, c1), h2 = __halves2bfloat162(a2, c2), h3 = __halves2bfloat162(a3, c3);
      w1[e] = *reinterpret_cast<uint32_t*>(&h1);
      w2[e] = *reinterpret_cast<uint32_t*>(&h2);
      w3[e] = *reinterpret_cast<uint32_t*>(&h3);
    }
    const uint32_t off = (((uint32_t)(hf * 4 + q)) ^ sw) << 4;
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + off), "r"(w1[0]), "r"(w1[1]), "r"(w1[2]), "r"(w1[3]) : "memory");
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + stride + off), "r"(w2[0]), "r"(w2[1]), "r"(w2[2]), "r"(w2[3]) : "memory");
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + 2 * stride + off), "r"(w3[0]), "r"(w3[1]), "r"(w3[2]), "r"(w3[3]) : "memory");
  }
}

// The 64 x 64 basis (row-major fp32 in global memory) as three swizzled bf16 tiles [64 rows x 128 B].
__device__ __forceinline__ void load_basis_split(const float* __restrict__ g, uint32_t sB) {
  // 256 threads: row = tid / 4, 16 columns each
  const int row = threadIdx.x >> 2, c0 = (threadIdx.x & 3) * 16;
  const uint32_t rowaddr = sB + (uint32_t)row * 128u;
  const uint32_t sw = (uint32_t)(row & 7);
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    uint32_t w1[4], w2[4], w3[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      __nv_bfloat16 a1, a2, a3, c1, c2, c3;
      split3(__ldg(g + row * 64 + c0 + 8 * q + 2 * e), a1, a2, a3);
      split3(__ldg(g + row * 64 + c0 + 8 * q + 2 * e + 1), c1, c2, c3);
      __nv_bfloat162 h1 = __halves2bfloat162(a1, c1), h2 = __halves2bfloat162(a2, c2), h3 = __halves2bfloat162(a3, c3);
      w1[e] = *reinterpret_cast<uint32_t*>(&h1);
      w2[e] = *reinterpret_cast<uint32_t*>(&h2);
      w3[e] = *reinterpret_cast<uint32_t*>(&h3);
    }
    const uint32_t off = (((uint32_t)(c0 / 8 + q)) ^ sw) << 4;
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + off), "r"(w1[0]), "r"(w1[1]), "r"(w1[2]), "r"(w1[3]) : "memory");
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + TC_B_TILE + off), "r"(w2[0]), "r"(w2[1]), "r"(w2[2]), "r"(w2[3]) : "memory");
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + 2 * TC_B_TILE + off), "r"(w3[0]), "r"(w3[1]), "r"(w3[2]), "r"(w3[3]) : "memory");
  }
}

// D[128 x 64] = A B with the six significant products of the 3-term splits.  a_mn: A tile holds K rows of
// 128 bytes of M (two 64-wide M blocks 8 KB apart); otherwise A tile holds 128 M rows of 128 bytes of K.
// b_mn: the basis tile is read with its rows as K (B = F); otherwise with its rows as N (B = F^T).
__device__ __forceinline__ void issue_split_gemm(uint32_t tD, uint32_t sA, uint32_t sB, bool a_mn, bool b_mn) {
  const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
                         ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
  const int ta[6] = {0, 0, 1, 0, 1, 2}, tb[6] = {0, 1, 0, 2, 1, 0};
  uint32_t first = 1;
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
    for (int t = 0; t < 6; ++t) {
      const uint32_t a0 = sA + (uint32_t)ta[t] * TC_A_TILE, b0 = sB + (uint32_t)tb[t] * TC_B_TILE;
      const uint64_t da = a_mn ? make_desc(a0 + kk * 2048u, 8192, 1024) : make_desc(a0 + kk * 32u, 16, 1024);
      const uint64_t db = b_mn ? make_desc(b0 + kk * 2048u, 8192, 1024) : make_desc(b0 + kk * 32u, 16, 1024);
      umma_bf16(tD, da, db, idesc, first ? 0u : 1u);
      first = 0;
    }
  }
}

__global__ void __launch_bounds__(NT, 2) aggregate_tc_kernel(const AggArgs a) {
  extern __shared__ uint8_t smem_raw_tc[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw_tc) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t bar_mma;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ TplrParamDesc s_desc[2];
  __shared__ long long s_gbase[2];                                 // element offset of each chunk of the pair, -1: none
  __shared__ int s_cols[2], s_skip[2];
  float* S = reinterpret_cast<float*>(smem);                       // [2][4096] sums, later the A tiles
  int* Cnt = reinterpret_cast<int*>(smem + 2 * 4096 * 4);          // [2][4096] contributor counts
  const uint32_t sA = smem_u32(smem), sB = sA + TC_ACC_BYTES;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qd = warp & 3, hf = warp >> 2;                         // TMEM lane quadrant, column half
  const int ch = qd >> 1, rin = (qd & 1) * 32 + lane;              // chunk of the pair, row inside the chunk
  const int trow = ch * 64 + rin;                                  // row of the stacked 128-row tiles
  const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
  volatile int* abort_flag = &s_abort;
  int cur_f = -1;
  uint32_t phase = 0;

  if (tid == 0) {
    s_abort = 0;
    mbar_init(smem_u32(&bar_mma), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 128;" ::"r"(smem_u32(&s_tmem_base)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tZ = s_tmem_base, tG = s_tmem_base + 64;
  const int n_pairs = (a.total_chunks + 1) / 2;
  bool ok = true;
  TplrParamDesc d = a.descs[0];

  // One pair ahead: thread t owns scatter task t of a pair (chunk of the pair, peer, index pair) and holds
  // that task's raw bytes for the NEXT pair in registers, so the dependent chain packed index -> value ->
  // table entry of a pair is already under way while the previous pair is in the tensor cores.  The loaded
  // registers are not touched before the scatter that consumes them.  Tasks beyond the first NT of a pair
  // (more than 8 peers at k = 32) are fetched in line as before.
  const bool ahead = (a.variant & 4) != 0;
  const int pf_pairs = max(1, d.k / 2), pf_per = max(1, a.n_peers) * pf_pairs;
  const int pf_c2 = tid / pf_per, pf_rem = tid - pf_c2 * pf_per;
  const int pf_peer = pf_rem / pf_pairs, pf_pr = pf_rem - pf_peer * pf_pairs;
  int pf_begin = d.chunk_begin, pf_n = d.n_chunks, pf_param = d.param_id;     // cached descriptor fields of the task's tensor
  long long pf_idx_off = d.idx_off, pf_val_off = d.val_off;
  unsigned pf_b0 = 0, pf_b1 = 0, pf_b2 = 0, pf_r0 = 0, pf_r1 = 0;
  float pf_sc = 1.f;
  bool pf_valid = false;
  auto fetch_ahead = [&](int qq) {
    pf_valid = false;
    if (!ahead || tid >= 2 * pf_per || qq >= n_pairs) return;
    const int cc = 2 * qq + pf_c2;
    if (cc >= a.total_chunks) return;
    if (!(cc >= pf_begin && cc < pf_begin + pf_n)) {
      const TplrParamDesc& dn = a.descs[find_desc(a.descs, a.n_desc, cc)];
      pf_begin = dn.chunk_begin; pf_n = dn.n_chunks; pf_param = dn.param_id;
      pf_idx_off = dn.idx_off; pf_val_off = dn.val_off;
    }
    if (a.skip && a.skip[pf_param]) return;
    const int cl2 = cc - pf_begin;
    const uint8_t* ip = a.pp.idx[pf_peer] + pf_idx_off + ((long long)cl2 * pf_pairs + pf_pr) * 3;
    const long long vo = pf_val_off + (long long)cl2 * (2 * pf_pairs) + 2 * pf_pr;
    pf_b0 = ip[0]; pf_b1 = ip[1]; pf_b2 = ip[2];
    if (a.val_dtype == 0) {
      pf_r0 = __float_as_uint(reinterpret_cast<const float*>(a.pp.val[pf_peer])[vo]);
      pf_r1 = __float_as_uint(reinterpret_cast<const float*>(a.pp.val[pf_peer])[vo + 1]);
    } else if (a.val_dtype == 1) {
      pf_r0 = reinterpret_cast<const unsigned short*>(a.pp.val[pf_peer])[vo];
      pf_r1 = reinterpret_cast<const unsigned short*>(a.pp.val[pf_peer])[vo + 1];
    } else {
      pf_r0 = reinterpret_cast<const uint8_t*>(a.pp.val[pf_peer])[vo];
      pf_r1 = reinterpret_cast<const uint8_t*>(a.pp.val[pf_peer])[vo + 1];
    }
    pf_sc = a.clip ? a.clip[(long long)pf_peer * a.n_params + pf_param] : 1.f;
    pf_valid = true;
  };
  fetch_ahead(blockIdx.x);

  for (int q = blockIdx.x; q < n_pairs && ok; q += gridDim.x) {
    // this thread's chunk of the pair
    const int c = 2 * q + ch;
    const bool active = c < a.total_chunks;
    {
      // consecutive chunks mostly belong to the same tensor: search the table only when the cached entry misses
      const int cc = active ? c : a.total_chunks - 1;
      if (!(cc >= d.chunk_begin && cc < d.chunk_begin + d.n_chunks)) d = a.descs[find_desc(a.descs, a.n_desc, cc)];
    }
    const int cl = c - d.chunk_begin;
    const int cy = d.chunk_row0 + cl / d.chunks_x, cx = cl % d.chunks_x;
    const long long base = d.elem_off + (long long)cy * 64 * d.cols + (long long)cx * 64;
    const bool skipped = a.skip && a.skip[d.param_id];
    __syncthreads();                                   // previous pair's tiles and accumulators are free
    if (rin == 0 && hf == 0) {                         // the scatter and the update below work on both chunks of the pair
      s_desc[ch] = d;
      s_gbase[ch] = active ? base : -1;
      s_cols[ch] = d.cols;
      s_skip[ch] = skipped ? 1 : 0;
    }
    if (d.fh_off != cur_f) {                           // uniform: every 64 x 64 chunk uses the same basis
      load_basis_split(a.basis + d.fh_off, sB);
      cur_f = d.fh_off;
    }
    for (int i = tid; i < TC_ACC_BYTES / 16; i += NT) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    // ---- pull + unpack + scale + scatter-add, both chunks --------------------------------
    if (ahead) {
      if (pf_valid) {                                  // this thread's task of the pair, fetched one pair ago
        const int i0 = (int)(pf_b0 | ((pf_b1 & 0xfu) << 8));
        const int i1 = (int)(((pf_b1 >> 4) & 0xfu) | (pf_b2 << 4));
        float v0, v1;
        if (a.val_dtype == 0) {
          v0 = __uint_as_float(pf_r0); v1 = __uint_as_float(pf_r1);
        } else if (a.val_dtype == 1) {
          v0 = __uint_as_float(pf_r0 << 16); v1 = __uint_as_float(pf_r1 << 16);
        } else {
          const float* qt = a.qtable + ((long long)pf_peer * a.n_params + pf_param) * (a.n_bins + 1);
          const float shift = qt[a.n_bins];
          v0 = qt[min((int)pf_r0, a.n_bins - 1)] + shift; v1 = qt[min((int)pf_r1, a.n_bins - 1)] + shift;
        }
        v0 *= pf_sc; v1 *= pf_sc;
        atomicAdd(&S[pf_c2 * 4096 + i0], v0); atomicAdd(&Cnt[pf_c2 * 4096 + i0], 1);
        atomicAdd(&S[pf_c2 * 4096 + i1], v1); atomicAdd(&Cnt[pf_c2 * 4096 + i1], 1);
      }
      fetch_ahead(q + gridDim.x);
    }
    {
      const int pairs = d.k / 2;                       // k is the same for all 64 x 64 chunks of a layout
      for (int t = ahead ? tid + NT : tid; t < 2 * a.n_peers * pairs; t += NT) {
        const int c2 = t / (a.n_peers * pairs), rem = t - c2 * (a.n_peers * pairs);
        const int cc = 2 * q + c2;
        if (cc >= a.total_chunks) continue;
        const TplrParamDesc& d2 = s_desc[c2];
        if (a.skip && a.skip[d2.param_id]) continue;
        const int cl2 = cc - d2.chunk_begin;
        const int peer = rem / pairs, pr = rem - peer * pairs;
        const uint8_t* ip = a.pp.idx[peer] + d2.idx_off + ((long long)cl2 * pairs + pr) * 3;
        const unsigned b0 = ip[0], b1 = ip[1], b2 = ip[2];
        const int i0 = (int)(b0 | ((b1 & 0xfu) << 8));
        const int i1 = (int)(((b1 >> 4) & 0xfu) | (b2 << 4));
        const long long vo = d2.val_off + (long long)cl2 * d2.k + 2 * pr;
        const float* qt = a.qtable ? a.qtable + ((long long)peer * a.n_params + d2.param_id) * (a.n_bins + 1) : nullptr;
        const float sc = a.clip ? a.clip[(long long)peer * a.n_params + d2.param_id] : 1.f;
        const float v0 = load_val(a.pp.val[peer], vo, a.val_dtype, qt, a.n_bins) * sc;
        const float v1 = load_val(a.pp.val[peer], vo + 1, a.val_dtype, qt, a.n_bins) * sc;
        atomicAdd(&S[c2 * 4096 + i0], v0); atomicAdd(&Cnt[c2 * 4096 + i0], 1);   // 12-bit indices: always < 4096
        atomicAdd(&S[c2 * 4096 + i1], v1); atomicAdd(&Cnt[c2 * 4096 + i1], 1);
      }
    }
    __syncthreads();
    // ---- mean, transposed read: row j of S_c^T, columns n = 32*hf .. ------------------------
    float v[32];
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      const int n = hf * 32 + e;
      const float s = S[ch * 4096 + n * 64 + rin];
      const int cnt = Cnt[ch * 4096 + n * 64 + rin];
      v[e] = cnt > 1 ? s / (float)cnt : s;
    }
    __syncthreads();                                   // accumulators are read out: their bytes become the A tiles
    store_split_row(sA, TC_A_TILE, trow, hf, v);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tcgen05_fence_before();
    __syncthreads();
    if (tid == 0) {
      tcgen05_fence_after();
      issue_split_gemm(tZ, sA, sB, /*a_mn=*/false, /*b_mn=*/true);      // Z = S^T F
      umma_commit(smem_u32(&bar_mma));
    }
    ok = mbar_wait(smem_u32(&bar_mma), phase, abort_flag);
    phase ^= 1;
    ok = __syncthreads_and(ok);
    if (!ok) break;
    tcgen05_fence_after();
    {
      uint32_t r[32];
      tmem_ld32(tZ + hf * 32 + lane_off, r);
#pragma unroll
      for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(r[e]);
    }
    // Z_c rows (index j) into block c of the tiles: read back M-contiguous by the second GEMM
    store_split_row(sA + (uint32_t)ch * 8192u, TC_A_TILE, rin, hf, v);
    // The update runs in a row-contiguous mapping: half a warp per row of the stacked 128 x 64 result, 16 bytes
    // per lane, so that every global access of a warp covers two whole 256-byte rows (the accumulator mapping,
    // one row per lane, touches 32 lines per instruction).  The snapshot values are requested here and used
    // after the second product.
    const int urow = tid >> 4, uc4 = tid & 15;
    float4 t0r[8];
    if (a.update_mode != 2) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int row = i * 16 + urow, c2 = row >> 6;
        const long long gb = s_gbase[c2];
        if (gb >= 0) t0r[i] = *reinterpret_cast<const float4*>(a.theta0 + gb + (long long)(row & 63) * s_cols[c2] + uc4 * 4);
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tcgen05_fence_before();
    __syncthreads();
    if (tid == 0) {
      tcgen05_fence_after();
      issue_split_gemm(tG, sA, sB, /*a_mn=*/true, /*b_mn=*/true);       // g = Z^T F
      umma_commit(smem_u32(&bar_mma));
    }
    ok = mbar_wait(smem_u32(&bar_mma), phase, abort_flag);
    phase ^= 1;
    ok = __syncthreads_and(ok);
    if (!ok) break;
    tcgen05_fence_after();
    uint32_t gr[32];
    tmem_ld32(tG + hf * 32 + lane_off, gr);
    tcgen05_fence_before();
    // ---- outer update ---------------------------------------------------------------------------
    // g leaves the accumulator mapping through shared memory (the tiles of the finished products are free):
    // row trow, 16-byte slots swizzled by the row so that both mappings are conflict-free.
    {
      const uint32_t st_own = sA + (uint32_t)trow * 256u + (uint32_t)hf * 128u;
      const uint32_t sw = (uint32_t)(trow & 7);
#pragma unroll
      for (int q4 = 0; q4 < 8; ++q4)
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(st_own + (((uint32_t)q4 ^ sw) << 4)), "r"(gr[4 * q4]),
                     "r"(gr[4 * q4 + 1]), "r"(gr[4 * q4 + 2]), "r"(gr[4 * q4 + 3]) : "memory");
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int row = i * 16 + urow, c2 = row >> 6;
      const long long gb = s_gbase[c2];
      if (gb < 0) continue;
      const bool skp = s_skip[c2] != 0;
      const float lr = skp ? 0.f : a.lr;
      const float decay = skp ? 1.f : (1.f - a.lr * a.weight_decay);
      const long long g0 = gb + (long long)(row & 63) * s_cols[c2] + uc4 * 4;
      float gv[4];
      asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(gv[0]), "=f"(gv[1]), "=f"(gv[2]), "=f"(gv[3])
                   : "r"(sA + (uint32_t)row * 256u + (uint32_t)(uc4 >> 3) * 128u + ((((uint32_t)uc4 & 7u) ^ (uint32_t)(row & 7)) << 4))
                   : "memory");
      if (skp) { gv[0] = gv[1] = gv[2] = gv[3] = 0.f; }
      if (a.grad_out) *reinterpret_cast<float4*>(a.grad_out + g0) = make_float4(gv[0], gv[1], gv[2], gv[3]);
      if (a.update_mode != 2) {
        const float tv[4] = {t0r[i].x, t0r[i].y, t0r[i].z, t0r[i].w};
        float o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float step = (a.update_mode == 1) ? (gv[e] > 0.f ? 1.f : (gv[e] < 0.f ? -1.f : 0.f)) : gv[e];
          o[e] = tv[e] * decay - lr * step;
        }
        *reinterpret_cast<float4*>(a.theta + g0) = make_float4(o[0], o[1], o[2], o[3]);
        if (a.theta_bf16) {
          __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]), hi = __floats2bfloat162_rn(o[2], o[3]);
          uint2 pk;
          pk.x = *reinterpret_cast<unsigned int*>(&lo);
          pk.y = *reinterpret_cast<unsigned int*>(&hi);
          *reinterpret_cast<uint2*>(a.theta_bf16 + g0) = pk;
        }
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 0) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 128;" ::"r"(s_tmem_base) : "memory");
  }
  if (tid == 0 && s_abort && a.status) atomicOr(a.status, TPLR_ST_WAIT_TIMEOUT);
}

// ------------------------------------------------------------------------------------- //
// Tensor-core path of the compress kernel (all chunks 64 x 64, one shared basis): the forward DCT
// Y = F X F^T and the dense inverse of the selected coefficients run as tcgen05 GEMMs (same 3-term
// split, same tile tricks as aggregate_tc_kernel); top-k selection, packing and the error-feedback
// update stay on the CUDA cores.  Two chunks per step: the 128 threads whose TMEM lanes hold a chunk
// select for it.  Thread (chunk ch, row rin, column half hf) owns X[rin][32*hf..] and, after the
// second GEMM, the coefficients Y[32*hf .. 32*hf+31][rin] (the GEMM pair leaves Y transposed).
// ------------------------------------------------------------------------------------- //
constexpr int TC_NCAND = 256;                // candidates of the threshold search per chunk (the histogram's storage)
constexpr int TC_X_BYTES = 128 * 64 * 4;     // fp32 copy of the two chunks (each thread re-reads only its own part)
constexpr int TC_SMEM_CMP = 3 * TC_A_TILE + 3 * TC_B_TILE + TC_X_BYTES + 1024;

__global__ void __launch_bounds__(NT, 2) compress_tc_kernel(const CompressArgs a) {
  extern __shared__ uint8_t smem_raw_tc[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw_tc) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t bar_mma;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ int s_hist[2][256];
  __shared__ int s_wsum[8];
  __shared__ int s_bin[2], s_krem[2];
  __shared__ __align__(16) unsigned int s_tmax[2][128];
  __shared__ unsigned int s_thr[2];
  __shared__ long long s_gbase[2];                       // element offset of each chunk of the pair, -1: none
  __shared__ int s_cols[2];
  __shared__ int s_sel_idx[2][TPLR_TILE];
  __shared__ float s_sel_val[2][TPLR_TILE];
  const uint32_t sA = smem_u32(smem), sB = sA + 3 * TC_A_TILE, sX = sB + 3 * TC_B_TILE;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qd = warp & 3, hf = warp >> 2;
  const int ch = qd >> 1, rin = (qd & 1) * 32 + lane;
  const int trow = ch * 64 + rin;
  const int lt = rin + hf * 64;                          // thread index inside the chunk's group of 128
  const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
  const uint32_t xaddr = sX + (uint32_t)trow * 256u + (uint32_t)hf * 128u;
  const uint32_t xsw = (uint32_t)(lane & 7);
  volatile int* abort_flag = &s_abort;
  int cur_f = -1;
  uint32_t phase = 0;

  if (tid == 0) {
    s_abort = 0;
    mbar_init(smem_u32(&bar_mma), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 128;" ::"r"(smem_u32(&s_tmem_base)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tZ = s_tmem_base, tY = s_tmem_base + 64;
  const int n_pairs = (a.total_chunks + 1) / 2;
  bool ok = true;

  TplrParamDesc d = a.descs[0];
  auto run_gemm = [&](uint32_t tD, bool a_mn, bool b_mn) -> bool {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tcgen05_fence_before();
    __syncthreads();
    if (tid == 0) {
      tcgen05_fence_after();
      issue_split_gemm(tD, sA, sB, a_mn, b_mn);
      umma_commit(smem_u32(&bar_mma));
    }
    bool o = mbar_wait(smem_u32(&bar_mma), phase, abort_flag);
    phase ^= 1;
    o = __syncthreads_and(o);
    tcgen05_fence_after();
    return o;
  };

  for (int q = blockIdx.x; q < n_pairs && ok; q += gridDim.x) {
    const int c = 2 * q + ch;
    const bool active = c < a.total_chunks;
    {
      const int cc = active ? c : a.total_chunks - 1;
      if (!(cc >= d.chunk_begin && cc < d.chunk_begin + d.n_chunks)) d = a.descs[find_desc(a.descs, a.n_desc, cc)];
    }
    const int k = d.k;
    const int cl = c - d.chunk_begin;
    const int cy = d.chunk_row0 + cl / d.chunks_x, cx = cl % d.chunks_x;
    const long long gbase = d.elem_off + (long long)cy * 64 * d.cols + (long long)cx * 64;
    __syncthreads();
    if (rin == 0 && hf == 0) { s_gbase[ch] = active ? gbase : -1; s_cols[ch] = d.cols; }
    if (d.fh_off != cur_f) {
      load_basis_split(a.basis + d.fh_off, sB);
      cur_f = d.fh_off;
    }
    __syncthreads();
    // ---- X = gamma*e + delta into the fp32 copy in shared memory ------------------------------------
    // Row-contiguous mapping: half a warp per row of the stacked 128 x 64 tile, 16 bytes per lane, so that every
    // global access of a warp covers two whole 256-byte rows (one row per lane would touch 32 lines per
    // instruction).  Slot (row, 16-byte column c4) of the copy: row * 256 + (c4 / 8) * 128 + ((c4 % 8) ^ (row % 8)) * 16.
    const int urow = tid >> 4, uc4 = tid & 15;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int row = i * 16 + urow, c2 = row >> 6;
      const long long gb = s_gbase[c2];
      float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
      if (gb >= 0 && !a.null_round) {
        const long long g = gb + (long long)(row & 63) * s_cols[c2] + uc4 * 4;
        const float4 e = *reinterpret_cast<const float4*>(a.ef + g);
        float4 dl = *reinterpret_cast<const float4*>(a.theta0 + g);
        if (a.delta_mode) {
          const float4 t = *reinterpret_cast<const float4*>(a.theta + g);
          dl.x -= t.x; dl.y -= t.y; dl.z -= t.z; dl.w -= t.w;
        }
        x.x = fmaf(a.gamma, e.x, dl.x); x.y = fmaf(a.gamma, e.y, dl.y);
        x.z = fmaf(a.gamma, e.z, dl.z); x.w = fmaf(a.gamma, e.w, dl.w);
      }
      asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(sX + (uint32_t)row * 256u + (uint32_t)(uc4 >> 3) * 128u +
                   ((((uint32_t)uc4 & 7u) ^ (uint32_t)(row & 7)) << 4)), "f"(x.x), "f"(x.y), "f"(x.z), "f"(x.w) : "memory");
    }
    __syncthreads();
    // this thread's 32 values (row trow, columns 32*hf ..) for the operand tile
    float v[32];
#pragma unroll
    for (int q4 = 0; q4 < 8; ++q4)
      asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v[4 * q4]), "=f"(v[4 * q4 + 1]), "=f"(v[4 * q4 + 2]),
                   "=f"(v[4 * q4 + 3]) : "r"(xaddr + (((uint32_t)q4 ^ xsw) << 4)) : "memory");
    store_split_row(sA, TC_A_TILE, trow, hf, v);
    if ((a.variant & 2) && !a.null_round) {
      // the next pair's 128 bytes of this thread in the three dense tensors, asked into L2 now
      const int cn = c + 2 * (int)gridDim.x;
      if (cn < a.total_chunks && cn < d.chunk_begin + d.n_chunks) {
        const int cln = cn - d.chunk_begin;
        const long long gn = d.elem_off + (long long)(d.chunk_row0 + cln / d.chunks_x) * 64 * d.cols +
                             (long long)(cln % d.chunks_x) * 64 + (long long)rin * d.cols + hf * 32;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(a.ef + gn));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(a.theta0 + gn));
        if (a.delta_mode) asm volatile("prefetch.global.L2 [%0];" ::"l"(a.theta + gn));
      }
    }
    if (!(ok = run_gemm(tZ, /*a_mn=*/false, /*b_mn=*/false))) break;          // Z = X F^T
    {
      uint32_t r[32];
      tmem_ld32(tZ + hf * 32 + lane_off, r);
#pragma unroll
      for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(r[e]);
    }
    store_split_row(sA + (uint32_t)ch * 8192u, TC_A_TILE, rin, hf, v);
    if (!(ok = run_gemm(tY, /*a_mn=*/true, /*b_mn=*/false))) break;           // Y^T = Z^T F^T
    {
      uint32_t r[32];
      tmem_ld32(tY + hf * 32 + lane_off, r);
#pragma unroll
      for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(r[e]);             // v[e] = Y[32*hf + e][rin]
    }
    tcgen05_fence_before();
    // ---- threshold of the k largest |Y| of each chunk (its 128 threads, 32 keys each) ---------
    // Result: prefix = the k-th largest key, krem = how many keys equal to it belong to the selection.
    // Fast path: the k-th largest of the 128 per-thread maxima is a lower bound of the k-th largest key
    // (k distinct keys are at least that large), so only the keys at or above it (a few dozen for k = 32)
    // are candidates; they are compacted into shared memory and the exact threshold is found by counting
    // among them.  No shared-memory atomics: the histogram of the radix select below serialises on the
    // few exponent values that the keys share.  More candidates than fit (many equal keys) or
    // k > 128 take the radix select.
    unsigned int prefix = 0u, mask = 0u;
    int krem = k;
    bool radix = true;
    if (k <= 128 && (a.variant & 1)) {
      unsigned int m = 0u;
#pragma unroll
      for (int i = 0; i < 32; ++i) m = max(m, __float_as_uint(v[i]) & 0x7fffffffu);
      s_tmax[ch][lt] = m;
      __syncthreads();
      {
        int rank = 0;
        const uint4* row = reinterpret_cast<const uint4*>(s_tmax[ch]);
#pragma unroll 8
        for (int j4 = 0; j4 < 32; ++j4) {
          const uint4 o = row[j4];
          const int j = 4 * j4;
          rank += (o.x > m) || (o.x == m && j < lt);
          rank += (o.y > m) || (o.y == m && j + 1 < lt);
          rank += (o.z > m) || (o.z == m && j + 2 < lt);
          rank += (o.w > m) || (o.w == m && j + 3 < lt);
        }
        if (rank == k - 1) s_thr[ch] = m;
      }
      __syncthreads();
      // zero keys never are candidates: a chunk with fewer than k non-zero coefficients (rows of the embedding that
      // no token touched, a null round) has t0 == 0 and is resolved without any search: all non-zero keys and the
      // first k - n_cand zeros in order
      const unsigned int t0 = s_thr[ch] ? s_thr[ch] : 1u;
      int cnt = 0;
#pragma unroll
      for (int i = 0; i < 32; ++i) cnt += (__float_as_uint(v[i]) & 0x7fffffffu) >= t0;
      int incl = cnt;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
      }
      if (lane == 31) s_wsum[warp] = incl;
      __syncthreads();
      // warps of chunk ch hold lt blocks in the order 2ch, 2ch+1, 2ch+4, 2ch+5
      const int w0 = s_wsum[2 * ch], w1 = s_wsum[2 * ch + 1], w2 = s_wsum[2 * ch + 4], w3 = s_wsum[2 * ch + 5];
      const int slot = (warp & 1) + 2 * (warp >> 2);
      int off = incl - cnt + (slot > 0 ? w0 : 0) + (slot > 1 ? w1 : 0) + (slot > 2 ? w2 : 0);
      const int n_cand = w0 + w1 + w2 + w3;
      // both chunks of the pair take the same path (the radix select synchronises the whole CTA)
      const int n_other = s_wsum[2 * (ch ^ 1)] + s_wsum[2 * (ch ^ 1) + 1] + s_wsum[2 * (ch ^ 1) + 4] + s_wsum[2 * (ch ^ 1) + 5];
      radix = n_cand > TC_NCAND || n_other > TC_NCAND;
      if (!radix) {
        unsigned int* cand = reinterpret_cast<unsigned int*>(s_hist[ch]);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const unsigned int key = __float_as_uint(v[i]) & 0x7fffffffu;
          if (key >= t0) cand[off++] = key;
        }
        __syncthreads();
        for (int j = lt; j < n_cand; j += 128) {
          const unsigned int cj = cand[j];
          int gt = 0, ge = 0;
          for (int i = 0; i < n_cand; ++i) {
            const unsigned int x = cand[i];
            gt += x > cj; ge += x >= cj;
          }
          if (gt < k && k <= ge) { s_bin[ch] = (int)cj; s_krem[ch] = k - gt; }   // ties write the same pair
        }
        __syncthreads();
        if (n_cand < k) { prefix = 0u; krem = k - n_cand; }      // sparse chunk (only possible with t0 == 1)
        else { prefix = (unsigned int)s_bin[ch]; krem = s_krem[ch]; }
      }
      __syncthreads();            // s_hist, s_wsum, s_bin and s_krem are reused below
    }
#pragma unroll 1
    for (int pass = 0; radix && pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      s_hist[0][tid] = 0; s_hist[1][tid] = 0;
      __syncthreads();
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const unsigned int key = __float_as_uint(v[i]) & 0x7fffffffu;
        if ((key & mask) == prefix) atomicAdd(&s_hist[ch][(key >> shift) & 255u], 1);
      }
      __syncthreads();
      if (warp < 2) {                                     // warp w scans the histogram of chunk w
        // every thread of a chunk carries the same (prefix, krem); warp w reads chunk w's from shared memory
        const int kr = pass == 0 ? k : s_krem[warp];
        const int hi = 255 - 8 * lane;
        int sum = 0;
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) sum += s_hist[warp][hi - jj];
        int incl = sum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          int t = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += t;
        }
        const int excl = incl - sum;
        int bin = -1, rem = 0;
        if (excl < kr && kr <= incl) {
          int run = excl;
          for (int jj = 0; jj < 8; ++jj) {
            const int cnt = s_hist[warp][hi - jj];
            if (run + cnt >= kr) { bin = hi - jj; rem = kr - run; break; }
            run += cnt;
          }
        }
        __syncwarp();
        if (bin >= 0) { s_bin[warp] = bin; s_krem[warp] = rem; }
      }
      __syncthreads();
      prefix |= ((unsigned int)s_bin[ch]) << shift;
      mask |= 255u << shift;
      krem = s_krem[ch];
      __syncthreads();
    }
    // ---- ordered compaction inside each chunk's four warps -----------------------------------
    int gcnt = 0, qcnt = 0;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const unsigned int key = __float_as_uint(v[i]) & 0x7fffffffu;
      gcnt += key > prefix; qcnt += key == prefix;
    }
    const int packed = gcnt | (qcnt << 16);
    int incl = packed;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) s_wsum[warp] = incl;
    __syncthreads();
    int woff = 0;
    {
      // warps of chunk ch in order: 2ch, 2ch+1, 2ch+4, 2ch+5
      const int order[4] = {2 * ch, 2 * ch + 1, 2 * ch + 4, 2 * ch + 5};
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) if (order[jj] != warp && ((order[jj] < warp && (order[jj] >> 2) == (warp >> 2)) || (order[jj] >> 2) < (warp >> 2))) woff += s_wsum[order[jj]];
    }
    const int excl = incl - packed + woff;
    int gb = excl & 0xffff, qb = excl >> 16;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const unsigned int key = __float_as_uint(v[i]) & 0x7fffffffu;
      int pos = -1;
      if (key > prefix) { pos = gb + min(qb, krem); ++gb; }
      else if (key == prefix) { if (qb < krem) pos = gb + qb; ++qb; }
      if (pos >= 0 && pos < TPLR_TILE) {
        s_sel_idx[ch][pos] = (hf * 32 + i) * 64 + rin;     // row-major index of Y[32*hf + i][rin]
        s_sel_val[ch][pos] = v[i];
      }
    }
    __syncthreads();
    // ---- payload ------------------------------------------------------------------------------
    if (active) {
      uint8_t* ip = a.idx_out + d.idx_off + (long long)cl * (k / 2) * 3;
      float* vp = a.val_out + d.val_off + (long long)cl * k;
      if (lt < k / 2) {
        const int i0 = s_sel_idx[ch][2 * lt], i1 = s_sel_idx[ch][2 * lt + 1];
        ip[3 * lt + 0] = (uint8_t)(i0 & 0xff);
        ip[3 * lt + 1] = (uint8_t)(((i0 >> 8) & 0xf) | ((i1 & 0xf) << 4));
        ip[3 * lt + 2] = (uint8_t)((i1 >> 4) & 0xff);
      }
      if (lt >= 64 && lt < 64 + k) vp[lt - 64] = s_sel_val[ch][lt - 64];
    }
    // ---- residual e <- X - F^T S F with S the selected coefficients ------------------------------
    float t32[32];
    if (a.write_residual) {
      for (int i = tid; i < 3 * TC_A_TILE / 16; i += NT) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
      __syncthreads();
      if (lt < k) {
        const int e = s_sel_idx[ch][lt];
        const int n = e >> 6, jx = e & 63;                 // S[n][jx] goes to row jx, column n of the S^T tile
        const int row = ch * 64 + jx;
        const uint32_t addr = (uint32_t)row * 128u + ((((uint32_t)(n >> 3)) ^ (uint32_t)(row & 7)) << 4) + (uint32_t)(n & 7) * 2u;
        __nv_bfloat16 b1, b2, b3;
        split3(s_sel_val[ch][lt], b1, b2, b3);
        *reinterpret_cast<__nv_bfloat16*>(smem + addr) = b1;
        *reinterpret_cast<__nv_bfloat16*>(smem + TC_A_TILE + addr) = b2;
        *reinterpret_cast<__nv_bfloat16*>(smem + 2 * TC_A_TILE + addr) = b3;
      }
      if (!(ok = run_gemm(tZ, /*a_mn=*/false, /*b_mn=*/true))) break;        // Z' = S^T F
      {
        uint32_t r[32];
        tmem_ld32(tZ + hf * 32 + lane_off, r);
#pragma unroll
        for (int e = 0; e < 32; ++e) t32[e] = __uint_as_float(r[e]);
      }
      store_split_row(sA + (uint32_t)ch * 8192u, TC_A_TILE, rin, hf, t32);
      if (!(ok = run_gemm(tY, /*a_mn=*/true, /*b_mn=*/true))) break;         // transmit = Z'^T F
      uint32_t r[32];
      tmem_ld32(tY + hf * 32 + lane_off, r);
      tcgen05_fence_before();
#pragma unroll
      for (int e = 0; e < 32; ++e) t32[e] = __uint_as_float(r[e]);
    } else {
#pragma unroll
      for (int e = 0; e < 32; ++e) t32[e] = 0.f;
    }
    // e <- X - transmit: subtracted in place in the shared copy (own slots), written out in the row-contiguous mapping
#pragma unroll
    for (int q4 = 0; q4 < 8; ++q4) {
      float4 x;
      const uint32_t ad = xaddr + (((uint32_t)q4 ^ xsw) << 4);
      asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(x.x), "=f"(x.y), "=f"(x.z), "=f"(x.w) : "r"(ad) : "memory");
      asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(ad), "f"(x.x - t32[4 * q4]), "f"(x.y - t32[4 * q4 + 1]),
                   "f"(x.z - t32[4 * q4 + 2]), "f"(x.w - t32[4 * q4 + 3]) : "memory");
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int row = i * 16 + urow, c2 = row >> 6;
      const long long gb = s_gbase[c2];
      if (gb < 0) continue;
      float4 x;
      asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(x.x), "=f"(x.y), "=f"(x.z), "=f"(x.w)
                   : "r"(sX + (uint32_t)row * 256u + (uint32_t)(uc4 >> 3) * 128u + ((((uint32_t)uc4 & 7u) ^ (uint32_t)(row & 7)) << 4))
                   : "memory");
      *reinterpret_cast<float4*>(a.ef + gb + (long long)(row & 63) * s_cols[c2] + uc4 * 4) = x;
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 0) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 128;" ::"r"(s_tmem_base) : "memory");
  }
  if (tid == 0 && s_abort && a.status) atomicOr(a.status, TPLR_ST_WAIT_TIMEOUT);
}

}  // namespace

// Same contract as tplr_compress_chunks with use_dct = 1 and one shared basis, for descriptor tables in which
// every chunk is 64 x 64 (element offsets and column counts multiples of 4).
TPLR_API int tplr_compress_chunks_tc(const void* descs, int n_desc, int total_chunks, const float* basis,
                                     float* ef, const float* theta0, const float* theta,
                                     uint8_t* idx_out, float* val_out, unsigned int* status,
                                     float gamma, int delta_mode, int null_round, int write_residual, void* stream) {
  TPLR_ENTER();
  if (total_chunks <= 0) return 0;
  CompressArgs a;
  a.descs = (const TplrParamDesc*)descs; a.basis = basis; a.ef = ef; a.theta0 = theta0; a.theta = theta;
  a.idx_out = idx_out; a.val_out = val_out; a.status = status; a.n_desc = n_desc;
  a.total_chunks = total_chunks; a.gamma = gamma; a.use_dct = 1; a.delta_mode = delta_mode;
  a.null_round = null_round; a.write_residual = write_residual; a.distinct = 0;
  a.variant = g_tc_variant.load(std::memory_order_relaxed);
  cudaError_t err = cudaFuncSetAttribute(compress_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_CMP);
  if (err != cudaSuccess) return (int)err;
  int grid = tplr_sm_count() * 2;
  const int n_pairs = (total_chunks + 1) / 2;
  if (grid > n_pairs) grid = n_pairs;
  compress_tc_kernel<<<grid, NT, TC_SMEM_CMP, (cudaStream_t)stream>>>(a);
  return (int)cudaGetLastError();
}

// Same contract as tplr_aggregate_apply with use_dct = 1 and one shared basis, for descriptor tables in
// which every chunk is 64 x 64 (element offsets and column counts multiples of 4).
TPLR_API int tplr_aggregate_apply_tc(const void* descs, int n_desc, int total_chunks, const float* basis,
                                     int n_peers, const void* const* idx_ptrs, const void* const* val_ptrs,
                                     int val_dtype, const float* qtable, int n_bins, int n_params,
                                     const float* clip, const int* skip, const float* theta0, float* theta,
                                     void* theta_bf16, float* grad_out, float lr, float weight_decay,
                                     int update_mode, unsigned int* status, void* stream) {
  TPLR_ENTER();
  if (total_chunks <= 0) return 0;
  if (n_peers > TPLR_MAX_PEERS || n_peers <= 0) return (int)cudaErrorInvalidValue;
  AggArgs a;
  a.descs = (const TplrParamDesc*)descs; a.basis = basis; a.clip = clip; a.skip = skip; a.qtable = qtable;
  a.theta0 = theta0; a.theta = theta; a.theta_bf16 = (__nv_bfloat16*)theta_bf16; a.grad_out = grad_out;
  a.status = status; a.n_desc = n_desc; a.total_chunks = total_chunks; a.n_peers = n_peers;
  a.n_params = n_params; a.n_bins = n_bins; a.lr = lr; a.weight_decay = weight_decay; a.use_dct = 1;
  a.update_mode = update_mode; a.val_dtype = val_dtype; a.distinct = 0;
  a.variant = g_tc_variant.load(std::memory_order_relaxed);
  for (int i = 0; i < n_peers; ++i) { a.pp.idx[i] = (const uint8_t*)idx_ptrs[i]; a.pp.val[i] = val_ptrs[i]; }
  cudaError_t err = cudaFuncSetAttribute(aggregate_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_AGG);
  if (err != cudaSuccess) return (int)err;
  int grid = tplr_sm_count() * 2;
  const int n_pairs = (total_chunks + 1) / 2;
  if (grid > n_pairs) grid = n_pairs;
  aggregate_tc_kernel<<<grid, NT, TC_SMEM_AGG, (cudaStream_t)stream>>>(a);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------- //
// 8-bit value quantisation of a whole payload (the reference's wire format, src/tplr/compress.py:585-636):
// per tensor  shift = mean(v), scale = range_in_sigmas * std(v - shift) / n_bins (1 when zero or non-finite),
// code = clamp(rint((v - shift) / scale + n_bins/2), 0, n_bins - 1), lookup[b] = mean of (v - shift) over the
// values with code b.  Output: codes (uint8, same offsets as the values) and a table [n_params][n_bins + 2]
// = lookup | shift | scale, whose first n_bins + 1 entries per row are what aggregate_kernel's uint8 decode
// reads.  Three launches: statistics, encode + per-bin sums, finalise.  The per-bin sums are taken in 64-bit
// fixed point (2^-20 of a bin width, exact for the fp32 quotient), so the tables do not depend on the order in
// which the atomics land: the same payload always encodes to the same bytes.
// ------------------------------------------------------------------------------------- //
#define QSPLIT 16
__global__ void __launch_bounds__(256) quant_sum_kernel(const TplrParamDesc* __restrict__ descs, const float* __restrict__ val,
                                                        float* __restrict__ part, int pass, const float* __restrict__ table,
                                                        int n_bins) {
  __shared__ float red[32];
  const TplrParamDesc d = descs[blockIdx.x];
  const long long n = (long long)d.n_chunks * d.k;
  const long long per = (n + QSPLIT - 1) / QSPLIT;
  const long long lo = per * blockIdx.y, hi = min(n, lo + per);
  const float shift = pass ? table[(long long)d.param_id * (n_bins + 2) + n_bins] : 0.f;
  float s = 0.f;
  for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = val[d.val_off + i] - shift;
    s += pass ? v * v : v;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) part[(long long)d.param_id * QSPLIT + blockIdx.y] = s;
}

// pass 0: shift = sum / n ; pass 1: scale from the centred sum of squares.  One thread per tensor.
#define QFIX 1048576.0            // fixed-point unit of the per-bin sums: 2^-20 of a bin width
__global__ void quant_stat_kernel(const TplrParamDesc* __restrict__ descs, int n_desc, const float* __restrict__ part,
                                  float* __restrict__ table, unsigned long long* __restrict__ bins, int pass, int n_bins,
                                  float range_in_sigmas) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_desc) return;
  const TplrParamDesc d = descs[i];
  const long long n = (long long)d.n_chunks * d.k;
  float s = 0.f;
  for (int j = 0; j < QSPLIT; ++j) s += part[(long long)d.param_id * QSPLIT + j];
  float* row = table + (long long)d.param_id * (n_bins + 2);
  if (pass == 0) {
    row[n_bins] = n > 0 ? s / (float)n : 0.f;
    for (int b = 0; b < 2 * n_bins; ++b) bins[(long long)d.param_id * 2 * n_bins + b] = 0ull;
  } else {
    const float stdv = sqrtf(s) / sqrtf((float)max(n - 1, 1LL));
    float scale = range_in_sigmas * stdv / (float)n_bins;
    if (!isfinite(scale) || scale == 0.f) scale = 1.f;
    row[n_bins + 1] = scale;
  }
}

__global__ void __launch_bounds__(256) quant_encode_kernel(const TplrParamDesc* __restrict__ descs, const float* __restrict__ val,
                                                           uint8_t* __restrict__ codes, const float* __restrict__ table,
                                                           unsigned long long* __restrict__ bins, int n_bins) {
  __shared__ unsigned long long s_sum[256];       // two's complement sums of (v - shift) / scale in units of 2^-20
  __shared__ unsigned int s_cnt[256];
  const TplrParamDesc d = descs[blockIdx.x];
  const long long n = (long long)d.n_chunks * d.k;
  const long long per = (n + QSPLIT - 1) / QSPLIT;
  const long long lo = per * blockIdx.y, hi = min(n, lo + per);
  const float* row = table + (long long)d.param_id * (n_bins + 2);
  const float shift = row[n_bins], inv = 1.f / row[n_bins + 1], offset = (float)(n_bins / 2);
  for (int b = threadIdx.x; b < n_bins; b += blockDim.x) { s_sum[b] = 0ull; s_cnt[b] = 0u; }
  __syncthreads();
  for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float c = val[d.val_off + i] - shift;
    const int q = (int)fminf(fmaxf(rintf(c * inv + offset), 0.f), (float)(n_bins - 1));
    codes[d.val_off + i] = (uint8_t)q;
    atomicAdd(&s_sum[q], (unsigned long long)__double2ll_rn((double)(c * inv) * QFIX));
    atomicAdd(&s_cnt[q], 1u);
  }
  __syncthreads();
  unsigned long long* bp = bins + (long long)d.param_id * 2 * n_bins;
  for (int b = threadIdx.x; b < n_bins; b += blockDim.x)
    if (s_cnt[b] > 0u) { atomicAdd(bp + b, s_sum[b]); atomicAdd(bp + n_bins + b, (unsigned long long)s_cnt[b]); }
}

__global__ void quant_lookup_kernel(const TplrParamDesc* __restrict__ descs, const unsigned long long* __restrict__ bins,
                                    float* __restrict__ table, int n_bins) {
  const TplrParamDesc d = descs[blockIdx.x];
  const unsigned long long* bp = bins + (long long)d.param_id * 2 * n_bins;
  float* row = table + (long long)d.param_id * (n_bins + 2);
  const double scale = (double)row[n_bins + 1];
  for (int b = threadIdx.x; b < n_bins; b += blockDim.x) {
    const unsigned long long cnt = bp[n_bins + b];
    row[b] = cnt ? (float)((double)(long long)bp[b] / QFIX / (double)cnt * scale) : 0.f;
  }
}

// descs: one descriptor per tensor (full-model table); val / codes: the payload's value buffer and its uint8 image;
// table: [n_params][n_bins + 2] (lookup | shift | scale); scratch: n_params * (QSPLIT + 4 * n_bins) floats, 8-byte
// aligned (QSPLIT partial sums per tensor, then 2 * n_bins 64-bit words per tensor).  n_bins <= 256.
TPLR_API int tplr_quantize_values(const void* descs, int n_desc, const float* val, uint8_t* codes, float* table,
                                  float* scratch, int n_params, int n_bins, float range_in_sigmas, void* stream) {
  TPLR_ENTER();
  if (n_desc <= 0) return 0;
  if (n_bins <= 0 || n_bins > 256) return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)stream;
  const TplrParamDesc* dd = (const TplrParamDesc*)descs;
  float* part = scratch;
  unsigned long long* bins = reinterpret_cast<unsigned long long*>(scratch + (long long)n_params * QSPLIT);
  if (reinterpret_cast<uintptr_t>(bins) & 7u) return (int)cudaErrorInvalidValue;
  dim3 grid(n_desc, QSPLIT);
  quant_sum_kernel<<<grid, 256, 0, st>>>(dd, val, part, 0, table, n_bins);
  quant_stat_kernel<<<(n_desc + 127) / 128, 128, 0, st>>>(dd, n_desc, part, table, bins, 0, n_bins, range_in_sigmas);
  quant_sum_kernel<<<grid, 256, 0, st>>>(dd, val, part, 1, table, n_bins);
  quant_stat_kernel<<<(n_desc + 127) / 128, 128, 0, st>>>(dd, n_desc, part, table, bins, 1, n_bins, range_in_sigmas);
  quant_encode_kernel<<<grid, 256, 0, st>>>(dd, val, codes, table, bins, n_bins);
  quant_lookup_kernel<<<n_desc, 256, 0, st>>>(dd, bins, table, n_bins);
  return (int)cudaGetLastError();
}

// Decode of a whole payload: out[i] = lookup[code[i]] + shift with the table written by tplr_quantize_values
// (or filled from a received payload's per-tensor parameters).  One launch over all tensors.
__global__ void __launch_bounds__(256) dequant_values_kernel(const TplrParamDesc* __restrict__ descs, const uint8_t* __restrict__ codes,
                                                             const float* __restrict__ table, float* __restrict__ out, int n_bins) {
  __shared__ float s_row[257];
  const TplrParamDesc d = descs[blockIdx.x];
  const long long n = (long long)d.n_chunks * d.k;
  const long long per = ((n + QSPLIT - 1) / QSPLIT + 3) & ~3LL;
  const long long lo = per * blockIdx.y, hi = min(n, lo + per);
  const float* row = table + (long long)d.param_id * (n_bins + 2);
  for (int b = threadIdx.x; b <= n_bins; b += blockDim.x) s_row[b] = row[b];
  __syncthreads();
  const float shift = s_row[n_bins];
  for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x)
    out[d.val_off + i] = s_row[min((int)codes[d.val_off + i], n_bins - 1)] + shift;
}

TPLR_API int tplr_dequantize_values(const void* descs, int n_desc, const uint8_t* codes, const float* table, float* out,
                                    int n_bins, void* stream) {
  TPLR_ENTER();
  if (n_desc <= 0) return 0;
  if (n_bins <= 0 || n_bins > 256) return (int)cudaErrorInvalidValue;
  dim3 grid(n_desc, QSPLIT);
  dequant_values_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const TplrParamDesc*)descs, codes, table, out, n_bins);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------- //
// Error feedback under quantisation.  The reference subtracts from the error feedback what a receiver will
// decode, i.e. the *dequantised* top-k values (src/tplr/neurons.py:157-171), so the quantisation error stays
// in the buffer and is sent later.  compress_kernel has already subtracted the exact values; this kernel
// adds back decode(v - deq(v)) per chunk (a rank-k product against the DCT basis, as in compress_kernel's
// residual) and overwrites the stored values with deq(v), so that the node's own payload is applied with the
// numbers every receiver sees.  idx / val / codes / table may live in a peer's memory (plain loads/stores).
// ------------------------------------------------------------------------------------- //
struct RequantArgs {
  const TplrParamDesc* descs;
  const float* basis;
  float* ef;
  const uint8_t* idx;
  float* val;
  const uint8_t* codes;
  const float* table;
  int n_desc, total_chunks, n_bins, use_dct, distinct;
};

// One chunk per CTA iteration.  The k selected entries are fetched by the first k threads (the next chunk's
// while this one is computed), the tensor's lookup row and the DCT matrices are cached in shared memory, and
// every thread accumulates a 4 x 4 patch of  sum_j diff_j * F_h[b_j][r] * F_w[d_j][l]  straight from the basis.
struct RequantEntry {
  unsigned b0, b1, b2;
  float v;
  int code;
};

static __device__ __forceinline__ RequantEntry requant_fetch(const RequantArgs& a, const TplrParamDesc& d, int cl, int tid) {
  RequantEntry e;
  const uint8_t* ip = a.idx + d.idx_off + ((long long)cl * (d.k / 2) + (tid >> 1)) * 3;
  const long long vi = d.val_off + (long long)cl * d.k + tid;
  e.b0 = ip[0]; e.b1 = ip[1]; e.b2 = ip[2];
  e.v = a.val[vi];
  e.code = a.codes[vi];
  return e;
}

__global__ void __launch_bounds__(NT, 4) requant_residual_kernel(const RequantArgs a) {
  __shared__ __align__(16) float Fh[TPLR_TILE_ELEMS];
  __shared__ __align__(16) float Fw2[TPLR_TILE_ELEMS];
  __shared__ float s_row[258];
  __shared__ int s_b[TPLR_TILE], s_d[TPLR_TILE];
  __shared__ float s_diff[TPLR_TILE];
  const float* Fw = a.distinct ? Fw2 : Fh;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  int cur_fh = -1, cur_fw = -1, cur_param = -1;
  int c = blockIdx.x;
  if (c >= a.total_chunks) return;
  TplrParamDesc d = a.descs[find_desc(a.descs, a.n_desc, c)];
  RequantEntry ent;
  if (tid < d.k) ent = requant_fetch(a, d, c - d.chunk_begin, tid);
  while (c < a.total_chunks) {
    const int h = d.h, w = d.w, k = d.k;
    const int cl = c - d.chunk_begin;
    const int cy = d.chunk_row0 + cl / d.chunks_x, cx = cl % d.chunks_x;
    const long long base = d.elem_off + (long long)cy * h * d.cols + (long long)cx * w;
    __syncthreads();  // previous chunk's shared memory fully consumed
    if (a.use_dct && (d.fh_off != cur_fh || d.fw_off != cur_fw)) {
      for (int i = tid; i < TPLR_TILE_ELEMS; i += NT) {
        const int r = i >> 6, cc = i & 63;
        Fh[i] = (r < h && cc < h) ? __ldg(a.basis + d.fh_off + r * h + cc) : 0.f;
        if (a.distinct) Fw2[i] = (r < w && cc < w) ? __ldg(a.basis + d.fw_off + r * w + cc) : 0.f;
      }
      cur_fh = d.fh_off;
      cur_fw = d.fw_off;
    }
    if (d.param_id != cur_param) {
      const float* row = a.table + (long long)d.param_id * (a.n_bins + 2);
      for (int i = tid; i <= a.n_bins; i += NT) s_row[i] = row[i];
      cur_param = d.param_id;
      __syncthreads();
    }
    if (tid < k) {
      const int e = min((tid & 1) ? (int)(((ent.b1 >> 4) & 0xfu) | (ent.b2 << 4)) : (int)(ent.b0 | ((ent.b1 & 0xfu) << 8)),
                        h * w - 1);
      const float deq = s_row[min(ent.code, a.n_bins - 1)] + s_row[a.n_bins];
      a.val[d.val_off + (long long)cl * k + tid] = deq;
      s_b[tid] = e / w;
      s_d[tid] = e % w;
      s_diff[tid] = ent.v - deq;
    }
    __syncthreads();
    // the next chunk's entries travel while this chunk is computed
    const int cn = c + gridDim.x;
    TplrParamDesc dn = d;
    if (cn < a.total_chunks) {
      if (!(cn >= d.chunk_begin && cn < d.chunk_begin + d.n_chunks)) dn = a.descs[find_desc(a.descs, a.n_desc, cn)];
      if (tid < dn.k) ent = requant_fetch(a, dn, cn - dn.chunk_begin, tid);
    }
    if (!a.use_dct) {
      if (tid < k) a.ef[base + (long long)s_b[tid] * d.cols + s_d[tid]] += s_diff[tid];
    } else {
      const bool vec = (w == 64) && ((d.cols & 3) == 0) && ((base & 3) == 0);
      // this thread's patch of the error feedback is loaded before the product and stored after it
      float4 x[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        x[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        const int r = 4 * ty + i;
        if (vec && r < h) x[i] = *reinterpret_cast<const float4*>(a.ef + base + (long long)r * d.cols + 4 * tx);
      }
      float acc[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
#pragma unroll 4
      for (int j = 0; j < k; ++j) {
        const float df = s_diff[j];
        const float4 fh = *reinterpret_cast<const float4*>(Fh + s_b[j] * LD + 4 * ty);
        const float4 fw = *reinterpret_cast<const float4*>(Fw + s_d[j] * LD + 4 * tx);
        const float av[4] = {fh.x * df, fh.y * df, fh.z * df, fh.w * df};
        const float bv[4] = {fw.x, fw.y, fw.z, fw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) acc[i][jj] = fmaf(av[i], bv[jj], acc[i][jj]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = 4 * ty + i;
        if (r >= h) continue;
        const long long g0 = base + (long long)r * d.cols + 4 * tx;
        if (vec) {
          *reinterpret_cast<float4*>(a.ef + g0) =
              make_float4(x[i].x + acc[i][0], x[i].y + acc[i][1], x[i].z + acc[i][2], x[i].w + acc[i][3]);
        } else {
#pragma unroll
          for (int jj = 0; jj < 4; ++jj)
            if (4 * tx + jj < w) a.ef[g0 + jj] += acc[i][jj];
        }
      }
    }
    c = cn;
    d = dn;
  }
}

// descs: the launch's chunk table (same as for tplr_compress_chunks); ef biased like there; table as written by
// tplr_quantize_values.  Chunks must be disjoint between concurrent launches (they update ef and val in place).
TPLR_API int tplr_requant_residual(const void* descs, int n_desc, int total_chunks, const float* basis, float* ef,
                                   const uint8_t* idx, float* val, const uint8_t* codes, const float* table,
                                   int n_bins, int use_dct, int distinct, void* stream) {
  TPLR_ENTER();
  if (total_chunks <= 0) return 0;
  if (n_bins <= 0 || n_bins > 256) return (int)cudaErrorInvalidValue;
  RequantArgs a;
  a.descs = (const TplrParamDesc*)descs; a.basis = basis; a.ef = ef; a.idx = idx; a.val = val; a.codes = codes;
  a.table = table; a.n_desc = n_desc; a.total_chunks = total_chunks; a.n_bins = n_bins; a.use_dct = use_dct;
  a.distinct = distinct;
  int grid = tplr_sm_count() * 4;
  if (grid > total_chunks) grid = total_chunks;
  requant_residual_kernel<<<grid, NT, 0, (cudaStream_t)stream>>>(a);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------- //
// Index-overlap check: for every pair of peers (i < j), the number of (chunk, index) selections they share,
// summed over all chunks of the payload.  One CTA per chunk (grid-stride): a 4096-bit membership bitmap per
// peer in shared memory, then popcount(AND) per pair.  counts[i * n_peers + j] (i < j) accumulates with 64-bit
// atomics.  Replaces the per-tensor torch scatter / gather of the reference's check
// (neurons/validator.py:3860-3990) with one launch over the packed payloads.
// ------------------------------------------------------------------------------------- //
__global__ void __launch_bounds__(256) index_overlap_kernel(const TplrParamDesc* __restrict__ descs, int n_desc, int total_chunks,
                                                            PeerPtrs pp, int n_peers, unsigned long long* __restrict__ counts) {
  extern __shared__ unsigned int s_bits[];               // [n_peers][128] words, then [n_peers * n_peers] partial counts
  unsigned int* s_cnt = s_bits + n_peers * 128;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < n_peers * n_peers; i += blockDim.x) s_cnt[i] = 0u;
  TplrParamDesc d = descs[0];
  for (int c = blockIdx.x; c < total_chunks; c += gridDim.x) {
    if (!(c >= d.chunk_begin && c < d.chunk_begin + d.n_chunks)) d = descs[find_desc(descs, n_desc, c)];
    const int cl = c - d.chunk_begin, pairs = d.k / 2;
    __syncthreads();
    for (int i = tid; i < n_peers * 128; i += blockDim.x) s_bits[i] = 0u;
    __syncthreads();
    for (int t = tid; t < n_peers * pairs; t += blockDim.x) {
      const int peer = t / pairs, pr = t - peer * pairs;
      const uint8_t* ip = pp.idx[peer] + d.idx_off + ((long long)cl * pairs + pr) * 3;
      const unsigned b0 = ip[0], b1 = ip[1], b2 = ip[2];
      const unsigned i0 = b0 | ((b1 & 0xfu) << 8), i1 = ((b1 >> 4) & 0xfu) | (b2 << 4);
      atomicOr(&s_bits[peer * 128 + (i0 >> 5)], 1u << (i0 & 31));
      atomicOr(&s_bits[peer * 128 + (i1 >> 5)], 1u << (i1 & 31));
    }
    __syncthreads();
    const int n_pairs = n_peers * (n_peers - 1) / 2;
    for (int q = warp; q < n_pairs; q += blockDim.x / 32) {
      int i = 0, rem = q;                               // q-th pair (i < j) in row-major order
      while (rem >= n_peers - 1 - i) { rem -= n_peers - 1 - i; ++i; }
      const int j = i + 1 + rem;
      unsigned int n = 0;
#pragma unroll
      for (int w = 0; w < 4; ++w) n += __popc(s_bits[i * 128 + lane * 4 + w] & s_bits[j * 128 + lane * 4 + w]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) n += __shfl_xor_sync(0xffffffffu, n, o);
      if (lane == 0) s_cnt[i * n_peers + j] += n;       // one warp owns a pair for the whole kernel
    }
  }
  __syncthreads();
  for (int i = tid; i < n_peers * n_peers; i += blockDim.x)
    if (s_cnt[i]) atomicAdd(counts + i, (unsigned long long)s_cnt[i]);
}

// counts: [n_peers * n_peers] uint64, zeroed by the caller.
TPLR_API int tplr_index_overlap(const void* descs, int n_desc, int total_chunks, int n_peers,
                                const void* const* idx_ptrs, unsigned long long* counts, void* stream) {
  TPLR_ENTER();
  if (total_chunks <= 0 || n_peers < 2) return 0;
  if (n_peers > TPLR_MAX_PEERS) return (int)cudaErrorInvalidValue;
  PeerPtrs pp;
  for (int i = 0; i < n_peers; ++i) { pp.idx[i] = (const uint8_t*)idx_ptrs[i]; pp.val[i] = nullptr; }
  const int smem = (n_peers * 128 + n_peers * n_peers) * (int)sizeof(unsigned int);
  int grid = tplr_sm_count() * 4;
  if (grid > total_chunks) grid = total_chunks;
  index_overlap_kernel<<<grid, 256, smem, (cudaStream_t)stream>>>((const TplrParamDesc*)descs, n_desc, total_chunks, pp,
                                                                 n_peers, counts);
  return (int)cudaGetLastError();
}

TPLR_API int tplr_param_desc_size() { return (int)sizeof(TplrParamDesc); }

// Selects the variants of the tensor-core compress / aggregate kernels (see g_tc_variant); returns the old value.
TPLR_API int tplr_compress_set_variant(int v) {
  return g_tc_variant.exchange(v & 7, std::memory_order_relaxed);
}
