// Bandwidth-bound model and optimizer kernels (sm_100a): RMSNorm, RoPE, SwiGLU,
// fused cross-entropy loss + logit gradient, embedding gather / scatter-add, fused AdamW
// with global-norm clipping and a bf16 shadow write, and deterministic sum-of-squares.
//
// All activations are bf16 with fp32 math; gradients of parameters are accumulated into
// an fp32 flat buffer (the reference reduces and accumulates gradients in fp32:
// src/tplr/model_factory.py:153,183).  Reference ops these replace: RMSNorm / RoPE / SwiGLU /
// CE of the torchtitan LLaMA (models/llama3/model/model.py:69-95, :236-237, :276-277;
// components/loss.py:18-22) and torch.optim.AdamW(fused=True) + clip_grad_norm_
// (neurons/trainer.py:280-298, :940).
#include "common.cuh"
#include "no_alloc.h"
#include <atomic>

typedef __nv_bfloat16 bf16;

struct alignas(16) bf16x8 { __nv_bfloat162 v[4]; };

static __device__ __forceinline__ void unpack8(const bf16x8& p, float* f) {
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(p.v[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
static __device__ __forceinline__ bf16x8 pack8(const float* f) {
  bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}

// ------------------------------------------------------------------------------------- //
// RMSNorm: one CTA per row, 8 bf16 per thread per trip, row cached in registers (D <= 8192)
// ------------------------------------------------------------------------------------- //
#define RMS_MAXV 4
__global__ void __launch_bounds__(256) rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                          bf16* __restrict__ y, float* __restrict__ rstd,
                                                          int D, float eps) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * D);
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  bf16x8* yr = reinterpret_cast<bf16x8*>(y + row * D);
  const int nv = D / 8;
  float xv[RMS_MAXV][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < RMS_MAXV; ++j) {
    const int i = threadIdx.x + j * 256;
    if (i < nv) {
      unpack8(xr[i], xv[j]);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss = fmaf(xv[j][e], xv[j][e], ss);
    }
  }
  for (int i = threadIdx.x + RMS_MAXV * 256; i < nv; i += 256) {
    float t[8]; unpack8(xr[i], t);
#pragma unroll
    for (int e = 0; e < 8; ++e) ss = fmaf(t[e], t[e], ss);
  }
  ss = block_sum(ss, red);
  const float r = rsqrtf(ss / (float)D + eps);
  if (threadIdx.x == 0 && rstd) rstd[row] = r;
#pragma unroll
  for (int j = 0; j < RMS_MAXV; ++j) {
    const int i = threadIdx.x + j * 256;
    if (i < nv) {
      float wv[8], o[8]; unpack8(wr[i], wv);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = xv[j][e] * r * wv[e];
      yr[i] = pack8(o);
    }
  }
  for (int i = threadIdx.x + RMS_MAXV * 256; i < nv; i += 256) {
    float t[8], wv[8], o[8]; unpack8(xr[i], t); unpack8(wr[i], wv);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = t[e] * r * wv[e];
    yr[i] = pack8(o);
  }
}

TPLR_API int tplr_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long T, int D,
                              float eps, void* stream) {
  TPLR_ENTER();
  if (D % 8) return (int)cudaErrorInvalidValue;
  if (T <= 0) return 0;
  rmsnorm_fwd_kernel<<<(unsigned)T, 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (const bf16*)w, (bf16*)y, rstd, D, eps);
  return (int)cudaGetLastError();
}

// dx = rstd * (g - xhat * mean(g * xhat)),  g = dy * w, xhat = x * rstd;  dw += sum_rows dy * xhat.
// Persistent CTAs walk rows with stride gridDim.x; each thread owns fixed columns so the dw
// partial stays in registers and is flushed once with fp32 atomics. D <= 8192.
__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                                          const bf16* __restrict__ w, const float* __restrict__ rstd,
                                                          bf16* __restrict__ dx, float* __restrict__ dw,
                                                          long long T, int D) {
  __shared__ float red[32];
  const int nv = D / 8;
  float wv[RMS_MAXV][8], dwv[RMS_MAXV][8];
#pragma unroll
  for (int j = 0; j < RMS_MAXV; ++j) {
    const int i = threadIdx.x + j * 256;
#pragma unroll
    for (int e = 0; e < 8; ++e) { dwv[j][e] = 0.f; wv[j][e] = 0.f; }
    if (i < nv) unpack8(reinterpret_cast<const bf16x8*>(w)[i], wv[j]);
  }
  for (long long row = blockIdx.x; row < T; row += gridDim.x) {
    const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * D);
    const bf16x8* gr = reinterpret_cast<const bf16x8*>(dy + row * D);
    bf16x8* dr = reinterpret_cast<bf16x8*>(dx + row * D);
    const float r = rstd[row];
    float xh[RMS_MAXV][8], g[RMS_MAXV][8];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < RMS_MAXV; ++j) {
      const int i = threadIdx.x + j * 256;
      if (i < nv) {
        float xv[8], dv[8]; unpack8(xr[i], xv); unpack8(gr[i], dv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          xh[j][e] = xv[e] * r;
          g[j][e] = dv[e] * wv[j][e];
          dwv[j][e] = fmaf(dv[e], xh[j][e], dwv[j][e]);
          dot = fmaf(g[j][e], xh[j][e], dot);
        }
      }
    }
    dot = block_sum(dot, red) / (float)D;
#pragma unroll
    for (int j = 0; j < RMS_MAXV; ++j) {
      const int i = threadIdx.x + j * 256;
      if (i < nv) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = r * (g[j][e] - xh[j][e] * dot);
        dr[i] = pack8(o);
      }
    }
  }
  if (dw) {
#pragma unroll
    for (int j = 0; j < RMS_MAXV; ++j) {
      const int i = threadIdx.x + j * 256;
      if (i < nv)
#pragma unroll
        for (int e = 0; e < 8; ++e) atomicAdd(dw + i * 8 + e, dwv[j][e]);
    }
  }
}

TPLR_API int tplr_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                              float* dw, long long T, int D, void* stream) {
  TPLR_ENTER();
  if (D % 8 || D > RMS_MAXV * 256 * 8) return (int)cudaErrorInvalidValue;
  if (T <= 0) return 0;
  long long grid = tplr_sm_count() * 4;
  if (grid > T) grid = T;
  rmsnorm_bwd_kernel<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w,
                                                                      rstd, (bf16*)dx, dw, T, D);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------- //
// Residual add fused with RMSNorm, one warp per row (D <= 2048): no block barrier, 8 rows in
// flight per CTA.
//   forward   h = res + delta (delta may be null: h = res);  y = h * rstd(h) * w;  h written when delta != null
//   backward  dx = dres + rstd * (g - xhat * mean(g * xhat))  (dres may be null);  dw += sum_rows dy * xhat
// The backward's dx is the gradient of both `res` and `delta`, so the residual stream needs no
// separate add kernel in either direction (the reference leaves `h + attn(norm(h))` to eager adds:
// torchtitan models/llama3/model/model.py:339-341).
// ------------------------------------------------------------------------------------- //
template <int VPL>
__global__ void __launch_bounds__(256) add_rmsnorm_fwd_warp_kernel(const bf16* __restrict__ res, const bf16* __restrict__ delta,
                                                                   const bf16* __restrict__ w, bf16* __restrict__ h_out,
                                                                   bf16* __restrict__ y, float* __restrict__ rstd,
                                                                   long long T, int D, float eps) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= T) return;
  const int nv = D / 8;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(res + row * D);
  const bf16x8* dr = delta ? reinterpret_cast<const bf16x8*>(delta + row * D) : nullptr;
  bf16x8 hv[VPL];
  float ss = 0.f;
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
    const int i = lane + 32 * v;
    if (i < nv) {
      float a[8]; unpack8(xr[i], a);
      if (dr) {
        float b[8]; unpack8(dr[i], b);
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] += b[e];
        hv[v] = pack8(a);                 // the norm sees the bf16-rounded sum, as the stored residual does
        unpack8(hv[v], a);
        reinterpret_cast<bf16x8*>(h_out + row * D)[i] = hv[v];
      } else {
        hv[v] = xr[i];
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) ss = fmaf(a[e], a[e], ss);
    }
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / (float)D + eps);
  if (lane == 0 && rstd) rstd[row] = r;
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
    const int i = lane + 32 * v;
    if (i < nv) {
      float a[8], wv[8], o[8];
      unpack8(hv[v], a); unpack8(reinterpret_cast<const bf16x8*>(w)[i], wv);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = a[e] * r * wv[e];
      reinterpret_cast<bf16x8*>(y + row * D)[i] = pack8(o);
    }
  }
}

template <int VPL>
__global__ void __launch_bounds__(256) add_rmsnorm_bwd_warp_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                                                   const bf16* __restrict__ w, const float* __restrict__ rstd,
                                                                   const bf16* __restrict__ dres, bf16* __restrict__ dx,
                                                                   float* __restrict__ dw, long long T, int D) {
  __shared__ float s_dw[8][32 * 8 + 1];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int nv = D / 8;
  float dwv[VPL][8];
  bf16x8 wp[VPL];
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
    const int i = lane + 32 * v;
#pragma unroll
    for (int e = 0; e < 8; ++e) dwv[v][e] = 0.f;
    if (i < nv) wp[v] = reinterpret_cast<const bf16x8*>(w)[i];
  }
  for (long long row = (long long)blockIdx.x * 8 + wid; row < T; row += (long long)gridDim.x * 8) {
    const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * D);
    const bf16x8* gr = reinterpret_cast<const bf16x8*>(dy + row * D);
    const float r = rstd[row];
    bf16x8 xp[VPL], gp[VPL];
    float dot = 0.f;
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      const int i = lane + 32 * v;
      if (i < nv) { xp[v] = xr[i]; gp[v] = gr[i]; }
    }
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      const int i = lane + 32 * v;
      if (i < nv) {
        float xv[8], dv[8], wv[8];
        unpack8(xp[v], xv); unpack8(gp[v], dv); unpack8(wp[v], wv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xh = xv[e] * r;
          dwv[v][e] = fmaf(dv[e], xh, dwv[v][e]);
          dot = fmaf(dv[e] * wv[e], xh, dot);
        }
      }
    }
    dot = warp_sum(dot) / (float)D;
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      const int i = lane + 32 * v;
      if (i < nv) {
        float xv[8], dv[8], wv[8], o[8];
        unpack8(xp[v], xv); unpack8(gp[v], dv); unpack8(wp[v], wv);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = r * (dv[e] * wv[e] - xv[e] * r * dot);
        if (dres) {
          float a[8]; unpack8(reinterpret_cast<const bf16x8*>(dres + row * D)[i], a);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] += a[e];
        }
        reinterpret_cast<bf16x8*>(dx + row * D)[i] = pack8(o);
      }
    }
  }
  if (!dw) return;
  // reduce the eight warps' partial dw through shared memory, one slab of 32 vectors at a time
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
    __syncthreads();
#pragma unroll
    for (int e = 0; e < 8; ++e) s_dw[wid][lane * 8 + e] = dwv[v][e];
    __syncthreads();
    const int col = threadIdx.x;                     // 256 columns of this slab
    const int i = (col >> 3) + 32 * v;
    if (i < nv) {
      float acc = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) acc += s_dw[k][col];
      atomicAdd(dw + (long long)i * 8 + (col & 7), acc);
    }
  }
}

// T rows of D (multiple of 8, <= 2048) bf16.  delta may be null (plain RMSNorm, h_out unused).
TPLR_API int tplr_add_rmsnorm_fwd(const void* res, const void* delta, const void* w, void* h_out, void* y, float* rstd,
                                  long long T, int D, float eps, void* stream) {
  TPLR_ENTER();
  if (D % 8 || D > 2048) return (int)cudaErrorInvalidValue;
  if (T <= 0) return 0;
  const int vpl = (D / 8 + 31) / 32;
  const unsigned grid = (unsigned)((T + 7) / 8);
  cudaStream_t st = (cudaStream_t)stream;
#define TPLR_ARN_FWD(V) add_rmsnorm_fwd_warp_kernel<V><<<grid, 256, 0, st>>>((const bf16*)res, (const bf16*)delta, \
      (const bf16*)w, (bf16*)h_out, (bf16*)y, rstd, T, D, eps)
  if (vpl <= 1) TPLR_ARN_FWD(1); else if (vpl <= 2) TPLR_ARN_FWD(2); else if (vpl <= 4) TPLR_ARN_FWD(4); else TPLR_ARN_FWD(8);
#undef TPLR_ARN_FWD
  return (int)cudaGetLastError();
}

// dres may be null; dw (fp32, D) is accumulated into with atomics and may be null.
TPLR_API int tplr_add_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                                  void* dx, float* dw, long long T, int D, void* stream) {
  TPLR_ENTER();
  if (D % 8 || D > 2048) return (int)cudaErrorInvalidValue;
  if (T <= 0) return 0;
  const int vpl = (D / 8 + 31) / 32;
  long long grid = (long long)tplr_sm_count() * (vpl > 4 ? 1 : 2);   // resident CTAs: 240 registers at 8 vectors per lane
  if (grid > (T + 7) / 8) grid = (T + 7) / 8;
  cudaStream_t st = (cudaStream_t)stream;
#define TPLR_ARN_BWD(V) add_rmsnorm_bwd_warp_kernel<V><<<(unsigned)grid, 256, 0, st>>>((const bf16*)dy, (const bf16*)x, \
      (const bf16*)w, rstd, (const bf16*)dres, (bf16*)dx, dw, T, D)
  if (vpl <= 1) TPLR_ARN_BWD(1); else if (vpl <= 2) TPLR_ARN_BWD(2); else if (vpl <= 4) TPLR_ARN_BWD(4); else TPLR_ARN_BWD(8);
#undef TPLR_ARN_BWD
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------- //
// RoPE on interleaved pairs, in place on a packed [tokens, row_stride] buffer whose first
// n_heads*Dh columns are rotary heads (q heads followed by k heads). inverse = backward.
// ------------------------------------------------------------------------------------- //
__global__ void __launch_bounds__(256) rope_kernel(bf16* __restrict__ buf, const float* __restrict__ cosb,
                                                   const float* __restrict__ sinb, long long tokens, int S,
                                                   int n_heads, int Dh, long long row_stride, int inverse) {
  const int vec_per_head = Dh / 8;
  const long long per_tok = (long long)n_heads * vec_per_head;
  const long long total = tokens * per_tok;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long tok = i / per_tok;
    const int rem = (int)(i - tok * per_tok);
    const int head = rem / vec_per_head, v = rem - head * vec_per_head;
    const int pos = (int)(tok % S);
    bf16x8* p = reinterpret_cast<bf16x8*>(buf + tok * row_stride + (long long)head * Dh + v * 8);
    float f[8], o[8];
    unpack8(*p, f);
    const float4 c = *reinterpret_cast<const float4*>(cosb + (long long)pos * (Dh / 2) + v * 4);
    float4 s = *reinterpret_cast<const float4*>(sinb + (long long)pos * (Dh / 2) + v * 4);
    if (inverse) { s.x = -s.x; s.y = -s.y; s.z = -s.z; s.w = -s.w; }
    const float cv[4] = {c.x, c.y, c.z, c.w}, sv[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      o[2 * e] = f[2 * e] * cv[e] - f[2 * e + 1] * sv[e];
      o[2 * e + 1] = f[2 * e] * sv[e] + f[2 * e + 1] * cv[e];
    }
    *p = pack8(o);
  }
}

TPLR_API int tplr_rope(void* buf, const float* cosb, const float* sinb, long long tokens, int S, int n_heads,
                       int Dh, long long row_stride, int inverse, void* stream) {
  TPLR_ENTER();
  if (Dh % 8 || row_stride % 8) return (int)cudaErrorInvalidValue;
  const long long total = tokens * n_heads * (Dh / 8);
  if (total <= 0) return 0;
  long long grid = (total + 255) / 256;
  const long long cap = (long long)tplr_sm_count() * 16;
  if (grid > cap) grid = cap;
  rope_kernel<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>((bf16*)buf, cosb, sinb, tokens, S, n_heads, Dh, row_stride, inverse);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------- //
// SwiGLU on a packed [T, 2F] projection (gate = first F columns, up = last F columns)
// ------------------------------------------------------------------------------------- //
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const bf16* __restrict__ h, bf16* __restrict__ y,
                                                         long long T, int F) {
  const int fv = F / 8;
  const long long total = T * fv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / fv;
    const int c = (int)(i - t * fv);
    float a[8], b[8], o[8];
    unpack8(reinterpret_cast<const bf16x8*>(h + t * 2 * F)[c], a);
    unpack8(reinterpret_cast<const bf16x8*>(h + t * 2 * F + F)[c], b);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = a[e] / (1.f + __expf(-a[e])) * b[e];
    reinterpret_cast<bf16x8*>(y + t * F)[c] = pack8(o);
  }
}

__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const bf16* __restrict__ h, const bf16* __restrict__ dy,
                                                         bf16* __restrict__ dh, long long T, int F) {
  const int fv = F / 8;
  const long long total = T * fv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / fv;
    const int c = (int)(i - t * fv);
    float a[8], b[8], g[8], da[8], db[8];
    unpack8(reinterpret_cast<const bf16x8*>(h + t * 2 * F)[c], a);
    unpack8(reinterpret_cast<const bf16x8*>(h + t * 2 * F + F)[c], b);
    unpack8(reinterpret_cast<const bf16x8*>(dy + t * F)[c], g);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float sg = 1.f / (1.f + __expf(-a[e]));
      const float silu = a[e] * sg;
      db[e] = g[e] * silu;
      da[e] = g[e] * b[e] * (sg + silu * (1.f - sg));
    }
    reinterpret_cast<bf16x8*>(dh + t * 2 * F)[c] = pack8(da);
    reinterpret_cast<bf16x8*>(dh + t * 2 * F + F)[c] = pack8(db);
  }
}

static inline unsigned ew_grid(long long total) {
  long long grid = (total + 255) / 256;
  const long long cap = (long long)tplr_sm_count() * 16;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  return (unsigned)grid;
}

TPLR_API int tplr_swiglu_fwd(const void* h, void* y, long long T, int F, void* stream) {
  TPLR_ENTER();
  if (F % 8) return (int)cudaErrorInvalidValue;
  if (T <= 0) return 0;
  swiglu_fwd_kernel<<<ew_grid(T * (F / 8)), 256, 0, (cudaStream_t)stream>>>((const bf16*)h, (bf16*)y, T, F);
  return (int)cudaGetLastError();
}
TPLR_API int tplr_swiglu_bwd(const void* h, const void* dy, void* dh, long long T, int F, void* stream) {
  TPLR_ENTER();
  if (F % 8) return (int)cudaErrorInvalidValue;
  if (T <= 0) return 0;
  swiglu_bwd_kernel<<<ew_grid(T * (F / 8)), 256, 0, (cudaStream_t)stream>>>((const bf16*)h, (const bf16*)dy, (bf16*)dh, T, F);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------- //
// Cross entropy: per-row loss and (optionally) the logit gradient written in place.
//   loss_row = logsumexp(z) - z[label];  dz = (softmax(z) - onehot) * grad_scale / n_valid
// Rows whose label == ignore_index give loss 0 and gradient 0.  So do rows whose label lies outside
// [0, V) (a shard tokenised with a larger vocabulary, a corrupt label): they are never used as an index,
// they do not count as valid rows, and TPLR_ST_BAD_INDEX is OR-ed into `status` when one is given.
// ------------------------------------------------------------------------------------- //
__global__ void count_valid_kernel(const long long* __restrict__ labels, long long T, long long ignore_index,
                                   long long V, int* __restrict__ out, unsigned int* __restrict__ status) {
  __shared__ float red[32];
  float c = 0.f, bad = 0.f;
  for (long long i = threadIdx.x; i < T; i += blockDim.x) {
    const long long l = labels[i];
    if (l == ignore_index) continue;
    if (l < 0 || l >= V) bad += 1.f;
    else c += 1.f;
  }
  c = block_sum(c, red);
  bad = block_sum(bad, red);
  if (threadIdx.x == 0) {
    out[0] = (int)(c + 0.5f);
    if (bad > 0.f && status) atomicOr(status, TPLR_ST_BAD_INDEX);
  }
}

__global__ void __launch_bounds__(512) ce_kernel(bf16* __restrict__ logits, const long long* __restrict__ labels,
                                                 float* __restrict__ losses, const int* __restrict__ n_valid,
                                                 float grad_scale, int V, long long ld, long long ignore_index,
                                                 int write_grad) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  bf16* z = logits + row * ld;
  const long long label = labels[row];
  const int nv = V / 8;
  if (label == ignore_index || label < 0 || label >= V) {
    if (threadIdx.x == 0) losses[row] = 0.f;
    if (write_grad) {
      bf16x8 zero;
#pragma unroll
      for (int i = 0; i < 4; ++i) zero.v[i] = __floats2bfloat162_rn(0.f, 0.f);
      for (int i = threadIdx.x; i < nv; i += blockDim.x) reinterpret_cast<bf16x8*>(z)[i] = zero;
      for (int i = nv * 8 + threadIdx.x; i < V; i += blockDim.x) z[i] = __float2bfloat16(0.f);
    }
    return;
  }
  float m = -INFINITY;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float f[8]; unpack8(reinterpret_cast<const bf16x8*>(z)[i], f);
#pragma unroll
    for (int e = 0; e < 8; ++e) m = fmaxf(m, f[e]);
  }
  for (int i = nv * 8 + threadIdx.x; i < V; i += blockDim.x) m = fmaxf(m, __bfloat162float(z[i]));
  m = block_max(m, red);
  float s = 0.f;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float f[8]; unpack8(reinterpret_cast<const bf16x8*>(z)[i], f);
#pragma unroll
    for (int e = 0; e < 8; ++e) s += __expf(f[e] - m);
  }
  for (int i = nv * 8 + threadIdx.x; i < V; i += blockDim.x) s += __expf(__bfloat162float(z[i]) - m);
  s = block_sum(s, red);
  const float lse = m + logf(s);
  const float zl = __bfloat162float(z[label]);
  __syncthreads();
  if (threadIdx.x == 0) losses[row] = lse - zl;
  if (!write_grad) return;
  const float sc = grad_scale / (float)max(n_valid[0], 1);
  const float inv = sc / s;
  const int lv = (int)(label / 8), le = (int)(label % 8);
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float f[8], o[8]; unpack8(reinterpret_cast<const bf16x8*>(z)[i], f);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = __expf(f[e] - m) * inv;
    if (i == lv) o[le] -= sc;
    reinterpret_cast<bf16x8*>(z)[i] = pack8(o);
  }
  for (int i = nv * 8 + threadIdx.x; i < V; i += blockDim.x) {
    float o = __expf(__bfloat162float(z[i]) - m) * inv;
    if (i == label) o -= sc;
    z[i] = __float2bfloat16(o);
  }
}

// Deterministic tree sum of `n` floats into out[0], scaled: out = scale * sum / max(*den, 1) when den != null.
__global__ void __launch_bounds__(1024) sum_rows_kernel(const float* __restrict__ x, long long n,
                                                        const int* __restrict__ den, float scale,
                                                        float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) s += x[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) out[0] = den ? scale * s / (float)max(den[0], 1) : scale * s;
}

TPLR_API int tplr_cross_entropy(void* logits, const long long* labels, float* losses, int* n_valid,
                                float* loss_out, float grad_scale, long long T, int V, long long ld,
                                long long ignore_index, int write_grad, unsigned int* status, void* stream) {
  TPLR_ENTER();
  if (T <= 0) return 0;
  // ce_kernel reads and writes rows as 16-byte vectors: the stride and the base must allow it, and a
  // row must not overlap the next one
  if ((ld % 8) || ld < V || V <= 0 || ((uintptr_t)logits & 15)) return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)stream;
  count_valid_kernel<<<1, 1024, 0, st>>>(labels, T, ignore_index, V, n_valid, status);
  ce_kernel<<<(unsigned)T, 512, 0, st>>>((bf16*)logits, labels, losses, n_valid, grad_scale, V, ld, ignore_index, write_grad);
  sum_rows_kernel<<<1, 1024, 0, st>>>(losses, T, n_valid, 1.f, loss_out);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------- //
// Embedding gather (bf16 rows) and its gradient scatter-add into the fp32 gradient table
// ------------------------------------------------------------------------------------- //
__global__ void __launch_bounds__(256) embedding_fwd_kernel(const long long* __restrict__ tok, const bf16* __restrict__ table,
                                                            bf16* __restrict__ out, long long T, int D, int V) {
  const int dv = D / 8;
  const long long total = T * dv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / dv;
    const int c = (int)(i - t * dv);
    long long id = tok[t];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);
    reinterpret_cast<bf16x8*>(out + t * D)[c] = reinterpret_cast<const bf16x8*>(table + id * D)[c];
  }
}
__global__ void __launch_bounds__(256) embedding_bwd_kernel(const long long* __restrict__ tok, const bf16* __restrict__ dy,
                                                            float* __restrict__ dtable, long long T, int D, int V) {
  const int dv = D / 8;
  const long long total = T * dv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / dv;
    const int c = (int)(i - t * dv);
    long long id = tok[t];
    if (id < 0 || id >= V) continue;
    float f[8]; unpack8(reinterpret_cast<const bf16x8*>(dy + t * D)[c], f);
    float* dst = dtable + id * D + c * 8;
#pragma unroll
    for (int e = 0; e < 8; ++e) atomicAdd(dst + e, f[e]);
  }
}
TPLR_API int tplr_embedding_fwd(const long long* tok, const void* table, void* out, long long T, int D, int V, void* stream) {
  TPLR_ENTER();
  if (D % 8) return (int)cudaErrorInvalidValue;
  if (T <= 0) return 0;
  embedding_fwd_kernel<<<ew_grid(T * (D / 8)), 256, 0, (cudaStream_t)stream>>>(tok, (const bf16*)table, (bf16*)out, T, D, V);
  return (int)cudaGetLastError();
}
TPLR_API int tplr_embedding_bwd(const long long* tok, const void* dy, float* dtable, long long T, int D, int V, void* stream) {
  TPLR_ENTER();
  if (D % 8) return (int)cudaErrorInvalidValue;
  if (T <= 0) return 0;
  embedding_bwd_kernel<<<ew_grid(T * (D / 8)), 256, 0, (cudaStream_t)stream>>>(tok, (const bf16*)dy, dtable, T, D, V);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------- //
// sum of squares (deterministic two-stage) and fused AdamW
// ------------------------------------------------------------------------------------- //
__global__ void __launch_bounds__(512) sumsq_partial_kernel(const float* __restrict__ x, long long n,
                                                            float* __restrict__ partial) {
  __shared__ float red[32];
  float s = 0.f;
  const long long n4 = n / 4;
  const float4* x4 = reinterpret_cast<const float4*>(x);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    const float4 v = x4[i];
    s = fmaf(v.x, v.x, s); s = fmaf(v.y, v.y, s); s = fmaf(v.z, v.z, s); s = fmaf(v.w, v.w, s);
  }
  if (blockIdx.x == 0)
    for (long long i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x) s = fmaf(x[i], x[i], s);
  s = block_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

// partial must hold tplr_sumsq_blocks() floats; out[0] = sum(x^2). x must be 16-byte aligned.
TPLR_API int tplr_sumsq_blocks() { return tplr_sm_count() * 4; }
TPLR_API int tplr_sumsq(const float* x, long long n, float* partial, float* out, void* stream) {
  TPLR_ENTER();
  cudaStream_t st = (cudaStream_t)stream;
  const int blocks = tplr_sumsq_blocks();
  sumsq_partial_kernel<<<blocks, 512, 0, st>>>(x, n, partial);
  sum_rows_kernel<<<1, 1024, 0, st>>>(partial, blocks, nullptr, 1.f, out);
  return (int)cudaGetLastError();
}

// p, m, v, g fp32 (16-byte aligned, n elements). The gradient is first multiplied by
// grad_scale and by the clip coefficient min(1, max_norm / (grad_scale*sqrt(*gnorm_sq) + 1e-6))
// when gnorm_sq != null. Decoupled weight decay. Writes p and (optionally) its bf16 copy,
// which may live in a peer GPU's memory (plain stores over NVLink).
struct AdamArgs {
  float* p; float* m; float* v; const float* g;
  bf16* shadow[TPLR_MAX_PEERS];
  int n_shadow;
  long long n;
  float lr, b1, b2, eps, wd, bc1, bc2, grad_scale, max_norm;
  const float* gnorm_sq;
  int zero_grad;
  float* g_mut;
};

__global__ void __launch_bounds__(256) adamw_kernel(const AdamArgs a) {
  float coef = a.grad_scale;
  if (a.gnorm_sq && a.max_norm > 0.f) {
    const float nrm = a.grad_scale * sqrtf(a.gnorm_sq[0]);
    coef *= fminf(1.f, a.max_norm / (nrm + 1e-6f));
  }
  const long long n4 = a.n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    float4 p = reinterpret_cast<float4*>(a.p)[i];
    float4 m = reinterpret_cast<float4*>(a.m)[i];
    float4 v = reinterpret_cast<float4*>(a.v)[i];
    const float4 g4 = reinterpret_cast<const float4*>(a.g)[i];
    float pv[4] = {p.x, p.y, p.z, p.w}, mv[4] = {m.x, m.y, m.z, m.w}, vv[4] = {v.x, v.y, v.z, v.w};
    const float gv[4] = {g4.x * coef, g4.y * coef, g4.z * coef, g4.w * coef};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      mv[e] = a.b1 * mv[e] + (1.f - a.b1) * gv[e];
      vv[e] = a.b2 * vv[e] + (1.f - a.b2) * gv[e] * gv[e];
      const float mh = mv[e] / a.bc1;
      const float vh = vv[e] / a.bc2;
      pv[e] = pv[e] * (1.f - a.lr * a.wd) - a.lr * mh / (sqrtf(vh) + a.eps);
    }
    reinterpret_cast<float4*>(a.p)[i] = make_float4(pv[0], pv[1], pv[2], pv[3]);
    reinterpret_cast<float4*>(a.m)[i] = make_float4(mv[0], mv[1], mv[2], mv[3]);
    reinterpret_cast<float4*>(a.v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (a.zero_grad) reinterpret_cast<float4*>(a.g_mut)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (a.n_shadow) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(pv[0], pv[1]), hi = __floats2bfloat162_rn(pv[2], pv[3]);
      uint2 pk;
      pk.x = *reinterpret_cast<unsigned int*>(&lo);
      pk.y = *reinterpret_cast<unsigned int*>(&hi);
      for (int s = 0; s < a.n_shadow; ++s) reinterpret_cast<uint2*>(a.shadow[s])[i] = pk;
    }
  }
}

TPLR_API int tplr_adamw(float* p, float* m, float* v, float* g, void* const* shadows, int n_shadow,
                        long long n, float lr, float b1, float b2, float eps, float wd, int step,
                        float grad_scale, float max_norm, const float* gnorm_sq, int zero_grad,
                        void* stream) {
  TPLR_ENTER();
  if (n % 4 || n_shadow > TPLR_MAX_PEERS) return (int)cudaErrorInvalidValue;
  if (n <= 0) return 0;
  AdamArgs a;
  a.p = p; a.m = m; a.v = v; a.g = g; a.g_mut = g; a.n = n; a.n_shadow = n_shadow;
  for (int i = 0; i < n_shadow; ++i) a.shadow[i] = (bf16*)shadows[i];
  a.lr = lr; a.b1 = b1; a.b2 = b2; a.eps = eps; a.wd = wd;
  a.bc1 = 1.f - powf(b1, (float)step); a.bc2 = 1.f - powf(b2, (float)step);
  a.grad_scale = grad_scale; a.max_norm = max_norm; a.gnorm_sq = gnorm_sq; a.zero_grad = zero_grad;
  adamw_kernel<<<ew_grid(n / 4), 256, 0, (cudaStream_t)stream>>>(a);
  return (int)cudaGetLastError();
}

// dst_bf16[i] = bf16(src[i])  (n % 4 == 0, 16-byte aligned src, 8-byte aligned dst)
__global__ void __launch_bounds__(256) cast_bf16_kernel(const float* __restrict__ src, bf16* __restrict__ dst, long long n4) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(src)[i];
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 pk;
    pk.x = *reinterpret_cast<unsigned int*>(&lo);
    pk.y = *reinterpret_cast<unsigned int*>(&hi);
    reinterpret_cast<uint2*>(dst)[i] = pk;
  }
}
TPLR_API int tplr_cast_bf16(const float* src, void* dst, long long n, void* stream) {
  TPLR_ENTER();
  if (n % 4) return (int)cudaErrorInvalidValue;
  if (n <= 0) return 0;
  cast_bf16_kernel<<<ew_grid(n / 4), 256, 0, (cudaStream_t)stream>>>(src, (bf16*)dst, n / 4);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------- //
// Mirror of a symmetric product computed as one triangle, fused with the Newton-Schulz combination:
//   out[i][j] = alpha * U[i][j] (+ beta * aux[i][j]) (+ diag when i == j)   where U[i][j] is read at (i, j) when the 256 x 256 tile of
//   (i, j) lies on or above the diagonal and at (j, i) otherwise (tplr_gemm2_syrk leaves the lower tiles unwritten).
// 32 x 32 tiles; a lower tile is the transpose of its mirror tile, staged through shared memory.
// ------------------------------------------------------------------------------------- //
__global__ void __launch_bounds__(256) sym_axpby_kernel(const bf16* __restrict__ U, long long ldu, int M, float alpha,
                                                        const bf16* __restrict__ aux, long long ldaux, float beta,
                                                        float diag, bf16* __restrict__ out, long long ldo) {
  __shared__ float tile[32][33];
  const int ti = blockIdx.y, tj = blockIdx.x;
  const bool upper = (tj * 32) / 256 >= (ti * 32) / 256;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;              // 32 x 8 threads, 4 rows each
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int li = ty * 4 + r;
    const int si = (upper ? ti : tj) * 32 + li, sj = (upper ? tj : ti) * 32 + tx;
    tile[li][tx] = (si < M && sj < M) ? __bfloat162float(U[(long long)si * ldu + sj]) : 0.f;
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int li = ty * 4 + r;
    const int i = ti * 32 + li, j = tj * 32 + tx;
    if (i >= M || j >= M) continue;
    float v = alpha * (upper ? tile[li][tx] : tile[tx][li]);
    if (aux) v += beta * __bfloat162float(aux[(long long)i * ldaux + j]);
    if (i == j) v += diag;
    out[(long long)i * ldo + j] = __float2bfloat16(v);
  }
}
TPLR_API int tplr_sym_axpby(const void* U, long long ldu, int M, float alpha, const void* aux, long long ldaux, float beta,
                            float diag, void* out, long long ldo, void* stream) {
  TPLR_ENTER();
  if (M <= 0) return 0;
  const unsigned t = (unsigned)((M + 31) / 32);
  sym_axpby_kernel<<<dim3(t, t), 256, 0, (cudaStream_t)stream>>>((const bf16*)U, ldu, M, alpha, (const bf16*)aux, ldaux,
                                                               beta, diag, (bf16*)out, ldo);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------- //
// Cross entropy without caller-provided scratch (see no_alloc.h). The per-row losses and the
// valid-row counter live in a file-scope device array. In host code the array's name is only a
// handle: its device address is looked up once per device with cudaGetSymbolAddress (with that
// device current) and that pointer is what the kernels receive.
// ------------------------------------------------------------------------------------- //
// layout: word 0 is the valid-row counter (int), words 64.. are the per-row losses (256-byte aligned)
#define CE_SCRATCH_HEADER 64
static __device__ __align__(256) float g_ce_scratch[CE_SCRATCH_HEADER + TPLR_CE_NOALLOC_MAX_ROWS];

#define TPLR_MAX_DEVICES 64
// null = not looked up yet on that device.  Host threads may race to fill a slot: every one of them
// would store the same address, and the atomic makes the store and the later loads well defined.
static std::atomic<float*> g_ce_scratch_addr[TPLR_MAX_DEVICES];

static int ce_scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= TPLR_MAX_DEVICES) return TPLR_ERR_NOALLOC_BAD_ARG;
  float* p = g_ce_scratch_addr[dev].load(std::memory_order_acquire);
  if (!p) {
    e = cudaGetSymbolAddress((void**)&p, g_ce_scratch);
    if (e != cudaSuccess) return (int)e;
    g_ce_scratch_addr[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return 0;
}

TPLR_API long long tplr_cross_entropy_noalloc_max_rows(void) { return TPLR_CE_NOALLOC_MAX_ROWS; }

TPLR_API int tplr_cross_entropy_noalloc(void* logits, const long long* labels, float* loss_out, float grad_scale,
                                        long long rows, int vocab, long long ld, long long ignore_index,
                                        int write_grad, void* stream) {
  TPLR_ENTER();
  if (rows > TPLR_CE_NOALLOC_MAX_ROWS) return TPLR_ERR_NOALLOC_TOO_LARGE;
  if (rows < 0 || vocab <= 0 || (ld % 8) || ld < vocab || !logits || !labels || !loss_out) return TPLR_ERR_NOALLOC_BAD_ARG;
  if ((uintptr_t)logits & 15) return TPLR_ERR_NOALLOC_BAD_ARG;   // rows are read and written as 16-byte vectors
  if (rows == 0) return 0;
  float* sc = nullptr;
  const int rc = ce_scratch_for_current_device(&sc);
  if (rc != 0) return rc;
  int* n_valid = reinterpret_cast<int*>(sc);
  float* losses = sc + CE_SCRATCH_HEADER;
  cudaStream_t st = (cudaStream_t)stream;
  // count_valid_kernel overwrites n_valid and ce_kernel writes losses[0..rows) before
  // sum_rows_kernel reads them, so whatever an earlier call left in the array is never used.
  count_valid_kernel<<<1, 1024, 0, st>>>(labels, rows, ignore_index, vocab, n_valid, nullptr);
  ce_kernel<<<(unsigned)rows, 512, 0, st>>>((bf16*)logits, labels, losses, n_valid, grad_scale, vocab, ld,
                                            ignore_index, write_grad);
  sum_rows_kernel<<<1, 1024, 0, st>>>(losses, rows, n_valid, 1.f, loss_out);
  return (int)cudaGetLastError();
}
