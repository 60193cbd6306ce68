// Shared declarations for the sm_100a kernels of this library.
//
// Every entry point is plain C ABI (called through ctypes with raw device pointers
// and the caller's stream), returns a cudaError_t-compatible int, and never
// allocates device memory: all workspaces are passed in by the caller.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define TPLR_API extern "C" __attribute__((visibility("default")))

// The CUDA runtime keeps a per-thread "last error"; another library's benign failure on the
// calling thread must not be reported as ours, so every entry point clears it first.
#define TPLR_ENTER() (void)cudaGetLastError()

#define TPLR_MAX_PEERS 32
#define TPLR_TILE 64            // maximum chunk edge (target_chunk)
#define TPLR_TILE_ELEMS 4096    // 64*64: indices fit 12 bits

// Status word bits written by kernels that validate their inputs instead of trapping.
enum : unsigned int {
  TPLR_ST_OK = 0u,
  TPLR_ST_BAD_INDEX = 1u,        // packed index >= elements in chunk
  TPLR_ST_NONFINITE = 2u,        // non-finite value met in a payload
  TPLR_ST_WAIT_TIMEOUT = 4u,     // bounded spin on a peer flag / mbarrier expired
  TPLR_ST_BAD_ARG = 8u,
};

// One entry per parameter tensor (or per contiguous range of chunk-rows of it) that a
// compress / aggregate launch covers.  Chunks are numbered row-major (y, x) inside the
// covered range; chunk c of the launch belongs to the entry with
// chunk_begin <= c < chunk_begin + n_chunks.
struct TplrParamDesc {
  long long elem_off;   // offset (elements) of the tensor's first element in the flat buffers
  long long idx_off;    // byte offset of this entry's first chunk in the packed-index buffer
  long long val_off;    // element offset of this entry's first chunk in the value buffer
  int rows, cols;       // logical 2-D shape (1-D tensors: rows = 1)
  int h, w;             // chunk edge per dimension (divisors of rows / cols, <= 64)
  int chunks_x;         // cols / w
  int chunk_row0;       // first chunk-row covered by this entry
  int chunk_begin;      // first launch-wide chunk id of this entry
  int n_chunks;         // chunks covered
  int k;                // even top-k for this tensor (<= h*w, <= 64)
  int fh_off, fw_off;   // float offsets of the h- and w-sized DCT matrices in the basis table
  int param_id;         // index into per-parameter side tables (norms, clip factors)
};

static __device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
static __device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum for blockDim.x <= 1024; `red` must hold 32 floats.
static __device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) red[wid] = v;
  __syncthreads();
  int nw = (blockDim.x + 31) >> 5;
  float r = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
  if (wid == 0) r = warp_sum(r);
  if (threadIdx.x == 0) red[0] = r;
  __syncthreads();
  return red[0];
}
static __device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) red[wid] = v;
  __syncthreads();
  int nw = (blockDim.x + 31) >> 5;
  float r = (threadIdx.x < nw) ? red[threadIdx.x] : -INFINITY;
  if (wid == 0) r = warp_max(r);
  if (threadIdx.x == 0) red[0] = r;
  __syncthreads();
  return red[0];
}

static inline int tplr_sm_count() {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  return sms;
}
