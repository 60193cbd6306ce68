// Peer-memory runtime (one process per GPU, NVLink/NVSwitch peer access through CUDA IPC):
// symmetric allocations, handle export/import, a flag barrier with bounded waits, and the
// copy/reduce kernels that move shards directly between GPUs with plain loads and stores.
//
// This is the transport under the sharded optimizer step and the compressed-gradient
// gather; the reference uses torch.distributed/NCCL for all of it
// (src/tplr/distributed.py:35-549, FSDP2 all-gather / reduce-scatter).
#include "common.cuh"
#include <string.h>

TPLR_API int tplr_heap_alloc(unsigned long long bytes, void** out) {
  TPLR_ENTER();
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(p, 0, bytes);
  *out = p;
  return (int)e;
}
TPLR_API int tplr_heap_free(void* p) {
  TPLR_ENTER(); return (int)cudaFree(p); }

TPLR_API int tplr_ipc_handle_size() { return (int)sizeof(cudaIpcMemHandle_t); }
TPLR_API int tplr_ipc_get(void* p, void* handle_out) {
  TPLR_ENTER();
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e == cudaSuccess) memcpy(handle_out, &h, sizeof(h));
  return (int)e;
}
TPLR_API int tplr_ipc_open(const void* handle, void** out) {
  TPLR_ENTER();
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  return (int)cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
}
TPLR_API int tplr_ipc_close(void* p) {
  TPLR_ENTER(); return (int)cudaIpcCloseMemHandle(p); }

// ------------------------------------------------------------------------------------- //
// Flag barrier. Every rank owns an array of `n_ranks` 64-bit slots in symmetric memory.
// Arrive: write `epoch` into slot[my_rank] of every rank (release, system scope).
// Wait: poll own slots until all >= epoch (acquire, system scope), at most `timeout_ns`;
// on expiry set TPLR_ST_WAIT_TIMEOUT in *status and return — nothing spins forever.
// ------------------------------------------------------------------------------------- //
struct BarrierArgs {
  unsigned long long* flags[TPLR_MAX_PEERS];
  int n_ranks, my_rank;
  unsigned long long epoch, timeout_ns;
  unsigned int* status;
};

static __device__ __forceinline__ unsigned long long gtime_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__global__ void barrier_kernel(const BarrierArgs a) {
  const int r = threadIdx.x;
  if (r >= a.n_ranks) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(a.flags[r] + a.my_rank), "l"(a.epoch) : "memory");
  const unsigned long long t0 = gtime_ns();
  const unsigned long long* mine = a.flags[a.my_rank] + r;
  for (;;) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(mine) : "memory");
    if (v >= a.epoch) break;
    if (gtime_ns() - t0 > a.timeout_ns) {
      if (a.status) atomicOr(a.status, TPLR_ST_WAIT_TIMEOUT);
      break;
    }
    __nanosleep(200);
  }
}

TPLR_API int tplr_barrier(void* const* flag_ptrs, int n_ranks, int my_rank, unsigned long long epoch,
                          unsigned long long timeout_ns, unsigned int* status, void* stream) {
  TPLR_ENTER();
  if (n_ranks > TPLR_MAX_PEERS || n_ranks <= 0) return (int)cudaErrorInvalidValue;
  BarrierArgs a;
  for (int i = 0; i < n_ranks; ++i) a.flags[i] = (unsigned long long*)flag_ptrs[i];
  a.n_ranks = n_ranks; a.my_rank = my_rank; a.epoch = epoch; a.timeout_ns = timeout_ns; a.status = status;
  barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(a);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------- //
// Reduce-scatter by pulling: own[lo : lo+n] += sum over the other ranks' buffers of the same
// range (fp32, read over NVLink with 16-byte loads). The caller orders it after a barrier.
// ------------------------------------------------------------------------------------- //
struct ReduceArgs {
  float* bufs[TPLR_MAX_PEERS];
  int n_ranks, my_rank;
  long long lo, n4;
};

__global__ void __launch_bounds__(256) reduce_shards_kernel(const ReduceArgs a) {
  float4* own = reinterpret_cast<float4*>(a.bufs[a.my_rank] + a.lo);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < a.n4;
       i += (long long)gridDim.x * blockDim.x) {
    float4 s = own[i];
    for (int r = 0; r < a.n_ranks; ++r) {
      if (r == a.my_rank) continue;
      const float4 v = reinterpret_cast<const float4*>(a.bufs[r] + a.lo)[i];
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    own[i] = s;
  }
}

TPLR_API int tplr_reduce_shards(void* const* bufs, int n_ranks, int my_rank, long long lo, long long n,
                                void* stream) {
  TPLR_ENTER();
  if (n_ranks > TPLR_MAX_PEERS || (n % 4) || (lo % 4)) return (int)cudaErrorInvalidValue;
  if (n <= 0) return 0;
  ReduceArgs a;
  for (int i = 0; i < n_ranks; ++i) a.bufs[i] = (float*)bufs[i];
  a.n_ranks = n_ranks; a.my_rank = my_rank; a.lo = lo; a.n4 = n / 4;
  long long grid = (a.n4 + 255) / 256;
  const long long cap = (long long)tplr_sm_count() * 8;
  if (grid > cap) grid = cap;
  reduce_shards_kernel<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(a);
  return (int)cudaGetLastError();
}

// dst_k[0:bytes] = src[0:bytes] for every destination (16-byte aligned, bytes % 16 == 0)
struct PushArgs {
  uint4* dst[TPLR_MAX_PEERS];
  const uint4* src;
  int n_dst;
  long long n16;
};
__global__ void __launch_bounds__(256) push_copy_kernel(const PushArgs a) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < a.n16;
       i += (long long)gridDim.x * blockDim.x) {
    const uint4 v = a.src[i];
    for (int d = 0; d < a.n_dst; ++d) a.dst[d][i] = v;
  }
}
TPLR_API int tplr_push_copy(const void* src, void* const* dsts, int n_dst, long long bytes, void* stream) {
  TPLR_ENTER();
  if (n_dst > TPLR_MAX_PEERS || (bytes % 16)) return (int)cudaErrorInvalidValue;
  if (bytes <= 0 || n_dst <= 0) return 0;
  PushArgs a;
  a.src = (const uint4*)src; a.n_dst = n_dst; a.n16 = bytes / 16;
  for (int i = 0; i < n_dst; ++i) a.dst[i] = (uint4*)dsts[i];
  long long grid = (a.n16 + 255) / 256;
  const long long cap = (long long)tplr_sm_count() * 8;
  if (grid > cap) grid = cap;
  push_copy_kernel<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(a);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------- //
// Block-table copy: the all-gather of sharded parameters.  `table` (device memory) holds `n_blocks` records
// {src, dst, bytes}: src points into a peer's shard (mapped through the symmetric heap) or into this
// GPU's own, dst into the local full-size buffer of the group being gathered; both 16-byte aligned, bytes a
// multiple of 16.  The CTAs keep no shared memory and few registers, so they run beside the CTAs of a GEMM
// that occupies every SM instead of waiting for one to retire; `max_ctas` bounds how many SMs they touch.
// Replaces the per-block all-gather of FSDP2 (torchtitan models/llama3/infra/parallelize.py:383-422).
// ------------------------------------------------------------------------------------- //
struct CopyBlock { const uint4* src; uint4* dst; long long bytes; };

__global__ void __launch_bounds__(256) copy_blocks_kernel(const CopyBlock* __restrict__ table, int n_blocks) {
  for (int b = blockIdx.x; b < n_blocks; b += gridDim.x) {
    const CopyBlock cb = table[b];
    const long long n16 = cb.bytes >> 4;
    long long i = threadIdx.x;
    for (; i + 3 * 256 < n16; i += 4 * 256) {        // four 16-byte loads in flight per thread
      const uint4 v0 = cb.src[i], v1 = cb.src[i + 256], v2 = cb.src[i + 512], v3 = cb.src[i + 768];
      cb.dst[i] = v0; cb.dst[i + 256] = v1; cb.dst[i + 512] = v2; cb.dst[i + 768] = v3;
    }
    for (; i < n16; i += 256) cb.dst[i] = cb.src[i];
  }
}

TPLR_API int tplr_copy_blocks(const void* table, int n_blocks, int max_ctas, void* stream) {
  TPLR_ENTER();
  if (n_blocks <= 0) return 0;
  int grid = n_blocks;
  if (max_ctas <= 0) max_ctas = tplr_sm_count();
  if (grid > max_ctas) grid = max_ctas;
  copy_blocks_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const CopyBlock*)table, n_blocks);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------- //
// Block-table reduce: dst[dst_off + i] += sum over ranks r of bufs[r][src_off + i] (fp32).  Used for the
// gradients that are accumulated locally in full size (embedding rows, norm weights) and reduced into the
// owner's gradient shard once per inner step; the matrices' gradients never take this path (their GEMM
// epilogue adds them into the owner's shard directly).  Records: {src_off, dst_off, n} in elements, all
// multiples of 4.  The caller orders it after a barrier.
// ------------------------------------------------------------------------------------- //
struct ReduceBlock { long long src_off, dst_off, n; };
struct ReduceBlocksArgs {
  const float* bufs[TPLR_MAX_PEERS];
  int n_ranks;
  const ReduceBlock* table;
  int n_blocks;
  float* dst;
};

__global__ void __launch_bounds__(256) reduce_blocks_kernel(const ReduceBlocksArgs a) {
  for (int b = blockIdx.x; b < a.n_blocks; b += gridDim.x) {
    const ReduceBlock rb = a.table[b];
    float4* out = reinterpret_cast<float4*>(a.dst + rb.dst_off);
    const long long n4 = rb.n >> 2;
    for (long long i = threadIdx.x; i < n4; i += 256) {
      float4 s = out[i];
      for (int r = 0; r < a.n_ranks; ++r) {
        const float4 v = reinterpret_cast<const float4*>(a.bufs[r] + rb.src_off)[i];
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
      out[i] = s;
    }
  }
}

TPLR_API int tplr_reduce_blocks(void* const* bufs, int n_ranks, const void* table, int n_blocks, void* dst,
                                void* stream) {
  TPLR_ENTER();
  if (n_ranks > TPLR_MAX_PEERS || n_ranks <= 0) return (int)cudaErrorInvalidValue;
  if (n_blocks <= 0) return 0;
  ReduceBlocksArgs a;
  for (int i = 0; i < n_ranks; ++i) a.bufs[i] = (const float*)bufs[i];
  a.n_ranks = n_ranks; a.table = (const ReduceBlock*)table; a.n_blocks = n_blocks; a.dst = (float*)dst;
  int grid = n_blocks;
  const int cap = tplr_sm_count() * 4;
  if (grid > cap) grid = cap;
  reduce_blocks_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(a);
  return (int)cudaGetLastError();
}

// One 64-bit store into (possibly peer) memory, stream ordered: the "this window's payload is in place" post of
// co-located nodes.  System-scope release so that the payload written before it is visible to whoever reads the cell.
__global__ void store_i64_kernel(long long* dst, long long value) {
  __threadfence_system();
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(value) : "memory");
}
TPLR_API int tplr_store_i64(void* dst, long long value, void* stream) {
  TPLR_ENTER();
  if (!dst || ((uintptr_t)dst & 7)) return (int)cudaErrorInvalidValue;
  store_i64_kernel<<<1, 1, 0, (cudaStream_t)stream>>>((long long*)dst, value);
  return (int)cudaGetLastError();
}
