// Cross-entropy entry point for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference implementation; it exists for hosts
// that embed this library where allocation is off the table: a process whose whole device
// memory is already handed out to a fixed arena by another runtime, a plugin called from a
// thread that is not allowed to touch the caching allocator, or a control loop that has to
// stay free of cudaMalloc/cudaFree because those calls synchronise the device and can fail
// late when memory is fragmented.  Such a caller owns the logits, labels and the output scalar,
// but has nowhere to put the per-row scratch that the regular entry point (tplr_cross_entropy)
// expects to be passed in.
//
// Here the scratch (one float per row plus a valid-row counter) lives in a fixed array inside
// the library image, sized for at most TPLR_CE_NOALLOC_MAX_ROWS rows.  Every GPU that loads the
// library carries that array (TPLR_CE_NOALLOC_MAX_ROWS * 4 + 256 bytes) until the process exits.
//
// Rules for callers:
//  * rows > TPLR_CE_NOALLOC_MAX_ROWS is refused with TPLR_ERR_NOALLOC_TOO_LARGE; nothing is launched.
//  * The first call on each device looks up the array's device address (once, with that device
//    current).  Make that first call before starting any stream capture.
//  * All calls share the one array and it keeps whatever the previous call left in it; the
//    kernels overwrite every slot they later read, so a call never sees stale values.  Two calls
//    that may run on the GPU at the same time (different streams, no ordering between them) race
//    on the array: order them yourself.
//  * A label that is neither ignore_index nor inside [0, vocab) is treated like ignore_index (loss 0,
//    zero gradient, not counted); it is never used as an index.
//  * `logits` must be 16-byte aligned, `ld` a multiple of 8 and at least `vocab`; anything else is
//    refused with TPLR_ERR_NOALLOC_BAD_ARG before a kernel is launched.
//  * This entry point itself calls no cudaMalloc, cudaFree or allocating library routine on any path.
//    (The CUDA driver loads a library's kernels the first time one of them is launched in a process;
//    that is the driver's own bookkeeping, happens once, and is another reason to make the first call
//    during set-up rather than inside a latency-critical section.)
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define TPLR_CE_NOALLOC_MAX_ROWS 131072
#define TPLR_ERR_NOALLOC_TOO_LARGE (-201)
#define TPLR_ERR_NOALLOC_BAD_ARG (-202)

// Same arithmetic as tplr_cross_entropy: mean cross entropy over rows whose label differs from
// ignore_index, written to *loss_out (device, fp32); with write_grad != 0 the bf16 logits are
// replaced in place by (softmax - onehot) * grad_scale / n_valid.  `ld` is the row stride of
// `logits` in elements (a multiple of 8).  Returns 0, a positive cudaError_t, or one of the
// negative TPLR_ERR_NOALLOC_* codes.
int tplr_cross_entropy_noalloc(void* logits, const long long* labels, float* loss_out, float grad_scale,
                               long long rows, int vocab, long long ld, long long ignore_index,
                               int write_grad, void* stream);

// Capacity query (rows); lets a caller check a shape up front.
long long tplr_cross_entropy_noalloc_max_rows(void);

#ifdef __cplusplus
}
#endif
