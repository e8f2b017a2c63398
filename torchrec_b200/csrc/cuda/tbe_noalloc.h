// C entry point for the fused embedding backward + optimizer update that allocates nothing.
//
// This entry point has no counterpart in the reference; it exists for callers of this library that
// must not allocate device memory while they run.
//
// Who needs it: code that runs where an allocation is not allowed or not wanted.  A serving or
// training loop that has handed all device memory to its own arena has nothing left for a
// cudaMalloc; a host thread that must not block cannot afford the implicit device synchronisation
// that cudaMalloc/cudaFree may perform; and a program that does not link the tensor library's
// caching allocator (a plain C or C++ host, a ctypes caller) has no allocator to ask.  The regular
// operator (`trb200::tbe_backward_apply`) asks the tensor library for four scratch buffers on every
// call; this one keeps the same scratch in a fixed array that lives in the module's device image.
//
// What it does: exactly the work of `trb200::tbe_backward_apply` for an already sorted plan (the
// tensors `tbe_build_plan` returns): segment-reduce the upstream gradient rows per embedding row
// and apply the optimizer in place.  Same kernels, same arithmetic, same order of summation.
//
// Limits (requests beyond them are rejected with TRB_NOALLOC_E_TOO_LARGE and a message, nothing is
// launched):
//   N (sorted entries)          <= TRB_NOALLOC_MAX_ENTRIES   (262144)
//   ceil(N/64) * max_D          <= TRB_NOALLOC_MAX_BLOCK_DIM (4096 * 128), i.e. 4 MiB of fp32 partials
//   max_D a multiple of 4, <= 1024
// The scratch array takes about 4.1 MiB of device memory per device from the moment the module is
// loaded on that device, whether or not this entry point is ever called.
//
// Set-up: the first call on each device looks up the device address of the scratch array (once per
// device, with that device current) and caches it.  That look-up may initialise the module on the
// device, so make the first call on a device before any stream capture begins on it.  Later calls
// do no set-up.
//
// Concurrency: there is ONE scratch array per device.  Two calls whose kernels can overlap on the
// same device (different streams, or different host threads on different streams) race on it and
// give wrong updates.  Calls on one stream are ordered and safe.  The call is asynchronous: it
// returns after enqueueing a small memset and three kernels on `stream`.
//
// The device that owns the pointers must be the current device of the calling thread.
#pragma once

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TRB_NOALLOC_MAX_ENTRIES 262144
#define TRB_NOALLOC_MAX_BLOCK_DIM (4096 * 128)

enum trb_noalloc_status {
  TRB_NOALLOC_OK = 0,
  TRB_NOALLOC_E_BAD_ARG = 1,    // null pointer, unknown dtype code, bad dim, missing optional input
  TRB_NOALLOC_E_TOO_LARGE = 2,  // beyond the limits above
  TRB_NOALLOC_E_DEVICE = 3,     // pointers are not on the current device
  TRB_NOALLOC_E_CUDA = 4,       // a CUDA runtime call failed; the message carries its error string
};

// dtype codes: 0 = fp32, 1 = fp16, 2 = bf16
typedef struct trb_tbe_bwd_noalloc_args {
  void* weights;              // all tables back to back, updated in place
  int32_t weights_dtype;
  int32_t grad_dtype;
  float* mom1;                // optimizer state, or null when the optimizer has none
  float* mom2;                // second state, or null
  float* dense_grad;          // only for opt_type 100 (write summed gradient, no update), else null
  const int64_t* meta;        // [5, F] per-feature metadata as built by TableBatchedEmbeddingBags
  const int64_t* sorted_keys; // [N] global row ids, ascending
  const int32_t* sorted_src;  // [N] pooled: bag id f*B+b; unpooled: position of the id
  const float* sorted_w;      // [N] per-sample weights in sorted order, or null
  const int32_t* src_feature; // unpooled only: feature of every position; null when pooled
  const float* bag_scale;     // mean pooling: 1/len per bag, or null
  const void* grad;           // upstream gradient rows
  int64_t grad_stride;        // elements per gradient row
  int64_t N;
  int32_t B;
  int32_t F;
  int32_t max_D;
  int32_t pooled;             // 1 pooled, 0 unpooled
  int32_t opt_type;           // same codes as the operator (0 SGD, 1 rowwise Adagrad, ...)
  int32_t step;               // optimizer step count (bias correction), >= 1
  float lr, eps, beta1, beta2, weight_decay, max_grad;
} trb_tbe_bwd_noalloc_args;

// Returns a trb_noalloc_status.  On failure, when `errbuf` is not null, a NUL-terminated message of
// at most `errbuf_len` bytes is written to it.  `stream` is a cudaStream_t (null = default stream).
int trb_tbe_backward_apply_noalloc(const trb_tbe_bwd_noalloc_args* args, void* stream, char* errbuf,
                                   size_t errbuf_len);

#ifdef __cplusplus
}
#endif
