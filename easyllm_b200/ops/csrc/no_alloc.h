// Entry points that never allocate.  They have no counterpart in the reference project.
//
// Some callers of the kernel library cannot hand over a scratch buffer and must not trigger an
// allocation either: a C or C++ host program that links the library without PyTorch (so there is no
// caching allocator to borrow from), or code running at a point where a device allocation would
// synchronise the device or fail (inside an out-of-memory handler, or while another thread holds the
// allocator).  For them the RMSNorm backward, whose weight-gradient reduction needs per-CTA partial
// sums, is offered with that scratch held in a fixed array inside the library's device image.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest problem the fixed scratch serves: cols <= ELL_STATIC_NORM_MAX_COLS (and a multiple of 8);
// rows are unlimited (the grid is capped so that grid * cols <= ELL_STATIC_NORM_SCRATCH_ELEMS floats = 4.5 MiB).
#define ELL_STATIC_NORM_MAX_COLS 8192
#define ELL_STATIC_NORM_SCRATCH_ELEMS (144 * 8192)

// Return codes.
#define ELL_STATIC_OK 0
#define ELL_STATIC_ERR_SHAPE (-1)      // cols not a multiple of 8, or rows < 0
#define ELL_STATIC_ERR_TOO_LARGE (-2)  // cols above ELL_STATIC_NORM_MAX_COLS: the fixed scratch cannot hold one partial row set
#define ELL_STATIC_ERR_SYMBOL (-3)     // the address of the scratch array could not be obtained on the current device
#define ELL_STATIC_ERR_DEVICE (-4)     // no current device, or a device ordinal beyond the table kept here (64)
// Positive values are cudaError_t codes from the launch.

// Same arithmetic and arguments as ell_rmsnorm_bwd minus the scratch pointer:
//   dh = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dres),   dw (+)= sum_rows dy * xhat      (dw is fp32 [cols])
// dy, h, dres, dh: bf16 [rows, cols];  w: bf16 [cols];  rstd: fp32 [rows];  dres may be null.
//
// The call allocates nothing: no cudaMalloc/cudaFree, no library routine that allocates.
// Set-up: the first call on each device (with that device current) looks up the device address of the
// scratch array and caches it; make that first call outside any stream capture.  The cached address belongs
// to the device's primary context and stays valid for as long as that context lives; after cudaDeviceReset
// (or a driver-API context that is not the primary one) the library must be reloaded before the next call.
// With rows == 0 the call launches no kernel; dw is set to zero when accumulate_dw is 0 and left alone otherwise.
// The scratch is shared by every call on a device and keeps its last contents.  Nothing in it has to
// start at zero: every partial row that the reduction reads is written in full by the same call first.
// Two calls on one device that overlap in time (different streams, or different threads) race on the
// scratch and give wrong weight gradients; serialise them on one stream or with events.
int ell_rmsnorm_bwd_static(const void* dy, const void* h, const void* w, const float* rstd, const void* dres,
                           void* dh, float* dw, int rows, int cols, int accumulate_dw, cudaStream_t stream);

// One-line text for a return code of the function above (static storage, never null).
const char* ell_static_strerror(int code);

#ifdef __cplusplus
}
#endif
