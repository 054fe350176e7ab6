// Arg-max over the last dimension for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference runtime; it exists only in this library.
//
// Who needs it: a caller that holds no allocator it may use at the point of the call - a plug-in that runs inside
// another framework's stream callback, a C host that links this library without any tensor library, or code that
// runs after the device's memory has been handed out in full.  ortb200_argmax() asks such a caller for a scratch
// buffer; this variant brings its own: a fixed array that lives in the library's device image.
//
//   x [rows, n] (row-major, dtype = ORTB200_F16 / ORTB200_BF16 / ORTB200_F32)  ->  out int64 [rows]
//   first maximum wins, NaN never wins, an all-NaN row yields 0 - the same contract as ortb200_argmax().
//
// Limits and rules:
//   * rows <= ORTB200_ARGMAX_NOALLOC_MAX_ROWS (4096) and 1 <= n <= 2^32 - 1.  Anything larger is refused with
//     ORTB200_NOALLOC_E_TOO_LARGE and nothing is launched; use ortb200_argmax() with your own scratch instead.
//   * The call allocates nothing and frees nothing, on the host or on the device.  It enqueues one clear of the
//     scratch array and one kernel on `stream` and returns without waiting for them.
//   * The scratch array's device address is looked up once per device, on the first call made with that device
//     current.  Make that first call (or call ortb200_argmax_noalloc_prepare()) during set-up, before any stream
//     capture begins on that device: the lookup may have to load this library's device code.
//   * There is one scratch array per device.  Two calls whose work overlaps on the same device (different streams,
//     or different host threads with different streams) race on it and give wrong answers; order them on one
//     stream or with events.
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ORTB200_ARGMAX_NOALLOC_MAX_ROWS 4096

#define ORTB200_NOALLOC_OK 0
#define ORTB200_NOALLOC_E_BAD_ARGUMENT (-1)   /* null pointer, negative rows, n out of range */
#define ORTB200_NOALLOC_E_BAD_DTYPE (-4)
#define ORTB200_NOALLOC_E_LAUNCH (-11)        /* the clear or the kernel launch was rejected by the CUDA runtime */
#define ORTB200_NOALLOC_E_TOO_LARGE (-20)     /* rows > ORTB200_ARGMAX_NOALLOC_MAX_ROWS */
#define ORTB200_NOALLOC_E_NO_SCRATCH (-21)    /* the scratch array's address could not be obtained on this device */

// Looks up (and remembers) the scratch address for the current device.  Optional: the first
// ortb200_argmax_noalloc() call on a device does the same.  Returns ORTB200_NOALLOC_OK or ORTB200_NOALLOC_E_NO_SCRATCH.
int ortb200_argmax_noalloc_prepare(void);

// `stream` is a cudaStream_t (0 = the legacy default stream).
int ortb200_argmax_noalloc(const void* x, int64_t* out, int64_t rows, int64_t n, int dtype, void* stream);

// A one-line description of a return code of the two functions above (never null).
const char* ortb200_argmax_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
