// Batch-norm forward (training) for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for embedders of this library.
//
// Who needs it: code that runs where the device heap is not ours to touch -- an application that handed
// all of the GPU's memory to its own pool at start-up, a latency-critical loop that cannot afford the
// implicit device-wide synchronisation and the unbounded latency of cudaMalloc/cudaFree, or a plug-in
// living inside a host program whose memory accounting would be thrown off by a foreign allocation.
// The regular entry point `rb_bn_fwd_train` asks such a caller for a zeroed scratch buffer of 2*C
// floats; this one needs nothing but the inputs and outputs.
//
// How: the per-channel sum / sum-of-squares scratch lives in a fixed array inside the library's device
// image (32 KiB, present on every GPU that loads the library until the process exits). That caps the
// channel count at RB_BN_NOALLOC_MAX_CHANNELS; larger requests are refused with RB_BN_NOALLOC_E_TOO_MANY_CHANNELS.
//
// Rules of use:
//  * The first call on each device looks up the device address of the scratch array (once per device,
//    with that device current). Make that first call during set-up, before any stream capture.
//  * Every call on a device shares the one array. The entry point clears the part it uses at the start
//    of each call (in stream order), so leftovers of an earlier call never leak into a result; but two
//    calls that overlap in time on the same GPU (different streams, or different host threads) race on
//    it. Serialise them: one stream, or events between streams.
//  * No cudaMalloc, cudaFree or any allocating library routine is called here, on any path.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RB_BN_NOALLOC_MAX_CHANNELS 4096

#define RB_BN_NOALLOC_OK 0
#define RB_BN_NOALLOC_E_CHANNEL_ALIGN (-10)       /* C must be a multiple of 8 */
#define RB_BN_NOALLOC_E_TOO_MANY_CHANNELS (-20)   /* C > RB_BN_NOALLOC_MAX_CHANNELS */
#define RB_BN_NOALLOC_E_DEVICE (-21)              /* current device could not be queried / index too large */
#define RB_BN_NOALLOC_E_SYMBOL (-22)              /* cudaGetSymbolAddress failed */
#define RB_BN_NOALLOC_E_LAUNCH (-1)               /* a kernel launch or the clearing memset failed */

// Same contract as rb_bn_fwd_train (bn.cu) without the `sums` argument:
//   x [rows][C] bf16 in, y [rows][C] bf16 out, mean/istd [C] fp32 out (batch statistics, kept for backward),
//   run_mean/run_var [C] fp32 in/out (may be null), gamma/beta [C] fp32 in, residual [rows][C] bf16 or null.
int rb_bn_fwd_train_noalloc(const void* x, long long rows, int C, int c_valid, float eps, float factor, float* mean,
                            float* istd, float* run_mean, float* run_var, const float* gamma, const float* beta,
                            const void* residual, void* y, int relu, cudaStream_t stream);

// Human-readable text for the codes above.
const char* rb_bn_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
