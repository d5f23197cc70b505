// Allocation-free entry point. It has no counterpart in the reference.
//
// Who it is for: host code that may not allocate device memory while it runs. Examples are a
// plugin living inside an application that has given all device memory to its own pool (a
// cudaMalloc there fails or fragments the pool), and a step loop that must never take the CUDA
// allocator's lock or risk the implicit device synchronisation an allocation can bring. The usual
// entry point (torch.ops.gdnet_b200.cross_entropy, driven from Python) needs temporaries from
// torch's allocator: a per-row loss buffer, the count of valid targets and the reduction result.
//
// This variant keeps that scratch in a fixed array inside the library instead (a file-scope
// __device__ array in loss_optim.cu, (GD_NOALLOC_MAX_ROWS + 64) floats = ~256 KB, held by every GPU
// that loads the library until the process exits). The caller passes only inputs and the output.
//
//   loss_out[0] = mean over rows with targets[row] != ignore_index of
//                 logsumexp(logits[row, :vocab]) - logits[row, targets[row]]
//
// logits: device, bf16, `rows` rows of pitch `ld` elements (ld % 8 == 0, 16-byte aligned base);
// only the first `vocab` columns take part. targets: device int64[rows]. loss_out: device float[1].
// A target that is neither `ignore_index` nor inside [0, vocab) is never used as an index: its row is
// left out of the sum and of the count, exactly like an ignored row (this entry point has no status
// word to report it through, so validate targets on the caller's side if bad ids must be noticed).
// stream: a cudaStream_t (as void*), may be null for the default stream. The logits are not modified.
//
// Return value: 0 on success, otherwise
//   1  rows > GD_NOALLOC_MAX_ROWS (or rows < 0): the fixed scratch cannot hold it; nothing was launched
//   2  bad argument (null pointer, misaligned logits, ld % 8 != 0, vocab out of range)
//   3  a CUDA call failed (looking up the scratch array's address, or a launch)
//
// Rules of use:
//  * The first call on each device looks up the device address of the scratch array
//    (cudaGetSymbolAddress, with that device current) and remembers it. Make that first call outside
//    any stream capture.
//  * Every call on a device shares the one scratch array and leaves its last contents there. Nothing
//    in it has to start at zero: a call overwrites the per-row slots [0, rows) before it reads them
//    and never reads beyond `rows`, so leftovers of a longer earlier call are harmless. Two calls
//    whose kernels overlap on the GPU (different streams, no ordering between them) race on the
//    scratch: order them.
//  * No cudaMalloc, cudaFree or allocating library routine is called, neither directly nor through
//    torch; the function launches two kernels on `stream` and returns without synchronising.
#pragma once

#include <stdint.h>

#define GD_NOALLOC_MAX_ROWS 65536

#ifdef __cplusplus
extern "C" {
#endif

int gd_cross_entropy_mean_noalloc(const void* logits_bf16, const int64_t* targets, int64_t rows, int vocab,
                                  int64_t ld, int ignore_index, float* loss_out, void* stream);

#ifdef __cplusplus
}
#endif
