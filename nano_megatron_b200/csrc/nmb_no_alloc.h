// Allocation-free entry point of the kernel library.
//
// This entry point has no counterpart in the reference project (which has no
// native code at all); it exists for callers that are not allowed to allocate
// device memory at the time of the call.
//
// Who cannot allocate: code that runs inside a region where cudaMalloc /
// cudaFree are illegal or harmful -- a caller with a fixed memory budget that
// was carved up at start-up, a real-time loop that must not take the
// allocator's (device-synchronising) lock, a plug-in called from a host
// framework that owns all device memory and hands out only the input and
// output buffers.  The regular entry point `nmb_col_reduce` needs an fp32
// scratch buffer of 2 * 16 * H elements from its caller (the Python layer
// allocates it with torch); such callers have nowhere to get it from.
//
// `nmb_col_sum_noalloc` therefore keeps that scratch inside the library, in a
// file-scope `__device__` array of fixed size that every GPU which loads the
// library holds until the process exits:
//
//     NMB_NOALLOC_MAX_COLS = 8192 columns  ->  2 * 16 * 8192 * 4 B = 1 MiB per GPU
//
// Contract
//   * out[c] (+)= sum over rows r of dy[r, c]  -- the bias-gradient reduction,
//     bf16 in / bf16 out, fp32 accumulation; same arithmetic as
//     `nmb_col_reduce(mode = 0)`.
//   * The caller passes every input and output pointer; the function calls no
//     cudaMalloc, cudaFree or any other allocating routine.
//   * cols > NMB_NOALLOC_MAX_COLS is rejected with a non-zero code and nothing
//     is launched; so are odd cols / ld, ld < cols, a `dy` that is not 4-byte
//     aligned (rows are read two bf16 at a time, so a view that starts at an
//     odd element of a wider row is refused rather than read misaligned) and an
//     `out` that is not 2-byte aligned.  `nmb_col_sum_noalloc_strerror` turns
//     the code into a sentence.
//   * rows == 0 is a sum over nothing: out is zeroed (left alone when
//     accumulating); cols == 0 does nothing.
//   * The first call on each device looks up the device address of the
//     scratch array (cudaGetSymbolAddress, with that device current) and caches
//     it.  Make that first call before starting any stream capture on the
//     device.
//   * All calls on one device share the one scratch array, and it keeps
//     whatever the previous call left there.  Nothing in it has to start at
//     zero -- each call overwrites every slot it later reads -- but two calls
//     whose kernels overlap on the GPU (different streams, no ordering between
//     them) race on it.  Order such calls yourself.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define NMB_NOALLOC_MAX_COLS 8192

enum {
  NMB_NOALLOC_OK = 0,
  NMB_NOALLOC_BAD_SHAPE = 3,   // cols or ld odd, ld < cols, dy not 4-byte / out not 2-byte aligned, null pointer
  NMB_NOALLOC_TOO_LARGE = 4,   // cols > NMB_NOALLOC_MAX_COLS
  NMB_NOALLOC_NO_SCRATCH = 5,  // the scratch symbol could not be resolved on this device
};

// dy: bf16 [rows, ld] with `cols` valid columns; out: bf16 [cols].
// accumulate != 0 adds to the previous contents of out.  `stream` is a
// cudaStream_t.  Returns NMB_NOALLOC_OK, one of the codes above, or
// 400 + cudaError_t if the launch itself failed.
int nmb_col_sum_noalloc(const void* dy, int ld, void* out, int rows, int cols, int accumulate, void* stream);

int nmb_col_sum_noalloc_max_cols(void);
const char* nmb_col_sum_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
