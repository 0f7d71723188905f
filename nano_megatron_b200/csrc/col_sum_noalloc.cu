// Column sum (bias gradient) that brings its own scratch memory.  See
// nmb_no_alloc.h for who needs this and for the full contract.
//
// The reduction is the two-stage scheme of `nmb_col_reduce(mode = 0)`:
// stage 1 splits the rows 16 ways and writes one fp32 partial sum per
// (split, column); stage 2 adds the 16 partials of a column.  The partials live
// in `g_noalloc_scratch` below instead of a caller-provided buffer.
#include "common.cuh"
#include "nmb_no_alloc.h"

namespace {

constexpr int kSplit = 16;
constexpr int kMaxDevices = 64;

// 16 splits x NMB_NOALLOC_MAX_COLS columns of fp32 = 512 KiB are used; the
// array is sized like the regular entry point's scratch (2 x that, 1 MiB) so
// both layouts fit.  Held by every GPU that loads the library, until exit.
static __device__ __align__(256) float g_noalloc_scratch[2 * kSplit * NMB_NOALLOC_MAX_COLS];

// Host-side cache of the array's *device* address, one slot per device.  The
// name `g_noalloc_scratch` in host code is only a handle for the runtime, not
// an address a kernel may dereference -- hence cudaGetSymbolAddress.
float* g_scratch_addr[kMaxDevices] = {nullptr};

__global__ void noalloc_stage1(const __nv_bfloat16* __restrict__ dy, float* __restrict__ partial, int rows,
                               int cols, int ld) {
  __shared__ float red[8][64];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int c = blockIdx.x * 64 + lane * 2;
  float a0 = 0.f, a1 = 0.f;
  if (c < cols) {
    for (int r = blockIdx.y * 8 + warp; r < rows; r += kSplit * 8) {
      const float2 g = __bfloat1622float2(
          *reinterpret_cast<const __nv_bfloat162*>(dy + static_cast<size_t>(r) * ld + c));
      a0 += g.x;
      a1 += g.y;
    }
  }
  red[warp][lane * 2] = a0;
  red[warp][lane * 2 + 1] = a1;
  __syncthreads();
  if (threadIdx.x < 64) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += red[w][threadIdx.x];
    const int cc = blockIdx.x * 64 + threadIdx.x;
    // Every (split, column < cols) slot is written here before stage 2 reads
    // it, so stale contents from an earlier call never leak into a result.
    if (cc < cols) partial[static_cast<size_t>(blockIdx.y) * cols + cc] = s;
  }
}

__global__ void noalloc_stage2(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out, int cols,
                               int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < kSplit; ++k) s += partial[static_cast<size_t>(k) * cols + c];
  if (accumulate) s += __bfloat162float(out[c]);
  out[c] = __float2bfloat16(s);
}

// Resolve (once per device, with that device current) the device address of
// the scratch array.  No allocation happens here: the array is part of the
// loaded module.
float* scratch_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (g_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch) != cudaSuccess) return nullptr;
    g_scratch_addr[dev] = p;
  }
  return g_scratch_addr[dev];
}

}  // namespace

extern "C" int nmb_col_sum_noalloc_max_cols(void) { return NMB_NOALLOC_MAX_COLS; }

extern "C" const char* nmb_col_sum_noalloc_strerror(int code) {
  switch (code) {
    case NMB_NOALLOC_OK: return "ok";
    case NMB_NOALLOC_BAD_SHAPE:
      return "cols and ld must be even, ld >= cols, dy 4-byte aligned, out 2-byte aligned, pointers non-null";
    case NMB_NOALLOC_TOO_LARGE: return "cols exceeds NMB_NOALLOC_MAX_COLS (8192): the built-in scratch is too small";
    case NMB_NOALLOC_NO_SCRATCH: return "the built-in scratch array could not be resolved on the current device";
    default: return "CUDA launch error (code - 400 is the cudaError_t)";
  }
}

extern "C" int nmb_col_sum_noalloc(const void* dy, int ld, void* out, int rows, int cols, int accumulate,
                                   void* stream) {
  if (cols <= 0) return NMB_NOALLOC_OK;
  if (out == nullptr || (reinterpret_cast<uintptr_t>(out) & 1) != 0) return NMB_NOALLOC_BAD_SHAPE;
  if (rows < 0) rows = 0;
  // Stage 1 reads dy two bf16 at a time (4-byte loads at dy + r * ld + c with c
  // even): the base must be 4-byte aligned and the pitch even, or the load is a
  // misaligned address on the device.
  if (rows > 0 && (dy == nullptr || (reinterpret_cast<uintptr_t>(dy) & 3) != 0)) return NMB_NOALLOC_BAD_SHAPE;
  if ((cols % 2) != 0 || (ld % 2) != 0 || ld < cols) return NMB_NOALLOC_BAD_SHAPE;
  if (cols > NMB_NOALLOC_MAX_COLS) return NMB_NOALLOC_TOO_LARGE;
  float* scratch = scratch_for_current_device();
  if (scratch == nullptr) return NMB_NOALLOC_NO_SCRATCH;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid((cols + 63) / 64, kSplit);
  noalloc_stage1<<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(dy), scratch, rows, cols, ld);
  noalloc_stage2<<<(cols + 255) / 256, 256, 0, s>>>(scratch, static_cast<__nv_bfloat16*>(out), cols, accumulate);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? NMB_NOALLOC_OK : 400 + static_cast<int>(e);
}
