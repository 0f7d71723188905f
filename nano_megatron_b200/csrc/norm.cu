// LayerNorm / RMSNorm forward and backward, bf16 in/out with fp32 statistics,
// plus the column reductions used for normalisation-parameter and bias
// gradients.  Replaces F.layer_norm and the four elementwise kernels of
// rms_norm in the reference (nano_megatron/reference/layers.py:18-35) and their
// autograd backward.
//
// One warp owns one row at a time (rows are 128 B .. 4 KiB, so the second and
// third sweeps over a row hit L1).  Statistics are two-pass (mean first, then
// centred variance), in fp32.
#include "common.cuh"

namespace nmb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// y = (x - mean) * rstd * w + b          (rms == 0)
// y = x * rstd * w, rstd = 1/sqrt(mean(x^2)+eps)   (rms == 1)
__global__ void norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ y,
                                float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows,
                                int H, float eps, int rms) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int pairs = H >> 1;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows;
       row += gridDim.x * warps_per_block) {
    const __nv_bfloat162* xr = reinterpret_cast<const __nv_bfloat162*>(x + static_cast<size_t>(row) * H);
    float mean = 0.f;
    if (!rms) {
      float s = 0.f;
      for (int i = lane; i < pairs; i += 32) {
        const float2 v = __bfloat1622float2(xr[i]);
        s += v.x + v.y;
      }
      mean = warp_sum(s) / H;
    }
    float sq = 0.f;
    for (int i = lane; i < pairs; i += 32) {
      const float2 v = __bfloat1622float2(xr[i]);
      const float a = v.x - mean, b = v.y - mean;
      sq += a * a + b * b;
    }
    const float var = warp_sum(sq) / H;
    // The reference's rms_norm divides by sqrt(mean(x^2) + eps).
    const float rstd = rsqrtf(var + eps);
    if (lane == 0) {
      if (mean_out != nullptr) mean_out[row] = mean;
      rstd_out[row] = rstd;
    }
    const __nv_bfloat162* wr = reinterpret_cast<const __nv_bfloat162*>(w);
    const __nv_bfloat162* br = reinterpret_cast<const __nv_bfloat162*>(bias);
    __nv_bfloat162* yr = reinterpret_cast<__nv_bfloat162*>(y + static_cast<size_t>(row) * H);
    for (int i = lane; i < pairs; i += 32) {
      const float2 v = __bfloat1622float2(xr[i]);
      const float2 g = __bfloat1622float2(wr[i]);
      float o0 = (v.x - mean) * rstd * g.x;
      float o1 = (v.y - mean) * rstd * g.y;
      if (!rms && bias != nullptr) {
        const float2 bb = __bfloat1622float2(br[i]);
        o0 += bb.x;
        o1 += bb.y;
      }
      yr[i] = __floats2bfloat162_rn(o0, o1);
    }
  }
}

// dx for one row:  g = dy * w ;  xhat = (x - mean) * rstd
//   layernorm: dx = rstd * (g - mean(g) - xhat * mean(g * xhat))
//   rmsnorm  : dx = rstd * (g - xhat * mean(g * xhat))
// `dx_add` (optional) is added to the result: the residual branch gradient.
__global__ void norm_bwd_dx_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ mean_in,
                                   const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dx_add,
                                   __nv_bfloat16* __restrict__ dx, int rows, int H, int rms) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int pairs = H >> 1;
  const __nv_bfloat162* wr = reinterpret_cast<const __nv_bfloat162*>(w);
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows;
       row += gridDim.x * warps_per_block) {
    const __nv_bfloat162* xr = reinterpret_cast<const __nv_bfloat162*>(x + static_cast<size_t>(row) * H);
    const __nv_bfloat162* gr = reinterpret_cast<const __nv_bfloat162*>(dy + static_cast<size_t>(row) * H);
    const float mean = rms ? 0.f : mean_in[row];
    const float rstd = rstd_in[row];
    float s1 = 0.f, s2 = 0.f;
    for (int i = lane; i < pairs; i += 32) {
      const float2 v = __bfloat1622float2(xr[i]);
      const float2 g = __bfloat1622float2(gr[i]);
      const float2 ww = __bfloat1622float2(wr[i]);
      const float g0 = g.x * ww.x, g1 = g.y * ww.y;
      s1 += g0 + g1;
      s2 += g0 * (v.x - mean) * rstd + g1 * (v.y - mean) * rstd;
    }
    s1 = rms ? 0.f : warp_sum(s1) / H;
    s2 = warp_sum(s2) / H;
    __nv_bfloat162* dr = reinterpret_cast<__nv_bfloat162*>(dx + static_cast<size_t>(row) * H);
    const __nv_bfloat162* ar =
        dx_add ? reinterpret_cast<const __nv_bfloat162*>(dx_add + static_cast<size_t>(row) * H) : nullptr;
    for (int i = lane; i < pairs; i += 32) {
      const float2 v = __bfloat1622float2(xr[i]);
      const float2 g = __bfloat1622float2(gr[i]);
      const float2 ww = __bfloat1622float2(wr[i]);
      float o0 = rstd * (g.x * ww.x - s1 - (v.x - mean) * rstd * s2);
      float o1 = rstd * (g.y * ww.y - s1 - (v.y - mean) * rstd * s2);
      if (ar != nullptr) {
        const float2 a = __bfloat1622float2(ar[i]);
        o0 += a.x;
        o1 += a.y;
      }
      dr[i] = __floats2bfloat162_rn(o0, o1);
    }
  }
}

// Column reductions over rows, two stages.
//   mode 0: out0[c] = sum_r dy[r,c]
//   mode 1: out0[c] = sum_r dy[r,c] * xhat[r,c] (dgamma), out1[c] = sum_r dy[r,c] (dbeta)
// Stage 1 writes partial[split][2][H] (fp32); stage 2 sums the splits and
// stores / accumulates bf16.
constexpr int kColSplit = 16;

__global__ void col_reduce_stage1(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                  const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                                  float* __restrict__ partial, int rows, int H, int ld, int mode, int rms) {
  // block = 32 lanes (column pairs) x 8 warps (rows); grid = (ceil(H/64), kColSplit)
  __shared__ float red[2][8][64];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int c = blockIdx.x * 64 + lane * 2;
  float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
  if (c < H) {
    for (int r = blockIdx.y * 8 + warp; r < rows; r += kColSplit * 8) {
      const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dy + static_cast<size_t>(r) * ld + c));
      if (mode == 1) {
        const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + static_cast<size_t>(r) * H + c));
        const float m = rms ? 0.f : mean_in[r];
        const float rs = rstd_in[r];
        a0 += g.x * (v.x - m) * rs;
        a1 += g.y * (v.y - m) * rs;
        b0 += g.x;
        b1 += g.y;
      } else {
        a0 += g.x;
        a1 += g.y;
      }
    }
  }
  red[0][warp][lane * 2] = a0;
  red[0][warp][lane * 2 + 1] = a1;
  red[1][warp][lane * 2] = b0;
  red[1][warp][lane * 2 + 1] = b1;
  __syncthreads();
  if (threadIdx.x < 128) {
    const int which = threadIdx.x >> 6;
    const int col = threadIdx.x & 63;
    float s = 0.f;
#pragma unroll
    for (int wv = 0; wv < 8; ++wv) s += red[which][wv][col];
    const int cc = blockIdx.x * 64 + col;
    if (cc < H) partial[(static_cast<size_t>(blockIdx.y) * 2 + which) * H + cc] = s;
  }
}

__global__ void col_reduce_stage2(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out0,
                                  __nv_bfloat16* __restrict__ out1, int H, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s0 = 0.f, s1 = 0.f;
#pragma unroll
  for (int k = 0; k < kColSplit; ++k) {
    s0 += partial[(static_cast<size_t>(k) * 2) * H + c];
    s1 += partial[(static_cast<size_t>(k) * 2 + 1) * H + c];
  }
  if (out0 != nullptr) {
    if (accumulate) s0 += __bfloat162float(out0[c]);
    out0[c] = __float2bfloat16(s0);
  }
  if (out1 != nullptr) {
    if (accumulate) s1 += __bfloat162float(out1[c]);
    out1[c] = __float2bfloat16(s1);
  }
}

}  // namespace nmb

using namespace nmb;

extern "C" int nmb_norm_fwd(const void* x, const void* w, const void* bias, void* y, float* mean, float* rstd,
                            int rows, int H, float eps, int rms, void* stream) {
  if (rows <= 0) return 0;
  if (H % 2 != 0) return kBadArgument;
  const int threads = 256;
  int blocks = (rows + 7) / 8;
  const int cap = sm_count() * 8;
  if (blocks > cap) blocks = cap;
  norm_fwd_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
      static_cast<const __nv_bfloat16*>(bias), static_cast<__nv_bfloat16*>(y), mean, rstd, rows, H, eps, rms);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + e;
}

extern "C" int nmb_norm_bwd_dx(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                               const void* dx_add, void* dx, int rows, int H, int rms, void* stream) {
  if (rows <= 0) return 0;
  if (H % 2 != 0) return kBadArgument;
  const int threads = 256;
  int blocks = (rows + 7) / 8;
  const int cap = sm_count() * 8;
  if (blocks > cap) blocks = cap;
  norm_bwd_dx_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
      static_cast<const __nv_bfloat16*>(w), mean, rstd, static_cast<const __nv_bfloat16*>(dx_add),
      static_cast<__nv_bfloat16*>(dx), rows, H, rms);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + e;
}

// `partial` is fp32 scratch of 2 * 16 * H elements.
extern "C" int nmb_col_reduce(const void* dy, int ld, const void* x, const float* mean, const float* rstd,
                              float* partial, void* out0, void* out1, int rows, int H, int mode, int rms,
                              int accumulate, void* stream) {
  if (rows <= 0 || H <= 0) return 0;
  if (H % 2 != 0 || ld % 2 != 0) return kBadArgument;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid((H + 63) / 64, kColSplit);
  col_reduce_stage1<<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(dy),
                                         static_cast<const __nv_bfloat16*>(x), mean, rstd, partial, rows, H, ld,
                                         mode, rms);
  col_reduce_stage2<<<(H + 255) / 256, 256, 0, s>>>(partial, static_cast<__nv_bfloat16*>(out0),
                                                    static_cast<__nv_bfloat16*>(out1), H, accumulate);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + e;
}
