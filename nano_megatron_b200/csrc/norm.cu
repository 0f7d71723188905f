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

// Vector variants: rows of H = 256 * V elements, every lane keeps its 8 * V
// elements of the row in registers (one 16-byte load per 256-column chunk), so
// the row is read from memory exactly once.
template <int V>
__global__ void norm_fwd_vec_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                    const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ y,
                                    float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, float eps,
                                    int rms) {
  constexpr int H = 256 * V;
  pdl_enter();
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows;
       row += gridDim.x * warps_per_block) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * H);
    float v[V][8];
    float s = 0.f;
#pragma unroll
    for (int c = 0; c < V; ++c) {
      const uint4 u = xr[c * 32 + lane];
      const uint32_t ww[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = unpack_bf16x2(ww[k]);
        v[c][2 * k] = f.x;
        v[c][2 * k + 1] = f.y;
        s += f.x + f.y;
      }
    }
    const float mean = rms ? 0.f : warp_sum(s) / H;
    float sq = 0.f;
#pragma unroll
    for (int c = 0; c < V; ++c)
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float d = v[c][k] - mean;
        sq += d * d;
      }
    const float rstd = rsqrtf(warp_sum(sq) / H + eps);
    if (lane == 0) {
      if (mean_out != nullptr) mean_out[row] = mean;
      rstd_out[row] = rstd;
    }
    uint4* yr = reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * H);
#pragma unroll
    for (int c = 0; c < V; ++c) {
      const uint4 gu = __ldg(reinterpret_cast<const uint4*>(w) + c * 32 + lane);
      const uint32_t gg[4] = {gu.x, gu.y, gu.z, gu.w};
      uint32_t bb[4] = {0, 0, 0, 0};
      if (!rms && bias != nullptr) {
        const uint4 bu = __ldg(reinterpret_cast<const uint4*>(bias) + c * 32 + lane);
        bb[0] = bu.x; bb[1] = bu.y; bb[2] = bu.z; bb[3] = bu.w;
      }
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 g = unpack_bf16x2(gg[k]);
        const float2 b2 = unpack_bf16x2(bb[k]);
        o[k] = pack_bf16x2((v[c][2 * k] - mean) * rstd * g.x + b2.x, (v[c][2 * k + 1] - mean) * rstd * g.y + b2.y);
      }
      yr[c * 32 + lane] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// dx plus per-block partial sums of dgamma / dbeta: every warp accumulates the
// column sums of the rows it processes in registers, the block combines its
// warps in shared memory and writes ONE partial row per block; a second tiny
// kernel adds the partial rows.  dy and x are read once.
template <int V>
__global__ void norm_bwd_vec_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                    const __nv_bfloat16* __restrict__ w, const float* __restrict__ mean_in,
                                    const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dx_add,
                                    __nv_bfloat16* __restrict__ dx, float* __restrict__ partial, int rows, int rms) {
  constexpr int H = 256 * V;
  extern __shared__ float red[];  // [warps][2][H]
  pdl_enter();
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int warps_per_block = blockDim.x >> 5;
  float wv[V][8];
#pragma unroll
  for (int c = 0; c < V; ++c) {
    const uint4 gu = __ldg(reinterpret_cast<const uint4*>(w) + c * 32 + lane);
    const uint32_t gg[4] = {gu.x, gu.y, gu.z, gu.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 g = unpack_bf16x2(gg[k]);
      wv[c][2 * k] = g.x;
      wv[c][2 * k + 1] = g.y;
    }
  }
  float dg[V][8], db[V][8];
#pragma unroll
  for (int c = 0; c < V; ++c)
#pragma unroll
    for (int k = 0; k < 8; ++k) dg[c][k] = db[c][k] = 0.f;
  for (int row = blockIdx.x * warps_per_block + warp; row < rows; row += gridDim.x * warps_per_block) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * H);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + static_cast<size_t>(row) * H);
    const float mean = rms ? 0.f : mean_in[row];
    const float rstd = rstd_in[row];
    float xh[V][8], g[V][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int c = 0; c < V; ++c) {
      const uint4 xu = xr[c * 32 + lane];
      const uint4 gu = gr[c * 32 + lane];
      const uint32_t xx[4] = {xu.x, xu.y, xu.z, xu.w};
      const uint32_t gg[4] = {gu.x, gu.y, gu.z, gu.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 a = unpack_bf16x2(xx[k]);
        const float2 b = unpack_bf16x2(gg[k]);
        xh[c][2 * k] = (a.x - mean) * rstd;
        xh[c][2 * k + 1] = (a.y - mean) * rstd;
        g[c][2 * k] = b.x;
        g[c][2 * k + 1] = b.y;
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        dg[c][k] += g[c][k] * xh[c][k];
        db[c][k] += g[c][k];
        const float gw = g[c][k] * wv[c][k];
        s1 += gw;
        s2 += gw * xh[c][k];
      }
    }
    s1 = rms ? 0.f : warp_sum(s1) / H;
    s2 = warp_sum(s2) / H;
    uint4* dr = reinterpret_cast<uint4*>(dx + static_cast<size_t>(row) * H);
    const uint4* ar = reinterpret_cast<const uint4*>(dx_add + static_cast<size_t>(row) * H);
#pragma unroll
    for (int c = 0; c < V; ++c) {
      float add[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (dx_add != nullptr) {  // gradient of the residual branch that bypassed the norm
        const uint4 au = ar[c * 32 + lane];
        const uint32_t aa[4] = {au.x, au.y, au.z, au.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 a = unpack_bf16x2(aa[k]);
          add[2 * k] = a.x;
          add[2 * k + 1] = a.y;
        }
      }
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        o[k] = pack_bf16x2(rstd * (g[c][2 * k] * wv[c][2 * k] - s1 - xh[c][2 * k] * s2) + add[2 * k],
                           rstd * (g[c][2 * k + 1] * wv[c][2 * k + 1] - s1 - xh[c][2 * k + 1] * s2) + add[2 * k + 1]);
      dr[c * 32 + lane] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
  float* mine = red + static_cast<size_t>(warp) * 2 * H;
#pragma unroll
  for (int c = 0; c < V; ++c) {
    float4* g4 = reinterpret_cast<float4*>(mine + (c * 32 + lane) * 8);
    float4* b4 = reinterpret_cast<float4*>(mine + H + (c * 32 + lane) * 8);
    g4[0] = make_float4(dg[c][0], dg[c][1], dg[c][2], dg[c][3]);
    g4[1] = make_float4(dg[c][4], dg[c][5], dg[c][6], dg[c][7]);
    b4[0] = make_float4(db[c][0], db[c][1], db[c][2], db[c][3]);
    b4[1] = make_float4(db[c][4], db[c][5], db[c][6], db[c][7]);
  }
  __syncthreads();
  float* prow = partial + static_cast<size_t>(blockIdx.x) * 2 * H;
  for (int i = threadIdx.x; i < 2 * H; i += blockDim.x) {
    float acc = 0.f;
    for (int wv2 = 0; wv2 < warps_per_block; ++wv2) acc += red[static_cast<size_t>(wv2) * 2 * H + i];
    prow[i] = acc;
  }
}

// Sums the per-block partial rows: 32 columns per block, 8 groups of partial
// rows summed in parallel and combined through shared memory.
// `accumulate`: add to what dgamma / dbeta already hold (gradient buffers).
__global__ void norm_bwd_finish_kernel(const float* __restrict__ partial, int n_partial, int H,
                                       __nv_bfloat16* __restrict__ dgamma, __nv_bfloat16* __restrict__ dbeta,
                                       int accumulate) {
  __shared__ float red[8][32];
  pdl_enter();
  const int cx = threadIdx.x & 31;
  const int px = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + cx;  // column in [0, 2H): dgamma then dbeta
  float acc = 0.f;
  for (int p = px; p < n_partial; p += 8) acc += partial[static_cast<size_t>(p) * 2 * H + col];
  red[px][cx] = acc;
  __syncthreads();
  if (px == 0) {
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) s += red[k][cx];
    __nv_bfloat16* dst = col < H ? dgamma + col : (dbeta != nullptr ? dbeta + (col - H) : nullptr);
    if (dst != nullptr) {
      if (accumulate) s += __bfloat162float(*dst);
      *dst = __float2bfloat16(s);
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
// stores / accumulates bf16.  With `fused_finish` stage 2 runs inside stage 1:
// the block that arrives last on its column group's counter (all splits of the
// 64 columns are then in memory) sums them, so one launch does the whole
// reduction.  The counters return to zero, ready for the next launch (graph
// replays included); launches that share the scratch must be stream-ordered.
constexpr int kColSplit = 64;
constexpr int kMaxColGroups = 1024;
__device__ unsigned int g_col_arrivals[kMaxColGroups];

__global__ void col_reduce_stage1(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                  const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                                  float* partial, int rows, int H, int ld, int mode, int rms, int fused_finish,
                                  __nv_bfloat16* out0, __nv_bfloat16* out1, int accumulate) {
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
    __threadfence();
  }
  if (!fused_finish) return;
  __shared__ int is_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(&g_col_arrivals[blockIdx.x], 1u);
    is_last = prev == gridDim.y - 1;
    if (is_last) g_col_arrivals[blockIdx.x] = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  {
    // 2 x 64 sums of kColSplit partials: each half of the block takes half the splits
    const int pair = threadIdx.x & 127;
    const int half = threadIdx.x >> 7;
    const int which = pair >> 6;
    const int cc = blockIdx.x * 64 + (pair & 63);
    float s = 0.f;
    if (cc < H && (which == 0 || out1 != nullptr)) {
#pragma unroll 8
      for (int k = half * (kColSplit / 2); k < (half + 1) * (kColSplit / 2); ++k)
        s += __ldcg(&partial[(static_cast<size_t>(k) * 2 + which) * H + cc]);
    }
    float* comb = &red[0][0][0];
    if (half == 1) comb[pair] = s;
    __syncthreads();
    if (half == 0 && cc < H) {
      s += comb[pair];
      __nv_bfloat16* dst = which == 0 ? out0 : out1;
      if (dst != nullptr) {
        if (accumulate) s += __bfloat162float(dst[cc]);
        dst[cc] = __float2bfloat16(s);
      }
    }
  }
}

// Vector form of stage 1 (+ in-kernel finish) for H % 8 == 0 and 16-byte
// aligned rows: a warp covers 256 columns with one 16-byte load per lane and
// keeps four rows in flight; block (g, s) reduces rows s*8+w, s*8+w+8*S, ... of
// column group g; the last block of a column group to finish adds the S
// partial rows with float4 loads (4 x 64 threads, one quarter of the splits
// each) and stores / accumulates the bf16 result.
// MODE is a template parameter so that the plain column sum (bias gradients,
// the common case) does not carry the registers of the dgamma / dbeta form and
// keeps four blocks per SM.
template <int MODE>
__global__ void __launch_bounds__(256, MODE == 0 ? 4 : 2)
col_reduce_vec_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                      const float* __restrict__ mean_in, const float* __restrict__ rstd_in, float* partial,
                      int rows, int H, int ld, int rms, __nv_bfloat16* out0, __nv_bfloat16* out1,
                      int accumulate) {
  constexpr int mode = MODE;
  __shared__ __align__(16) float red[2][8][256];
  __shared__ int is_last;
  pdl_enter();
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int S = gridDim.y;
  const int c = blockIdx.x * 256 + lane * 8;
  float a[8], b[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) a[k] = b[k] = 0.f;
  if (c < H) {
    const int stride = S * 8;
    for (int r0 = blockIdx.y * 8 + warp; r0 < rows; r0 += 4 * stride) {
      uint4 g[4], v[4];
      float m[4], rs[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int r = r0 + u * stride;
        g[u] = make_uint4(0, 0, 0, 0);
        v[u] = make_uint4(0, 0, 0, 0);
        m[u] = 0.f;
        rs[u] = 0.f;
        if (r < rows) {
          g[u] = *reinterpret_cast<const uint4*>(dy + static_cast<size_t>(r) * ld + c);
          if (mode == 1) {
            v[u] = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * H + c);
            m[u] = rms ? 0.f : mean_in[r];
            rs[u] = rstd_in[r];
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t gg[4] = {g[u].x, g[u].y, g[u].z, g[u].w};
        const uint32_t vv[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 gf = unpack_bf16x2(gg[k]);
          if (mode == 1) {
            const float2 xf = unpack_bf16x2(vv[k]);
            a[2 * k] += gf.x * (xf.x - m[u]) * rs[u];
            a[2 * k + 1] += gf.y * (xf.y - m[u]) * rs[u];
            b[2 * k] += gf.x;
            b[2 * k + 1] += gf.y;
          } else {
            a[2 * k] += gf.x;
            a[2 * k + 1] += gf.y;
          }
        }
      }
    }
  }
  float4* ra = reinterpret_cast<float4*>(&red[0][warp][lane * 8]);
  float4* rb = reinterpret_cast<float4*>(&red[1][warp][lane * 8]);
  ra[0] = make_float4(a[0], a[1], a[2], a[3]);
  ra[1] = make_float4(a[4], a[5], a[6], a[7]);
  rb[0] = make_float4(b[0], b[1], b[2], b[3]);
  rb[1] = make_float4(b[4], b[5], b[6], b[7]);
  __syncthreads();
  {
    const int col = threadIdx.x;  // 256 columns of this group
    const int cc = blockIdx.x * 256 + col;
    if (cc < H) {
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int wv = 0; wv < 8; ++wv) {
        s0 += red[0][wv][col];
        s1 += red[1][wv][col];
      }
      partial[(static_cast<size_t>(blockIdx.y) * 2) * H + cc] = s0;
      if (mode == 1) partial[(static_cast<size_t>(blockIdx.y) * 2 + 1) * H + cc] = s1;
    }
    __threadfence();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(&g_col_arrivals[blockIdx.x], 1u);
    is_last = prev == gridDim.y - 1;
    if (is_last) g_col_arrivals[blockIdx.x] = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const int quarter = threadIdx.x >> 6;           // which quarter of the splits
  const int c4 = (threadIdx.x & 63) * 4;          // 4 columns per thread
  const int cc = blockIdx.x * 256 + c4;
  const int n_out = mode == 1 ? 2 : 1;
  float4 acc[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
  if (cc < H) {
    for (int which = 0; which < n_out; ++which) {
#pragma unroll 4
      for (int k = quarter; k < S; k += 4) {
        const float4 p4 = __ldcg(reinterpret_cast<const float4*>(&partial[(static_cast<size_t>(k) * 2 + which) * H + cc]));
        acc[which].x += p4.x;
        acc[which].y += p4.y;
        acc[which].z += p4.z;
        acc[which].w += p4.w;
      }
    }
  }
  float4* comb = reinterpret_cast<float4*>(&red[0][0][0]);  // [which][quarter][64]
  comb[(0 * 4 + quarter) * 64 + (threadIdx.x & 63)] = acc[0];
  comb[(1 * 4 + quarter) * 64 + (threadIdx.x & 63)] = acc[1];
  __syncthreads();
  if (threadIdx.x < 64 * n_out && blockIdx.x * 256 + (threadIdx.x & 63) * 4 < H) {
    const int which = threadIdx.x >> 6;
    const int idx = threadIdx.x & 63;
    float4 t = comb[(which * 4) * 64 + idx];
#pragma unroll
    for (int q = 1; q < 4; ++q) {
      const float4 o = comb[(which * 4 + q) * 64 + idx];
      t.x += o.x;
      t.y += o.y;
      t.z += o.z;
      t.w += o.w;
    }
    __nv_bfloat16* dst = which == 0 ? out0 : out1;
    if (dst != nullptr) {
      dst += blockIdx.x * 256 + idx * 4;  // H % 8 == 0: all four columns exist
      float r4[4] = {t.x, t.y, t.z, t.w};
      if (accumulate) {
        const uint2 old = *reinterpret_cast<const uint2*>(dst);
        const float2 o0 = unpack_bf16x2(old.x), o1 = unpack_bf16x2(old.y);
        r4[0] += o0.x;
        r4[1] += o0.y;
        r4[2] += o1.x;
        r4[3] += o1.y;
      }
      *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16x2(r4[0], r4[1]), pack_bf16x2(r4[2], r4[3]));
    }
  }
}

__global__ void col_reduce_stage2(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out0,
                                  __nv_bfloat16* __restrict__ out1, int H, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s0 = 0.f, s1 = 0.f;
#pragma unroll 8
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

template <int V>
static void launch_fwd_vec(const void* x, const void* w, const void* bias, void* y, float* mean, float* rstd, int rows,
                           float eps, int rms, int blocks, cudaStream_t s) {
  launch_pdl(norm_fwd_vec_kernel<V>, dim3(blocks), dim3(256), 0, s, static_cast<const __nv_bfloat16*>(x),
             static_cast<const __nv_bfloat16*>(w), static_cast<const __nv_bfloat16*>(bias),
             static_cast<__nv_bfloat16*>(y), mean, rstd, rows, eps, rms);
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

extern "C" int nmb_norm_fwd(const void* x, const void* w, const void* bias, void* y, float* mean, float* rstd,
                            int rows, int H, float eps, int rms, void* stream) {
  if (rows <= 0) return 0;
  if (H % 2 != 0) return kBadArgument;
  const int threads = 256;
  int blocks = (rows + 7) / 8;
  const int cap = sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (H % 256 == 0 && H <= 2048 && aligned16(x) && aligned16(w) && aligned16(y) && (bias == nullptr || aligned16(bias))) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (H / 256) {
      case 1: launch_fwd_vec<1>(x, w, bias, y, mean, rstd, rows, eps, rms, blocks, s); break;
      case 2: launch_fwd_vec<2>(x, w, bias, y, mean, rstd, rows, eps, rms, blocks, s); break;
      case 3: launch_fwd_vec<3>(x, w, bias, y, mean, rstd, rows, eps, rms, blocks, s); break;
      case 4: launch_fwd_vec<4>(x, w, bias, y, mean, rstd, rows, eps, rms, blocks, s); break;
      case 6: launch_fwd_vec<6>(x, w, bias, y, mean, rstd, rows, eps, rms, blocks, s); break;
      case 8: launch_fwd_vec<8>(x, w, bias, y, mean, rstd, rows, eps, rms, blocks, s); break;
      default: goto generic;
    }
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : 400 + e;
  }
generic:
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

template <int V>
static int configure_bwd_vec() {
  cudaError_t e = cudaFuncSetAttribute(norm_bwd_vec_kernel<V>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       8 * 2 * 256 * V * static_cast<int>(sizeof(float)));
  return e == cudaSuccess ? 0 : 300 + e;
}

extern "C" int nmb_norm_configure() {
  return configure_bwd_vec<1>() | configure_bwd_vec<2>() | configure_bwd_vec<3>() | configure_bwd_vec<4>();
}

template <int V>
static void launch_bwd_vec(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                           const void* dx_add, void* dx, float* partial, int rows, int rms, int blocks, cudaStream_t s) {
  launch_pdl(norm_bwd_vec_kernel<V>, dim3(blocks), dim3(256), 8 * 2 * 256 * V * sizeof(float), s,
             static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
             static_cast<const __nv_bfloat16*>(w), mean, rstd, static_cast<const __nv_bfloat16*>(dx_add),
             static_cast<__nv_bfloat16*>(dx), partial, rows, rms);
}

// Fused backward: dx, dgamma, dbeta in one pass over dy and x.  Needs
// H % 256 == 0, H <= 1024 (register budget) and 16-byte aligned rows; returns
// -1 when the shape is not covered (callers then use the generic kernels).
// `partial` is fp32 scratch of kNormBwdBlocks * 2 * H elements.  `dx_add`
// (optional, same shape as dx) is added to dx; `accumulate` adds the parameter
// gradients to the contents of dgamma / dbeta instead of overwriting them.
constexpr int kNormBwdBlocks = 148;
extern "C" int nmb_norm_bwd_fused_blocks() { return kNormBwdBlocks; }

extern "C" int nmb_norm_bwd_fused(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                                  const void* dx_add, void* dx, void* dgamma, void* dbeta, float* partial, int rows,
                                  int H, int rms, int accumulate, void* stream) {
  if (rows <= 0) return 0;
  if (H % 256 != 0 || H > 1024 || !aligned16(dy) || !aligned16(x) || !aligned16(w) || !aligned16(dx) ||
      !aligned16(dx_add))
    return -1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int blocks = (rows + 7) / 8;
  if (blocks > kNormBwdBlocks) blocks = kNormBwdBlocks;
  switch (H / 256) {
    case 1: launch_bwd_vec<1>(dy, x, w, mean, rstd, dx_add, dx, partial, rows, rms, blocks, s); break;
    case 2: launch_bwd_vec<2>(dy, x, w, mean, rstd, dx_add, dx, partial, rows, rms, blocks, s); break;
    case 3: launch_bwd_vec<3>(dy, x, w, mean, rstd, dx_add, dx, partial, rows, rms, blocks, s); break;
    case 4: launch_bwd_vec<4>(dy, x, w, mean, rstd, dx_add, dx, partial, rows, rms, blocks, s); break;
    default: return -1;
  }
  launch_pdl(norm_bwd_finish_kernel, dim3(2 * H / 32), dim3(256), 0, s, static_cast<const float*>(partial), blocks, H,
             static_cast<__nv_bfloat16*>(dgamma), static_cast<__nv_bfloat16*>(dbeta), accumulate);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + e;
}

// `partial` is fp32 scratch of 2 * 64 * H elements.
extern "C" int nmb_col_reduce(const void* dy, int ld, const void* x, const float* mean, const float* rstd,
                              float* partial, void* out0, void* out1, int rows, int H, int mode, int rms,
                              int accumulate, void* stream) {
  if (rows <= 0 || H <= 0) return 0;
  if (H % 2 != 0 || ld % 2 != 0) return kBadArgument;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (H % 8 == 0 && ld % 8 == 0 && aligned16(dy) && (mode != 1 || aligned16(x)) && (H + 255) / 256 <= kMaxColGroups &&
      (out0 == nullptr || (reinterpret_cast<uintptr_t>(out0) & 7) == 0) &&
      (out1 == nullptr || (reinterpret_cast<uintptr_t>(out1) & 7) == 0)) {
    const int groups = (H + 255) / 256;
    int split = 8;  // at least two blocks per SM, at most kColSplit partial rows
    while (split < kColSplit && groups * split < 2 * sm_count()) split *= 2;
    while (split > 1 && split * 8 > rows) split /= 2;
    if (mode == 1)
      launch_pdl(col_reduce_vec_kernel<1>, dim3(groups, split), dim3(256), 0, s,
                 static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), mean, rstd, partial, rows,
                 H, ld, rms, static_cast<__nv_bfloat16*>(out0), static_cast<__nv_bfloat16*>(out1), accumulate);
    else
      launch_pdl(col_reduce_vec_kernel<0>, dim3(groups, split), dim3(256), 0, s,
                 static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), mean, rstd, partial, rows,
                 H, ld, rms, static_cast<__nv_bfloat16*>(out0), static_cast<__nv_bfloat16*>(out1), accumulate);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : 400 + e;
  }
  dim3 grid((H + 63) / 64, kColSplit);
  const int fused_finish = grid.x <= kMaxColGroups ? 1 : 0;
  col_reduce_stage1<<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(dy),
                                         static_cast<const __nv_bfloat16*>(x), mean, rstd, partial, rows, H, ld,
                                         mode, rms, fused_finish, static_cast<__nv_bfloat16*>(out0),
                                         static_cast<__nv_bfloat16*>(out1), accumulate);
  if (!fused_finish)
    col_reduce_stage2<<<(H + 255) / 256, 256, 0, s>>>(partial, static_cast<__nv_bfloat16*>(out0),
                                                      static_cast<__nv_bfloat16*>(out1), H, accumulate);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + e;
}
