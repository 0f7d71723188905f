// Softmax cross entropy over (optionally vocabulary-sharded) bf16 logits with
// fp32 statistics.  Replaces the ~15 ATen kernels of the reference's
// vocab-parallel CE (nano_megatron/parallel/vocab_parallel.py:103-176) and
// F.cross_entropy (nano_megatron/reference/loss.py:18-23).
//
//   stage A (per rank)   : row max, sum exp(x - max), target logit (if owned)
//   stage B (all ranks)  : combine the per-rank triples -> lse, loss, count
//   backward             : dlogits = (exp(x - lse) - onehot) * gscale, written
//                          straight from the logits (no saved softmax)
// Rows whose target is `ignore_index` contribute neither loss nor gradient.
#include "common.cuh"

namespace nmb {

constexpr int kCeThreads = 256;

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, other) : v + other;
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = scratch[0];
  for (int w = 1; w < (blockDim.x >> 5); ++w) r = is_max ? fmaxf(r, scratch[w]) : r + scratch[w];
  return r;
}

// stats[row] = {local max, local sum exp(x - local max), target logit or 0}
__global__ void ce_stats_kernel(const __nv_bfloat16* __restrict__ logits, long long ld,
                                const long long* __restrict__ target, int vocab_start, int vloc,
                                float* __restrict__ stats, int rows) {
  __shared__ float scratch[32];
  const int row = blockIdx.x;
  if (row >= rows) return;
  const __nv_bfloat16* x = logits + row * ld;
  const bool vec = (vloc % 8 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
  float mx = -INFINITY;
  if (vec) {
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    for (int i = threadIdx.x; i < vloc / 8; i += blockDim.x) {
      const uint4 u = xv[i];
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 f = unpack_bf16x2(w[t]);
        mx = fmaxf(mx, fmaxf(f.x, f.y));
      }
    }
  } else {
    for (int i = threadIdx.x; i < vloc; i += blockDim.x) mx = fmaxf(mx, __bfloat162float(x[i]));
  }
  mx = block_reduce(mx, true, scratch);
  float se = 0.f;
  if (vec) {
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    for (int i = threadIdx.x; i < vloc / 8; i += blockDim.x) {
      const uint4 u = xv[i];
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 f = unpack_bf16x2(w[t]);
        se += __expf(f.x - mx) + __expf(f.y - mx);
      }
    }
  } else {
    for (int i = threadIdx.x; i < vloc; i += blockDim.x) se += __expf(__bfloat162float(x[i]) - mx);
  }
  se = block_reduce(se, false, scratch);
  if (threadIdx.x == 0) {
    const long long t = target[row] - vocab_start;
    float tl = 0.f;
    if (t >= 0 && t < vloc) tl = __bfloat162float(x[t]);
    stats[row * 3 + 0] = mx;
    stats[row * 3 + 1] = se;
    stats[row * 3 + 2] = tl;
  }
}

// all_stats[rank][row][3] -> lse[row], loss[row]; accum[0] += sum loss, accum[1] += #valid
__global__ void ce_combine_kernel(const float* __restrict__ all_stats, int n_ranks,
                                  const long long* __restrict__ target, int ignore_index,
                                  float* __restrict__ lse, float* __restrict__ loss_rows,
                                  float* __restrict__ accum, int rows) {
  __shared__ float scratch[32];
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  float my_loss = 0.f, my_cnt = 0.f;
  if (row < rows) {
    float gmax = -INFINITY;
    for (int r = 0; r < n_ranks; ++r) gmax = fmaxf(gmax, all_stats[(static_cast<size_t>(r) * rows + row) * 3]);
    float se = 0.f, tl = 0.f;
    for (int r = 0; r < n_ranks; ++r) {
      const float* s = all_stats + (static_cast<size_t>(r) * rows + row) * 3;
      se += s[1] * __expf(s[0] - gmax);
      tl += s[2];
    }
    const float l = gmax + logf(se);
    lse[row] = l;
    const bool valid = target[row] != ignore_index;
    const float ls = valid ? (l - tl) : 0.f;
    if (loss_rows != nullptr) loss_rows[row] = ls;
    my_loss = ls;
    my_cnt = valid ? 1.f : 0.f;
  }
  const float tot = block_reduce(my_loss, false, scratch);
  const float cnt = block_reduce(my_cnt, false, scratch);
  if (threadIdx.x == 0) {
    atomicAdd(&accum[0], tot);
    atomicAdd(&accum[1], cnt);
  }
}

// dlogits[row, c] = (exp(x - lse) - [c == target]) * gscale[0]   (0 for ignored rows)
__global__ void ce_bwd_kernel(const __nv_bfloat16* __restrict__ logits, long long ld,
                              const long long* __restrict__ target, int vocab_start, int vloc,
                              int ignore_index, const float* __restrict__ lse,
                              const float* __restrict__ gscale, __nv_bfloat16* __restrict__ dlogits,
                              long long ldd, int rows) {
  const int row = blockIdx.x;
  if (row >= rows) return;
  const __nv_bfloat16* x = logits + row * ld;
  __nv_bfloat16* dx = dlogits + row * ldd;
  const long long tg = target[row];
  const bool valid = tg != ignore_index;
  const float gs = valid ? gscale[0] : 0.f;
  const float l = lse[row];
  const long long t = tg - vocab_start;
  const bool vec = (vloc % 8 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                   ((reinterpret_cast<uintptr_t>(dx) & 15) == 0);
  if (vec) {
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    uint4* dv = reinterpret_cast<uint4*>(dx);
    for (int i = threadIdx.x; i < vloc / 8; i += blockDim.x) {
      const uint4 u = xv[i];
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = unpack_bf16x2(w[k]);
        const int c = i * 8 + k * 2;
        float g0 = __expf(f.x - l), g1 = __expf(f.y - l);
        if (c == t) g0 -= 1.f;
        if (c + 1 == t) g1 -= 1.f;
        o[k] = pack_bf16x2(g0 * gs, g1 * gs);
      }
      dv[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  } else {
    for (int i = threadIdx.x; i < vloc; i += blockDim.x) {
      float g = __expf(__bfloat162float(x[i]) - l);
      if (i == t) g -= 1.f;
      dx[i] = __float2bfloat16(g * gs);
    }
  }
}

}  // namespace nmb

using namespace nmb;

extern "C" int nmb_ce_stats(const void* logits, long long ld, const long long* target, int vocab_start, int vloc,
                            float* stats, int rows, void* stream) {
  if (rows <= 0) return 0;
  ce_stats_kernel<<<rows, kCeThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(logits), ld, target, vocab_start, vloc, stats, rows);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + e;
}

// accum: two zero-initialised floats {sum of losses, number of valid rows}
extern "C" int nmb_ce_combine(const float* all_stats, int n_ranks, const long long* target, int ignore_index,
                              float* lse, float* loss_rows, float* accum, int rows, void* stream) {
  if (rows <= 0) return 0;
  ce_combine_kernel<<<(rows + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      all_stats, n_ranks, target, ignore_index, lse, loss_rows, accum, rows);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + e;
}

extern "C" int nmb_ce_bwd(const void* logits, long long ld, const long long* target, int vocab_start, int vloc,
                          int ignore_index, const float* lse, const float* gscale, void* dlogits, long long ldd,
                          int rows, void* stream) {
  if (rows <= 0) return 0;
  ce_bwd_kernel<<<rows, kCeThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(logits), ld, target, vocab_start, vloc, ignore_index, lse, gscale,
      static_cast<__nv_bfloat16*>(dlogits), ldd, rows);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + e;
}
