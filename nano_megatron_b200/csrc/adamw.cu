// Fused multi-tensor AdamW: every parameter of a model is updated by one
// launch.  Replaces the per-parameter Python loop of ~10 ATen kernels in the
// reference optimizer (nano_megatron/reference/optimizer.py:41-93) with the
// same arithmetic: decoupled weight decay, fp32 moments, bias correction,
// params (bf16 or fp32) up-cast, updated and cast back.
//
// The step counter and the hyper-parameters live in device memory so that a
// captured CUDA graph replays the right values.
#include "common.cuh"

namespace nmb {

struct AdamTensor {
  void* param;
  const void* grad;
  float* exp_avg;
  float* exp_avg_sq;
  long long numel;
  long long first_block;  // index of this tensor's first block in the launch
  int param_bf16;
  int grad_bf16;
};

constexpr int kAdamBlockElems = 4096;
constexpr int kAdamThreads = 256;

// hyper = {lr, beta1, beta2, eps, weight_decay}; step_count[0] = steps done so far
__global__ void adamw_kernel(const AdamTensor* __restrict__ table, int n_tensors,
                             const float* __restrict__ hyper, const int* __restrict__ step_count) {
  // locate the tensor this block works on
  int lo = 0, hi = n_tensors - 1;
  const long long blk = blockIdx.x;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (table[mid].first_block <= blk) lo = mid; else hi = mid - 1;
  }
  const AdamTensor t = table[lo];
  const long long base = (blk - t.first_block) * kAdamBlockElems;
  const float lr = hyper[0], b1 = hyper[1], b2 = hyper[2], eps = hyper[3], wd = hyper[4];
  const float step = static_cast<float>(step_count[0] + 1);
  const float corr1 = 1.f - powf(b1, step);
  const float corr2 = 1.f - powf(b2, step);
  const float step_size = lr / corr1;
  const float inv_sqrt_corr2 = 1.f / sqrtf(corr2);
  const float decay = 1.f - lr * wd;
  auto update = [&](float g, float& w, float& m, float& v) {
    if (wd != 0.f) w *= decay;
    m = m * b1 + g * (1.f - b1);
    v = v * b2 + g * g * (1.f - b2);
    const float denom = sqrtf(v) * inv_sqrt_corr2 + eps;
    w -= step_size * (m / denom);
  };
  const long long remaining = t.numel - base;
  const int count = remaining < kAdamBlockElems ? static_cast<int>(remaining) : kAdamBlockElems;
  const uintptr_t align_bits = reinterpret_cast<uintptr_t>(t.param) | reinterpret_cast<uintptr_t>(t.grad) |
                               reinterpret_cast<uintptr_t>(t.exp_avg) | reinterpret_cast<uintptr_t>(t.exp_avg_sq);
  const bool vec = t.param_bf16 && t.grad_bf16 && (align_bits & 15) == 0 && (base % 8) == 0;
  int done = 0;
  if (vec) {
    // 8 elements per thread per trip: one 16-byte load of param and grad, two of each moment.
    const int groups = count / 8;
    __nv_bfloat16* pw = static_cast<__nv_bfloat16*>(t.param) + base;
    const __nv_bfloat16* pg = static_cast<const __nv_bfloat16*>(t.grad) + base;
    float* pm = t.exp_avg + base;
    float* pv = t.exp_avg_sq + base;
    for (int gi = threadIdx.x; gi < groups; gi += kAdamThreads) {
      const uint4 wu = reinterpret_cast<const uint4*>(pw)[gi];
      const uint4 gu = reinterpret_cast<const uint4*>(pg)[gi];
      float4 m0 = reinterpret_cast<float4*>(pm)[gi * 2], m1 = reinterpret_cast<float4*>(pm)[gi * 2 + 1];
      float4 v0 = reinterpret_cast<float4*>(pv)[gi * 2], v1 = reinterpret_cast<float4*>(pv)[gi * 2 + 1];
      const uint32_t ww[4] = {wu.x, wu.y, wu.z, wu.w};
      const uint32_t gg[4] = {gu.x, gu.y, gu.z, gu.w};
      float w[8], g[8];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 a = unpack_bf16x2(ww[k]);
        const float2 c = unpack_bf16x2(gg[k]);
        w[2 * k] = a.x; w[2 * k + 1] = a.y;
        g[2 * k] = c.x; g[2 * k + 1] = c.y;
      }
      float* mm[8] = {&m0.x, &m0.y, &m0.z, &m0.w, &m1.x, &m1.y, &m1.z, &m1.w};
      float* vv[8] = {&v0.x, &v0.y, &v0.z, &v0.w, &v1.x, &v1.y, &v1.z, &v1.w};
#pragma unroll
      for (int k = 0; k < 8; ++k) update(g[k], w[k], *mm[k], *vv[k]);
      reinterpret_cast<float4*>(pm)[gi * 2] = m0;
      reinterpret_cast<float4*>(pm)[gi * 2 + 1] = m1;
      reinterpret_cast<float4*>(pv)[gi * 2] = v0;
      reinterpret_cast<float4*>(pv)[gi * 2 + 1] = v1;
      uint4 out;
      out.x = pack_bf16x2(w[0], w[1]);
      out.y = pack_bf16x2(w[2], w[3]);
      out.z = pack_bf16x2(w[4], w[5]);
      out.w = pack_bf16x2(w[6], w[7]);
      reinterpret_cast<uint4*>(pw)[gi] = out;
    }
    done = groups * 8;
  }
  for (int i = done + threadIdx.x; i < count; i += kAdamThreads) {
    const long long idx = base + i;
    const float g = t.grad_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(t.grad)[idx])
                                : static_cast<const float*>(t.grad)[idx];
    float w = t.param_bf16 ? __bfloat162float(static_cast<__nv_bfloat16*>(t.param)[idx])
                           : static_cast<float*>(t.param)[idx];
    float m = t.exp_avg[idx], v = t.exp_avg_sq[idx];
    update(g, w, m, v);
    t.exp_avg[idx] = m;
    t.exp_avg_sq[idx] = v;
    if (t.param_bf16) static_cast<__nv_bfloat16*>(t.param)[idx] = __float2bfloat16(w);
    else static_cast<float*>(t.param)[idx] = w;
  }
}

__global__ void adamw_advance_kernel(int* step_count) { step_count[0] += 1; }

}  // namespace nmb

using namespace nmb;

extern "C" int nmb_adamw_table_entry_size() { return static_cast<int>(sizeof(AdamTensor)); }

extern "C" long long nmb_adamw_blocks_for(long long numel) {
  return (numel + kAdamBlockElems - 1) / kAdamBlockElems;
}

extern "C" int nmb_adamw_step(const void* table_dev, int n_tensors, long long total_blocks, const float* hyper,
                              int* step_count, void* stream) {
  if (n_tensors <= 0 || total_blocks <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  adamw_kernel<<<static_cast<unsigned>(total_blocks), kAdamThreads, 0, s>>>(
      static_cast<const AdamTensor*>(table_dev), n_tensors, hyper, step_count);
  adamw_advance_kernel<<<1, 1, 0, s>>>(step_count);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + e;
}
