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
  for (int i = threadIdx.x; i < kAdamBlockElems; i += kAdamThreads) {
    const long long idx = base + i;
    if (idx >= t.numel) break;
    const float g = t.grad_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(t.grad)[idx])
                                : static_cast<const float*>(t.grad)[idx];
    float w = t.param_bf16 ? __bfloat162float(static_cast<__nv_bfloat16*>(t.param)[idx])
                           : static_cast<float*>(t.param)[idx];
    if (wd != 0.f) w *= decay;
    const float m = t.exp_avg[idx] * b1 + g * (1.f - b1);
    const float v = t.exp_avg_sq[idx] * b2 + g * g * (1.f - b2);
    t.exp_avg[idx] = m;
    t.exp_avg_sq[idx] = v;
    const float denom = sqrtf(v) * inv_sqrt_corr2 + eps;
    w -= step_size * (m / denom);
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
