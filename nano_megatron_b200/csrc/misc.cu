// Small memory-bound kernels: embedding gather / scatter-add (vocabulary
// sharded), GELU / SwiGLU forward and backward, rotary embedding, and the
// loss-scaling helpers.  They replace the ATen elementwise chains of the
// reference (nano_megatron/reference/layers.py:38-81,
// nano_megatron/parallel/vocab_parallel.py:86-100).
#include "common.cuh"

namespace nmb {

// out[n, :] = tok[id - vocab_start] (zero when the id is not in this shard) + pos[position]
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const long long* __restrict__ positions,
                                     const __nv_bfloat16* __restrict__ tok, const __nv_bfloat16* __restrict__ pos,
                                     __nv_bfloat16* __restrict__ out, int n, int H, int vocab_start, int vloc) {
  const int row = blockIdx.x;
  if (row >= n) return;
  const long long id = ids[row] - vocab_start;
  const bool own = id >= 0 && id < vloc;
  const __nv_bfloat162* tr = own ? reinterpret_cast<const __nv_bfloat162*>(tok + id * H) : nullptr;
  const __nv_bfloat162* pr =
      pos != nullptr ? reinterpret_cast<const __nv_bfloat162*>(pos + positions[row] * H) : nullptr;
  __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(out + static_cast<size_t>(row) * H);
  for (int i = threadIdx.x; i < H / 2; i += blockDim.x) {
    float2 v = make_float2(0.f, 0.f);
    if (own) v = __bfloat1622float2(tr[i]);
    if (pr != nullptr) {
      const float2 q = __bfloat1622float2(pr[i]);
      v.x += q.x;
      v.y += q.y;
    }
    o[i] = __floats2bfloat162_rn(v.x, v.y);
  }
}

// dtok[id - vocab_start] += dy[n] (owned ids only) ; dpos[position] += dy[n]
__global__ void embedding_bwd_kernel(const long long* __restrict__ ids, const long long* __restrict__ positions,
                                     const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dtok,
                                     __nv_bfloat16* __restrict__ dpos, int n, int H, int vocab_start, int vloc) {
  const int row = blockIdx.x;
  if (row >= n) return;
  const long long id = ids[row] - vocab_start;
  const bool own = dtok != nullptr && id >= 0 && id < vloc;
  const __nv_bfloat162* g = reinterpret_cast<const __nv_bfloat162*>(dy + static_cast<size_t>(row) * H);
  __nv_bfloat162* tr = own ? reinterpret_cast<__nv_bfloat162*>(dtok + id * H) : nullptr;
  __nv_bfloat162* pr = dpos != nullptr ? reinterpret_cast<__nv_bfloat162*>(dpos + positions[row] * H) : nullptr;
  for (int i = threadIdx.x; i < H / 2; i += blockDim.x) {
    const __nv_bfloat162 v = g[i];
    if (own) atomicAdd(tr + i, v);
    if (pr != nullptr) atomicAdd(pr + i, v);
  }
}

__global__ void gelu_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n2) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n2) return;
  const float2 v = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(x)[i]);
  reinterpret_cast<__nv_bfloat162*>(y)[i] = __floats2bfloat162_rn(gelu_erf_f(v.x), gelu_erf_f(v.y));
}

__global__ void gelu_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                __nv_bfloat16* __restrict__ dx, long long n2) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n2) return;
  const float2 v = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(x)[i]);
  const float2 g = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(dy)[i]);
  reinterpret_cast<__nv_bfloat162*>(dx)[i] =
      __floats2bfloat162_rn(g.x * gelu_erf_grad_f(v.x), g.y * gelu_erf_grad_f(v.y));
}

// x = [gate | up] per row (each F wide); y = silu(gate) * up
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long long rows,
                                  int F) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long half = F / 2;
  if (i >= rows * half) return;
  const long long r = i / half;
  const int c = i % half;
  const float2 g = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(x + r * 2 * F)[c]);
  const float2 u = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(x + r * 2 * F + F)[c]);
  const float s0 = g.x / (1.f + __expf(-g.x)), s1 = g.y / (1.f + __expf(-g.y));
  reinterpret_cast<__nv_bfloat162*>(y + r * F)[c] = __floats2bfloat162_rn(s0 * u.x, s1 * u.y);
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                  __nv_bfloat16* __restrict__ dx, long long rows, int F) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long half = F / 2;
  if (i >= rows * half) return;
  const long long r = i / half;
  const int c = i % half;
  const float2 g = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(x + r * 2 * F)[c]);
  const float2 u = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(x + r * 2 * F + F)[c]);
  const float2 d = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(dy + r * F)[c]);
  const float sg0 = 1.f / (1.f + __expf(-g.x)), sg1 = 1.f / (1.f + __expf(-g.y));
  const float dg0 = d.x * u.x * sg0 * (1.f + g.x * (1.f - sg0));
  const float dg1 = d.y * u.y * sg1 * (1.f + g.y * (1.f - sg1));
  reinterpret_cast<__nv_bfloat162*>(dx + r * 2 * F)[c] = __floats2bfloat162_rn(dg0, dg1);
  reinterpret_cast<__nv_bfloat162*>(dx + r * 2 * F + F)[c] = __floats2bfloat162_rn(d.x * g.x * sg0, d.y * g.y * sg1);
}

// In-place rotation of interleaved pairs of a [B, S, heads, d] view.
// angle = positions[b, s] * inv_freq[i]; `sign` = +1 forward, -1 backward.
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, long long sb, long long ss, long long sh,
                            const long long* __restrict__ positions, const float* __restrict__ inv_freq, int B,
                            int S, int heads, int d, float sign) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int half = d / 2;
  const long long total = static_cast<long long>(B) * S * heads * half;
  if (i >= total) return;
  const int pi = i % half;
  long long t = i / half;
  const int h = t % heads;
  t /= heads;
  const int s = t % S;
  const int b = t / S;
  const float ang = static_cast<float>(positions[static_cast<long long>(b) * S + s]) * inv_freq[pi];
  float sn, cs;
  sincosf(ang, &sn, &cs);
  sn *= sign;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(x + b * sb + s * ss + h * sh) + pi;
  const float2 v = __bfloat1622float2(*p);
  *p = __floats2bfloat162_rn(v.x * cs - v.y * sn, v.x * sn + v.y * cs);
}

// y = a * alpha[0] ; used for device-side loss scaling without a host sync
__global__ void scale_by_device_scalar_kernel(float* __restrict__ y, const float* __restrict__ num,
                                              const float* __restrict__ den, float mul) {
  // y[0] = num[0] / max(den[0], 1) * mul
  const float d = den[0] > 0.f ? den[0] : 1.f;
  y[0] = num[0] / d * mul;
}

}  // namespace nmb

using namespace nmb;

#define NMB_LAUNCH_CHECK()                      \
  do {                                          \
    cudaError_t e = cudaGetLastError();         \
    return e == cudaSuccess ? 0 : 400 + e;      \
  } while (0)

extern "C" int nmb_embedding_fwd(const long long* ids, const long long* positions, const void* tok, const void* pos,
                                 void* out, int n, int H, int vocab_start, int vloc, void* stream) {
  if (n <= 0) return 0;
  if (H % 2) return kBadArgument;
  embedding_fwd_kernel<<<n, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      ids, positions, static_cast<const __nv_bfloat16*>(tok), static_cast<const __nv_bfloat16*>(pos),
      static_cast<__nv_bfloat16*>(out), n, H, vocab_start, vloc);
  NMB_LAUNCH_CHECK();
}

extern "C" int nmb_embedding_bwd(const long long* ids, const long long* positions, const void* dy, void* dtok,
                                 void* dpos, int n, int H, int vocab_start, int vloc, void* stream) {
  if (n <= 0) return 0;
  if (H % 2) return kBadArgument;
  embedding_bwd_kernel<<<n, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      ids, positions, static_cast<const __nv_bfloat16*>(dy), static_cast<__nv_bfloat16*>(dtok),
      static_cast<__nv_bfloat16*>(dpos), n, H, vocab_start, vloc);
  NMB_LAUNCH_CHECK();
}

extern "C" int nmb_gelu_fwd(const void* x, void* y, long long n, void* stream) {
  if (n <= 0) return 0;
  if (n % 2) return kBadArgument;
  const long long n2 = n / 2;
  gelu_fwd_kernel<<<static_cast<unsigned>((n2 + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), n2);
  NMB_LAUNCH_CHECK();
}

extern "C" int nmb_gelu_bwd(const void* x, const void* dy, void* dx, long long n, void* stream) {
  if (n <= 0) return 0;
  if (n % 2) return kBadArgument;
  const long long n2 = n / 2;
  gelu_bwd_kernel<<<static_cast<unsigned>((n2 + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy), static_cast<__nv_bfloat16*>(dx), n2);
  NMB_LAUNCH_CHECK();
}

extern "C" int nmb_swiglu_fwd(const void* x, void* y, long long rows, int F, void* stream) {
  if (rows <= 0) return 0;
  if (F % 2) return kBadArgument;
  const long long n = rows * (F / 2);
  swiglu_fwd_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), rows, F);
  NMB_LAUNCH_CHECK();
}

extern "C" int nmb_swiglu_bwd(const void* x, const void* dy, void* dx, long long rows, int F, void* stream) {
  if (rows <= 0) return 0;
  if (F % 2) return kBadArgument;
  const long long n = rows * (F / 2);
  swiglu_bwd_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy), static_cast<__nv_bfloat16*>(dx), rows, F);
  NMB_LAUNCH_CHECK();
}

extern "C" int nmb_rope(void* x, long long sb, long long ss, long long sh, const long long* positions,
                        const float* inv_freq, int B, int S, int heads, int d, float sign, void* stream) {
  const long long n = static_cast<long long>(B) * S * heads * (d / 2);
  if (n <= 0) return 0;
  rope_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(x), sb, ss, sh, positions, inv_freq, B, S, heads, d, sign);
  NMB_LAUNCH_CHECK();
}

extern "C" int nmb_scalar_ratio(float* y, const float* num, const float* den, float mul, void* stream) {
  scale_by_device_scalar_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(y, num, den, mul);
  NMB_LAUNCH_CHECK();
}

// 1: the GEMM, attention, norm and column-sum kernels are launched with
// programmatic stream serialization (see pdl_wait in common.cuh); 0: plain
// stream order for every kernel.
extern "C" void nmb_set_pdl(int enabled) { nmb::g_pdl_enabled = enabled ? 1 : 0; }

