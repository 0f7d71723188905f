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

// ---------------------------------------------------------------------------
// Forward in ONE launch, with the cross-rank exchange inside the kernel.
//
// The reference's vocabulary-parallel CE issues three all-reduces of [tokens]
// (max, target logit, sum-exp: nano_megatron/parallel/vocab_parallel.py:118-140).
// Here one block per token row reads its logits ONCE (online max / sum-exp:
// the running sum is rescaled when the maximum grows), thread 0 stores the
// row's triple straight into slot [my rank] of every rank's gather buffer (peer
// stores), and the last block of the grid to finish -- on every rank -- raises a
// flag on the peers, waits (bounded) for theirs, and combines all ranks' triples
// of all rows into the log-sum-exp per row, the loss sum and the token count.
// With one rank the exchange disappears and the same kernel is the plain CE.
//
// The gather buffer is one of two, picked by the parity of a device-side epoch
// that the last block advances: a rank that has finished call k may already be
// storing call k+1's triples while a slower peer still combines call k, and it
// cannot reach call k+2 before that peer has raised its flag for k+1.
struct CeComm {
  float4* gathered[2][kMaxRanks];  // per parity, per rank: [n_ranks][rows]
  uint32_t* flags[kMaxRanks];      // per rank: [kMaxRanks] "rank r has stored every row of this epoch"
  uint32_t* sync;                  // [0] epoch of the last finished call, [1] blocks of this call that are done
  int rank, n_ranks;
  long long budget;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
  const float mm = fmaxf(m, m2);
  // exp(-inf - -inf) would be NaN: an empty partner contributes nothing
  const float a = (m == -INFINITY) ? 0.f : s * __expf(m - mm);
  const float b = (m2 == -INFINITY) ? 0.f : s2 * __expf(m2 - mm);
  m = mm;
  s = a + b;
}

__global__ void __launch_bounds__(kCeThreads)
ce_forward_fused_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, const long long* __restrict__ target,
                        int vocab_start, int vloc, int ignore_index, const __grid_constant__ CeComm cc,
                        float* __restrict__ lse, float* __restrict__ accum, int rows, int* status) {
  __shared__ float sm[32], ss[32];
  __shared__ int is_last;
  __shared__ uint32_t epoch_s;
  const int row = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) epoch_s = cc.sync[0] + 1;
  const __nv_bfloat16* x = logits + row * ld;
  const bool vec = (vloc % 8 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
  float m = -INFINITY, s = 0.f;
  if (vec) {
    // Four independent 16-byte loads in flight per thread (one row is ~100 KB and
    // the kernel is otherwise bound by load latency), then one FFMA + ex2 per
    // element: exp(f - m) = 2^(f * log2e - m * log2e).
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    const int nvec = vloc / 8;
    const int step = blockDim.x;
    constexpr float kLog2e = 1.4426950408889634f;
    float ml = -INFINITY;  // m * log2e
    auto take = [&](const uint4& u) {
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
      float f[8];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 p = unpack_bf16x2(w[t]);
        f[2 * t] = p.x;
        f[2 * t + 1] = p.y;
      }
      float m8 = f[0];
#pragma unroll
      for (int t = 1; t < 8; ++t) m8 = fmaxf(m8, f[t]);
      if (m8 > m) {
        s *= fast_exp2(ml - m8 * kLog2e);  // m == -inf: s is 0 and 2^(-inf) = 0
        m = m8;
        ml = m8 * kLog2e;
      }
#pragma unroll
      for (int t = 0; t < 8; ++t) s += fast_exp2(fmaf(f[t], kLog2e, -ml));
    };
    int i = threadIdx.x;
    for (; i + 3 * step < nvec; i += 4 * step) {
      uint4 u[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) u[j] = xv[i + j * step];
#pragma unroll
      for (int j = 0; j < 4; ++j) take(u[j]);
    }
    for (; i < nvec; i += step) take(xv[i]);
  } else {
    for (int i = threadIdx.x; i < vloc; i += blockDim.x) {
      const float v = __bfloat162float(x[i]);
      if (v > m) {
        s *= __expf(m - v);
        m = v;
      }
      s += __expf(v - m);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
    online_merge(m, s, m2, s2);
  }
  if (lane == 0) {
    sm[warp] = m;
    ss[warp] = s;
  }
  __syncthreads();
  const uint32_t e = epoch_s;
  float4* const* gathered = cc.gathered[e & 1];
  if (threadIdx.x == 0) {
    for (int w = 1; w < (blockDim.x >> 5); ++w) online_merge(m, s, sm[w], ss[w]);
    const long long t = target[row] - vocab_start;
    const float tl = (t >= 0 && t < vloc) ? __bfloat162float(x[t]) : 0.f;
    const float4 triple = make_float4(m, s, tl, 0.f);
    for (int p = 0; p < cc.n_ranks; ++p)
      gathered[(cc.rank + p) % cc.n_ranks][static_cast<size_t>(cc.rank) * rows + row] = triple;
    __threadfence_system();
    const unsigned done = atomicAdd(&cc.sync[1], 1u);
    is_last = done == gridDim.x - 1;
  }
  __syncthreads();
  if (!is_last) return;

  // ---- last block of this rank: exchange flags, then combine every row ----
  __shared__ int ok_s;
  if (threadIdx.x == 0) {
    cc.sync[1] = 0;
    cc.sync[0] = e;
    ok_s = 1;
    __threadfence_system();
  }
  __syncthreads();
  if (cc.n_ranks > 1 && threadIdx.x < cc.n_ranks && static_cast<int>(threadIdx.x) != cc.rank) {
    st_release_sys(cc.flags[threadIdx.x] + cc.rank, e);
    if (!wait_flag_sys(cc.flags[cc.rank] + threadIdx.x, e, cc.budget)) {
      report_status(status, kPeerTimeout, 21);
      ok_s = 0;
    }
  }
  __syncthreads();
  float my_loss = 0.f, my_cnt = 0.f;
  if (ok_s) {
    const float4* mine = gathered[cc.rank];
    for (int r = threadIdx.x; r < rows; r += blockDim.x) {
      float gm = -INFINITY;
      for (int p = 0; p < cc.n_ranks; ++p) gm = fmaxf(gm, mine[static_cast<size_t>(p) * rows + r].x);
      float se = 0.f, tl = 0.f;
      for (int p = 0; p < cc.n_ranks; ++p) {
        const float4 t4 = mine[static_cast<size_t>(p) * rows + r];
        se += t4.y * __expf(t4.x - gm);
        tl += t4.z;
      }
      const float l = gm + logf(se);
      lse[r] = l;
      if (target[r] != ignore_index) {
        my_loss += l - tl;
        my_cnt += 1.f;
      }
    }
  }
  const float tot = block_reduce(my_loss, false, sm);
  const float cnt = block_reduce(my_cnt, false, ss);
  if (threadIdx.x == 0) {
    accum[0] = tot;
    accum[1] = cnt;
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

// One-launch forward (see CeComm).  `comm` has the layout of nmb::CeComm; with
// n_ranks == 1 only gathered[*][0] (a local [rows] float4 scratch) is used.
extern "C" int nmb_ce_forward_fused(const void* logits, long long ld, const long long* target, int vocab_start,
                                    int vloc, int ignore_index, const void* comm, float* lse, float* accum, int rows,
                                    int* status, void* stream) {
  if (rows <= 0) return 0;
  const nmb::CeComm* cc = static_cast<const nmb::CeComm*>(comm);
  if (cc->n_ranks < 1 || cc->n_ranks > kMaxRanks) return kBadArgument;
  ce_forward_fused_kernel<<<rows, kCeThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(logits), ld, target, vocab_start, vloc, ignore_index, *cc, lse, accum, rows,
      status);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + e;
}

extern "C" int nmb_ce_comm_size() { return static_cast<int>(sizeof(nmb::CeComm)); }

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
