// Peer-memory collectives over NVLink / NVSwitch: kernels that read and write
// other GPUs' buffers directly (symmetric allocations exchanged through CUDA
// IPC) and synchronise through flags in a symmetric "signal pad".
//
// They replace NCCL calls of the reference where a collective is fused with
// arithmetic: the bucketed gradient all-reduce + divide of its DDP
// (nano_megatron/distributed/bucket.py:85-100) becomes one kernel that reads the
// peers' buckets, sums in fp32, scales by 1/(dp*cp) and writes the result.
//
// Synchronisation.  A signal pad is `kChannels x kMaxBlocks x kMaxRanks` 32-bit
// flags per rank.  Block b of a kernel on channel c signals by storing its
// epoch into slot [c][b][my_rank] of every peer's pad and waits until its own
// pad's slots [c][b][*] have reached that epoch.  The epoch of (c, b) lives in
// device memory owned by that block, so a replayed CUDA graph keeps counting.
// All ranks of a group must launch the same kernels on a channel in the same
// order.  Every wait is bounded; a timed-out wait stores kPeerTimeout in the
// status word and the block stops touching peer memory.
//
// Only plain peer loads / stores are used (no multimem, no TMA multicast).
#include "common.cuh"

#include <string.h>

namespace nmb {

struct PeerPtrs {
  void* p[kMaxRanks];
};

// Block-level barrier with the same block index on every rank of the group.
// `budget` in clock cycles.  Returns false (for the whole block) on a timeout.
__device__ bool block_barrier(const PeerPtrs& pads, int channel, int rank, int n, uint32_t epoch, int* status,
                              long long budget, int where) {
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();  // the block's earlier writes are ordered before the signal
  if (threadIdx.x < n) {
    __threadfence_system();
    st_release_sys(pad_slot(pads.p[threadIdx.x], channel, blockIdx.x, rank), epoch);
    const uint32_t* mine = pad_slot(pads.p[rank], channel, blockIdx.x, threadIdx.x);
    const long long t0 = clock64();
    // epochs only grow; compare as signed distance so wrap-around is harmless
    while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
      if (clock64() - t0 > budget) {
        report_status(status, kPeerTimeout, where);
        failed = 1;
        break;
      }
    }
  }
  __syncthreads();
  const bool ok = failed == 0;
  __syncthreads();  // `failed` is reused by the next barrier of this block
  return ok;
}

template <typename T>
struct Vec16;
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int kElems = 8;
  static __device__ __forceinline__ void add(float* acc, const uint4& u) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = unpack_bf16x2(w[k]);
      acc[2 * k] += f.x;
      acc[2 * k + 1] += f.y;
    }
  }
  static __device__ __forceinline__ uint4 pack(const float* acc, float scale) {
    uint4 o;
    o.x = pack_bf16x2(acc[0] * scale, acc[1] * scale);
    o.y = pack_bf16x2(acc[2] * scale, acc[3] * scale);
    o.z = pack_bf16x2(acc[4] * scale, acc[5] * scale);
    o.w = pack_bf16x2(acc[6] * scale, acc[7] * scale);
    return o;
  }
};
template <>
struct Vec16<float> {
  static constexpr int kElems = 4;
  static __device__ __forceinline__ void add(float* acc, const uint4& u) {
    acc[0] += __uint_as_float(u.x);
    acc[1] += __uint_as_float(u.y);
    acc[2] += __uint_as_float(u.z);
    acc[3] += __uint_as_float(u.w);
  }
  static __device__ __forceinline__ uint4 pack(const float* acc, float scale) {
    return make_uint4(__float_as_uint(acc[0] * scale), __float_as_uint(acc[1] * scale),
                      __float_as_uint(acc[2] * scale), __float_as_uint(acc[3] * scale));
  }
};

// In-place all-reduce (sum) * scale of a symmetric buffer, two-shot:
//   block b owns the b-th slice of the buffer on every rank; inside it rank r
//   reduces the r-th sub-slice (reading all peers), then every rank copies the
//   other ranks' reduced sub-slices.  Dependencies therefore stay between
//   blocks of equal index, which is what `block_barrier` synchronises.
//   U = independent 16-byte loads in flight per thread (NVLink latency is ~2 us).
template <typename T, int U>
__device__ __forceinline__ void allreduce_scale_body(const PeerPtrs& bufs, const PeerPtrs& pads, uint32_t* epochs,
                                                     int channel, int rank, int n, long long n_vec, float scale,
                                                     int* status, long long budget) {
  using V = Vec16<T>;
  __shared__ uint32_t epoch_s;
  uint32_t* my_epoch = epochs + channel * kMaxBlocks + blockIdx.x;
  if (threadIdx.x == 0) epoch_s = *my_epoch;
  __syncthreads();
  const uint32_t e0 = epoch_s;
  const long long per_block = (n_vec + gridDim.x - 1) / gridDim.x;
  const long long blk_lo = per_block * blockIdx.x;
  long long blk_hi = blk_lo + per_block;
  if (blk_hi > n_vec) blk_hi = n_vec;
  const long long blk_len = blk_hi > blk_lo ? blk_hi - blk_lo : 0;
  const long long per_rank = (blk_len + n - 1) / n;

  bool ok = block_barrier(pads, channel, rank, n, e0 + 1, status, budget, 61);  // peers' inputs are ready
  if (ok) {
    const long long lo = blk_lo + per_rank * rank;
    long long hi = lo + per_rank;
    if (hi > blk_hi) hi = blk_hi;
    uint4* mine = static_cast<uint4*>(bufs.p[rank]);
    for (long long base = lo + threadIdx.x; base < hi; base += static_cast<long long>(blockDim.x) * U) {
      float acc[U][V::kElems];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int k = 0; k < V::kElems; ++k) acc[u][k] = 0.f;
#pragma unroll 1
      for (int k = 0; k < n; ++k) {
        const uint4* src = static_cast<const uint4*>(bufs.p[(rank + k) % n]);  // start at home, spread the peers
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = base + static_cast<long long>(u) * blockDim.x;
          v[u] = i < hi ? src[i] : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) V::add(acc[u], v[u]);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = base + static_cast<long long>(u) * blockDim.x;
        if (i < hi) mine[i] = V::pack(acc[u], scale);
      }
    }
  }
  ok = ok && block_barrier(pads, channel, rank, n, e0 + 2, status, budget, 62);  // all sub-slices reduced
  if (ok) {
    uint4* mine = static_cast<uint4*>(bufs.p[rank]);
    for (int k = 1; k < n; ++k) {
      const int src = (rank + k) % n;
      const long long lo = blk_lo + per_rank * src;
      long long hi = lo + per_rank;
      if (hi > blk_hi) hi = blk_hi;
      const uint4* theirs = static_cast<const uint4*>(bufs.p[src]);
      for (long long base = lo + threadIdx.x; base < hi; base += static_cast<long long>(blockDim.x) * U) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = base + static_cast<long long>(u) * blockDim.x;
          if (i < hi) v[u] = theirs[i];
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = base + static_cast<long long>(u) * blockDim.x;
          if (i < hi) mine[i] = v[u];
        }
      }
    }
  }
  // nobody may overwrite a buffer a peer is still copying from
  block_barrier(pads, channel, rank, n, e0 + 3, status, budget, 63);
  if (threadIdx.x == 0) *my_epoch = e0 + 3;
}

// Latency-first variant: 512 threads, 8 loads in flight each; it fills the SMs
// it runs on, so nothing else shares them.
template <typename T>
__global__ void __launch_bounds__(512)
allreduce_scale_kernel(const __grid_constant__ PeerPtrs bufs, const __grid_constant__ PeerPtrs pads, uint32_t* epochs, int channel, int rank, int n,
                       long long n_vec, float scale, int* status, long long budget) {
  allreduce_scale_body<T, 8>(bufs, pads, epochs, channel, rank, n, n_vec, scale, status, budget);
}

// Overlap-first variant for gradient buckets reduced during backward.  A block
// must fit beside a resident persistent GEMM CTA (10 warps x 144 registers)
// instead of waiting for, or displacing, it.  The register file is split over
// the four SM sub-partitions (16 K registers each) and warps are dealt to them
// round-robin, so the GEMM's 10 warps leave 16384 - 3 * 4608 = 2560 registers
// on the fullest sub-partitions: room for ONE more warp of at most 80
// registers per thread there, i.e. a block of 4 warps.
constexpr int kLightThreads = 128;
template <typename T>
__global__ void __maxnreg__(80)
allreduce_scale_light_kernel(const __grid_constant__ PeerPtrs bufs, const __grid_constant__ PeerPtrs pads, uint32_t* epochs, int channel, int rank, int n,
                             long long n_vec, float scale, int* status, long long budget) {
  allreduce_scale_body<T, 4>(bufs, pads, epochs, channel, rank, n, n_vec, scale, status, budget);
}

// ---------------------------------------------------------------------------
// In-switch all-reduce (NVLS): the buffer is mapped at the same offset of a
// multicast address on every rank.  `multimem.ld_reduce` on that address makes
// the NVSwitch read the element from all ranks and return the sum (accumulated
// in fp32), `multimem.st` writes a value to all ranks at once.  Block b owns the
// b-th slice of the buffer, inside it rank r reduces and broadcasts the r-th
// sub-slice: every element crosses this GPU's links once in and once out,
// instead of (n-1)/n of the buffer twice with peer loads, and a thread issues
// one load and one store per 16 bytes whatever the number of ranks.  The flag
// rounds before and after are the plain peer-memory ones (`block_barrier`).
// This is multicast *addressing* for reductions; no TMA or bulk load with
// cluster multicast is involved.
template <typename T>
struct Multimem;
template <>
struct Multimem<__nv_bfloat16> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc)
                 : "memory");
    return v;
  }
  static __device__ __forceinline__ uint4 scale(const uint4& v, float s) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = unpack_bf16x2(w[k]);
      o[k] = pack_bf16x2(f.x * s, f.y * s);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
  }
};
template <>
struct Multimem<float> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc)
                 : "memory");
    return v;
  }
  static __device__ __forceinline__ uint4 scale(const uint4& v, float s) {
    return make_uint4(__float_as_uint(__uint_as_float(v.x) * s), __float_as_uint(__uint_as_float(v.y) * s),
                      __float_as_uint(__uint_as_float(v.z) * s), __float_as_uint(__uint_as_float(v.w) * s));
  }
};
__device__ __forceinline__ void multimem_st(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

template <typename T, int U>
__device__ __forceinline__ void multimem_allreduce_body(uint8_t* mc, const PeerPtrs& pads, uint32_t* epochs, int channel,
                                                        int rank, int n, long long n_vec, float scale, int* status,
                                                        long long budget) {
  __shared__ uint32_t epoch_s;
  uint32_t* my_epoch = epochs + channel * kMaxBlocks + blockIdx.x;
  if (threadIdx.x == 0) epoch_s = *my_epoch;
  __syncthreads();
  const uint32_t e0 = epoch_s;
  const long long per_block = (n_vec + gridDim.x - 1) / gridDim.x;
  const long long blk_lo = per_block * blockIdx.x;
  long long blk_hi = blk_lo + per_block;
  if (blk_hi > n_vec) blk_hi = n_vec;
  const long long blk_len = blk_hi > blk_lo ? blk_hi - blk_lo : 0;
  const long long per_rank = (blk_len + n - 1) / n;
  bool ok = block_barrier(pads, channel, rank, n, e0 + 1, status, budget, 71);  // every rank's input is ready
  if (ok) {
    const long long lo = blk_lo + per_rank * rank;
    long long hi = lo + per_rank;
    if (hi > blk_hi) hi = blk_hi;
    for (long long base = lo + threadIdx.x; base < hi; base += static_cast<long long>(blockDim.x) * U) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = base + static_cast<long long>(u) * blockDim.x;
        if (i < hi) v[u] = Multimem<T>::ld_reduce(mc + i * 16);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = base + static_cast<long long>(u) * blockDim.x;
        if (i < hi) multimem_st(mc + i * 16, Multimem<T>::scale(v[u], scale));
      }
    }
  }
  // every rank's sub-slice has been written everywhere (and nobody still reads the inputs)
  block_barrier(pads, channel, rank, n, e0 + 2, status, budget, 72);
  if (threadIdx.x == 0) *my_epoch = e0 + 2;
}

template <typename T>
__global__ void __launch_bounds__(512)
multimem_allreduce_kernel(uint8_t* mc, const __grid_constant__ PeerPtrs pads, uint32_t* epochs, int channel, int rank,
                          int n, long long n_vec, float scale, int* status, long long budget) {
  multimem_allreduce_body<T, 4>(mc, pads, epochs, channel, rank, n, n_vec, scale, status, budget);
}

// Overlap-first variant (see allreduce_scale_light_kernel for the sizing).
template <typename T>
__global__ void __maxnreg__(80)
multimem_allreduce_light_kernel(uint8_t* mc, const __grid_constant__ PeerPtrs pads, uint32_t* epochs, int channel,
                                int rank, int n, long long n_vec, float scale, int* status, long long budget) {
  multimem_allreduce_body<T, 4>(mc, pads, epochs, channel, rank, n, n_vec, scale, status, budget);
}

// All-gather through peer stores: every rank writes its `n_vec` 16-byte vectors
// into slot [rank] of every rank's `[n][n_vec]` destination, then the blocks of
// equal index meet in a barrier.  Small-message replacement for NCCL
// all-gather (CE statistics, sequence-parallel replicated-parameter grads,
// embedding gradients) that can sit inside a captured CUDA graph.
__global__ void __launch_bounds__(512)
peer_allgather_kernel(const uint4* __restrict__ src, PeerPtrs dst, PeerPtrs pads, uint32_t* epochs, int channel,
                      int rank, int n, long long n_vec, int* status, long long budget) {
  __shared__ uint32_t epoch_s;
  uint32_t* my_epoch = epochs + channel * kMaxBlocks + blockIdx.x;
  if (threadIdx.x == 0) epoch_s = *my_epoch;
  __syncthreads();
  const uint32_t e0 = epoch_s;
  const long long per_block = (n_vec + gridDim.x - 1) / gridDim.x;
  const long long lo = per_block * blockIdx.x;
  long long hi = lo + per_block;
  if (hi > n_vec) hi = n_vec;
  for (int k = 0; k < n; ++k) {
    uint4* out = static_cast<uint4*>(dst.p[(rank + k) % n]) + static_cast<long long>(rank) * n_vec;
    for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) out[i] = src[i];
  }
  block_barrier(pads, channel, rank, n, e0 + 1, status, budget, 66);
  if (threadIdx.x == 0) *my_epoch = e0 + 1;
}

// Vocabulary-parallel embedding without a reduction: every token's row has
// exactly one producer (the rank that owns its vocabulary id), which writes
// token + position embedding straight into the output buffers of the ranks that
// need the row -- the owner of the token's sequence shard (sequence parallel,
// `to_all == 0`, output `[B * S/ranks, H]`) or every rank (`to_all != 0`,
// output `[B * S, H]`).
__global__ void embedding_scatter_kernel(const long long* __restrict__ ids, const long long* __restrict__ positions,
                                         const __nv_bfloat16* __restrict__ tok, const __nv_bfloat16* __restrict__ pos,
                                         PeerPtrs out, int n_ranks, int n_tokens, int H, int vocab_start, int vloc,
                                         int seq_len, int shard_len, int to_all) {
  const int row = blockIdx.x;
  if (row >= n_tokens) return;
  const long long id = ids[row] - vocab_start;
  if (id < 0 || id >= vloc) return;
  const int s = row % seq_len;
  const int owner = s / shard_len;
  const long long local = to_all ? row : static_cast<long long>(row / seq_len) * shard_len + s % shard_len;
  const uint4* tr = reinterpret_cast<const uint4*>(tok + id * H);
  const uint4* pr = pos != nullptr ? reinterpret_cast<const uint4*>(pos + positions[row] * H) : nullptr;
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
    uint4 v = tr[i];
    if (pr != nullptr) {
      const uint4 q = pr[i];
      const uint32_t a[4] = {v.x, v.y, v.z, v.w};
      const uint32_t b[4] = {q.x, q.y, q.z, q.w};
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 x = unpack_bf16x2(a[k]);
        const float2 y = unpack_bf16x2(b[k]);
        o[k] = pack_bf16x2(x.x + y.x, x.y + y.y);
      }
      v = make_uint4(o[0], o[1], o[2], o[3]);
    }
    if (to_all) {
      for (int r = 0; r < n_ranks; ++r)
        reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(out.p[r]) + local * H)[i] = v;
    } else {
      reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(out.p[owner]) + local * H)[i] = v;
    }
  }
}

// Context-parallel attention backward, owner side: dK and dV of this rank's
// key/value shard are the sums of the contributions of every rank that can see
// the shard (ranks `first` .. n-1; each stored its tiles into slot [its rank] of
// this rank's staging buffers from inside its attention-backward kernel).  One
// launch: blocks of equal index on all ranks meet in a flag round (a rank gets
// here only after its attention backward has finished, so all contributions
// have been stored), then every block sums its share of the slots in fp32, in
// slot order, and writes bf16 results to the (strided) gradient tensors.  With a
// rotary table dK is un-rotated on the way out.  This replaces the reference's
// reduce-scatter of the gathered dK / dV
// (nano_megatron/parallel/context_parallel.py:175-181).
__device__ __forceinline__ void unrope8_bf(float (&x)[8], const float2* table, long long pos, int half, int pair0) {
  const float4* tp = reinterpret_cast<const float4*>(table + pos * half + pair0);
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    const float4 cs = __ldg(tp + q);
    const float a0 = x[4 * q], a1 = x[4 * q + 1], b0 = x[4 * q + 2], b1 = x[4 * q + 3];
    x[4 * q] = a0 * cs.x + a1 * cs.y;
    x[4 * q + 1] = -a0 * cs.y + a1 * cs.x;
    x[4 * q + 2] = b0 * cs.z + b1 * cs.w;
    x[4 * q + 3] = -b0 * cs.w + b1 * cs.z;
  }
}

__global__ void __launch_bounds__(256)
cp_dkv_reduce_kernel(const __nv_bfloat16* __restrict__ stage_k, const __nv_bfloat16* __restrict__ stage_v,
                     __nv_bfloat16* __restrict__ out_k, __nv_bfloat16* __restrict__ out_v, long long out_sb,
                     long long out_ss, long long out_sh, int B, int S, int H, int d, int first, PeerPtrs pads,
                     uint32_t* epochs, int channel, int rank, int n, const float2* __restrict__ rope_table,
                     const long long* __restrict__ rope_pos, int* status, long long budget) {
  __shared__ uint32_t epoch_s;
  uint32_t* my_epoch = epochs + channel * kMaxBlocks + blockIdx.x;
  if (threadIdx.x == 0) epoch_s = *my_epoch;
  __syncthreads();
  const bool ok = block_barrier(pads, channel, rank, n, epoch_s + 1, status, budget, 67);
  if (threadIdx.x == 0) *my_epoch = epoch_s + 1;
  if (!ok) return;
  const int per_row = d / 8;
  const long long slot_vecs = static_cast<long long>(B) * S * H * per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < 2 * slot_vecs;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const bool is_v = i >= slot_vecs;
    const long long j = is_v ? i - slot_vecs : i;
    const uint4* stage = reinterpret_cast<const uint4*>(is_v ? stage_v : stage_k);
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    for (int slot = first; slot < n; ++slot) Vec16<__nv_bfloat16>::add(acc, stage[slot * slot_vecs + j]);
    const int c8 = static_cast<int>(j % per_row);
    const long long row = j / per_row;  // (b * S + s) * H + h
    const int h = row % H;
    const long long bs = row / H;
    if (!is_v && rope_table != nullptr) unrope8_bf(acc, rope_table, rope_pos[bs], d / 2, c8 * 4);
    __nv_bfloat16* dst = (is_v ? out_v : out_k) + (bs / S) * out_sb + (bs % S) * out_ss + h * out_sh + c8 * 8;
    *reinterpret_cast<uint4*>(dst) = Vec16<__nv_bfloat16>::pack(acc, 1.f);
  }
}

// Stand-alone barrier (one block), e.g. "my buffer is published" between kernels.
__global__ void barrier_kernel(PeerPtrs pads, uint32_t* epochs, int channel, int rank, int n, int* status,
                               long long budget) {
  __shared__ uint32_t epoch_s;
  uint32_t* my_epoch = epochs + channel * kMaxBlocks + blockIdx.x;
  if (threadIdx.x == 0) epoch_s = *my_epoch;
  __syncthreads();
  block_barrier(pads, channel, rank, n, epoch_s + 1, status, budget, 64);
  if (threadIdx.x == 0) *my_epoch = epoch_s + 1;
}

// Waits for a flag that nobody sets unless `release` is non-zero: used by the
// tests of the bounded-wait path (the wait must end with kPeerTimeout and the
// context must stay usable).
__global__ void bounded_wait_probe_kernel(const uint32_t* flag, uint32_t want, int* status, long long budget) {
  const long long t0 = clock64();
  while (static_cast<int32_t>(ld_acquire_sys(flag) - want) < 0) {
    if (clock64() - t0 > budget) {
      report_status(status, kPeerTimeout, 65);
      return;
    }
  }
}

// out[rows, cols] = sum over `n` slots of partial[slot][rows, cols] (+ bias[cols]) (+ residual[rows, cols]).
// Second half of the GEMM -> reduce-scatter path: every peer has stored its
// partial tile for this rank's rows into slot [peer] of this rank's staging.
__global__ void slot_sum_kernel(const __nv_bfloat16* __restrict__ partial, int n, long long slot_elems,
                                const __nv_bfloat16* __restrict__ bias, const __nv_bfloat16* __restrict__ residual,
                                __nv_bfloat16* __restrict__ out, long long rows, int cols) {
  const long long vecs = slot_elems / 8;
  const int cvec = cols / 8;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < vecs;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    for (int s = 0; s < n; ++s)
      Vec16<__nv_bfloat16>::add(acc, reinterpret_cast<const uint4*>(partial + s * slot_elems)[i]);
    if (bias != nullptr) Vec16<__nv_bfloat16>::add(acc, reinterpret_cast<const uint4*>(bias)[i % cvec]);
    if (residual != nullptr) Vec16<__nv_bfloat16>::add(acc, reinterpret_cast<const uint4*>(residual)[i]);
    reinterpret_cast<uint4*>(out)[i] = Vec16<__nv_bfloat16>::pack(acc, 1.f);
  }
}

}  // namespace nmb

using namespace nmb;

// ---------------------------------------------------------------- allocation --
extern "C" int nmb_symm_alloc(long long bytes, void** ptr, unsigned char* handle64) {
  cudaError_t e = cudaMalloc(ptr, static_cast<size_t>(bytes));
  if (e != cudaSuccess) return 400 + e;
  e = cudaMemset(*ptr, 0, static_cast<size_t>(bytes));
  if (e != cudaSuccess) return 400 + e;
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, *ptr);
  if (e != cudaSuccess) return 400 + e;
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle64, &h, 64);
  return 0;
}

extern "C" int nmb_symm_open(const unsigned char* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? 0 : 400 + e;
}

extern "C" int nmb_symm_close(void* ptr) {
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  return e == cudaSuccess ? 0 : 400 + e;
}

extern "C" int nmb_symm_free(void* ptr) {
  cudaError_t e = cudaFree(ptr);
  return e == cudaSuccess ? 0 : 400 + e;
}

static void fill(PeerPtrs& t, void* const* src, int n) {
  for (int i = 0; i < kMaxRanks; ++i) t.p[i] = i < n ? src[i] : nullptr;
}

// The overlap-first all-reduce asks for the same shared-memory carve-out as the
// GEMM / attention kernels it runs beside: an SM keeps one carve-out at a time,
// so with the default (small) carve-out its blocks and the 190 KB GEMM CTAs
// would exclude each other.
extern "C" int nmb_comm_configure() {
  cudaError_t e = cudaFuncSetAttribute(allreduce_scale_light_kernel<__nv_bfloat16>,
                                       cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(allreduce_scale_light_kernel<float>, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(multimem_allreduce_light_kernel<__nv_bfloat16>,
                             cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(multimem_allreduce_light_kernel<float>, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
  return e == cudaSuccess ? 0 : 300 + e;
}

extern "C" int nmb_comm_limits(int* max_ranks, int* max_blocks, int* channels) {
  *max_ranks = kMaxRanks;
  *max_blocks = kMaxBlocks;
  *channels = kChannels;
  return 0;
}


// bufs[n], pads[n]: per-rank device pointers (peer-mapped); numel elements of
// bf16 (is_bf16) or fp32.  numel * elem_size must be a multiple of 16.
// blocks < 0 selects the overlap-first variant with -blocks blocks.
extern "C" int nmb_allreduce_scale(void* const* bufs, void* const* pads, void* epochs, int channel, int rank,
                                   int n, long long numel, int is_bf16, float scale, int blocks, int* status,
                                   long long budget_cycles, void* stream) {
  if (n < 1 || n > kMaxRanks || channel < 0 || channel >= kChannels) return kBadArgument;
  const int per = is_bf16 ? 8 : 4;
  if (numel % per != 0) return kBadArgument;
  const bool light = blocks < 0;
  if (light) blocks = -blocks;
  if (blocks < 1) blocks = 1;
  if (blocks > kMaxBlocks) blocks = kMaxBlocks;
  PeerPtrs b, p;
  fill(b, bufs, n);
  fill(p, pads, n);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (light && is_bf16)
    allreduce_scale_light_kernel<__nv_bfloat16><<<blocks, kLightThreads, 0, s>>>(b, p, static_cast<uint32_t*>(epochs), channel,
                                                                      rank, n, numel / per, scale, status, budget_cycles);
  else if (light)
    allreduce_scale_light_kernel<float><<<blocks, kLightThreads, 0, s>>>(b, p, static_cast<uint32_t*>(epochs), channel, rank, n,
                                                               numel / per, scale, status, budget_cycles);
  else if (is_bf16)
    allreduce_scale_kernel<__nv_bfloat16><<<blocks, 512, 0, s>>>(b, p, static_cast<uint32_t*>(epochs), channel, rank, n,
                                                                numel / per, scale, status, budget_cycles);
  else
    allreduce_scale_kernel<float><<<blocks, 512, 0, s>>>(b, p, static_cast<uint32_t*>(epochs), channel, rank, n,
                                                         numel / per, scale, status, budget_cycles);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + e;
}

// In-place all-reduce (sum) * scale through the multicast mapping `mc` of a
// buffer of `numel` elements (same layout rules as nmb_allreduce_scale).
extern "C" int nmb_multimem_allreduce_scale(void* mc, void* const* pads, void* epochs, int channel, int rank, int n,
                                            long long numel, int is_bf16, float scale, int blocks, int* status,
                                            long long budget_cycles, void* stream) {
  if (mc == nullptr || n < 2 || n > kMaxRanks || channel < 0 || channel >= kChannels) return kBadArgument;
  if (reinterpret_cast<uintptr_t>(mc) & 15) return kBadArgument;
  const int per = is_bf16 ? 8 : 4;
  if (numel % per != 0) return kBadArgument;
  const bool light = blocks < 0;
  if (light) blocks = -blocks;
  if (blocks < 1) blocks = 1;
  if (blocks > kMaxBlocks) blocks = kMaxBlocks;
  PeerPtrs p;
  fill(p, pads, n);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t* m = static_cast<uint8_t*>(mc);
  uint32_t* ep = static_cast<uint32_t*>(epochs);
  const long long n_vec = numel / per;
  if (light && is_bf16)
    multimem_allreduce_light_kernel<__nv_bfloat16><<<blocks, kLightThreads, 0, s>>>(m, p, ep, channel, rank, n, n_vec, scale, status, budget_cycles);
  else if (light)
    multimem_allreduce_light_kernel<float><<<blocks, kLightThreads, 0, s>>>(m, p, ep, channel, rank, n, n_vec, scale, status, budget_cycles);
  else if (is_bf16)
    multimem_allreduce_kernel<__nv_bfloat16><<<blocks, 512, 0, s>>>(m, p, ep, channel, rank, n, n_vec, scale, status, budget_cycles);
  else
    multimem_allreduce_kernel<float><<<blocks, 512, 0, s>>>(m, p, ep, channel, rank, n, n_vec, scale, status, budget_cycles);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + e;
}

// src: numel*elem bytes (multiple of 16); dsts[n]: every rank's [n][same bytes] buffer.
extern "C" int nmb_peer_allgather(const void* src, void* const* dsts, void* const* pads, void* epochs, int channel,
                                  int rank, int n, long long nbytes, int* status, long long budget_cycles,
                                  void* stream) {
  if (n < 1 || n > kMaxRanks || channel < 0 || channel >= kChannels || nbytes % 16 != 0) return kBadArgument;
  PeerPtrs d, p;
  fill(d, dsts, n);
  fill(p, pads, n);
  const long long n_vec = nbytes / 16;
  int blocks = static_cast<int>((n_vec + 4095) / 4096);
  if (blocks < 1) blocks = 1;
  if (blocks > 64) blocks = 64;
  peer_allgather_kernel<<<blocks, 512, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), d, p, static_cast<uint32_t*>(epochs), channel, rank, n, n_vec, status,
      budget_cycles);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + e;
}

extern "C" int nmb_embedding_scatter(const long long* ids, const long long* positions, const void* tok,
                                     const void* pos, void* const* outs, int n_ranks, int n_tokens, int H,
                                     int vocab_start, int vloc, int seq_len, int shard_len, int to_all, void* stream) {
  if (n_tokens <= 0) return 0;
  if (H % 8 != 0 || n_ranks < 1 || n_ranks > kMaxRanks || shard_len < 1) return kBadArgument;
  PeerPtrs o;
  fill(o, outs, n_ranks);
  embedding_scatter_kernel<<<n_tokens, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      ids, positions, static_cast<const __nv_bfloat16*>(tok), static_cast<const __nv_bfloat16*>(pos), o, n_ranks,
      n_tokens, H, vocab_start, vloc, seq_len, shard_len, to_all);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + e;
}

extern "C" int nmb_symm_barrier(void* const* pads, void* epochs, int channel, int rank, int n, int* status,
                                long long budget_cycles, void* stream) {
  if (n < 1 || n > kMaxRanks || channel < 0 || channel >= kChannels) return kBadArgument;
  PeerPtrs p;
  fill(p, pads, n);
  barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p, static_cast<uint32_t*>(epochs), channel, rank, n,
                                                                  status, budget_cycles);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + e;
}

// stage_k / stage_v: this rank's [n][B, S, H, d] staging buffers; out_k / out_v:
// [B, S, H, d] views with element strides (out_sb, out_ss, out_sh), 16-byte
// aligned rows.  All ranks of the group launch it with the same shapes.
extern "C" int nmb_cp_dkv_reduce(const void* stage_k, const void* stage_v, void* out_k, void* out_v, long long out_sb,
                                 long long out_ss, long long out_sh, int B, int S, int H, int d, int first,
                                 void* const* pads, void* epochs, int channel, int rank, int n,
                                 const void* rope_table, const long long* rope_pos, int* status,
                                 long long budget_cycles, void* stream) {
  if (n < 1 || n > kMaxRanks || channel < 0 || channel >= kChannels || d % 8 != 0 || first < 0 || first >= n)
    return kBadArgument;
  if ((out_sb | out_ss | out_sh) % 8 != 0) return kBadArgument;
  PeerPtrs p;
  fill(p, pads, n);
  const long long vecs = 2LL * B * S * H * (d / 8);
  int blocks = static_cast<int>((vecs + 1023) / 1024);
  if (blocks < 1) blocks = 1;
  if (blocks > 2 * 148) blocks = 2 * 148;
  if (blocks > kMaxBlocks) blocks = kMaxBlocks;
  cp_dkv_reduce_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(stage_k), static_cast<const __nv_bfloat16*>(stage_v),
      static_cast<__nv_bfloat16*>(out_k), static_cast<__nv_bfloat16*>(out_v), out_sb, out_ss, out_sh, B, S, H, d, first,
      p, static_cast<uint32_t*>(epochs), channel, rank, n, static_cast<const float2*>(rope_table), rope_pos, status,
      budget_cycles);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + e;
}

extern "C" int nmb_bounded_wait_probe(const void* flag, unsigned want, int* status, long long budget_cycles,
                                      void* stream) {
  bounded_wait_probe_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint32_t*>(flag), want,
                                                                            status, budget_cycles);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + e;
}

extern "C" int nmb_slot_sum(const void* partial, int n, long long slot_elems, const void* bias, const void* residual,
                            void* out, long long rows, int cols, void* stream) {
  if (slot_elems % 8 != 0 || cols % 8 != 0) return kBadArgument;
  const long long vecs = slot_elems / 8;
  int blocks = static_cast<int>((vecs + 255) / 256);
  const int cap = sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  slot_sum_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(partial), n, slot_elems, static_cast<const __nv_bfloat16*>(bias),
      static_cast<const __nv_bfloat16*>(residual), static_cast<__nv_bfloat16*>(out), rows, cols);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + e;
}
