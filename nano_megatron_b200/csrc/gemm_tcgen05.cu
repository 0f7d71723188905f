// bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in
// TMEM, operands staged by TMA) with fused epilogues.
//
//   C[M,N] = epilogue( sum_k A[m,k] * B[n,k] )
//
// Either operand may be stored K-major (row = M/N index, K contiguous) or
// MN-major (row = K index, M/N contiguous), which covers the three products a
// linear layer needs without any transposed copy:
//   forward  Y  = X  W^T   : A = X   (K-major),  B = W  (K-major)
//   dgrad    dX = dY W     : A = dY  (K-major),  B = W  (MN-major)
//   wgrad    dW = dY^T X   : A = dY  (MN-major), B = X  (MN-major)
// This replaces the cuBLAS calls behind `F.linear` in the reference
// (nano_megatron/parallel/mappings.py:419,450) and the separate bias / GELU /
// residual elementwise kernels that follow them
// (nano_megatron/reference/layers.py:39, :343, :352).
//
// Structure: persistent CTAs (one per SM), 320 threads:
//   warp 0      TMA producer (one elected lane), STAGES-deep smem ring
//   warp 1      TMEM owner + single-thread tcgen05.mma issuer
//   warps 2..9  epilogue: tcgen05.ld -> registers -> bias/GELU/residual -> a per-warp
//               shared-memory transpose -> global in 128-byte row runs
//               (two warps per TMEM lane quadrant, each takes half of the columns)
// Two TMEM accumulator buffers let the epilogue of tile i overlap the main
// loop of tile i+1.  Every CTA loads its own tiles (no multicast load); the
// CTA-pair variant further down (cta_group::2, clusters of two) is what the
// dispatcher picks for shapes with enough tiles.  The kernels are launched with
// programmatic stream serialization and wait for the previous kernel only
// after their barrier / TMEM set-up.
#include "common.cuh"

#include <string.h>

namespace nmb {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kGemmThreads = 320;  // TMA warp, MMA warp, 8 epilogue warps

enum EpilogueMode : int {
  kEpiPlain = 0,   // C = acc (+bias) (+residual) (+C_old)
  kEpiGelu = 1,    // aux_out = acc+bias ; C = gelu(acc+bias)
  kEpiDGelu = 2,   // C = acc * gelu'(aux_in)
  kEpiRope = 3,    // C = rope(acc + bias) on the first rope_cols columns (interleaved pairs), rest unchanged
  kEpiSwiGLU = 4,  // B rows are [gate; up] (F each): aux_out = [gate | up] + bias ; C[:, :F] = silu(gate) * up
  kEpiDSwiGLU = 5, // acc = d(act) [M, F]: C[:, :F] = d gate, C[:, F:] = d up, from aux_in = [gate | up]
};

struct GemmEpilogue {
  void* c;                  // bf16 (or fp32 when out_f32) [M, ldc]
  const __nv_bfloat16* bias;      // [N] or null
  const __nv_bfloat16* residual;  // [M, ldr] or null
  __nv_bfloat16* aux_out;         // [M, ld_aux] (kEpiGelu)
  const __nv_bfloat16* aux_in;    // [M, ld_aux] (kEpiDGelu)
  int ldc;
  int ldr;
  int ld_aux;
  int mode;
  int accumulate;           // add the previous contents of C
  int out_f32;              // C is fp32
  float alpha;              // scale applied to the accumulator first
  // kEpiRope: rotary position embedding fused into the projection that produces q and k
  // (the reference rotates after the projection with ~10 elementwise kernels per tensor,
  // nano_megatron/reference/layers.py:67-81).  Pair i of a head is rotated by the angle
  // whose (cos, sin) is rope_table[rope_pos[row]][i].
  const float2* rope_table;     // [positions][rope_half]
  const long long* rope_pos;    // [M]
  int rope_cols;                // leading columns that hold q and k heads
  int rope_half;                // head_dim / 2
  int swiglu_f;                 // kEpiSwiGLU / kEpiDSwiGLU: F
  // split-K (weight gradients whose tiles fill a fraction of the machine): the K
  // range of every tile is cut into `splits` pieces computed by different CTAs;
  // all but the last store their fp32 partial tile into `splitk_ws` [tile][split][128 * BN]
  // and count themselves in on `splitk_counters[tile]`; the last split adds them to
  // its own accumulator in split order (deterministic) and runs the epilogue.
  float* splitk_ws;
  unsigned* splitk_counters;
  int splits;
};

// Extra epilogue arguments of the C entry points (all optional).
struct NmbEpilogueExtra {
  const void* rope_table;
  const long long* rope_pos;
  int rope_cols;
  int rope_half;
  int swiglu_f;
};

// Collective fused into the GEMM (both optional, normally one at a time).
//
//  * all-gather of A (sequence-parallel input): A's rows are sharded over the
//    ranks by sequence position.  The last `ag_copy_ctas` CTAs of the launch do
//    not compute: they pull the peers' shards over NVLink into this rank's full
//    A buffer, 128-row tile by tile, and publish a ready flag per tile; the GEMM
//    CTAs walk the tiles local-shard-first and wait for a tile's flag before
//    issuing its first TMA load, so the transfer hides behind the math.  Every
//    remote tile crosses NVLink once and is then read from local memory.
//  * reduce-scatter / all-reduce of C: every 128-row block of C has an owner
//    rank (the owner of its sequence shard).  A rank computes the blocks of the
//    other owners FIRST and stores each partial tile straight into slot
//    [my_rank] of the owner's staging buffer (peer stores), followed by one
//    release store to the tile's flag on the owner.  Its own blocks come LAST:
//    by then the peers' partials have normally landed, the epilogue of an own
//    tile waits for the tile's flags (bounded), adds the peers' partials, bias
//    and residual to its accumulator and writes the final tile -- to its own
//    shard (reduce-scatter) or to every rank's output followed by a second flag
//    (all-reduce; the kernel ends by waiting for the final tiles of the other
//    owners).  There is no grid-wide round and no separate reduction pass.
//
// Flags hold the launch's epoch (a device-side counter that the last CTA to
// leave the kernel advances, so a replayed CUDA graph keeps counting); they
// only grow and never need clearing.  Ranks of a group must launch the same
// fused GEMMs in the same order.
//
// Buffer reuse.  Peers write into this rank's staging / output buffers, so a
// peer may only start writing for launch j once this rank is done with the
// previous launch that used the same buffers (including whatever its stream
// did with the result afterwards).  Every launch therefore announces "I have
// started the launch with epoch e" to all peers (`rs_started`), every buffer
// remembers the epoch of the last launch that used it (`rs_last`, the same
// value on all ranks because the sequences are identical), and before its first
// peer store a CTA waits until every peer has started a launch later than that
// one.  The caller alternates two buffers per shape, which makes this wait a
// formality (finishing a launch needs the peers' tiles of that launch, so a
// rank is never more than one launch ahead); with a single buffer, or when a
// replayed CUDA graph follows another one that ended on the same buffer, it
// degrades to a rendezvous at the start of the launch instead of a race.
constexpr int kMaxFusedTiles = 4096;  // per owner: (rows_per_rank / 128) * ceil(N / BN)

struct FusedComm {
  const void* ag_src[kMaxRanks];
  void* ag_dst;
  uint32_t* ag_ready;
  int ag_copy_ctas;
  int rs_mode;  // 0 off, 1 reduce-scatter, 2 all-reduce
  void* rs_stage[kMaxRanks];
  void* rs_out[kMaxRanks];
  uint32_t* rs_flags[kMaxRanks];  // per rank: [2][kMaxFusedTiles][kMaxRanks]: partial stored / final stored
  uint32_t* rs_started[kMaxRanks];  // per rank: [kMaxRanks] "rank r has started the launch with this epoch"
  uint32_t* rs_last[2];             // local: epoch of the last launch that used the staging / output buffer
  const __nv_bfloat16* rs_bias;
  const __nv_bfloat16* rs_residual;
  void* pads[kMaxRanks];
  uint32_t* sync;  // [0] epoch of the last finished fused launch, [1] CTAs of this launch that have left
  int channel;
  int rank, n_ranks;
  int seq_len, shard_len, rows_per_rank;
  long long budget;
};

__device__ __forceinline__ uint32_t* fused_flag(const FusedComm& fc, int on_rank, int kind, int tile, int from_rank) {
  return fc.rs_flags[on_rank] + (static_cast<size_t>(kind) * kMaxFusedTiles + tile) * kMaxRanks + from_rank;
}

// Rows are [batch][sequence]; a sequence is cut into n_ranks contiguous shards.
__device__ __forceinline__ int row_owner(const FusedComm& fc, int row) { return (row % fc.seq_len) / fc.shard_len; }
__device__ __forceinline__ int row_local(const FusedComm& fc, int row) {
  return (row / fc.seq_len) * fc.shard_len + (row % fc.seq_len) % fc.shard_len;
}
__device__ __forceinline__ int row_global(const FusedComm& fc, int owner, int local) {
  return (local / fc.shard_len) * fc.seq_len + owner * fc.shard_len + local % fc.shard_len;
}

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = STAGES * kStageBytes;
  // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], tile_done[2], decided[2], tmem slot, abort, epoch,
  // need, last[2]
  static constexpr int kTotal = kBarOffset + (2 * STAGES + 8) * 8 + 32;
};

// Copy CTA of the fused all-gather: pulls remote 128-row tiles of A into the
// local full buffer and publishes one ready flag per tile.  NVLink needs a
// couple of megabytes in flight to run at full rate (bandwidth x ~2.5 us of
// latency), far more than a few CTAs' worth of register loads: one thread per
// copy CTA drives bulk asynchronous copies instead (peer memory -> shared
// memory -> local memory, a ring of 32 KB pieces, five loads in flight per CTA;
// plain bulk copies, no cluster multicast).
constexpr int kCopyPiece = 32768;
constexpr int kCopyStages = 6;

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ uint32_t gather_copy_role(const FusedComm& fc, int M, int K, int copy_idx, int* status, uint8_t* smem) {
  __shared__ uint32_t epoch_s;
  __shared__ int ok_s;
  __shared__ int abort_s;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kCopyStages * kCopyPiece);
  if (threadIdx.x == 0) {
    epoch_s = fc.sync[0] + 1;
    ok_s = 1;
    abort_s = 0;
    for (int i = 0; i < kCopyStages; ++i) mbar_init(&bars[i], 1);
    fence_mbar_init();
  }
  __syncthreads();
  const uint32_t e = epoch_s;
  // Peers' shards are complete once their copy CTA of the same index got here
  // (it runs after everything earlier in that rank's stream).
  if (threadIdx.x < fc.n_ranks) {
    __threadfence_system();
    st_release_sys(pad_slot(fc.pads[threadIdx.x], fc.channel, 1 + copy_idx, fc.rank), e);
    if (!wait_flag_sys(pad_slot(fc.pads[fc.rank], fc.channel, 1 + copy_idx, threadIdx.x), e, fc.budget)) {
      report_status(status, kPeerTimeout, 6);
      ok_s = 0;
    }
  }
  __syncthreads();
  const int tpc = fc.shard_len / kBM;
  const int nb = M / fc.seq_len;
  const int per_owner = nb * tpc;
  const int remote = (fc.n_ranks - 1) * per_owner;
  const size_t tile_bytes = static_cast<size_t>(kBM) * K * 2;
  const int pieces = static_cast<int>((tile_bytes + kCopyPiece - 1) / kCopyPiece);
  const int my_tiles = remote > copy_idx ? (remote - copy_idx + fc.ag_copy_ctas - 1) / fc.ag_copy_ctas : 0;
  const int total = my_tiles * pieces;
  if (threadIdx.x == 0) {
    // item j = (j / pieces)-th tile of this CTA, piece j % pieces
    auto locate = [&](int j, int& m_blk, size_t& off, uint32_t& bytes, int& owner) {
      const int i = copy_idx + (j / pieces) * fc.ag_copy_ctas;
      const int k = 1 + i / per_owner;  // distance from my rank
      const int rem = i % per_owner;
      owner = (fc.rank + k) % fc.n_ranks;
      m_blk = ((rem / tpc) * fc.seq_len + owner * fc.shard_len) / kBM + rem % tpc;
      const size_t in_tile = static_cast<size_t>(j % pieces) * kCopyPiece;
      off = static_cast<size_t>(m_blk) * tile_bytes + in_tile;
      const size_t left = tile_bytes - in_tile;
      bytes = static_cast<uint32_t>(left < kCopyPiece ? left : kCopyPiece);
    };
    int loaded = 0;
    bool ok = ok_s != 0;
    for (int stored = 0; stored < total; ++stored) {
      while (ok && loaded < total && loaded - stored < kCopyStages - 1) {
        // the piece stored from this stage two stores ago has left shared memory
        if (loaded >= kCopyStages) bulk_wait_read_1();
        int m_blk, owner;
        size_t off;
        uint32_t bytes;
        locate(loaded, m_blk, off, bytes, owner);
        uint64_t* bar = &bars[loaded % kCopyStages];
        mbar_expect_tx(bar, bytes);
        bulk_load(smem + (loaded % kCopyStages) * kCopyPiece, static_cast<const uint8_t*>(fc.ag_src[owner]) + off, bytes,
                  bar);
        ++loaded;
      }
      int m_blk, owner;
      size_t off;
      uint32_t bytes;
      locate(stored, m_blk, off, bytes, owner);
      if (ok) {
        if (!mbar_wait(&bars[stored % kCopyStages], (stored / kCopyStages) & 1, &abort_s, status, 17)) ok = false;
      }
      if (ok) {
        bulk_store(static_cast<uint8_t*>(fc.ag_dst) + off, smem + (stored % kCopyStages) * kCopyPiece, bytes);
        bulk_commit();
      }
      if (stored % pieces == pieces - 1) {
        // the tile is complete in local memory: publish it (also after a failed
        // wait, so that no GEMM CTA spins on it; the status word tells the host)
        bulk_wait_all();
        __threadfence();
        fence_proxy_async_all();
        st_release_gpu(&fc.ag_ready[m_blk], e);
      }
    }
    bulk_wait_all();
    if (!ok) {
      // loads may still be landing in shared memory: let them before the CTA exits
      for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
  }
  // Closing round: no peer is still reading this rank's shard when a later
  // kernel overwrites it.  The copy CTAs are done long before the compute CTAs,
  // so this wait is normally hidden.
  __syncthreads();
  if (threadIdx.x < fc.n_ranks && ok_s) {
    __threadfence_system();
    st_release_sys(pad_slot(fc.pads[threadIdx.x], fc.channel, 65 + copy_idx, fc.rank), e);
    if (!wait_flag_sys(pad_slot(fc.pads[fc.rank], fc.channel, 65 + copy_idx, threadIdx.x), e, fc.budget))
      report_status(status, kPeerTimeout, 7);
  }
  return e;
}

// Every CTA of a fused launch (compute and copy CTAs alike, also after an
// aborted wait) leaves through here: the last one advances the epoch.
__device__ __forceinline__ void fused_leave(const FusedComm& fc, uint32_t epoch) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned left = atomicAdd(&fc.sync[1], 1u);
    if (left == gridDim.x - 1) {
      fc.sync[1] = 0;
      fc.sync[0] = epoch;
      if (fc.rs_mode != 0) {
        *fc.rs_last[0] = epoch;
        if (fc.rs_last[1] != nullptr) *fc.rs_last[1] = epoch;
      }
      __threadfence();
    }
  }
}

// Store of one 32-column bf16 chunk of a warp's 32 accumulator rows.  In the
// accumulator a lane owns a row, so a store from registers writes 16 bytes to 32
// different rows per instruction (half-filled sectors, four instructions per
// chunk).  With a staging buffer the warp transposes the chunk through 2 KB of
// shared memory of its own (16-byte pieces XOR-swizzled so that both phases are
// free of bank conflicts) and writes 8 rows x 64 contiguous bytes per
// instruction.  `dst` points at column 0 of the chunk in the warp's first row;
// rows >= rows_valid are not written.  All 32 lanes must call it.
struct ChunkStore {
  uint4* wbuf;
  int lane;
  __nv_bfloat16* dst;
  size_t ld;
  int rows_valid;
  // 16-byte piece q (of 4) of this lane's row
  __device__ __forceinline__ void put(int q, const uint4& o) const {
    if (wbuf != nullptr) {
      wbuf[lane * 4 + (q ^ ((lane >> 1) & 3))] = o;
    } else if (lane < rows_valid) {
      reinterpret_cast<uint4*>(dst + static_cast<size_t>(lane) * ld)[q] = o;
    }
  }
  __device__ __forceinline__ void flush() const {
    if (wbuf == nullptr) return;
    __syncwarp();
    const int seg = lane & 3;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = i * 8 + (lane >> 2);
      const uint4 u = wbuf[r * 4 + (seg ^ ((r >> 1) & 3))];
      if (r < rows_valid) *reinterpret_cast<uint4*>(dst + static_cast<size_t>(r) * ld + seg * 8) = u;
    }
    __syncwarp();
  }
};

// Epilogue of one 128-row accumulator tile for one warp: drains its half of
// the BN columns of TMEM lane quadrant `t_row` (32 columns at a time), applies
// alpha / bias / GELU / dGELU / residual / accumulate and stores row `row`.
// FULL adds the rotary and SwiGLU-backward epilogues (only compiled into the
// kernel instantiation that also carries the fused collectives).
// `ws_row` (split-K, last split of a tile): the other splits' partial tiles are added
// to this split's own part in TMEM, in split order.  It points at this lane's first
// float4 of split 0's partial (layout [chunk][quad][q][lane] float4, so a warp reads
// 512-byte runs); splits are 128 * BN floats apart.
template <int BN, bool FULL>
__device__ __forceinline__ void epilogue_columns(const GemmEpilogue& ep, const FusedComm& fc, uint32_t t_row, int row,
                                                 bool row_ok, int n0, int half, int N, const float* ws_row = nullptr,
                                                 uint4* wbuf = nullptr, int lane = 0, int M = 0) {
  // With a staging buffer every lane takes part in every store: a lane whose row
  // lies beyond M works on the last valid row instead (its result is not written).
  const bool staged = wbuf != nullptr && !ep.out_f32 && (N % 32) == 0;
  if (!staged) wbuf = nullptr;
  const int wrow0 = row - (staged ? lane : 0);  // first row of the warp (staged) / this lane's row (direct)
  const int rows_valid = staged ? (M - wrow0 < 32 ? M - wrow0 : 32) : 32;
  if (staged && !row_ok) {
    row = M - 1;
    row_ok = true;
  }
  const int slane = staged ? lane : 0;
#pragma unroll 1
  for (int c = half * (BN / 64); c < (half + 1) * (BN / 64); ++c) {
    const int col0 = n0 + c * 32;
    if (col0 >= N) break;  // uniform across the warp
    float v[32];
    {
      uint32_t r[32];
      tmem_ld_32x32(t_row + c * 32, r);
      if (ws_row != nullptr) {
        // split-K: the other splits' partials, two splits' loads in flight at a time
        const float4* src = reinterpret_cast<const float4*>(ws_row) + c * 1024;
        float4 f[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) f[q] = __ldcg(src + q * 32);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        for (int sp = 0; sp < ep.splits - 1; ++sp) {
          float4 g[8];
          const bool more = sp + 2 < ep.splits;
          if (more) {
#pragma unroll
            for (int q = 0; q < 8; ++q) g[q] = __ldcg(src + static_cast<size_t>(sp + 1) * (kBM * BN / 4) + q * 32);
          }
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            v[4 * q] += f[q].x;
            v[4 * q + 1] += f[q].y;
            v[4 * q + 2] += f[q].z;
            v[4 * q + 3] += f[q].w;
          }
          if (more) {
#pragma unroll
            for (int q = 0; q < 8; ++q) f[q] = g[q];
          }
        }
        if (!row_ok) continue;
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] *= ep.alpha;
      } else {
        tmem_ld_wait();
        if (!row_ok) continue;
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * ep.alpha;
      }
    }
    const bool full_chunk = (col0 + 32 <= N);
    if (full_chunk) {
      if (ep.bias != nullptr) {
        const uint4* bp = reinterpret_cast<const uint4*>(ep.bias + col0);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 u = __ldg(bp + q);
          const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float2 f = unpack_bf16x2(w[t]);
            v[q * 8 + t * 2] += f.x;
            v[q * 8 + t * 2 + 1] += f.y;
          }
        }
      }
      if (FULL && ep.mode == kEpiRope && col0 < ep.rope_cols) {
        // 16 interleaved pairs of one head; their angles are consecutive table entries
        const int pair0 = (col0 % (2 * ep.rope_half)) >> 1;
        const float4* tp = reinterpret_cast<const float4*>(ep.rope_table + ep.rope_pos[row] * ep.rope_half + pair0);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const float4 cs = __ldg(tp + q);
          const float a0 = v[4 * q], a1 = v[4 * q + 1], b0 = v[4 * q + 2], b1 = v[4 * q + 3];
          v[4 * q] = a0 * cs.x - a1 * cs.y;
          v[4 * q + 1] = a0 * cs.y + a1 * cs.x;
          v[4 * q + 2] = b0 * cs.z - b1 * cs.w;
          v[4 * q + 3] = b0 * cs.w + b1 * cs.z;
        }
      }
      if (FULL && ep.mode == kEpiDSwiGLU) {
        // v = d(act); gate / up pre-activations from the forward pass
        const __nv_bfloat16* pre = ep.aux_in + static_cast<size_t>(row) * ep.ld_aux + col0;
        // two output streams: d gate now, d up kept in registers until the buffer is free again
        __nv_bfloat16* c0 = static_cast<__nv_bfloat16*>(ep.c) + static_cast<size_t>(wrow0) * ep.ldc + col0;
        const ChunkStore sg{wbuf, slane, c0, static_cast<size_t>(ep.ldc), rows_valid};
        const ChunkStore su{wbuf, slane, c0 + ep.swiglu_f, static_cast<size_t>(ep.ldc), rows_valid};
        uint4 ou4[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 gu = reinterpret_cast<const uint4*>(pre)[q];
          const uint4 uu = reinterpret_cast<const uint4*>(pre + ep.swiglu_f)[q];
          const uint32_t gw[4] = {gu.x, gu.y, gu.z, gu.w};
          const uint32_t uw[4] = {uu.x, uu.y, uu.z, uu.w};
          uint32_t og[4], ou[4];
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float2 g = unpack_bf16x2(gw[t]);
            const float2 u = unpack_bf16x2(uw[t]);
            const float d0 = v[q * 8 + t * 2], d1 = v[q * 8 + t * 2 + 1];
            const float s0 = 1.f / (1.f + __expf(-g.x)), s1 = 1.f / (1.f + __expf(-g.y));
            og[t] = pack_bf16x2(d0 * u.x * s0 * (1.f + g.x * (1.f - s0)), d1 * u.y * s1 * (1.f + g.y * (1.f - s1)));
            ou[t] = pack_bf16x2(d0 * g.x * s0, d1 * g.y * s1);
          }
          sg.put(q, make_uint4(og[0], og[1], og[2], og[3]));
          ou4[q] = make_uint4(ou[0], ou[1], ou[2], ou[3]);
        }
        sg.flush();
#pragma unroll
        for (int q = 0; q < 4; ++q) su.put(q, ou4[q]);
        su.flush();
        continue;
      }
      if (ep.mode == kEpiGelu) {
        const ChunkStore sa{wbuf, slane, ep.aux_out + static_cast<size_t>(wrow0) * ep.ld_aux + col0,
                            static_cast<size_t>(ep.ld_aux), rows_valid};
#pragma unroll
        for (int q = 0; q < 4; ++q)
          sa.put(q, make_uint4(pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]), pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]),
                               pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]), pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7])));
        sa.flush();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          // GELU of the value the backward pass will see (bf16-rounded).
          const float h = __bfloat162float(__float2bfloat16(v[j]));
          v[j] = gelu_erf_f(h);
        }
      } else if (ep.mode == kEpiDGelu) {
        const uint4* ap =
            reinterpret_cast<const uint4*>(ep.aux_in + static_cast<size_t>(row) * ep.ld_aux + col0);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 u = ap[q];
          const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float2 f = unpack_bf16x2(w[t]);
            v[q * 8 + t * 2] *= gelu_erf_grad_f(f.x);
            v[q * 8 + t * 2 + 1] *= gelu_erf_grad_f(f.y);
          }
        }
      }
      if (ep.residual != nullptr) {
        const uint4* rp =
            reinterpret_cast<const uint4*>(ep.residual + static_cast<size_t>(row) * ep.ldr + col0);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 u = rp[q];
          const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float2 f = unpack_bf16x2(w[t]);
            v[q * 8 + t * 2] += f.x;
            v[q * 8 + t * 2 + 1] += f.y;
          }
        }
      }
      if (ep.out_f32) {
        float4* cp = reinterpret_cast<float4*>(static_cast<float*>(ep.c) +
                                               static_cast<size_t>(row) * ep.ldc + col0);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          float4 o = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
          if (ep.accumulate) {
            const float4 old = cp[q];
            o.x += old.x;
            o.y += old.y;
            o.z += old.z;
            o.w += old.w;
          }
          cp[q] = o;
        }
      } else {
        __nv_bfloat16* c_row = static_cast<__nv_bfloat16*>(ep.c) + static_cast<size_t>(row) * ep.ldc;
        uint4* cp = reinterpret_cast<uint4*>(c_row + col0);
        const ChunkStore sc{wbuf, slane, static_cast<__nv_bfloat16*>(ep.c) + static_cast<size_t>(wrow0) * ep.ldc + col0,
                            static_cast<size_t>(ep.ldc), rows_valid};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          if (ep.accumulate) {
            const uint4 u = cp[q];
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const float2 f = unpack_bf16x2(w[t]);
              v[q * 8 + t * 2] += f.x;
              v[q * 8 + t * 2 + 1] += f.y;
            }
          }
          sc.put(q, make_uint4(pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]), pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]),
                               pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]), pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7])));
        }
        sc.flush();
      }
    } else {
      // Ragged last chunk of the N dimension: scalar path.
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int col = col0 + j;
        if (col >= N) continue;
        float x = v[j];
        if (ep.bias != nullptr) x += __bfloat162float(ep.bias[col]);
        if (ep.mode == kEpiGelu) {
          const __nv_bfloat16 hb = __float2bfloat16(x);
          ep.aux_out[static_cast<size_t>(row) * ep.ld_aux + col] = hb;
          x = gelu_erf_f(__bfloat162float(hb));
        } else if (ep.mode == kEpiDGelu) {
          x *= gelu_erf_grad_f(__bfloat162float(ep.aux_in[static_cast<size_t>(row) * ep.ld_aux + col]));
        }
        if (ep.residual != nullptr)
          x += __bfloat162float(ep.residual[static_cast<size_t>(row) * ep.ldr + col]);
        if (ep.out_f32) {
          float* cp = static_cast<float*>(ep.c) + static_cast<size_t>(row) * ep.ldc + col;
          *cp = ep.accumulate ? (*cp + x) : x;
        } else {
          __nv_bfloat16* cp = static_cast<__nv_bfloat16*>(ep.c) + static_cast<size_t>(row) * ep.ldc + col;
          if (ep.accumulate) x += __bfloat162float(*cp);
          *cp = __float2bfloat16(x);
        }
      }
    }
  }
}

// SwiGLU forward epilogue (BN = 256): accumulator columns 0..127 are the gate,
// 128..255 the up projection of output features [n0/2, n0/2 + 128).  Each warp
// takes 64 features: stores gate + bias and up + bias into aux_out = [gate | up]
// (what the backward pass needs) and silu(gate) * up into C.  The activation is
// computed from the bf16-rounded pre-activations, as the backward will see them.
__device__ __forceinline__ void epilogue_swiglu(const GemmEpilogue& ep, uint32_t t_row, int row, bool row_ok, int n0,
                                                int half, uint4* wbuf, int lane, int M) {
  const int F = ep.swiglu_f;
  const int wrow0 = row - lane;
  const int rows_valid = M - wrow0 < 32 ? M - wrow0 : 32;
  (void)row_ok;
#pragma unroll 1
  for (int c = 2 * half; c < 2 * half + 2; ++c) {
    const int col0 = (n0 >> 1) + c * 32;
    if (col0 >= F) break;  // uniform across the warp (F is a multiple of 32)
    uint32_t rg[32], ru[32];
    tmem_ld_32x32(t_row + c * 32, rg);
    tmem_ld_32x32(t_row + 128 + c * 32, ru);
    tmem_ld_wait();
    __nv_bfloat16* pre = ep.aux_out + static_cast<size_t>(wrow0) * ep.ld_aux + col0;
    const ChunkStore sg{wbuf, lane, pre, static_cast<size_t>(ep.ld_aux), rows_valid};
    const ChunkStore su{wbuf, lane, pre + F, static_cast<size_t>(ep.ld_aux), rows_valid};
    const ChunkStore sa{wbuf, lane, static_cast<__nv_bfloat16*>(ep.c) + static_cast<size_t>(wrow0) * ep.ldc + col0,
                        static_cast<size_t>(ep.ldc), rows_valid};
    uint4 pu4[4], pa4[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float g[8], u[8];
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        g[t] = __uint_as_float(rg[q * 8 + t]) * ep.alpha;
        u[t] = __uint_as_float(ru[q * 8 + t]) * ep.alpha;
      }
      if (ep.bias != nullptr) {
        const uint4 bg = __ldg(reinterpret_cast<const uint4*>(ep.bias + col0) + q);
        const uint4 bu = __ldg(reinterpret_cast<const uint4*>(ep.bias + F + col0) + q);
        const uint32_t wg[4] = {bg.x, bg.y, bg.z, bg.w};
        const uint32_t wu[4] = {bu.x, bu.y, bu.z, bu.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float2 a = unpack_bf16x2(wg[t]);
          const float2 b = unpack_bf16x2(wu[t]);
          g[2 * t] += a.x;
          g[2 * t + 1] += a.y;
          u[2 * t] += b.x;
          u[2 * t + 1] += b.y;
        }
      }
      uint32_t pg[4], pu[4], pa[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        pg[t] = pack_bf16x2(g[2 * t], g[2 * t + 1]);
        pu[t] = pack_bf16x2(u[2 * t], u[2 * t + 1]);
        const float2 gr = unpack_bf16x2(pg[t]);
        const float2 ur = unpack_bf16x2(pu[t]);
        pa[t] = pack_bf16x2(gr.x / (1.f + __expf(-gr.x)) * ur.x, gr.y / (1.f + __expf(-gr.y)) * ur.y);
      }
      sg.put(q, make_uint4(pg[0], pg[1], pg[2], pg[3]));
      pu4[q] = make_uint4(pu[0], pu[1], pu[2], pu[3]);
      pa4[q] = make_uint4(pa[0], pa[1], pa[2], pa[3]);
    }
    sg.flush();
#pragma unroll
    for (int q = 0; q < 4; ++q) su.put(q, pu4[q]);
    su.flush();
#pragma unroll
    for (int q = 0; q < 4; ++q) sa.put(q, pa4[q]);
    sa.flush();
  }
}

// Epilogue of a tile whose rows take part in a fused reduce-scatter /
// all-reduce (N is a multiple of 32 there, rows are whole 128-row blocks).
//   own == false: the tile belongs to another rank: store the bf16 partial into
//                 slot [my rank] of the owner's staging buffer;
//   own == true : add the peers' partials (already in my staging buffer), bias
//                 and residual, and write the final tile to my shard
//                 (reduce-scatter) or to every rank's output (all-reduce).
// In the accumulator a lane owns a ROW (32 consecutive columns per tcgen05.ld),
// so storing from registers would issue 16-byte writes to 32 different rows per
// instruction -- over NVLink that is one tiny packet per lane.  The warp
// therefore transposes 64 columns at a time through a 4 KB shared-memory buffer
// of its own (16-byte chunks XOR-swizzled by the row) and writes rows out in
// 128-byte runs, four rows per instruction.
constexpr int kEpiStageBytes = 8 * 4096;  // one 32 x 64 bf16 buffer per epilogue warp

template <int BN>
__device__ __forceinline__ void epilogue_columns_reduce(const GemmEpilogue& ep, const FusedComm& fc, uint32_t t_row,
                                                        int m0, int quad, int lane, int owner, int n0, int half, int N,
                                                        bool own, uint4* wbuf) {
  const int row = m0 + quad * 32 + lane;         // the accumulator row this lane drains
  const int lrow = row_local(fc, row);
  const int lrow0 = lrow - lane;                  // local index of the warp's first row (a tile never straddles shards)
  const int grow0 = row - lane;
#pragma unroll 1
  for (int c2 = half * (BN / 128); c2 < (half + 1) * (BN / 128); ++c2) {
    const int col0 = n0 + c2 * 64;
    if (col0 >= N) break;  // uniform across the warp
    const int ncols = (N - col0) < 64 ? (N - col0) : 64;  // 32 or 64
#pragma unroll 1
    for (int h2 = 0; h2 * 32 < ncols; ++h2) {
      const int cc = col0 + h2 * 32;
      uint32_t r[32];
      tmem_ld_32x32(t_row + (c2 * 2 + h2) * 32, r);
      tmem_ld_wait();
      float v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * ep.alpha;
      if (own) {
        auto add4 = [&](const uint4* src) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint4 u = src[q];
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const float2 f = unpack_bf16x2(w[t]);
              v[q * 8 + t * 2] += f.x;
              v[q * 8 + t * 2 + 1] += f.y;
            }
          }
        };
        const __nv_bfloat16* mine = static_cast<const __nv_bfloat16*>(fc.rs_stage[fc.rank]);
        for (int p = 1; p < fc.n_ranks; ++p) {
          const int src = (fc.rank + p) % fc.n_ranks;
          add4(reinterpret_cast<const uint4*>(mine + (static_cast<size_t>(src) * fc.rows_per_rank + lrow) * N + cc));
        }
        if (fc.rs_bias != nullptr) add4(reinterpret_cast<const uint4*>(fc.rs_bias + cc));
        // reduce-scatter: residual is this rank's [rows_per_rank, N] shard; all-reduce: the full [M, N]
        const size_t rrow = fc.rs_mode == 1 ? static_cast<size_t>(lrow) : static_cast<size_t>(row);
        if (fc.rs_residual != nullptr) add4(reinterpret_cast<const uint4*>(fc.rs_residual + rrow * N + cc));
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 o;
        o.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
        o.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
        o.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
        o.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
        wbuf[lane * 8 + ((h2 * 4 + q) ^ (lane & 7))] = o;
      }
    }
    __syncwarp();
    const int segs = ncols / 8;  // 16-byte chunks per row: 4 or 8
    const int seg = lane & 7;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int rr = i * 4 + (lane >> 3);
      if (seg >= segs) continue;
      const uint4 o = wbuf[rr * 8 + (seg ^ (rr & 7))];
      const size_t col = static_cast<size_t>(col0) + seg * 8;
      if (!own) {
        __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(fc.rs_stage[owner]) +
                             (static_cast<size_t>(fc.rank) * fc.rows_per_rank + lrow0 + rr) * N + col;
        *reinterpret_cast<uint4*>(dst) = o;
      } else if (fc.rs_mode == 1) {
        __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(fc.rs_out[fc.rank]) + static_cast<size_t>(lrow0 + rr) * N + col;
        *reinterpret_cast<uint4*>(dst) = o;
      } else {
        for (int p = 0; p < fc.n_ranks; ++p) {
          __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(fc.rs_out[(fc.rank + p) % fc.n_ranks]) +
                               static_cast<size_t>(grow0 + rr) * N + col;
          *reinterpret_cast<uint4*>(dst) = o;
        }
      }
    }
    __syncwarp();
  }
}

// FUSED selects the instantiation that carries the optional code paths (copy
// CTAs and reduce epilogue of the fused collectives, rotary / SwiGLU
// epilogues); the plain one stays at the register count that lets a block of
// the overlapped gradient all-reduce share its SM.
template <int BN, int STAGES, bool A_MN, bool B_MN, bool FUSED, bool SPLITK>
__device__ __forceinline__ void gemm_bf16_body(const CUtensorMap& tma_a, const CUtensorMap& tma_b, const GemmEpilogue& ep,
                                               const FusedComm& fc, int M, int N, int K, int* status) {
  using L = GemmSmem<BN, STAGES>;
  const int n_gemm_ctas = FUSED ? gridDim.x - fc.ag_copy_ctas : gridDim.x;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // SWIZZLE_128B operands need 1024-byte aligned stage bases.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  if (FUSED && static_cast<int>(blockIdx.x) >= n_gemm_ctas) {
    static_assert(kCopyStages * kCopyPiece + kCopyStages * 8 <= L::kTotal, "copy ring must fit the GEMM's shared memory");
    const uint32_t e = gather_copy_role(fc, M, K, blockIdx.x - n_gemm_ctas, status, smem);
    fused_leave(fc, e);
    return;
  }
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint64_t* tile_done = acc_empty + 2;  // fused reduce / split-K: the 8 epilogue warps have stored a tile
  uint64_t* decided = tile_done + 2;    // split-K: "is this CTA the last split of the tile" has been decided
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(decided + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint32_t* epoch_slot = tmem_slot + 2;
  uint32_t* need_slot = tmem_slot + 3;  // fused reduce: peers must have started a launch with at least this epoch

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (M + kBM - 1) / kBM;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + kBK - 1) / kBK;
  // split-K: work unit u = split (u / num_tiles) of tile (u % num_tiles); the splits of
  // a tile run on different CTAs at the same time
  const int splits = SPLITK ? ep.splits : 1;
  const int num_units = num_tiles * splits;
  const int kb_per_split = (num_kb + splits - 1) / splits;
  constexpr uint32_t kTmemCols = 2 * BN;  // 256 or 512: powers of two
  const bool gathered = FUSED && fc.ag_copy_ctas > 0;
  const bool reducing = FUSED && fc.rs_mode != 0;
  const bool fused = gathered || reducing;
  // tile -> (m block, n block).  Plain GEMM: m fastest.  Gathered A: all n
  // blocks of an m block together, m blocks ordered local shard first, then the
  // peers by distance, so the first waves need no remote data.
  // Fused reduce: the other owners' blocks first (their partials have to travel),
  // this rank's own blocks last (the peers' partials for them have arrived by then).
  auto tile_coords = [&](int tile, int& m_blk, int& n_blk, int& owner) {
    if (!fused) {
      m_blk = tile % tiles_m;
      n_blk = tile / tiles_m;
      owner = fc.rank;
      return;
    }
    const int i_m = tile / tiles_n;
    n_blk = tile % tiles_n;
    const int tpc = fc.shard_len / kBM;           // m tiles per (batch, owner) chunk
    const int nb = M / fc.seq_len;
    const int k = i_m / (nb * tpc) + (gathered ? 0 : 1);
    const int rem = i_m % (nb * tpc);
    owner = (fc.rank + k) % fc.n_ranks;
    m_blk = ((rem / tpc) * fc.seq_len + owner * fc.shard_len) / kBM + rem % tpc;
  };

  // The fused forms read and publish protocol words in global memory during set-up:
  // they order themselves after the previous kernel first.  The plain form sets up
  // barriers and TMEM first and waits just before its first load.
  if constexpr (FUSED) pdl_enter();
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);  // one arrival per epilogue warp
      mbar_init(&tile_done[b], 8);
      mbar_init(&decided[b], 1);
    }
    *abort_flag = 0;
    *epoch_slot = fused ? fc.sync[0] + 1 : 0;
    if (reducing) {
      uint32_t last = *fc.rs_last[0];
      if (fc.rs_last[1] != nullptr && static_cast<int32_t>(*fc.rs_last[1] - last) > 0) last = *fc.rs_last[1];
      *need_slot = last + 1;
    }
    fence_mbar_init();
  }
  if (reducing && blockIdx.x == 0 && threadIdx.x < fc.n_ranks && static_cast<int>(threadIdx.x) != fc.rank) {
    // everything earlier in this rank's stream is complete: peers may reuse my buffers
    st_release_sys(fc.rs_started[threadIdx.x] + fc.rank, fc.sync[0] + 1);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if constexpr (!FUSED) pdl_enter();

  if (warp == 0) {
    // ------------------------------------------------------------ producer --
    if (lane == 0) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint32_t ag_epoch = *epoch_slot;
      for (int unit = blockIdx.x; unit < num_units && ok; unit += n_gemm_ctas) {
        const int tile = SPLITK ? unit % num_tiles : unit;
        const int kb_lo = SPLITK ? (unit / num_tiles) * kb_per_split : 0;
        const int kb_hi = SPLITK ? (kb_lo + kb_per_split < num_kb ? kb_lo + kb_per_split : num_kb) : num_kb;
        int m_blk, n_blk, owner;
        tile_coords(tile, m_blk, n_blk, owner);
        const int m0 = m_blk * kBM;
        const int n0 = n_blk * BN;
        if (gathered && owner != fc.rank) {
          // rows of this tile are being copied in by the copy CTAs
          const long long t0 = clock64();
          while (static_cast<int32_t>(ld_acquire_gpu(&fc.ag_ready[m_blk]) - ag_epoch) < 0) {
            if (*abort_flag != 0 || clock64() - t0 > fc.budget) {
              report_status(status, kPeerTimeout, 5);
              *abort_flag = 1;
              ok = false;
              break;
            }
          }
          if (!ok) break;
          fence_proxy_async_all();
        }
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, status, 1)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          mbar_expect_tx(&full_bar[stage], L::kStageBytes);
          if (!A_MN) {
            tma_load_2d(sa, &tma_a, &full_bar[stage], kb * kBK, m0);
          } else {
#pragma unroll
            for (int c = 0; c < kBM / 64; ++c)
              tma_load_2d(sa + c * 8192, &tma_a, &full_bar[stage], m0 + c * 64, kb * kBK);
          }
          if (!B_MN) {
            if (FUSED && BN == 256 && ep.mode == kEpiSwiGLU) {
              // 128 gate rows and the 128 up rows of the same output features
              tma_load_2d(sb, &tma_b, &full_bar[stage], kb * kBK, n0 >> 1);
              tma_load_2d(sb + 16384, &tma_b, &full_bar[stage], kb * kBK, ep.swiglu_f + (n0 >> 1));
            } else {
              tma_load_2d(sb, &tma_b, &full_bar[stage], kb * kBK, n0);
            }
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sb + c * 8192, &tma_b, &full_bar[stage], n0 + c * 64, kb * kBK);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer --
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(kBM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < num_units && ok; unit += n_gemm_ctas, ++local) {
        const int buf = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        const int kb_lo = SPLITK ? (unit / num_tiles) * kb_per_split : 0;
        const int kb_hi = SPLITK ? (kb_lo + kb_per_split < num_kb ? kb_lo + kb_per_split : num_kb) : num_kb;
        if (!mbar_wait(&acc_empty[buf], acc_phase ^ 1, abort_flag, status, 2)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, status, 3)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint32_t sb = sa + L::kABytes;
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            // One UMMA_K = 16 slice: 32 B along a K-major row, 16 rows of an
            // MN-major slab.
            const uint64_t da = A_MN ? make_smem_desc(sa + k * 2048, 8192, 1024)
                                     : make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + k * 2048, 8192, 1024)
                                     : make_smem_desc(sb + k * 32, 16, 1024);
            tc_mma_bf16(d_tmem, da, db, idesc, ((kb - kb_lo) | k) != 0 ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);  // frees the smem stage once the MMAs have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) tc_commit(&acc_full[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue --
    const int quad = warp & 3;          // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;   // which half of the tile's columns this warp drains
    const uint32_t epoch = *epoch_slot;
    int local = 0;
    int first_tile = blockIdx.x;
    if (reducing) {
      // peers' buffers are free for this launch once they have got far enough (see FusedComm)
      bool ok = true;
      if (lane < fc.n_ranks && lane != fc.rank)
        ok = wait_flag_sys(fc.rs_started[fc.rank] + lane, *need_slot, fc.budget);
      if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0) {
          report_status(status, kPeerTimeout, 11);
          *abort_flag = 1;
        }
        first_tile = num_units;
      }
    }
    for (int unit = first_tile; unit < num_units; unit += n_gemm_ctas, ++local) {
      const int tile = SPLITK ? unit % num_tiles : unit;
      const int buf = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      int m_blk, n_blk, owner;
      tile_coords(tile, m_blk, n_blk, owner);
      const int m0 = m_blk * kBM;
      const int n0 = n_blk * BN;
      if (!mbar_wait(&acc_full[buf], acc_phase, abort_flag, status, 4)) break;
      tc_fence_after();
      const int row = m0 + quad * 32 + lane;
      const bool row_ok = row < M;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * BN;
      if constexpr (SPLITK) {
        // Splits 0 .. splits-2 store their fp32 partial tile; the LAST split of a tile
        // keeps its own part in TMEM, waits for the others (they have lower unit
        // numbers, so they were started earlier and never wait themselves), adds them
        // in split order and runs the epilogue.  Workspace layout per (tile, split):
        // [chunk of 32 columns][quad][q][lane] float4, i.e. every store or load of a
        // warp is one 512-byte run.
        const int sp = unit / num_tiles;
        float4* ws_tile = reinterpret_cast<float4*>(ep.splitk_ws + static_cast<size_t>(tile) * (splits - 1) * kBM * BN);
        unsigned* cnt = ep.splitk_counters + tile;
        const unsigned all_in = 8u * static_cast<unsigned>(splits - 1);
        if (sp < splits - 1) {
          float4* mine = ws_tile + static_cast<size_t>(sp) * (kBM * BN / 4) + quad * 256 + lane;
#pragma unroll 1
          for (int c = half * (BN / 64); c < (half + 1) * (BN / 64); ++c) {
            uint32_t r[32];
            tmem_ld_32x32(t_row + c * 32, r);
            tmem_ld_wait();
            float4* dst = mine + c * 1024;
#pragma unroll
            for (int q = 0; q < 8; ++q)
              __stcg(dst + q * 32, make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                               __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3])));
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(&acc_empty[buf]);
            __threadfence();
            atomicAdd(cnt, 1u);
          }
          continue;
        }
        bool ok = true;
        if (lane == 0) {
          const long long t0 = clock64();
          while (ld_acquire_gpu(cnt) < all_in) {
            if (*abort_flag != 0 || clock64() - t0 > kWaitBudgetCycles) {
              if (*abort_flag == 0) report_status(status, kMbarTimeout, 18);
              *abort_flag = 1;
              ok = false;
              break;
            }
          }
        }
        if (!__all_sync(0xffffffffu, ok)) break;
        epilogue_columns<BN, false>(ep, fc, t_row, row, row_ok, n0, half, N,
                                    reinterpret_cast<const float*>(ws_tile + quad * 256 + lane),
                                    reinterpret_cast<uint4*>(smem + L::kTotal) + (warp - 2) * 256, lane, M);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&acc_empty[buf]);
          // the last of the eight warps to finish reading re-arms the counter
          if (atomicAdd(cnt, 1u) == all_in + 7u) atomicExch(cnt, 0u);
        }
        continue;
      }
      if (!reducing) {
        if (FUSED && BN == 256 && ep.mode == kEpiSwiGLU)
          epilogue_swiglu(ep, t_row, row, row_ok, n0, half,
                          reinterpret_cast<uint4*>(smem + L::kTotal) + (warp - 2) * 256, lane, M);
        else
          epilogue_columns<BN, FUSED>(ep, fc, t_row, row, row_ok, n0, half, N, nullptr,
                                      reinterpret_cast<uint4*>(smem + L::kTotal) + (warp - 2) * 256, lane, M);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);
        continue;
      }
      if constexpr (FUSED) {
      const bool own = owner == fc.rank;
      const int ftile = (row_local(fc, m0) / kBM) * tiles_n + n_blk;
      if (own) {
        // the peers computed this tile first: their partials are normally here already
        bool ok = true;
        if (lane < fc.n_ranks && lane != fc.rank)
          ok = wait_flag_sys(fused_flag(fc, fc.rank, 0, ftile, lane), epoch, fc.budget);
        if (!__all_sync(0xffffffffu, ok)) {
          if (lane == 0) {
            report_status(status, kPeerTimeout, 8);
            *abort_flag = 1;
          }
          break;
        }
      }
      epilogue_columns_reduce<BN>(ep, fc, t_row, m0, quad, lane, owner, n0, half, N, own,
                                  reinterpret_cast<uint4*>(smem + L::kTotal) + (warp - 2) * 256);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&acc_empty[buf]);
        mbar_arrive(&tile_done[buf]);
      }
      // One warp (a different one every tile) publishes the tile once all eight
      // have stored their part: a single system-scope fence + flag per tile.
      if (warp == 2 + (local & 7) && (!own || fc.rs_mode == 2)) {
        bool ok = true;
        if (lane == 0) ok = mbar_wait(&tile_done[buf], acc_phase, abort_flag, status, 9);
        if (!__all_sync(0xffffffffu, ok)) break;
        if (lane == 0) __threadfence_system();
        __syncwarp();
        if (!own) {
          if (lane == 0) st_release_sys(fused_flag(fc, owner, 0, ftile, fc.rank), epoch);
        } else if (lane < fc.n_ranks && lane != fc.rank) {
          st_release_sys(fused_flag(fc, lane, 1, ftile, fc.rank), epoch);
        }
      }
      }  // FUSED
    }
  }

  // Unwind.  After an aborted wait TMA writes may still be in flight: give
  // them time to land before the shared memory is handed back.
  if (*abort_flag != 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (reducing && fc.rs_mode == 2 && *abort_flag == 0) {
    // all-reduce: the kernel may only end once the other owners' final tiles
    // have landed in this rank's output (each CTA checks a share of them)
    const int per_owner = (fc.rows_per_rank / kBM) * tiles_n;
    const int total = (fc.n_ranks - 1) * per_owner;
    const uint32_t epoch = *epoch_slot;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += n_gemm_ctas * blockDim.x) {
      const int owner = (fc.rank + 1 + i / per_owner) % fc.n_ranks;
      if (!wait_flag_sys(fused_flag(fc, fc.rank, 1, i % per_owner, owner), epoch, fc.budget)) {
        report_status(status, kPeerTimeout, 10);
        break;
      }
    }
  }
  if (fused) fused_leave(fc, *epoch_slot);
}

// Two entry points around one body.  The plain GEMM is capped at 144 registers per
// thread: with 10 warps that leaves room on every SM sub-partition for one warp
// of the overlapped gradient all-reduce (<= 80 registers), which is what lets a
// block of it share the SM with a resident GEMM CTA.  The instantiation that
// carries the fused collectives, the rotary / SwiGLU epilogues or split-K may use
// what `__launch_bounds__` allows.
template <int BN, int STAGES, bool A_MN, bool B_MN>
__global__ void __maxnreg__(144)
gemm_plain_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, GemmEpilogue ep,
                  const __grid_constant__ FusedComm fc, int M, int N, int K, int* status) {
  gemm_bf16_body<BN, STAGES, A_MN, B_MN, false, false>(tma_a, tma_b, ep, fc, M, N, K, status);
}

template <int BN, int STAGES, bool A_MN, bool B_MN, bool FUSED, bool SPLITK = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 GemmEpilogue ep, const __grid_constant__ FusedComm fc, int M, int N, int K, int* status) {
  gemm_bf16_body<BN, STAGES, A_MN, B_MN, FUSED, SPLITK>(tma_a, tma_b, ep, fc, M, N, K, status);
}

// ---------------------------------------------------------------------------
// CTA-pair variant (tcgen05.mma.cta_group::2): a cluster of two CTAs computes a
// 256 x 256 tile.  Each CTA loads its own 128 rows of A and its own 128 rows
// (half) of B, so a k-block costs 32 KB of shared-memory fill and operand reads
// per CTA instead of 48 KB for the same 128 x 256 of output, which is what
// bounds the single-CTA kernel.  No multicast load: the halves differ.
//
//   warp 0      TMA producer (both CTAs): waits on its own CTA's empty barrier,
//               counts the bytes of its loads on the EVEN CTA's full barrier
//   warp 1      even CTA only: MMA issuer for the pair
//   warps 2..9  epilogue (both CTAs, own 128 rows of D)
// No thread relays a signal between the CTAs: the issuer's tcgen05.commit arrives
// on the empty / acc_full barrier of both CTAs at once, the odd CTA's loads
// complete on the even CTA's full barrier (its producer expects the bytes of
// both), and the odd CTA's epilogue warps arrive on the even CTA's acc_empty
// barriers once per tile.
// Optional cycle accounting of the roles of pair 0 (built only with
// -DNMB_GEMM_PROF; the counters go to the buffer passed as `aux_in` of a plain
// epilogue): where each role's time goes between waiting and working.
#ifdef NMB_GEMM_PROF
#define GP_DECL long long gp_t = clock64(); long long gp_acc[4] = {0, 0, 0, 0}; \
  long long* gp_out = (pair == 0 && ep.mode == kEpiPlain) ? reinterpret_cast<long long*>(const_cast<__nv_bfloat16*>(ep.aux_in)) : nullptr;
#define GP_LAP(k) do { const long long t = clock64(); gp_acc[k] += t - gp_t; gp_t = t; } while (0)
#define GP_STORE(base) do { if (gp_out != nullptr) for (int k = 0; k < 4; ++k) gp_out[(base) + k] = gp_acc[k]; } while (0)
#else
#define GP_DECL
#define GP_LAP(k)
#define GP_STORE(base)
#endif

struct GemmPairSmem {
  static constexpr int kStages = 6;
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = 128 * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = kStages * kStageBytes;
  // full, empty [kStages]; acc_full[2], acc_empty[2]; tmem slot, abort
  static constexpr int kTotal = kBarOffset + (2 * kStages + 4) * 8 + 16;
};

template <bool A_MN, bool B_MN>
__global__ void __maxnreg__(144)  // same cap and reason as gemm_plain_kernel
gemm_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 GemmEpilogue ep, const __grid_constant__ FusedComm fc, int M, int N, int K, int* status) {
  using L = GemmPairSmem;
  constexpr int BN = 256;
  constexpr int STAGES = L::kStages;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();
  const bool leader = cta == 0;
  const int pair = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;
  const int tiles_m = (M + 255) / 256;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + kBK - 1) / kBK;
  constexpr uint32_t kTmemCols = 512;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 16);  // 8 epilogue warps of each CTA
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);  // the whole TMEM: base 0 in both CTAs
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anyone signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_enter();  // set-up above touches no global memory

  if (warp == 0) {
    // ------------------------------------------------------------ producer --
    if (lane == 0) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // Both CTAs' loads count their bytes on the even CTA's full barrier.
      const uint32_t full0 = cluster_addr(&full_bar[0], 0);
      GP_DECL
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
        const int m0 = (tile % tiles_m) * 256 + static_cast<int>(cta) * 128;
        const int nb0 = (tile / tiles_m) * BN + static_cast<int>(cta) * 128;
        for (int kb = 0; kb < num_kb; ++kb) {
          // released in both CTAs at once by the issuer's commit
          if (!mbar_wait_cluster(&empty_bar[stage], phase ^ 1, abort_flag, status, 11)) {
            ok = false;
            break;
          }
          GP_LAP(0);  // waited for an empty stage
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          const uint32_t fb = full0 + stage * 8;
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * L::kStageBytes);
          if (!A_MN) {
            tma_load_2d_pair(sa, &tma_a, fb, kb * kBK, m0);
          } else {
#pragma unroll
            for (int c = 0; c < 2; ++c) tma_load_2d_pair(sa + c * 8192, &tma_a, fb, m0 + c * 64, kb * kBK);
          }
          if (!B_MN) {
            tma_load_2d_pair(sb, &tma_b, fb, kb * kBK, nb0);
          } else {
#pragma unroll
            for (int c = 0; c < 2; ++c) tma_load_2d_pair(sb + c * 8192, &tma_b, fb, nb0 + c * 64, kb * kBK);
          }
          GP_LAP(1);  // issued the loads
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      GP_STORE(leader ? 0 : 4);
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      // ---------------------------------------------- MMA issuer of the pair --
      constexpr uint32_t idesc = make_idesc_bf16(256, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      GP_DECL
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs, ++local) {
        const int buf = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait_cluster(&acc_empty[buf], acc_phase ^ 1, abort_flag, status, 12)) break;
        tc_fence_after();
        GP_LAP(0);  // waited for a free accumulator
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_cluster(&full_bar[stage], phase, abort_flag, status, 13)) {
            ok = false;
            break;
          }
          GP_LAP(1);  // waited for both CTAs' loads
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint32_t sb = sa + L::kABytes;
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t da = A_MN ? make_smem_desc(sa + k * 2048, 8192, 1024)
                                     : make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + k * 2048, 8192, 1024)
                                     : make_smem_desc(sb + k * 32, 16, 1024);
            tc_mma_bf16_pair(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          // the stage may be refilled in both CTAs once these MMAs have read it
          tc_commit_pair_both(&empty_bar[stage]);
          GP_LAP(3);  // issued MMAs + commit
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) tc_commit_pair_both(&acc_full[buf]);
      }
      GP_STORE(8);
    }
  } else {
    // ------------------------------------------------------------ epilogue --
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    int local = 0;
    for (int tile = pair; tile < num_tiles; tile += n_pairs, ++local) {
      const int buf = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      const int m0 = (tile % tiles_m) * 256 + static_cast<int>(cta) * 128;
      const int n0 = (tile / tiles_m) * BN;
      if (!mbar_wait_cluster(&acc_full[buf], acc_phase, abort_flag, status, 16)) break;
      tc_fence_after();
      const int row = m0 + quad * 32 + lane;
      const bool row_ok = row < M;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * BN;
      epilogue_columns<BN, false>(ep, fc, t_row, row, row_ok, n0, half, N, nullptr,
                                  reinterpret_cast<uint4*>(smem + L::kTotal) + (warp - 2) * 256, lane, M);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(cluster_addr(&acc_empty[buf], 0));
    }
  }

  if (*abort_flag != 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // nobody signals a CTA that has left, nobody's operands vanish under the issuer
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

static int g_pair_enabled = 1;
static int g_pair_clusters[2][2] = {{0, 0}, {0, 0}};  // co-resident clusters per variant (0 = not asked yet)

template <bool A_MN, bool B_MN>
static int launch_gemm_pair(const void* A, int lda, const void* B, int ldb, const GemmEpilogue& ep,
                            const FusedComm& fc, int M, int N, int K, int* status, cudaStream_t stream) {
  using L = GemmPairSmem;
  CUtensorMap ta, tb;
  int rc;
  if (!A_MN) {
    const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(lda) * 2};
    const uint32_t box[2] = {kBK, kBM};
    rc = make_tmap_bf16(&ta, A, 2, dims, strides, box);
  } else {
    const uint64_t dims[2] = {static_cast<uint64_t>(M), static_cast<uint64_t>(K)};
    const uint64_t strides[1] = {static_cast<uint64_t>(lda) * 2};
    const uint32_t box[2] = {64, kBK};
    rc = make_tmap_bf16(&ta, A, 2, dims, strides, box);
  }
  if (rc != 0) return 100 + rc;
  if (!B_MN) {
    const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
    const uint64_t strides[1] = {static_cast<uint64_t>(ldb) * 2};
    const uint32_t box[2] = {kBK, 128};
    rc = make_tmap_bf16(&tb, B, 2, dims, strides, box);
  } else {
    const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(K)};
    const uint64_t strides[1] = {static_cast<uint64_t>(ldb) * 2};
    const uint32_t box[2] = {64, kBK};
    rc = make_tmap_bf16(&tb, B, 2, dims, strides, box);
  }
  if (rc != 0) return 200 + rc;

  auto kern = gemm_pair_kernel<A_MN, B_MN>;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = L::kTotal + 1024 + kEpiStageBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // see pdl_wait()
  attr[1].val.programmaticStreamSerializationAllowed = g_pdl_enabled;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  int& resident = g_pair_clusters[A_MN][B_MN];
  if (resident == 0) {
    cfg.gridDim = dim3(2 * (sm_count() / 2));
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1) {
      (void)cudaGetLastError();
      n = sm_count() / 2 - 2;
    }
    resident = n;
  }
  const int tiles = ((M + 255) / 256) * ((N + 255) / 256);
  const int pairs = tiles < resident ? tiles : resident;
  cfg.gridDim = dim3(2 * pairs);
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ta, tb, ep, fc, M, N, K, status);
  return e == cudaSuccess ? 0 : 400 + static_cast<int>(e);
}

template <int BN, int STAGES, bool A_MN, bool B_MN, bool FUSED, bool SPLITK = false>
static int launch_gemm_impl(const void* A, int lda, const void* B, int ldb, const GemmEpilogue& ep, const FusedComm& fc,
                            int M, int N, int K, int* status, cudaStream_t stream) {
  using L = GemmSmem<BN, STAGES>;
  CUtensorMap ta, tb;
  int rc;
  if (!A_MN) {
    const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(lda) * 2};
    const uint32_t box[2] = {kBK, kBM};
    rc = make_tmap_bf16(&ta, A, 2, dims, strides, box);
  } else {
    const uint64_t dims[2] = {static_cast<uint64_t>(M), static_cast<uint64_t>(K)};
    const uint64_t strides[1] = {static_cast<uint64_t>(lda) * 2};
    const uint32_t box[2] = {64, kBK};
    rc = make_tmap_bf16(&ta, A, 2, dims, strides, box);
  }
  if (rc != 0) return 100 + rc;
  if (!B_MN) {
    const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
    const uint64_t strides[1] = {static_cast<uint64_t>(ldb) * 2};
    const uint32_t box[2] = {kBK, ep.mode == kEpiSwiGLU ? 128u : static_cast<uint32_t>(BN)};
    rc = make_tmap_bf16(&tb, B, 2, dims, strides, box);
  } else {
    const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(K)};
    const uint64_t strides[1] = {static_cast<uint64_t>(ldb) * 2};
    const uint32_t box[2] = {64, kBK};
    rc = make_tmap_bf16(&tb, B, 2, dims, strides, box);
  }
  if (rc != 0) return 200 + rc;

  void (*kern)(CUtensorMap, CUtensorMap, GemmEpilogue, FusedComm, int, int, int, int*);
  if constexpr (!FUSED && !SPLITK)
    kern = gemm_plain_kernel<BN, STAGES, A_MN, B_MN>;
  else
    kern = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN, FUSED, SPLITK>;
  const int smem_bytes = L::kTotal + 1024 + kEpiStageBytes;
  const int tiles = ((M + kBM - 1) / kBM) * ((N + BN - 1) / BN) * (SPLITK ? ep.splits : 1);
  int grid = tiles < sm_count() ? tiles : sm_count();
  if (fc.ag_copy_ctas > 0) {
    // the copy CTAs take SMs of their own; everything must be co-resident
    const int compute = sm_count() - fc.ag_copy_ctas;
    grid = (tiles < compute ? tiles : compute) + fc.ag_copy_ctas;
  }
  cudaError_t e;
  if (fc.rs_mode == 0 && fc.ag_copy_ctas == 0) {
    e = launch_pdl(kern, dim3(grid), dim3(kGemmThreads), smem_bytes, stream, ta, tb, ep, fc, M, N, K, status);
  } else {
    // kernels that wait for other GPUs keep plain stream ordering
    kern<<<grid, kGemmThreads, smem_bytes, stream>>>(ta, tb, ep, fc, M, N, K, status);
    e = cudaGetLastError();
  }
  return e == cudaSuccess ? 0 : 400 + static_cast<int>(e);
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
static int launch_gemm(const void* A, int lda, const void* B, int ldb, const GemmEpilogue& ep, const FusedComm& fc,
                       int M, int N, int K, int* status, cudaStream_t stream) {
  if (fc.rs_mode != 0 || fc.ag_copy_ctas > 0 || ep.mode >= kEpiRope) {
    // the fused collectives and the rotary / SwiGLU epilogues exist for K-major A only
    if constexpr (!A_MN)
      return launch_gemm_impl<BN, STAGES, A_MN, B_MN, true>(A, lda, B, ldb, ep, fc, M, N, K, status, stream);
    else
      return kBadArgument;
  }
  return launch_gemm_impl<BN, STAGES, A_MN, B_MN, false>(A, lda, B, ldb, ep, fc, M, N, K, status, stream);
}

// Split-K workspace of each device (registered by the host program: the launchers
// allocate nothing).  One workspace per device: split-K launches of one device
// must be ordered on one stream.
constexpr int kMaxDevices = 64;
static float* g_splitk_ws[kMaxDevices] = {nullptr};
static long long g_splitk_ws_bytes[kMaxDevices] = {0};
static unsigned* g_splitk_counters[kMaxDevices] = {nullptr};
static int g_splitk_n_counters[kMaxDevices] = {0};

// How many ways to cut K.  Cost model in units of one k-block of MMA time: a unit
// (tile x split) costs its k-blocks plus a fixed ~6 for the pipeline fill and the
// epilogue (+2 when partial tiles are exchanged), and the kernel takes as many
// rounds as the units need on the SMs.  A split is taken when the model says at
// least 10 % less than the unsplit kernel, each piece keeping >= 8 k-blocks.
static int choose_splits(int tiles, int num_kb, int dev) {
  if (dev < 0 || dev >= kMaxDevices || g_splitk_ws[dev] == nullptr) return 1;
  if (num_kb < 16 || tiles > g_splitk_n_counters[dev]) return 1;
  const int sms = sm_count();
  const long long base = static_cast<long long>((tiles + sms - 1) / sms) * (num_kb + 6);
  int best = 1;
  long long best_cost = base;
  for (int s = 2; s <= 8 && num_kb / s >= 8; ++s) {
    if (static_cast<long long>(tiles) * (s - 1) * kBM * 256 * 4 > g_splitk_ws_bytes[dev]) break;
    const long long rounds = (static_cast<long long>(tiles) * s + sms - 1) / sms;
    const long long cost = rounds * ((num_kb + s - 1) / s + 8);
    if (cost < best_cost) {
      best_cost = cost;
      best = s;
    }
  }
  return best_cost * 10 <= base * 9 ? best : 1;
}

template <bool A_MN, bool B_MN>
static int dispatch_tile(const void* A, int lda, const void* B, int ldb, const GemmEpilogue& ep, const FusedComm& fc,
                         int M, int N, int K, int* status, cudaStream_t stream) {
  if (ep.mode == kEpiSwiGLU) return launch_gemm<256, 4, A_MN, B_MN>(A, lda, B, ldb, ep, fc, M, N, K, status, stream);
  if constexpr (A_MN && B_MN) {
    // weight gradients: K is the token count, the output is small
    if (fc.ag_copy_ctas == 0 && fc.rs_mode == 0 && ep.mode == kEpiPlain && N > 128) {
      int dev = -1;
      cudaGetDevice(&dev);
      const int tiles = ((M + kBM - 1) / kBM) * ((N + 255) / 256);
      const int splits = choose_splits(tiles, (K + kBK - 1) / kBK, dev);
      if (splits > 1) {
        GemmEpilogue eps = ep;
        eps.splits = splits;
        eps.splitk_ws = g_splitk_ws[dev];
        eps.splitk_counters = g_splitk_counters[dev];
        return launch_gemm_impl<256, 4, A_MN, B_MN, false, true>(A, lda, B, ldb, eps, fc, M, N, K, status, stream);
      }
    }
  }
  if (g_pair_enabled && fc.ag_copy_ctas == 0 && fc.rs_mode == 0 && N >= 256 && ep.mode < kEpiRope) {
    const int pair_tiles = ((M + 255) / 256) * ((N + 255) / 256);
    if (pair_tiles * 3 >= sm_count() / 2)
      return launch_gemm_pair<A_MN, B_MN>(A, lda, B, ldb, ep, fc, M, N, K, status, stream);
  }
  const int tiles256 = ((M + kBM - 1) / kBM) * ((N + 255) / 256);
  // A 128 x 128 UMMA reads 8 KiB of operands from shared memory per 64 clocks,
  // i.e. the full 128 B/clk of the SM, and the TMA writes compete for the same
  // bandwidth; the 128 x 256 shape needs 25% less per FLOP.  Narrow tiles only
  // pay when the wide ones would leave most of the machine idle.
  if (N > 128 && tiles256 * 3 >= sm_count())
    return launch_gemm<256, 4, A_MN, B_MN>(A, lda, B, ldb, ep, fc, M, N, K, status, stream);
  return launch_gemm<128, 6, A_MN, B_MN>(A, lda, B, ldb, ep, fc, M, N, K, status, stream);
}

template <int BN, int STAGES, bool A_MN, bool B_MN, bool FUSED>
static int configure_gemm_impl() {
  void (*kern)(CUtensorMap, CUtensorMap, GemmEpilogue, FusedComm, int, int, int, int*);
  if constexpr (!FUSED)
    kern = gemm_plain_kernel<BN, STAGES, A_MN, B_MN>;
  else
    kern = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN, FUSED>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       GemmSmem<BN, STAGES>::kTotal + 1024 + kEpiStageBytes);
  // Every large kernel of the library asks for the maximum shared-memory
  // carve-out, and so do the communication kernels meant to run beside them: an
  // SM keeps one carve-out at a time, so kernels that prefer different ones
  // cannot share it and would serialise instead of overlapping.
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  return e == cudaSuccess ? 0 : 300 + static_cast<int>(e);
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
static int configure_gemm() {
  int rc = configure_gemm_impl<BN, STAGES, A_MN, B_MN, false>();
  if constexpr (!A_MN) rc |= configure_gemm_impl<BN, STAGES, A_MN, B_MN, true>();
  return rc;
}

template <bool A_MN, bool B_MN>
static int configure_gemm_pair() {
  cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       GemmPairSmem::kTotal + 1024 + kEpiStageBytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(gemm_pair_kernel<A_MN, B_MN>, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
  return e == cudaSuccess ? 0 : 300 + static_cast<int>(e);
}

}  // namespace nmb

// Opt every GEMM variant in to its dynamic shared memory size on the current
// device.  Called once per process (per device) right after the library is
// loaded, from the thread that loads it.
// Register (or, with null pointers, withdraw) the split-K workspace of the current
// device: `ws_bytes` of fp32 scratch and `n_counters` zero-initialised 32-bit
// counters, both owned by the caller for as long as GEMMs are launched.
extern "C" int nmb_gemm_set_splitk_workspace(void* ws, long long ws_bytes, void* counters, int n_counters) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= nmb::kMaxDevices) return nmb::kBadArgument;
  nmb::g_splitk_ws[dev] = static_cast<float*>(ws);
  nmb::g_splitk_ws_bytes[dev] = ws_bytes;
  nmb::g_splitk_counters[dev] = static_cast<unsigned*>(counters);
  nmb::g_splitk_n_counters[dev] = n_counters;
  return 0;
}

extern "C" int nmb_gemm_configure() {
  using namespace nmb;
  int rc = 0;
  {
    auto kern = gemm_bf16_kernel<256, 4, true, true, false, true>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<256, 4>::kTotal + 1024 + kEpiStageBytes);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) rc |= 300 + static_cast<int>(e);
  }
  rc |= configure_gemm<256, 4, false, false>();
  rc |= configure_gemm<256, 4, false, true>();
  rc |= configure_gemm<256, 4, true, true>();
  rc |= configure_gemm<256, 4, true, false>();
  rc |= configure_gemm<128, 6, false, false>();
  rc |= configure_gemm<128, 6, false, true>();
  rc |= configure_gemm<128, 6, true, true>();
  rc |= configure_gemm<128, 6, true, false>();
  rc |= configure_gemm_pair<false, false>();
  rc |= configure_gemm_pair<false, true>();
  rc |= configure_gemm_pair<true, true>();
  rc |= configure_gemm_pair<true, false>();
  return rc;
}

// Route eligible GEMMs (no fused collective, N >= 256, enough tiles) to the
// CTA-pair kernel.  Returns the previous setting.
extern "C" int nmb_gemm_set_pair(int enabled) {
  const int prev = nmb::g_pair_enabled;
  nmb::g_pair_enabled = enabled ? 1 : 0;
  return prev;
}

// C[M,N] = epilogue(alpha * A B^T).  `a_mn` / `b_mn` say that the operand is
// stored with its M/N index contiguous (i.e. as [K, M] / [K, N]).  Leading
// dimensions are in elements and must be multiples of 8 (TMA: 16-byte pitch);
// base pointers must be 16-byte aligned.  Returns 0 or a launch error code;
// device-side timeouts are reported through `status`.
static int gemm_entry(const void* A, int lda, int a_mn, const void* B, int ldb, int b_mn, void* C, int ldc, int M,
                      int N, int K, const void* bias, const void* residual, int ldr, void* aux_out,
                      const void* aux_in, int ld_aux, int mode, int accumulate, int out_f32, float alpha,
                      const nmb::FusedComm& fc, const nmb::NmbEpilogueExtra* extra, int* status, void* stream) {
  using namespace nmb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  (void)cudaGetLastError();  // a stale error of this host thread is not ours to report
  if ((lda % 8) != 0 || (ldb % 8) != 0) return kBadArgument;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return kBadArgument;
  GemmEpilogue ep;
  ep.c = C;
  ep.bias = static_cast<const __nv_bfloat16*>(bias);
  ep.residual = static_cast<const __nv_bfloat16*>(residual);
  ep.aux_out = static_cast<__nv_bfloat16*>(aux_out);
  ep.aux_in = static_cast<const __nv_bfloat16*>(aux_in);
  ep.ldc = ldc;
  ep.ldr = ldr;
  ep.ld_aux = ld_aux;
  ep.mode = mode;
  ep.accumulate = accumulate;
  ep.out_f32 = out_f32;
  ep.alpha = alpha;
  ep.rope_table = extra != nullptr ? static_cast<const float2*>(extra->rope_table) : nullptr;
  ep.rope_pos = extra != nullptr ? extra->rope_pos : nullptr;
  ep.rope_cols = extra != nullptr ? extra->rope_cols : 0;
  ep.rope_half = extra != nullptr ? extra->rope_half : 0;
  ep.swiglu_f = extra != nullptr ? extra->swiglu_f : 0;
  ep.splits = 1;
  ep.splitk_ws = nullptr;
  ep.splitk_counters = nullptr;
  if (mode == kEpiRope) {
    // whole 32-column chunks inside one head, 16-byte aligned table rows
    if (ep.rope_table == nullptr || ep.rope_pos == nullptr || ep.rope_half < 16 || (ep.rope_half % 16) != 0 ||
        (ep.rope_cols % (2 * ep.rope_half)) != 0 || ep.rope_cols > N || (N % 32) != 0 || out_f32 || accumulate ||
        (reinterpret_cast<uintptr_t>(ep.rope_table) & 15))
      return kBadArgument;
  }
  if (mode == kEpiSwiGLU) {
    // N = 2F rows of B = [gate; up]; C is [M, F], aux_out [M, 2F]
    if (ep.swiglu_f <= 0 || N != 2 * ep.swiglu_f || (ep.swiglu_f % 32) != 0 || a_mn || b_mn || aux_out == nullptr ||
        out_f32 || accumulate || residual != nullptr || fc.rs_mode != 0)
      return kBadArgument;
  }
  if (mode == kEpiDSwiGLU) {
    // N = F; C is [M, 2F] (d gate | d up), aux_in [M, 2F]
    if (ep.swiglu_f != N || (N % 32) != 0 || aux_in == nullptr || out_f32 || accumulate || residual != nullptr ||
        bias != nullptr || fc.rs_mode != 0)
      return kBadArgument;
  }
  const int celt = out_f32 ? 4 : 8;
  if (fc.rs_mode == 0 && ((ldc % celt) != 0 || (reinterpret_cast<uintptr_t>(C) & 15))) return kBadArgument;
  if (residual != nullptr && ((ldr % 8) != 0 || (reinterpret_cast<uintptr_t>(residual) & 15))) return kBadArgument;
  if ((aux_out != nullptr || aux_in != nullptr) && (ld_aux % 8) != 0) return kBadArgument;
  if (bias != nullptr && (reinterpret_cast<uintptr_t>(bias) & 15)) return kBadArgument;
  if (fc.rs_mode != 0 || fc.ag_copy_ctas > 0) {
    // fused collectives: whole 128-row tiles per shard, whole 32-column chunks
    if (fc.n_ranks < 2 || fc.n_ranks > kMaxRanks || fc.shard_len % kBM != 0 || M % fc.seq_len != 0 ||
        fc.seq_len != fc.shard_len * fc.n_ranks || N % 32 != 0 || out_f32 || accumulate)
      return kBadArgument;
    if (fc.rs_mode != 0 && (bias != nullptr || residual != nullptr || mode != kEpiPlain)) return kBadArgument;
    if (fc.rs_mode != 0 && (fc.rows_per_rank / kBM) * ((N + 127) / 128) > kMaxFusedTiles) return kTooLarge;
    if (fc.rs_mode != 0 && fc.ag_copy_ctas > 0) return kBadArgument;  // the two tile orders exclude each other
    if (fc.ag_copy_ctas > 0 && (a_mn || fc.ag_copy_ctas >= sm_count() / 2 || fc.ag_copy_ctas > 63)) return kBadArgument;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!a_mn && !b_mn) return dispatch_tile<false, false>(A, lda, B, ldb, ep, fc, M, N, K, status, s);
  if (!a_mn && b_mn) return dispatch_tile<false, true>(A, lda, B, ldb, ep, fc, M, N, K, status, s);
  if (a_mn && b_mn) return dispatch_tile<true, true>(A, lda, B, ldb, ep, fc, M, N, K, status, s);
  return dispatch_tile<true, false>(A, lda, B, ldb, ep, fc, M, N, K, status, s);
}

// C[M,N] = epilogue(alpha * A B^T).  `a_mn` / `b_mn` say that the operand is
// stored with its M/N index contiguous (i.e. as [K, M] / [K, N]).  Leading
// dimensions are in elements and must be multiples of 8 (TMA: 16-byte pitch);
// base pointers must be 16-byte aligned.  Returns 0 or a launch error code;
// device-side timeouts are reported through `status`.
extern "C" int nmb_gemm_bf16(const void* A, int lda, int a_mn, const void* B, int ldb, int b_mn,
                             void* C, int ldc, int M, int N, int K, const void* bias,
                             const void* residual, int ldr, void* aux_out, const void* aux_in,
                             int ld_aux, int mode, int accumulate, int out_f32, float alpha,
                             const void* extra, int* status, void* stream) {
  nmb::FusedComm fc;
  memset(&fc, 0, sizeof(fc));
  return gemm_entry(A, lda, a_mn, B, ldb, b_mn, C, ldc, M, N, K, bias, residual, ldr, aux_out, aux_in, ld_aux, mode,
                    accumulate, out_f32, alpha, fc, static_cast<const nmb::NmbEpilogueExtra*>(extra), status, stream);
}

// The same GEMM with a collective fused in (see FusedComm).  `comm` has the
// layout of nmb::FusedComm.  With a fused reduce, `bias` is added by the owner
// of each row block after the reduction (comm->rs_bias / rs_residual).
extern "C" int nmb_gemm_bf16_fused(const void* A, int lda, int a_mn, const void* B, int ldb, int b_mn, void* C,
                                   int ldc, int M, int N, int K, const void* bias, void* aux_out,
                                   int mode, float alpha, const void* comm, const void* extra, int* status,
                                   void* stream) {
  const nmb::FusedComm* fc = static_cast<const nmb::FusedComm*>(comm);
  const bool rs = fc->rs_mode != 0;
  return gemm_entry(A, lda, a_mn, B, ldb, b_mn, C, ldc, M, N, K, rs ? nullptr : bias, nullptr, 0,
                    rs ? nullptr : aux_out, nullptr, mode == nmb::kEpiSwiGLU ? N : N, rs ? nmb::kEpiPlain : mode, 0, 0,
                    alpha, *fc, static_cast<const nmb::NmbEpilogueExtra*>(extra), status, stream);
}

extern "C" int nmb_fused_max_tiles() { return nmb::kMaxFusedTiles; }

extern "C" int nmb_fused_comm_size() { return static_cast<int>(sizeof(nmb::FusedComm)); }
