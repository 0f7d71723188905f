// Causal flash attention forward / backward on tcgen05 tensor cores.
//
// Replaces the flash-attn 2.x calls of the reference
// (nano_megatron/parallel/attention_backend.py:216-223 forward,
// :497-514 chunked backward) and, because the key/value side is described by
// up to eight tensor maps ("chunks"), also the context-parallel path
// (:355-530, :549-635): each chunk may live in another GPU's memory and is
// fetched tile by tile with plain (non-multicast) TMA loads, so no gathered
// K/V copy is ever materialised and the online-softmax merge across chunks
// happens in registers.
//
// Layout: all tensors are addressed through 4-D tensor maps
// {head_dim, seq, heads, batch} with arbitrary strides, so the fused-QKV GEMM
// output [B*S, 3H] is consumed in place and the context is written in the
// [B*S, H] layout the output projection reads -- none of the
// split-heads / merge-heads / repeat_kv copies of the reference
// (nano_megatron/model/tp_gpt.py:171-187) exist here.
//
// Forward CTA = one 128-row query tile of one head; 320 threads:
//   warps 0-7  online softmax (two threads per query row, 64 columns each), O rescale, epilogue
//   warp 8     TMA producer (K/V double buffered)
//   warp 9     TMEM owner + tcgen05.mma issuer
// Both kernels run on one-dimensional grids ordered longest work first.
// S = Q K^T lives in TMEM (128 fp32 columns), P is written back to shared
// memory as a K-major bf16 operand, O accumulates in TMEM.
//
// Backward CTA = one 128-row key/value tile of one KV head, looping over the
// query tiles that can see it; dK/dV accumulate in TMEM, dQ tiles are added
// to an fp32 buffer with reductions.
#include "common.cuh"

namespace nmb {

constexpr int kMaxChunks = 8;
constexpr int kAttnThreads = 320;  // 8 softmax warps, TMA warp, MMA warp
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;  // log2 of the growth tolerated before O is rescaled

// Bulk (TMA) reduce-add of a contiguous fp32 span from shared to global memory.
__device__ __forceinline__ void bulk_reduce_add_f32(float* gdst, const float* ssrc, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(gdst),
               "r"(smem_u32(ssrc)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// 64-thread barrier of the two warps that share TMEM lane quadrant `quad`
// (barriers 1..4; 0 is __syncthreads).  Immediate ids keep the kernel's barrier
// count at five.
__device__ __forceinline__ void quad_pair_sync(int quad) {
  switch (quad) {
    case 0: asm volatile("bar.sync 1, 64;" ::: "memory"); break;
    case 1: asm volatile("bar.sync 2, 64;" ::: "memory"); break;
    case 2: asm volatile("bar.sync 3, 64;" ::: "memory"); break;
    default: asm volatile("bar.sync 4, 64;" ::: "memory"); break;
  }
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Cycle accounting of the forward kernel (profiling builds, -DNMB_ATTN_PROF): the
// first softmax thread and the MMA thread of CTA (0, 0, 0) add up where their time
// goes; nmb_attn_fwd_prof_read() copies the counters out.
#ifdef NMB_ATTN_PROF
__device__ long long g_attn_fwd_prof[16];
__device__ unsigned long long g_attn_fwd_span[4096][2];  // per CTA: start / end of its life, ns (globaltimer)
__device__ unsigned long long g_attn_fwd_marks[4096][4];  // per CTA: set-up done, first S, loop end, O written
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define FP_DECL(on) const bool fp_on = (on) && blockIdx.x == 0; long long fp_t = clock64(); long long fp_acc[6] = {0, 0, 0, 0, 0, 0};
#define FP_LAP(k) do { if (fp_on) { const long long t = clock64(); fp_acc[k] += t - fp_t; fp_t = t; } } while (0)
#define FP_STORE(base) do { if (fp_on) for (int k = 0; k < 6; ++k) g_attn_fwd_prof[(base) + k] = fp_acc[k]; } while (0)
#else
#define FP_DECL(on)
#define FP_LAP(k)
#define FP_STORE(base)
#endif

struct AttnFwdParams {
  CUtensorMap q_map;
  CUtensorMap k_map[kMaxChunks];
  CUtensorMap v_map[kMaxChunks];
  __nv_bfloat16* o;
  float* lse;  // [B, Hq, Sq]
  long long o_stride_b, o_stride_s, o_stride_h;
  int B, Hq, Hkv, Sq;
  int chunk_len, n_chunks;
  int d;       // true head dim (64, 96 or 128)
  int q_pos0;  // global position of query row 0 (context parallel offset)
  float scale;
  int* status;
};

template <int HD>
struct AttnFwdSmem {
  static constexpr int kSlabs = HD / 64;
  static constexpr int kTile = kSlabs * 16384;   // one 128 x HD bf16 tile
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kTile;          // 2 stages
  static constexpr int kV = kK + 2 * kTile;      // 2 stages
  static constexpr int kP = kV + 2 * kTile;      // 128 x 128 bf16
  static constexpr int kBar = kP + 32768;
  static constexpr int kNumBars = 9;
  static constexpr int kXch = kBar + kNumBars * 8 + 16;  // tile maxima of the two threads of a row, bf16 [2][128]
  static constexpr int kTotal = kXch + 512;
};

template <int HD>
__global__ void __launch_bounds__(kAttnThreads, HD == 64 ? 2 : 1)
attn_fwd_kernel(const __grid_constant__ AttnFwdParams p) {
  using L = AttnFwdSmem<HD>;
  constexpr int NS = L::kSlabs;
#ifdef NMB_ATTN_PROF
  if (threadIdx.x == 0 && blockIdx.x < 4096) g_attn_fwd_span[blockIdx.x][0] = global_ns();
#endif
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBar);
  uint64_t* q_full = &bars[0];
  uint64_t* kv_full = &bars[1];   // [2]
  uint64_t* kv_empty = &bars[3];  // [2]
  uint64_t* s_full = &bars[5];
  uint64_t* s_empty = &bars[6];
  uint64_t* p_full = &bars[7];
  uint64_t* o_full = &bars[8];
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(&bars[L::kNumBars]);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // One-dimensional grid, longest work first across the WHOLE grid: block i takes
  // query tile n_q_tiles - 1 - i / (heads * batch), so the causal tiles with the
  // most key tiles start first on every SM and the short ones fill the tail
  // (with (tile, head, batch) as a 3-D grid the tile index ran fastest, long and
  // short CTAs were interleaved and the last long ones started late).
  const int n_q_tiles = (p.Sq + 127) / 128;
  const int n_hb = p.Hq * p.B;
  const int qt = n_q_tiles - 1 - static_cast<int>(blockIdx.x) / n_hb;
  const int h = (static_cast<int>(blockIdx.x) % n_hb) % p.Hq;
  const int b = (static_cast<int>(blockIdx.x) % n_hb) / p.Hq;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qt * 128;
  const int skv_total = p.chunk_len * p.n_chunks;
  int q_last = q0 + 127;
  if (q_last > p.Sq - 1) q_last = p.Sq - 1;
  int n_kv = (p.q_pos0 + q_last + 128) / 128;  // ceil((last_pos + 1) / 128)
  const int max_kv = (skv_total + 127) / 128;
  if (n_kv > max_kv) n_kv = max_kv;
  constexpr uint32_t kTmemCols = 256;  // S: 128, O: HD <= 128
  constexpr uint32_t kSCol = 0, kOCol = 128;

  if ((smem_u32(smem) & 1023u) != 0) {  // swizzled operands need 1 KiB alignment
    if (threadIdx.x == 0) report_status(p.status, kBadArgument, 20);
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_empty, 256);
    mbar_init(p_full, 256);
    mbar_init(o_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_enter();  // the set-up above touches no global memory
#ifdef NMB_ATTN_PROF
  if (threadIdx.x == 0 && blockIdx.x < 4096) g_attn_fwd_marks[blockIdx.x][0] = global_ns();
#endif

  if (warp == 8) {
    // ------------------------------------------------------------ producer --
    if (lane == 0) {
      tma_prefetch_desc(&p.q_map);
      mbar_expect_tx(q_full, L::kTile);
#pragma unroll
      for (int c = 0; c < NS; ++c)
        tma_load_4d(smem + L::kQ + c * 16384, &p.q_map, q_full, c * 64, q0, h, b);
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        if (j >= 2 && !mbar_wait(&kv_empty[st], ((j >> 1) - 1) & 1, abort_flag, p.status, 21)) break;
        const int chunk = (j * 128) / p.chunk_len;
        const int row0 = j * 128 - chunk * p.chunk_len;
        mbar_expect_tx(&kv_full[st], 2 * L::kTile);
#pragma unroll
        for (int c = 0; c < NS; ++c) {
          tma_load_4d(smem + L::kK + st * L::kTile + c * 16384, &p.k_map[chunk], &kv_full[st], c * 64,
                      row0, hk, b);
          tma_load_4d(smem + L::kV + st * L::kTile + c * 16384, &p.v_map[chunk], &kv_full[st], c * 64,
                      row0, hk, b);
        }
      }
    }
  } else if (warp == 9) {
    // ---------------------------------------------------------- MMA issuer --
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(128, HD, false, true);
      const uint32_t sQ = smem_u32(smem + L::kQ);
      const uint32_t sP = smem_u32(smem + L::kP);
      auto issue_qk = [&](int j) {
        const uint32_t sK = smem_u32(smem + L::kK + (j & 1) * L::kTile);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          tc_mma_bf16(tmem_base + kSCol, make_smem_desc(sQ + off, 16, 1024),
                      make_smem_desc(sK + off, 16, 1024), idesc_qk, k != 0 ? 1u : 0u);
        }
        tc_commit(s_full);
      };
      FP_DECL(true)
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, 22) &&
                mbar_wait(&kv_full[0], 0, abort_flag, p.status, 23);
      if (ok) {
        tc_fence_after();
        issue_qk(0);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) {
          // S is single buffered: the next QK^T may start once the softmax
          // warps have read S_j; it then overlaps their P write / O rescale.
          if (!mbar_wait(&kv_full[(j + 1) & 1], ((j + 1) >> 1) & 1, abort_flag, p.status, 24) ||
              !mbar_wait(s_empty, j & 1, abort_flag, p.status, 25)) {
            ok = false;
            break;
          }
          FP_LAP(0);  // waited for K/V of the next tile and for S to be read
          tc_fence_after();
          issue_qk(j + 1);
          FP_LAP(1);  // issued QK^T
        }
        if (!mbar_wait(p_full, j & 1, abort_flag, p.status, 26)) {
          ok = false;
          break;
        }
        FP_LAP(2);  // waited for P
        tc_fence_after();
        const uint32_t sV = smem_u32(smem + L::kV + (j & 1) * L::kTile);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          tc_mma_bf16(tmem_base + kOCol,
                      make_smem_desc(sP + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024),
                      make_smem_desc(sV + k * 2048, 16384, 1024), idesc_pv, (j | k) != 0 ? 1u : 0u);
        }
        tc_commit(o_full);
        tc_commit(&kv_empty[j & 1]);
        FP_LAP(3);  // issued PV
      }
      FP_STORE(8);
    }
  } else {
    // ------------------------------------------------- softmax + epilogue --
    // Eight warps, two threads per query row: warp w owns TMEM lanes (rows)
    // 32 * (w & 3) .. + 31 and columns 64 * (w >> 2) .. + 63 of S, and the same
    // half of O's columns.  The two threads of a row agree on the tile maximum
    // through shared memory (each rounds its own maximum UP to bf16 first, so
    // both compute the same value from the same pair) under a 64-thread named
    // barrier of their quad, and add their row sums at the end.
    const int quad = warp & 3;
    const int half = warp >> 2;
    const int r = quad * 32 + lane;  // query row in the tile == TMEM lane
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    __nv_bfloat16* xch = reinterpret_cast<__nv_bfloat16*>(smem + L::kXch);  // [2 halves][128 rows]
    const int q_row = q0 + r;
    const int q_pos = p.q_pos0 + q_row;
    const float sl2 = p.scale * kLog2e;
    float m_run = -INFINITY;
    float l_run = 0.f;
    bool ok = true;
    FP_DECL(threadIdx.x == 0)
    for (int j = 0; j < n_kv; ++j) {
      if (!mbar_wait(s_full, j & 1, abort_flag, p.status, 27)) {
        ok = false;
        break;
      }
      FP_LAP(0);  // waited for S
#ifdef NMB_ATTN_PROF
      if (j == 0 && threadIdx.x == 0 && blockIdx.x < 4096) g_attn_fwd_marks[blockIdx.x][1] = global_ns();
#endif
      tc_fence_after();
      const int kv0 = j * 128;
      // A tile is "full" when every key of it is visible to every query row of
      // this CTA: then no per-element masking is needed (CTA-uniform test).
      const bool tile_full = (kv0 + 127 <= p.q_pos0 + q0) && (kv0 + 128 <= skv_total);
      int limit = q_pos - kv0;                       // columns <= limit are visible
      if (skv_total - 1 - kv0 < limit) limit = skv_total - 1 - kv0;
      // pass 1: maximum of this thread's 64 columns
      float mx = -INFINITY;
      if (tile_full) {
        uint32_t sa[32], sb[32];
        tmem_ld_32x32(t_lane + kSCol + half * 64, sa);
        tmem_ld_32x32(t_lane + kSCol + half * 64 + 32, sb);
        tmem_ld_wait();
        float m0 = __uint_as_float(sa[0]), m1 = __uint_as_float(sb[0]);
#pragma unroll
        for (int jj = 1; jj < 32; ++jj) {
          m0 = fmaxf(m0, __uint_as_float(sa[jj]));
          m1 = fmaxf(m1, __uint_as_float(sb[jj]));
        }
        mx = fmaxf(m0, m1);
      } else {
#pragma unroll 1
        for (int c = half * 2; c < half * 2 + 2; ++c) {
          uint32_t sr[32];
          tmem_ld_32x32(t_lane + kSCol + c * 32, sr);
          tmem_ld_wait();
#pragma unroll
          for (int jj = 0; jj < 32; ++jj)
            if (c * 32 + jj <= limit) mx = fmaxf(mx, __uint_as_float(sr[jj]));
        }
      }
      FP_LAP(1);  // pass 1
      {
        const __nv_bfloat16 mine = __float2bfloat16_ru(mx);
        xch[half * 128 + r] = mine;
        quad_pair_sync(quad);
        mx = fmaxf(__bfloat162float(mine), __bfloat162float(xch[(half ^ 1) * 128 + r]));
        quad_pair_sync(quad);  // both have read before either writes the next tile's value
      }
      FP_LAP(2);  // exchanged the maximum
      // Lazy rescaling: the reference maximum only moves when the tile maximum
      // exceeds it by more than 2^8 in the exponent domain, so most tiles need
      // no pass over O; the final division by l makes the result exact.
      float m_new = m_run;
      if (mx > m_run + kRescaleThreshold / sl2) m_new = mx;
      const float alpha = (m_new == m_run) ? 1.f : ((m_run == -INFINITY) ? 0.f : fast_exp2((m_run - m_new) * sl2));
      const float neg_m = (m_new == -INFINITY) ? 0.f : -m_new * sl2;
      // pass 2: probabilities of this thread's 64 columns
      uint32_t pk[32];
      float rowsum = 0.f;
      if (tile_full) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t sr[32];
          tmem_ld_32x32(t_lane + kSCol + half * 64 + c * 32, sr);
          tmem_ld_wait();
          float r0 = 0.f, r1 = 0.f;
#pragma unroll
          for (int jj = 0; jj < 32; jj += 2) {
            const float p0 = fast_exp2(fmaf(__uint_as_float(sr[jj]), sl2, neg_m));
            const float p1 = fast_exp2(fmaf(__uint_as_float(sr[jj + 1]), sl2, neg_m));
            r0 += p0;
            r1 += p1;
            pk[c * 16 + jj / 2] = pack_bf16x2(p0, p1);
          }
          rowsum += r0 + r1;
        }
      } else {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t sr[32];
          tmem_ld_32x32(t_lane + kSCol + half * 64 + c * 32, sr);
          tmem_ld_wait();
          const int col0 = half * 64 + c * 32;
#pragma unroll
          for (int jj = 0; jj < 32; jj += 2) {
            const float p0 = (col0 + jj <= limit) ? fast_exp2(fmaf(__uint_as_float(sr[jj]), sl2, neg_m)) : 0.f;
            const float p1 = (col0 + jj + 1 <= limit) ? fast_exp2(fmaf(__uint_as_float(sr[jj + 1]), sl2, neg_m)) : 0.f;
            rowsum += p0 + p1;
            pk[c * 16 + jj / 2] = pack_bf16x2(p0, p1);
          }
        }
      }
      tc_fence_before();
      mbar_arrive(s_empty);
      FP_LAP(3);  // pass 2
      l_run = l_run * alpha + rowsum;
      m_run = m_new;
      if (j > 0) {
        if (!mbar_wait(o_full, (j - 1) & 1, abort_flag, p.status, 28)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
          for (int c = half * (HD / 64); c < (half + 1) * (HD / 64); ++c) {
            uint32_t orr[32];
            tmem_ld_32x32(t_lane + kOCol + c * 32, orr);
            tmem_ld_wait();
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) orr[jj] = __float_as_uint(__uint_as_float(orr[jj]) * alpha);
            tmem_st_32x32(t_lane + kOCol + c * 32, orr);
          }
          tmem_st_wait();
        }
      }
      FP_LAP(4);  // waited for the previous PV, rescaled O if needed
      // P -> shared memory, K-major, 128-byte swizzle: this thread's 64 columns
      // are one row of slab `half`.
      uint8_t* sp = smem + L::kP + half * 16384;
#pragma unroll
      for (int c16 = 0; c16 < 8; ++c16) {
        uint4 u = make_uint4(pk[c16 * 4], pk[c16 * 4 + 1], pk[c16 * 4 + 2], pk[c16 * 4 + 3]);
        *reinterpret_cast<uint4*>(sp + swz128_offset(r, c16)) = u;
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_full);
      FP_LAP(5);  // stored P
    }
    FP_STORE(0);
#ifdef NMB_ATTN_PROF
    if (threadIdx.x == 0 && blockIdx.x < 4096) g_attn_fwd_marks[blockIdx.x][2] = global_ns();
#endif
    if (ok && mbar_wait(o_full, (n_kv - 1) & 1, abort_flag, p.status, 29)) {
      tc_fence_after();
      // every MMA has completed: the P buffer is free and carries the row sums
      float* lx = reinterpret_cast<float*>(smem + L::kP);
      lx[half * 128 + r] = l_run;
      quad_pair_sync(quad);
      const float l_tot = l_run + lx[(half ^ 1) * 128 + r];
      const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
      __nv_bfloat16* orow = p.o + b * p.o_stride_b + static_cast<long long>(q_row) * p.o_stride_s +
                            h * p.o_stride_h;
#pragma unroll 1
      for (int c = half * (HD / 64); c < (half + 1) * (HD / 64); ++c) {
        uint32_t orr[32];
        tmem_ld_32x32(t_lane + kOCol + c * 32, orr);
        tmem_ld_wait();
        if (q_row < p.Sq && c * 32 < p.d) {
          uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 u;
            u.x = pack_bf16x2(__uint_as_float(orr[q * 8 + 0]) * inv, __uint_as_float(orr[q * 8 + 1]) * inv);
            u.y = pack_bf16x2(__uint_as_float(orr[q * 8 + 2]) * inv, __uint_as_float(orr[q * 8 + 3]) * inv);
            u.z = pack_bf16x2(__uint_as_float(orr[q * 8 + 4]) * inv, __uint_as_float(orr[q * 8 + 5]) * inv);
            u.w = pack_bf16x2(__uint_as_float(orr[q * 8 + 6]) * inv, __uint_as_float(orr[q * 8 + 7]) * inv);
            dst[q] = u;
          }
        }
      }
      if (half == 0 && q_row < p.Sq)
        p.lse[(static_cast<long long>(b) * p.Hq + h) * p.Sq + q_row] = m_run * p.scale + logf(l_tot);
    }
  }

#ifdef NMB_ATTN_PROF
  if (threadIdx.x == 0 && blockIdx.x < 4096) g_attn_fwd_marks[blockIdx.x][3] = global_ns();
#endif
  if (*abort_flag != 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
#ifdef NMB_ATTN_PROF
  if (threadIdx.x == 0 && blockIdx.x < 4096) g_attn_fwd_span[blockIdx.x][1] = global_ns();
#endif
}

// ------------------------------------------------------------------ backward --
struct AttnBwdParams {
  CUtensorMap q_map;
  CUtensorMap do_map;
  CUtensorMap k_map[kMaxChunks];
  CUtensorMap v_map[kMaxChunks];
  __nv_bfloat16* dk[kMaxChunks];  // per chunk: where this rank's dK / dV tiles go
  __nv_bfloat16* dv[kMaxChunks];
  long long dkv_stride_b, dkv_stride_s, dkv_stride_h;
  const float* lse;    // [B, Hq, Sq]
  const float* delta;  // [B, Hq, Sq]  rowsum(dO * O)
  float* dq_acc;       // [B, Hq, Sq, d] fp32 (chunk-swizzled rows), zero-initialised
  int B, Hq, Hkv, Sq;
  int chunk_len, n_chunks;
  int d;
  int q_pos0;
  float scale;
  int* status;
#ifdef NMB_ATTN_PROF
  long long* prof;  // [8] cycle counters of CTA (0,0,0), thread 0 (profiling builds only)
#endif
};

#ifdef NMB_ATTN_PROF
#define NMB_PROF_DECL long long pt0 = 0, pacc[6] = {0, 0, 0, 0, 0, 0}; const bool prof_on = blockIdx.x == 0 && threadIdx.x == 0;
#define NMB_PROF_START() do { if (prof_on) pt0 = clock64(); } while (0)
#define NMB_PROF_LAP(k) do { if (prof_on) { const long long t = clock64(); pacc[k] += t - pt0; pt0 = t; } } while (0)
#define NMB_PROF_STORE() do { if (prof_on) { for (int k = 0; k < 6; ++k) p.prof[k] = pacc[k]; p.prof[6] = n_iter; } } while (0)
#else
#define NMB_PROF_DECL
#define NMB_PROF_START()
#define NMB_PROF_LAP(k)
#define NMB_PROF_STORE()
#endif

template <int HD>
struct AttnBwdSmem {
  static constexpr int kSlabs = HD / 64;
  static constexpr int kTile = kSlabs * 16384;
  static constexpr int kQStages = HD == 64 ? 2 : 1;
  static constexpr int kK = 0;
  static constexpr int kV = kK + kTile;
  static constexpr int kQ = kV + kTile;
  static constexpr int kDO = kQ + kQStages * kTile;
  static constexpr int kP = kDO + kQStages * kTile;
  static constexpr int kDS = kP + 32768;
  // fp32 staging of the dQ tile for the bulk reduce-add (128 rows x d floats,
  // 16-byte chunks XOR-swizzled by the row so that row-per-thread writes are
  // conflict free).  HD == 64: its own buffer; HD == 128: aliases P + dS.
  static constexpr bool kStageAlias = HD > 64;
  static constexpr int kStage = kStageAlias ? kP : kDS + 32768;
  static constexpr int kStageBytes = kStageAlias ? 0 : 128 * HD * 4;
  static constexpr int kBar = kDS + 32768 + kStageBytes;
  static constexpr int kNumBars = 1 + 2 * kQStages + 8;
  static constexpr int kTotal = kBar + kNumBars * 8 + 16;
};

constexpr int kBwdThreads = 320;       // 8 compute warps, TMA warp, MMA warp
constexpr int kBwdCompute = 256;

template <int HD>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ AttnBwdParams p) {
  using L = AttnBwdSmem<HD>;
  constexpr int NS = L::kSlabs;
  constexpr int QS = L::kQStages;
  constexpr bool kAliasDQ = HD > 64;  // dQ reuses the S columns when TMEM is full
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBar);
  uint64_t* kv_full = &bars[0];
  uint64_t* q_full = &bars[1];          // [QS]
  uint64_t* q_empty = &bars[1 + QS];    // [QS]
  uint64_t* sdp_full = &bars[1 + 2 * QS];
  uint64_t* pds_full = sdp_full + 1;    // P / dS written to shared memory (256 arrivals)
  uint64_t* dq_full = sdp_full + 2;     // [2] dQ MMAs of tile j done: barrier j & 1, phase j >> 1
  uint64_t* dq_empty = sdp_full + 4;    // [2] dQ of tile j read out of TMEM (256 arrivals)
  uint64_t* pds_free = sdp_full + 6;    // dV / dK (and dQ) MMAs done: P / dS / Q / dO stage reusable
  uint64_t* sdp_read = sdp_full + 7;    // S / dP copied to registers (256 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(&bars[L::kNumBars]);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // One-dimensional grid, longest work first: the lowest key tiles are visible to
  // the most query tiles, so all (head, batch) pairs of key tile 0 come first.
  const int n_hb = p.Hkv * p.B;
  const int kvt = static_cast<int>(blockIdx.x) / n_hb;
  const int hk = (static_cast<int>(blockIdx.x) % n_hb) % p.Hkv;
  const int b = (static_cast<int>(blockIdx.x) % n_hb) / p.Hkv;
  const int group = p.Hq / p.Hkv;
  const int kv0 = kvt * 128;
  const int chunk = kv0 / p.chunk_len;
  const int kv_row0 = kv0 - chunk * p.chunk_len;
  const int skv_total = p.chunk_len * p.n_chunks;
  const int n_q_tiles = (p.Sq + 127) / 128;
  int qt_first = 0;
  if (kv0 > p.q_pos0) qt_first = (kv0 - p.q_pos0) / 128;
  const int per_head = n_q_tiles > qt_first ? n_q_tiles - qt_first : 0;
  const int n_iter = per_head * group;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kSCol = 0, kDPCol = 128, kDVCol = 256, kDKCol = 256 + HD;
  // HD == 64 leaves room for two dQ accumulators (tile j uses j & 1)
  constexpr uint32_t kDQCol = kAliasDQ ? 0 : 256 + 2 * HD;
  constexpr uint32_t kDQStep = kAliasDQ ? 0 : HD;

  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) report_status(p.status, kBadArgument, 40);
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < QS; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
    }
    mbar_init(sdp_full, 1);
    mbar_init(pds_full, kBwdCompute);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&dq_full[s], 1);
      mbar_init(&dq_empty[s], kBwdCompute);
    }
    mbar_init(pds_free, 1);
    mbar_init(sdp_read, kBwdCompute);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_enter();  // the set-up above touches no global memory

  if (warp == 8) {
    // ------------------------------------------------------------ producer --
    if (lane == 0 && n_iter > 0) {
      mbar_expect_tx(kv_full, 2 * L::kTile);
#pragma unroll
      for (int c = 0; c < NS; ++c) {
        tma_load_4d(smem + L::kK + c * 16384, &p.k_map[chunk], kv_full, c * 64, kv_row0, hk, b);
        tma_load_4d(smem + L::kV + c * 16384, &p.v_map[chunk], kv_full, c * 64, kv_row0, hk, b);
      }
      for (int i = 0; i < n_iter; ++i) {
        const int st = i % QS;
        const int use = i / QS;
        if (use >= 1 && !mbar_wait(&q_empty[st], (use - 1) & 1, abort_flag, p.status, 41)) break;
        const int hq = hk * group + i / per_head;
        const int q0 = (qt_first + i % per_head) * 128;
        mbar_expect_tx(&q_full[st], 2 * L::kTile);
#pragma unroll
        for (int c = 0; c < NS; ++c) {
          tma_load_4d(smem + L::kQ + st * L::kTile + c * 16384, &p.q_map, &q_full[st], c * 64, q0, hq, b);
          tma_load_4d(smem + L::kDO + st * L::kTile + c * 16384, &p.do_map, &q_full[st], c * 64, q0, hq, b);
        }
      }
    }
  } else if (warp == 9) {
    // ---------------------------------------------------------- MMA issuer --
    if (lane == 0 && n_iter > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);   // S, dP
      constexpr uint32_t idesc_kv = make_idesc_bf16(128, HD, true, true);     // dV, dK
      constexpr uint32_t idesc_dq = make_idesc_bf16(128, HD, false, true);    // dQ
      const uint32_t sK = smem_u32(smem + L::kK);
      const uint32_t sV = smem_u32(smem + L::kV);
      const uint32_t sP = smem_u32(smem + L::kP);
      const uint32_t sDS = smem_u32(smem + L::kDS);
      auto issue_sdp = [&](int i) {
        const uint32_t sQ = smem_u32(smem + L::kQ + (i % QS) * L::kTile);
        const uint32_t sDO = smem_u32(smem + L::kDO + (i % QS) * L::kTile);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          tc_mma_bf16(tmem_base + kSCol, make_smem_desc(sQ + off, 16, 1024),
                      make_smem_desc(sK + off, 16, 1024), idesc_s, k != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          tc_mma_bf16(tmem_base + kDPCol, make_smem_desc(sDO + off, 16, 1024),
                      make_smem_desc(sV + off, 16, 1024), idesc_s, k != 0 ? 1u : 0u);
        }
        tc_commit(sdp_full);
      };
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.status, 42) &&
                mbar_wait(&q_full[0], 0, abort_flag, p.status, 43);
      if (ok) {
        tc_fence_after();
        issue_sdp(0);
      }
      for (int i = 0; i < n_iter && ok; ++i) {
        if (!kAliasDQ && i + 1 < n_iter) {
          // S / dP live in registers once read: the next tile's scores are
          // computed while the compute warps are still busy with this tile.
          if (!mbar_wait(sdp_read, i & 1, abort_flag, p.status, 53)) break;
          if (!mbar_wait(&q_full[(i + 1) % QS], ((i + 1) / QS) & 1, abort_flag, p.status, 46)) break;
          tc_fence_after();
          issue_sdp(i + 1);
        }
        if (!mbar_wait(pds_full, i & 1, abort_flag, p.status, 44)) break;
        if (!kAliasDQ && i > 1 && !mbar_wait(&dq_empty[i & 1], ((i - 2) >> 1) & 1, abort_flag, p.status, 45)) break;
        tc_fence_after();
        const uint32_t sQ = smem_u32(smem + L::kQ + (i % QS) * L::kTile);
        const uint32_t sDO = smem_u32(smem + L::kDO + (i % QS) * L::kTile);
        // dQ first: the compute warps stream it out while dV / dK accumulate.
#pragma unroll
        for (int k = 0; k < 8; ++k)  // dQ = dS K
          tc_mma_bf16(tmem_base + kDQCol + (i & 1) * kDQStep,
                      make_smem_desc(sDS + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024),
                      make_smem_desc(sK + k * 2048, 16384, 1024), idesc_dq, k != 0 ? 1u : 0u);
        tc_commit(&dq_full[i & 1]);
#pragma unroll
        for (int k = 0; k < 8; ++k)  // dV += P^T dO
          tc_mma_bf16(tmem_base + kDVCol, make_smem_desc(sP + k * 2048, 16384, 1024),
                      make_smem_desc(sDO + k * 2048, 16384, 1024), idesc_kv, (i | k) != 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 8; ++k)  // dK += dS^T Q
          tc_mma_bf16(tmem_base + kDKCol, make_smem_desc(sDS + k * 2048, 16384, 1024),
                      make_smem_desc(sQ + k * 2048, 16384, 1024), idesc_kv, (i | k) != 0 ? 1u : 0u);
        tc_commit(pds_free);
        tc_commit(&q_empty[i % QS]);
        if (kAliasDQ && i + 1 < n_iter) {
          const int st = (i + 1) % QS;
          if (!mbar_wait(&q_full[st], ((i + 1) / QS) & 1, abort_flag, p.status, 46)) break;
          if (!mbar_wait(&dq_empty[i & 1], (i >> 1) & 1, abort_flag, p.status, 47)) break;
          tc_fence_after();
          issue_sdp(i + 1);
        }
      }
    }
  } else {
    // ------------------------------------------------------------- compute --
    // Two threads per query row: warps w and w + 4 share a TMEM lane quadrant
    // and each takes one half of the columns.
    const int quad = warp & 3;
    const int half = warp >> 2;
    const int r = quad * 32 + lane;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const float sl2 = p.scale * kLog2e;
    float* stage = reinterpret_cast<float*>(smem + L::kStage);
    float* stage_row = stage + r * p.d;
    bool ok = true;
    NMB_PROF_DECL

    // dQ of tile j: TMEM -> fp32 staging tile (swizzled) -> ONE bulk reduce-add
    // of the whole tile into the global accumulator, whose tiles use the same
    // swizzled element order (attn_dq_store_kernel undoes it).  A failed wait
    // must not leave the other threads stuck in a named barrier: a thread that
    // gave up executes the barriers only (`ok` is kept warp-uniform for the
    // .sync.aligned TMEM instructions).
    auto dq_out = [&](int j) {
      if (ok && !mbar_wait(&dq_full[j & 1], (j >> 1) & 1, abort_flag, p.status, 49)) ok = false;
      // aliased staging: the dV / dK MMAs read P / dS until pds_free
      if (L::kStageAlias && ok && !mbar_wait(pds_free, j & 1, abort_flag, p.status, 51)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after();
      NMB_PROF_LAP(3);  // waited for the dQ MMAs
      if (!L::kStageAlias) {
        if (threadIdx.x == 0) bulk_wait_read();  // the previous tile's reduce has read the buffer
        asm volatile("bar.sync 1, 256;" ::: "memory");
      }
      constexpr int kDqChunks = HD / 64;  // 32-column chunks per thread
      if (ok) {
        uint32_t qr[kDqChunks][32];
#pragma unroll
        for (int cc = 0; cc < kDqChunks; ++cc)
          tmem_ld_32x32(t_lane + kDQCol + (j & 1) * kDQStep + (half * kDqChunks + cc) * 32, qr[cc]);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(&dq_empty[j & 1]);
#pragma unroll
        for (int cc = 0; cc < kDqChunks; ++cc) {
          const int c = half * kDqChunks + cc;
          if (c * 32 < p.d) {
#pragma unroll
            for (int q4 = 0; q4 < 8; ++q4) {
              const int ch = c * 8 + q4;                                  // 16-byte chunk of the row
              const int phys = (ch & ~7) | ((ch ^ r) & 7);                // XOR swizzle inside 128-byte groups
              *reinterpret_cast<uint4*>(stage_row + phys * 4) =
                  make_uint4(qr[cc][q4 * 4], qr[cc][q4 * 4 + 1], qr[cc][q4 * 4 + 2], qr[cc][q4 * 4 + 3]);
            }
          }
        }
      }
      fence_proxy_async_smem();
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (threadIdx.x == 0 && ok) {
        const int hq = hk * group + j / per_head;
        const int q0 = (qt_first + j % per_head) * 128;
        int rows_valid = p.Sq - q0;
        if (rows_valid > 128) rows_valid = 128;
        float* dq_tile = p.dq_acc + ((static_cast<long long>(b) * p.Hq + hq) * p.Sq + q0) * p.d;
        bulk_reduce_add_f32(dq_tile, stage, static_cast<uint32_t>(rows_valid) * p.d * 4);
        bulk_commit();
      }
      NMB_PROF_LAP(4);  // dQ write-out
    };

    NMB_PROF_START();
    for (int i = 0; i < n_iter; ++i) {
      const int hq = hk * group + i / per_head;
      const int q0 = (qt_first + i % per_head) * 128;
      const int q_row = q0 + r;
      const bool valid = q_row < p.Sq;
      const long long stat_idx = (static_cast<long long>(b) * p.Hq + hq) * p.Sq + q_row;
      const float lse2 = valid ? p.lse[stat_idx] * kLog2e : 0.f;
      const float dlt_s = valid ? p.delta[stat_idx] * p.scale : 0.f;
      int limit = p.q_pos0 + q_row - kv0;
      if (skv_total - 1 - kv0 < limit) limit = skv_total - 1 - kv0;
      if (!valid) limit = -1;
      // CTA-uniform: every (query, key) pair of this tile is visible and valid.
      const bool tile_full = (kv0 + 127 <= p.q_pos0 + q0) && (q0 + 127 < p.Sq) && (kv0 + 128 <= skv_total);
      if (ok && !mbar_wait(sdp_full, i & 1, abort_flag, p.status, 48)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after();
      NMB_PROF_LAP(0);  // waited for S / dP
      // this thread's 64 columns of P and dS, packed to bf16 pairs
      uint32_t pp[2][16], dd[2][16];
      if (ok) {
        uint32_t sr[2][32], dpr[2][32];  // all four TMEM loads in flight at once
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          tmem_ld_32x32(t_lane + kSCol + (half * 2 + cc) * 32, sr[cc]);
          tmem_ld_32x32(t_lane + kDPCol + (half * 2 + cc) * 32, dpr[cc]);
        }
        tmem_ld_wait();
        if (!kAliasDQ) {
          tc_fence_before();
          mbar_arrive(sdp_read);
        }
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int c = half * 2 + cc;
          if (tile_full) {
#pragma unroll
            for (int jj = 0; jj < 32; jj += 2) {
              const float p0 = fast_exp2(fmaf(__uint_as_float(sr[cc][jj]), sl2, -lse2));
              const float p1 = fast_exp2(fmaf(__uint_as_float(sr[cc][jj + 1]), sl2, -lse2));
              const float d0 = p0 * fmaf(__uint_as_float(dpr[cc][jj]), p.scale, -dlt_s);
              const float d1 = p1 * fmaf(__uint_as_float(dpr[cc][jj + 1]), p.scale, -dlt_s);
              pp[cc][jj / 2] = pack_bf16x2(p0, p1);
              dd[cc][jj / 2] = pack_bf16x2(d0, d1);
            }
          } else {
#pragma unroll
            for (int jj = 0; jj < 32; jj += 2) {
              const bool v0 = c * 32 + jj <= limit;
              const bool v1 = c * 32 + jj + 1 <= limit;
              const float p0 = v0 ? fast_exp2(fmaf(__uint_as_float(sr[cc][jj]), sl2, -lse2)) : 0.f;
              const float p1 = v1 ? fast_exp2(fmaf(__uint_as_float(sr[cc][jj + 1]), sl2, -lse2)) : 0.f;
              const float d0 = p0 * fmaf(__uint_as_float(dpr[cc][jj]), p.scale, -dlt_s);
              const float d1 = p1 * fmaf(__uint_as_float(dpr[cc][jj + 1]), p.scale, -dlt_s);
              pp[cc][jj / 2] = pack_bf16x2(p0, p1);
              dd[cc][jj / 2] = pack_bf16x2(d0, d1);
            }
          }
        }
      }
      NMB_PROF_LAP(1);  // computed P / dS
      // The shared P / dS tiles are still being read by the previous tile's
      // dV / dK MMAs; those ran while this tile's values were computed.
      if (ok && i > 0 && !mbar_wait(pds_free, (i - 1) & 1, abort_flag, p.status, 50)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      if (L::kStageAlias && i > 0) {
        // The dQ staging tile aliases P / dS: the bulk reduce must have finished
        // reading it before anyone overwrites it.
        if (threadIdx.x == 0) bulk_wait_read();
        asm volatile("bar.sync 1, 256;" ::: "memory");
      }
      if (ok) {
        uint8_t* sp = smem + L::kP;
        uint8_t* sds = smem + L::kDS;
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int c = half * 2 + cc;
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const uint32_t off = (c >> 1) * 16384 + swz128_offset(r, (c & 1) * 4 + t);
            *reinterpret_cast<uint4*>(sp + off) =
                make_uint4(pp[cc][t * 4], pp[cc][t * 4 + 1], pp[cc][t * 4 + 2], pp[cc][t * 4 + 3]);
            *reinterpret_cast<uint4*>(sds + off) =
                make_uint4(dd[cc][t * 4], dd[cc][t * 4 + 1], dd[cc][t * 4 + 2], dd[cc][t * 4 + 3]);
          }
        }
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(pds_full);
      }
      NMB_PROF_LAP(2);  // waited for the P / dS buffers, stored
      // With two dQ accumulators the previous tile's dQ is written out while the
      // tensor core works on this tile; with one, this tile's right away.
      if (kAliasDQ) {
        dq_out(i);
      } else if (i > 0) {
        dq_out(i - 1);
      }
    }
    if (!kAliasDQ && n_iter > 0) dq_out(n_iter - 1);
    NMB_PROF_STORE();
    bulk_wait_all();
    // dK / dV of this tile (rows = keys): wait for the last dV / dK MMAs.
    if (ok && n_iter > 0 && !mbar_wait(pds_free, (n_iter - 1) & 1, abort_flag, p.status, 52)) ok = false;
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    const int kv_row = kv_row0 + r;
    const long long off = b * p.dkv_stride_b + static_cast<long long>(kv_row) * p.dkv_stride_s + hk * p.dkv_stride_h;
    constexpr int kHalfCols = HD / 2;
    if (ok && n_iter == 0 && kv_row < p.chunk_len) {
      // no query sees this tile: its gradient is zero
      for (int c = half * kHalfCols; c < (half + 1) * kHalfCols && c < p.d; c += 8) {
        *reinterpret_cast<uint4*>(p.dk[chunk] + off + c) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(p.dv[chunk] + off + c) = make_uint4(0, 0, 0, 0);
      }
    }
    if (ok && n_iter > 0) {
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* row = (which == 0 ? p.dv[chunk] : p.dk[chunk]) + off;
        const uint32_t col = which == 0 ? kDVCol : kDKCol;
#pragma unroll 1
        for (int cc = 0; cc < kHalfCols / 32; ++cc) {
          const int c = half * (kHalfCols / 32) + cc;
          uint32_t ar[32];
          tmem_ld_32x32(t_lane + col + c * 32, ar);
          tmem_ld_wait();
          if (kv_row < p.chunk_len && c * 32 < p.d) {
            uint4* dst = reinterpret_cast<uint4*>(row + c * 32);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 u;
              u.x = pack_bf16x2(__uint_as_float(ar[q * 8 + 0]), __uint_as_float(ar[q * 8 + 1]));
              u.y = pack_bf16x2(__uint_as_float(ar[q * 8 + 2]), __uint_as_float(ar[q * 8 + 3]));
              u.z = pack_bf16x2(__uint_as_float(ar[q * 8 + 4]), __uint_as_float(ar[q * 8 + 5]));
              u.w = pack_bf16x2(__uint_as_float(ar[q * 8 + 6]), __uint_as_float(ar[q * 8 + 7]));
              dst[q] = u;
            }
          }
        }
      }
    }
  }

  if (*abort_flag != 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// delta[b,h,s] = sum_d dO * O ; also clears the fp32 dQ accumulator.
// d / 8 threads per (b, s, h) row, 16 bytes of O and dO per thread.
__global__ void attn_bwd_prep_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dO,
                                     long long o_sb, long long o_ss, long long o_sh, long long do_sb,
                                     long long do_ss, long long do_sh, float* __restrict__ delta,
                                     float* __restrict__ dq_acc, int B, int H, int S, int d) {
  pdl_enter();
  const int per_row = d >> 3;                       // 8, 12 or 16 threads per row
  const int group = per_row <= 8 ? 8 : 16;          // shuffle width (power of two)
  const long long gid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long row = gid / group;
  const int part = gid % group;
  const long long total = static_cast<long long>(B) * S * H;
  float acc = 0.f;
  if (row < total && part < per_row) {
    const int h = row % H;
    const long long bs = row / H;
    const int s = bs % S;
    const int b = bs / S;
    const uint4 a = *reinterpret_cast<const uint4*>(o + b * o_sb + s * o_ss + h * o_sh + part * 8);
    const uint4 g = *reinterpret_cast<const uint4*>(dO + b * do_sb + s * do_ss + h * do_sh + part * 8);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 x = unpack_bf16x2(aw[k]);
      const float2 y = unpack_bf16x2(gw[k]);
      acc += x.x * y.x + x.y * y.y;
    }
    float4* dq = reinterpret_cast<float4*>(dq_acc + row * d + part * 8);
    dq[0] = make_float4(0.f, 0.f, 0.f, 0.f);
    dq[1] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (int o2 = group >> 1; o2 > 0; o2 >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o2, 16);
  if (row < total && part == 0) {
    const int h = row % H;
    const long long bs = row / H;
    delta[(static_cast<long long>(bs / S) * H + h) * S + (bs % S)] = acc;
  }
}

// Inverse rotary rotation of 8 consecutive elements (4 interleaved pairs starting
// at pair `pair0` of the head) of the row at position `pos`: the gradient with
// respect to the un-rotated projection output, R(-angle) applied to the gradient
// of the rotated one.
__device__ __forceinline__ void unrope8(float (&x)[8], const float2* table, long long pos, int half, int pair0) {
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

// Last kernel of the backward pass.
//   * dq (bf16, strided) <- dq_acc (fp32, [B, H, S, d] with the 16-byte chunks of
//     a row XOR-swizzled by (s % 128) & 7 inside each group of eight); 8 elements
//     per thread;
//   * with a rotary table (q and k were rotated by the epilogue of the QKV
//     projection): dq is un-rotated on the way out and dk (already written by
//     the main kernel, bf16) is un-rotated in place by the threads past the dq
//     range -- so the projection's backward sees plain gradients and no separate
//     rotation kernel runs (the reference differentiates through ~10 elementwise
//     kernels per tensor, nano_megatron/reference/layers.py:67-81).
__global__ void attn_dq_store_kernel(const float* __restrict__ dq_acc, __nv_bfloat16* __restrict__ dq,
                                     long long dq_sb, long long dq_ss, long long dq_sh, int B, int H,
                                     int S, int d, const float2* __restrict__ rope_table,
                                     const long long* __restrict__ rope_pos, __nv_bfloat16* __restrict__ dk,
                                     long long dk_sb, long long dk_ss, long long dk_sh, int Hkv) {
  pdl_enter();
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long total = static_cast<long long>(B) * S * H * d / 8;
  const int per_row = d / 8;
  if (idx >= total) {
    if (rope_table == nullptr || dk == nullptr) return;
    const long long j = idx - total;
    if (j >= static_cast<long long>(B) * S * Hkv * per_row) return;
    const int c8 = static_cast<int>(j % per_row);
    const long long row = j / per_row;              // (b * S + s) * Hkv + h
    const int h = row % Hkv;
    const long long bs = row / Hkv;
    const int s = bs % S;
    const int b = bs / S;
    uint4* p = reinterpret_cast<uint4*>(dk + b * dk_sb + s * dk_ss + h * dk_sh + c8 * 8);
    const uint4 u = *p;
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    float x[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = unpack_bf16x2(w[k]);
      x[2 * k] = f.x;
      x[2 * k + 1] = f.y;
    }
    unrope8(x, rope_table, rope_pos[static_cast<long long>(b) * S + s], d / 2, c8 * 4);
    *p = make_uint4(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]), pack_bf16x2(x[4], x[5]),
                    pack_bf16x2(x[6], x[7]));
    return;
  }
  const int c8 = static_cast<int>(idx % per_row);   // which 8 columns of the row
  const long long row = idx / per_row;              // (b * H + h) * S + s
  const int s = row % S;
  const long long bh = row / S;
  const int h = bh % H;
  const int b = bh / H;
  const int r = s & 127;
  const float* src = dq_acc + row * d;
  const int c0 = 2 * c8, c1 = 2 * c8 + 1;           // the two 16-byte chunks
  const float4 v0 = *reinterpret_cast<const float4*>(src + ((c0 & ~7) | ((c0 ^ r) & 7)) * 4);
  const float4 v1 = *reinterpret_cast<const float4*>(src + ((c1 & ~7) | ((c1 ^ r) & 7)) * 4);
  float x[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
  if (rope_table != nullptr) unrope8(x, rope_table, rope_pos[static_cast<long long>(b) * S + s], d / 2, c8 * 4);
  uint4 out;
  out.x = pack_bf16x2(x[0], x[1]);
  out.y = pack_bf16x2(x[2], x[3]);
  out.z = pack_bf16x2(x[4], x[5]);
  out.w = pack_bf16x2(x[6], x[7]);
  *reinterpret_cast<uint4*>(dq + b * dq_sb + s * dq_ss + h * dq_sh + c8 * 8) = out;
}

static int make_attn_map(CUtensorMap* m, const void* ptr, int d, int S, int H, int B, long long ss,
                         long long sh, long long sb) {
  const uint64_t dims[4] = {static_cast<uint64_t>(d), static_cast<uint64_t>(S), static_cast<uint64_t>(H),
                            static_cast<uint64_t>(B)};
  const uint64_t strides[3] = {static_cast<uint64_t>(ss) * 2, static_cast<uint64_t>(sh) * 2,
                               static_cast<uint64_t>(sb) * 2};
  const uint32_t box[4] = {64, 128, 1, 1};
  return make_tmap_bf16(m, ptr, 4, dims, strides, box);
}

}  // namespace nmb

using namespace nmb;

// Tensor descriptor passed from Python: pointer + element strides of the
// (batch, seq, head) dimensions; head_dim is contiguous.
struct NmbTensor4 {
  void* ptr;
  long long stride_b, stride_s, stride_h;
};

// Opt the attention kernels in to their dynamic shared memory sizes (once per
// process and device, right after the library is loaded).
extern "C" int nmb_attn_configure() {
  cudaError_t e;
  e = cudaFuncSetAttribute(attn_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnFwdSmem<64>::kTotal);
  if (e != cudaSuccess) return 300 + e;
  e = cudaFuncSetAttribute(attn_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnFwdSmem<128>::kTotal);
  if (e != cudaSuccess) return 300 + e;
  e = cudaFuncSetAttribute(attn_bwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnBwdSmem<64>::kTotal);
  if (e != cudaSuccess) return 300 + e;
  e = cudaFuncSetAttribute(attn_bwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnBwdSmem<128>::kTotal);
  if (e != cudaSuccess) return 300 + e;
  // same carve-out as the GEMMs and the overlapped communication kernels
  const int carve = cudaSharedmemCarveoutMaxShared;
  e = cudaFuncSetAttribute(attn_fwd_kernel<64>, cudaFuncAttributePreferredSharedMemoryCarveout, carve);
  if (e != cudaSuccess) return 300 + e;
  e = cudaFuncSetAttribute(attn_fwd_kernel<128>, cudaFuncAttributePreferredSharedMemoryCarveout, carve);
  if (e != cudaSuccess) return 300 + e;
  e = cudaFuncSetAttribute(attn_bwd_kernel<64>, cudaFuncAttributePreferredSharedMemoryCarveout, carve);
  if (e != cudaSuccess) return 300 + e;
  e = cudaFuncSetAttribute(attn_bwd_kernel<128>, cudaFuncAttributePreferredSharedMemoryCarveout, carve);
  if (e != cudaSuccess) return 300 + e;
  return 0;
}

#ifdef NMB_ATTN_PROF
extern "C" int nmb_attn_fwd_prof_read(long long* host16) {
  return static_cast<int>(cudaMemcpyFromSymbol(host16, nmb::g_attn_fwd_prof, 16 * sizeof(long long)));
}
extern "C" int nmb_attn_fwd_marks_read(unsigned long long* host, int n_ctas) {
  return static_cast<int>(cudaMemcpyFromSymbol(host, nmb::g_attn_fwd_marks, sizeof(unsigned long long) * 4 * n_ctas));
}
extern "C" int nmb_attn_fwd_span_read(unsigned long long* host, int n_ctas) {
  return static_cast<int>(cudaMemcpyFromSymbol(host, nmb::g_attn_fwd_span, sizeof(unsigned long long) * 2 * n_ctas));
}
#endif

extern "C" int nmb_attn_fwd(const NmbTensor4* q, const NmbTensor4* k_chunks, const NmbTensor4* v_chunks,
                            int n_chunks, int chunk_len, const NmbTensor4* o, float* lse, int B, int Hq,
                            int Hkv, int Sq, int d, int q_pos0, float scale, int* status, void* stream) {
  if (n_chunks < 1 || n_chunks > kMaxChunks) return kBadArgument;
  if (d != 64 && d != 96 && d != 128) return kBadArgument;
  if (n_chunks > 1 && (chunk_len % 128) != 0) return kBadArgument;
  (void)cudaGetLastError();
  AttnFwdParams p;
  if (make_attn_map(&p.q_map, q->ptr, d, Sq, Hq, B, q->stride_s, q->stride_h, q->stride_b)) return 101;
  for (int c = 0; c < n_chunks; ++c) {
    if (make_attn_map(&p.k_map[c], k_chunks[c].ptr, d, chunk_len, Hkv, B, k_chunks[c].stride_s,
                      k_chunks[c].stride_h, k_chunks[c].stride_b))
      return 102;
    if (make_attn_map(&p.v_map[c], v_chunks[c].ptr, d, chunk_len, Hkv, B, v_chunks[c].stride_s,
                      v_chunks[c].stride_h, v_chunks[c].stride_b))
      return 103;
  }
  p.o = static_cast<__nv_bfloat16*>(o->ptr);
  p.o_stride_b = o->stride_b;
  p.o_stride_s = o->stride_s;
  p.o_stride_h = o->stride_h;
  p.lse = lse;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.Sq = Sq;
  p.chunk_len = chunk_len; p.n_chunks = n_chunks;
  p.d = d; p.q_pos0 = q_pos0; p.scale = scale; p.status = status;
  dim3 grid(((Sq + 127) / 128) * Hq * B);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (d == 64) {
    e = launch_pdl(attn_fwd_kernel<64>, grid, dim3(kAttnThreads), AttnFwdSmem<64>::kTotal, s, p);
  } else {
    e = launch_pdl(attn_fwd_kernel<128>, grid, dim3(kAttnThreads), AttnFwdSmem<128>::kTotal, s, p);
  }
  return e == cudaSuccess ? 0 : 400 + e;
}

// dq_acc: fp32 scratch [B, Sq, Hq, d]; delta: fp32 scratch [B, Hq, Sq].
extern "C" int nmb_attn_bwd(const NmbTensor4* q, const NmbTensor4* k_chunks, const NmbTensor4* v_chunks,
                            int n_chunks, int chunk_len, const NmbTensor4* o, const NmbTensor4* dout,
                            const float* lse, float* delta, float* dq_acc, const NmbTensor4* dq,
                            const NmbTensor4* dk_chunks, const NmbTensor4* dv_chunks, int B, int Hq, int Hkv,
                            int Sq, int d, int q_pos0, int n_visible_kv_tiles, float scale,
                            const void* rope_table, const long long* rope_pos, int* status, void* stream) {
  if (n_chunks < 1 || n_chunks > kMaxChunks) return kBadArgument;
  if (d != 64 && d != 96 && d != 128) return kBadArgument;
  if (n_chunks > 1 && (chunk_len % 128) != 0) return kBadArgument;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  (void)cudaGetLastError();
  {
    const long long rows = static_cast<long long>(B) * Sq * Hq;
    const int threads = 256;
    const long long blocks = (rows * (d <= 64 ? 8 : 16) + threads - 1) / threads;
    launch_pdl(attn_bwd_prep_kernel, dim3(static_cast<unsigned>(blocks)), dim3(threads), 0, s,
               static_cast<const __nv_bfloat16*>(o->ptr), static_cast<const __nv_bfloat16*>(dout->ptr), o->stride_b,
               o->stride_s, o->stride_h, dout->stride_b, dout->stride_s, dout->stride_h, delta, dq_acc, B, Hq, Sq, d);
  }
  AttnBwdParams p;
  if (make_attn_map(&p.q_map, q->ptr, d, Sq, Hq, B, q->stride_s, q->stride_h, q->stride_b)) return 101;
  if (make_attn_map(&p.do_map, dout->ptr, d, Sq, Hq, B, dout->stride_s, dout->stride_h, dout->stride_b)) return 104;
  for (int c = 0; c < n_chunks; ++c) {
    if (make_attn_map(&p.k_map[c], k_chunks[c].ptr, d, chunk_len, Hkv, B, k_chunks[c].stride_s,
                      k_chunks[c].stride_h, k_chunks[c].stride_b))
      return 102;
    if (make_attn_map(&p.v_map[c], v_chunks[c].ptr, d, chunk_len, Hkv, B, v_chunks[c].stride_s,
                      v_chunks[c].stride_h, v_chunks[c].stride_b))
      return 103;
    p.dk[c] = static_cast<__nv_bfloat16*>(dk_chunks[c].ptr);
    p.dv[c] = static_cast<__nv_bfloat16*>(dv_chunks[c].ptr);
  }
  p.dkv_stride_b = dk_chunks[0].stride_b;
  p.dkv_stride_s = dk_chunks[0].stride_s;
  p.dkv_stride_h = dk_chunks[0].stride_h;
  p.lse = lse; p.delta = delta; p.dq_acc = dq_acc;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.Sq = Sq;
  p.chunk_len = chunk_len; p.n_chunks = n_chunks;
  p.d = d; p.q_pos0 = q_pos0; p.scale = scale; p.status = status;
#ifdef NMB_ATTN_PROF
  p.prof = reinterpret_cast<long long*>(delta) - 8;  // profiling builds: the caller over-allocates delta by 8 slots in front
#endif
  dim3 grid(n_visible_kv_tiles * Hkv * B);
  cudaError_t e;
  if (d == 64) {
    e = launch_pdl(attn_bwd_kernel<64>, grid, dim3(kBwdThreads), AttnBwdSmem<64>::kTotal, s, p);
  } else {
    e = launch_pdl(attn_bwd_kernel<128>, grid, dim3(kBwdThreads), AttnBwdSmem<128>::kTotal, s, p);
  }
  if (e != cudaSuccess) return 400 + e;
  {
    // dk is un-rotated in place when the whole key sequence is one local chunk of the
    // query's length; with several chunks (context parallelism) dk still has to be
    // summed over ranks, and the kernel that sums it un-rotates it
    const bool unrope_k = rope_table != nullptr && n_chunks == 1 && chunk_len == Sq;
    long long octets = static_cast<long long>(B) * Sq * Hq * d / 8;
    if (unrope_k) octets += static_cast<long long>(B) * Sq * Hkv * d / 8;
    const int threads = 256;
    e = launch_pdl(attn_dq_store_kernel, dim3(static_cast<unsigned>((octets + threads - 1) / threads)), dim3(threads), 0,
                   s, static_cast<const float*>(dq_acc), static_cast<__nv_bfloat16*>(dq->ptr), dq->stride_b, dq->stride_s,
                   dq->stride_h, B, Hq, Sq, d, static_cast<const float2*>(rope_table), rope_pos,
                   unrope_k ? static_cast<__nv_bfloat16*>(dk_chunks[0].ptr) : static_cast<__nv_bfloat16*>(nullptr),
                   dk_chunks[0].stride_b, dk_chunks[0].stride_s, dk_chunks[0].stride_h, Hkv);
  }
  return e == cudaSuccess ? 0 : 500 + e;
}
