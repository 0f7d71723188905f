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
// Structure: persistent CTAs (one per SM), 192 threads:
//   warp 0      TMA producer (one elected lane), STAGES-deep smem ring
//   warp 1      TMEM owner + single-thread tcgen05.mma issuer
//   warps 2..9  epilogue: tcgen05.ld -> registers -> bias/GELU/residual -> global
//               (two warps per TMEM lane quadrant, each takes half of the columns)
// Two TMEM accumulator buffers let the epilogue of tile i overlap the main
// loop of tile i+1.  No cluster launch, no multicast: every CTA loads its own
// tiles.
#include "common.cuh"

namespace nmb {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kGemmThreads = 320;  // TMA warp, MMA warp, 8 epilogue warps

enum EpilogueMode : int {
  kEpiPlain = 0,   // C = acc (+bias) (+residual) (+C_old)
  kEpiGelu = 1,    // aux_out = acc+bias ; C = gelu(acc+bias)
  kEpiDGelu = 2,   // C = acc * gelu'(aux_in)
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
};

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = STAGES * kStageBytes;
  // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], tmem slot, abort
  static constexpr int kTotal = kBarOffset + (2 * STAGES + 4) * 8 + 16;
};

template <int BN, int STAGES, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 GemmEpilogue ep, int M, int N, int K, int* status) {
  using L = GemmSmem<BN, STAGES>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // SWIZZLE_128B operands need 1024-byte aligned stage bases.
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
  const int tiles_m = (M + kBM - 1) / kBM;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + kBK - 1) / kBK;
  constexpr uint32_t kTmemCols = 2 * BN;  // 256 or 512: powers of two

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ producer --
    if (lane == 0) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % tiles_m) * kBM;
        const int n0 = (tile / tiles_m) * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
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
            tma_load_2d(sb, &tma_b, &full_bar[stage], kb * kBK, n0);
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
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int buf = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&acc_empty[buf], acc_phase ^ 1, abort_flag, status, 2)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
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
            tc_mma_bf16(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
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
    int local = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      const int m0 = (tile % tiles_m) * kBM;
      const int n0 = (tile / tiles_m) * BN;
      if (!mbar_wait(&acc_full[buf], acc_phase, abort_flag, status, 4)) break;
      tc_fence_after();
      const int row = m0 + quad * 32 + lane;
      const bool row_ok = row < M;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = half * (BN / 64); c < (half + 1) * (BN / 64); ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= N) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_ld_wait();
        if (!row_ok) continue;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * ep.alpha;
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
          if (ep.mode == kEpiGelu) {
            uint4* ap = reinterpret_cast<uint4*>(ep.aux_out + static_cast<size_t>(row) * ep.ld_aux + col0);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 u;
              u.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
              u.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
              u.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
              u.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
              ap[q] = u;
            }
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
            uint4* cp = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(ep.c) +
                                                 static_cast<size_t>(row) * ep.ldc + col0);
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
              uint4 o;
              o.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
              o.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
              o.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
              o.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
              cp[q] = o;
            }
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
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
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
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
static int launch_gemm(const void* A, int lda, const void* B, int ldb, const GemmEpilogue& ep, int M,
                       int N, int K, int* status, cudaStream_t stream) {
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
    const uint32_t box[2] = {kBK, BN};
    rc = make_tmap_bf16(&tb, B, 2, dims, strides, box);
  } else {
    const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(K)};
    const uint64_t strides[1] = {static_cast<uint64_t>(ldb) * 2};
    const uint32_t box[2] = {64, kBK};
    rc = make_tmap_bf16(&tb, B, 2, dims, strides, box);
  }
  if (rc != 0) return 200 + rc;

  auto kern = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN>;
  const int smem_bytes = L::kTotal + 1024;
  const int tiles = ((M + kBM - 1) / kBM) * ((N + BN - 1) / BN);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, kGemmThreads, smem_bytes, stream>>>(ta, tb, ep, M, N, K, status);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + static_cast<int>(e);
}

template <bool A_MN, bool B_MN>
static int dispatch_tile(const void* A, int lda, const void* B, int ldb, const GemmEpilogue& ep,
                         int M, int N, int K, int* status, cudaStream_t stream) {
  const int tiles256 = ((M + kBM - 1) / kBM) * ((N + 255) / 256);
  // A 128 x 128 UMMA reads 8 KiB of operands from shared memory per 64 clocks,
  // i.e. the full 128 B/clk of the SM, and the TMA writes compete for the same
  // bandwidth; the 128 x 256 shape needs 25% less per FLOP.  Narrow tiles only
  // pay when the wide ones would leave most of the machine idle.
  if (N > 128 && tiles256 * 3 >= sm_count())
    return launch_gemm<256, 4, A_MN, B_MN>(A, lda, B, ldb, ep, M, N, K, status, stream);
  return launch_gemm<128, 6, A_MN, B_MN>(A, lda, B, ldb, ep, M, N, K, status, stream);
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
static int configure_gemm() {
  cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<BN, STAGES, A_MN, B_MN>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<BN, STAGES>::kTotal + 1024);
  return e == cudaSuccess ? 0 : 300 + static_cast<int>(e);
}

}  // namespace nmb

// Opt every GEMM variant in to its dynamic shared memory size on the current
// device.  Called once per process (per device) right after the library is
// loaded, from the thread that loads it.
extern "C" int nmb_gemm_configure() {
  using namespace nmb;
  int rc = 0;
  rc |= configure_gemm<256, 4, false, false>();
  rc |= configure_gemm<256, 4, false, true>();
  rc |= configure_gemm<256, 4, true, true>();
  rc |= configure_gemm<256, 4, true, false>();
  rc |= configure_gemm<128, 6, false, false>();
  rc |= configure_gemm<128, 6, false, true>();
  rc |= configure_gemm<128, 6, true, true>();
  rc |= configure_gemm<128, 6, true, false>();
  return rc;
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
                             int* status, void* stream) {
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
  // The vector epilogue needs 16-byte aligned rows; otherwise every chunk is
  // treated as ragged by shrinking nothing here and letting the kernel fall
  // back per chunk -- so require alignment up front instead.
  const int celt = out_f32 ? 4 : 8;
  if ((ldc % celt) != 0 || (reinterpret_cast<uintptr_t>(C) & 15)) return kBadArgument;
  if (residual != nullptr && ((ldr % 8) != 0 || (reinterpret_cast<uintptr_t>(residual) & 15))) return kBadArgument;
  if ((aux_out != nullptr || aux_in != nullptr) && (ld_aux % 8) != 0) return kBadArgument;
  if (bias != nullptr && (reinterpret_cast<uintptr_t>(bias) & 15)) return kBadArgument;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!a_mn && !b_mn) return dispatch_tile<false, false>(A, lda, B, ldb, ep, M, N, K, status, s);
  if (!a_mn && b_mn) return dispatch_tile<false, true>(A, lda, B, ldb, ep, M, N, K, status, s);
  if (a_mn && b_mn) return dispatch_tile<true, true>(A, lda, B, ldb, ep, M, N, K, status, s);
  return dispatch_tile<true, false>(A, lda, B, ldb, ep, M, N, K, status, s);
}
