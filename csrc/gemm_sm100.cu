// Persistent, warp-specialised bf16 GEMM for sm_100a.
//
//   C[b][M,N] (+)= A[b] * B[b]          fp32 accumulation in TMEM
//
// A is either "K-major" (row-major [M,K]) or "MN-major" (row-major [K,M], i.e. the
// transposed operand is read in place); likewise B is K-major (row-major [N,K]) or
// MN-major (row-major [K,N]). That covers forward (x * W[in,out]), dgrad (dy * W^T)
// and wgrad (x^T * dy) of a dense layer without a transpose pass.
//
// Roles per CTA (192 threads): warp 0 = TMA producer, warp 1 = tcgen05 MMA issuer
// (owns TMEM alloc/free), warps 2..5 = epilogue (one TMEM lane quarter each).
// smem ring of kStages {A 128x64, B BNx64} tiles in the 128-byte swizzle that both
// TMA and the UMMA descriptors use; two accumulators in TMEM so the epilogue of tile
// i overlaps the main loop of tile i+1. No cluster multicast is used anywhere.
//
// Epilogues: plain store (bf16 or fp32, optional C += ), residual add, and the
// T5.1.1 gated-GELU (B = [wi_0 | wi_1], out = gelu(h0) * h1, optionally saving
// h0/h1 for the backward pass).
#include <algorithm>

#include "gemm_common.cuh"

namespace t5x {

static thread_local long long* g_gemm_trace = nullptr;  // t5x_gemm_set_trace
long long* gemm_trace_buffer() { return g_gemm_trace; }

template <int BN>
struct GemmSmem {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kBarrierBytes = 1024;
  static constexpr int kEpiStageBytes = 4 * kEpiStageBytesPerWarp;  // coalesced epilogue stores
  static constexpr int kTotal =
      kStages * kStageBytes + kBarrierBytes + kEpiStageBytes + 1024;  // +1024 align slack
};

template <int BN, int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmB2, const GemmParams p) {
  using S = GemmSmem<BN>;
  constexpr int kStages = S::kStages;
  // columns of C produced by one tile
  constexpr int kTileN = (EPI == kEpiGatedGelu) ? BN / 2 : BN;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + kStages * S::kABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * S::kStageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + kStages;
  uint64_t* tmem_full = bars + 2 * kStages;
  uint64_t* tmem_empty = bars + 2 * kStages + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* epi_stage = reinterpret_cast<float*>(smem + kStages * S::kStageBytes + S::kBarrierBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  chain_release();  // the next kernel on the stream may set itself up behind this one
  if (threadIdx.x == 0) {
    T5X_GEMM_TRACE(0);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (EPI == kEpiGatedGelu) tma_prefetch_desc(&tmB2);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) T5X_GEMM_TRACE(1);

  const int num_kb = (p.K + kBK - 1) / kBK;
  const int tiles_per_batch = p.tiles_m * p.tiles_n;
  const int total_tiles = tiles_per_batch * p.batch;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      auto load_a = [&](int stage, int k0, int m0, int b) {
        uint8_t* a_dst = sA + stage * S::kABytes;
        if (!p.a_mn) {
          tma_load_3d(a_dst, &tmA, &full[stage], k0, m0, b);  // box {64, 128, 1}
        } else {
#pragma unroll
          for (int j = 0; j < kBM / 64; ++j)  // box {64 (m), 64 (k), 1}
            tma_load_3d(a_dst + j * 8192, &tmA, &full[stage], m0 + 64 * j, k0, b);
        }
      };
      auto load_b = [&](int stage, int k0, int n0, int b) {
        uint8_t* b_dst = sB + stage * S::kBBytes;
        if (EPI == kEpiGatedGelu) {
          constexpr int kHalf = BN / 2;  // 128 columns of each of wi_0 and wi_1
          if (!p.b_mn) {
            tma_load_3d(b_dst, &tmB, &full[stage], k0, n0, b);
            tma_load_3d(b_dst + kHalf * 128, &tmB2, &full[stage], k0, n0, b);
          } else {
#pragma unroll
            for (int j = 0; j < kHalf / 64; ++j) {
              tma_load_3d(b_dst + j * 8192, &tmB, &full[stage], n0 + 64 * j, k0, b);
              tma_load_3d(b_dst + (kHalf / 64 + j) * 8192, &tmB2, &full[stage], n0 + 64 * j, k0, b);
            }
          }
        } else {
          if (!p.b_mn) {
#pragma unroll
            for (int j = 0; j < BN / 128; ++j)  // box {64, 128, 1}
              tma_load_3d(b_dst + j * 16384, &tmB, &full[stage], k0, n0 + 128 * j, b);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)  // box {64 (n), 64 (k), 1}
              tma_load_3d(b_dst + j * 8192, &tmB, &full[stage], n0 + 64 * j, k0, b);
          }
        }
      };
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // B is constant (weights that no kernel in flight writes): the B halves of the first
      // stages are requested before the wait for the preceding kernel, the A halves after it.
      int preloaded = 0;
      if (p.b_constant && blockIdx.x < total_tiles) {
        int b, mt, nt;
        gemm_tile_coords(p, blockIdx.x, tiles_per_batch, b, mt, nt);
        preloaded = min(kStages, num_kb);
        for (int kb = 0; kb < preloaded; ++kb) {
          mbar_expect_tx(&full[kb], S::kStageBytes);
          load_b(kb, kb * kBK, nt * kTileN, b);
        }
        chain_wait();
        for (int kb = 0; kb < preloaded; ++kb) load_a(kb, kb * kBK, mt * kBM, b);
        T5X_GEMM_TRACE(2);
        if (preloaded == kStages) phase = 1;
        else stage = preloaded;
      } else {
        chain_wait();
      }
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int b, mt, nt;
        gemm_tile_coords(p, tile, tiles_per_batch, b, mt, nt);
        const int m0 = mt * kBM;
        const int n0 = nt * kTileN;
        for (int kb = preloaded; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) {
            report_status(p.status, kStatusTimeoutProducer, kKernelIdGemm, tile, kb);
            *abort_flag = 1;
            ok = false;
            break;
          }
          mbar_expect_tx(&full[stage], S::kStageBytes);
          const int k0 = kb * kBK;
          load_a(stage, k0, m0, b);
          load_b(stage, k0, n0, b);
          if (tile == blockIdx.x && kb == 0) T5X_GEMM_TRACE(2);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        preloaded = 0;
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(kBM, BN, p.a_mn, p.b_mn);
      // K-major: +32 B per UMMA_K=16 inside the 128 B swizzle row; SBO = 1024.
      // MN-major: +2048 B per UMMA_K (two 8-row k groups); LBO = 8192 (next 64 MN elements).
      const uint32_t a_kstep = p.a_mn ? 2048u : 32u;
      const uint32_t b_kstep = p.b_mn ? 2048u : 32u;
      const uint32_t a_lbo = p.a_mn ? 8192u : 16u;
      const uint32_t b_lbo = p.b_mn ? 8192u : 16u;
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag)) {
          report_status(p.status, kStatusTimeoutMma, kKernelIdGemm, tile, -1);
          *abort_flag = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag)) {
            report_status(p.status, kStatusTimeoutMma, kKernelIdGemm, tile, kb);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          if (local == 0 && kb == 0) T5X_GEMM_TRACE(3);
          const uint32_t a_addr = smem_u32(sA + stage * S::kABytes);
          const uint32_t b_addr = smem_u32(sB + stage * S::kBBytes);
#pragma unroll
          for (int s = 0; s < kBK / 16; ++s) {
            const uint64_t ad = make_smem_desc_sw128(a_addr + s * a_kstep, a_lbo, 1024);
            const uint64_t bd = make_smem_desc_sw128(b_addr + s * b_kstep, b_lbo, 1024);
            umma_bf16(d_tmem, ad, bd, idesc, (kb | s) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&tmem_full[acc]);
        if (local == 0) T5X_GEMM_TRACE(4);
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int q = warp & 3;  // TMEM lanes [32q, 32q+32) belong to warps with id % 4 == q
    int local = 0;
    bool ok = true;
    chain_wait();  // the epilogue reads residuals and writes C
    const bool c_vec_ok = (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      int b, mt, nt;
      gemm_tile_coords(p, tile, tiles_per_batch, b, mt, nt);
      const int m0 = mt * kBM;
      const int n0 = nt * kTileN;
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag)) {
        if (lane == 0) report_status(p.status, kStatusTimeoutEpilogue, kKernelIdGemm, tile, 0);
        *abort_flag = 1;
        ok = false;
        break;
      }
      tc_fence_after();
      if (local == 0 && warp == 2 && lane == 0) T5X_GEMM_TRACE(5);
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      if (EPI == kEpiCeStats)
        gemm_epilogue_ce_stats<BN>(p, t_row, m0, n0, nt, q, lane);
      else if (EPI == kEpiCeGrad)
        gemm_epilogue_ce_grad<BN>(p, t_row, m0, n0, q, lane, c_vec_ok);
      else
        gemm_epilogue_tile<BN, EPI>(p, t_row, m0, n0, b, q, lane, c_vec_ok,
                                    epi_stage + (warp - 2) * (kEpiStageBytesPerWarp / 4));
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      if (local == 0 && warp == 2 && lane == 0) T5X_GEMM_TRACE(6);
    }
  }

  // Teardown. Every TMA load that was issued has been waited for by the MMA role
  // (or, after an abort, is given a bounded time to land) before the CTA leaves.
  __syncwarp();
  if (*abort_flag && warp == 0 && lane == 0) {
    for (int it = 0; it < 2000; ++it) __nanosleep(1000);  // ~2 ms for copies in flight to land
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
    if (lane == 0) T5X_GEMM_TRACE(7);
  }
}

template <int BN, int EPI>
static int launch_gemm(const CUtensorMap* tA, const CUtensorMap* tB, const CUtensorMap* tB2,
                       GemmParams& p, int max_ctas, cudaStream_t stream) {
  using S = GemmSmem<BN>;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<BN, EPI>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal);
    if (e != cudaSuccess) return set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    attr_set[dev] = true;
  }
  const int total = p.tiles_m * p.tiles_n * p.batch;
  int grid = std::min(total, num_sms());
  if (max_ctas > 0) grid = std::min(grid, max_ctas);
  if (grid <= 0) return 0;
  p.b_constant = chained_launches_constant_b() ? 1 : 0;
  p.trace = g_gemm_trace;
  cudaError_t e = launch_chained(gemm_bf16_kernel<BN, EPI>, dim3(grid), dim3(kGemmThreads),
                                 S::kTotal, stream, *tA, *tB, *tB2, p);
  count_launches(1);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("gemm launch failed: %s", cudaGetErrorString(e));
  return 0;
}

static const CUtensorMap* operand_map(const void* ptr, int mn_major, long long rows_mn,
                                      long long k, long long ld, long long batch_stride, int batch,
                                      int box_rows_kmajor) {
  // K-major: memory is [rows_mn, k] (k contiguous, row stride ld). box {64 k, box_rows, 1}
  // MN-major: memory is [k, rows_mn] (mn contiguous, row stride ld). box {64 mn, 64 k, 1}
  uint64_t dims[3];
  uint64_t strides[2];
  uint32_t box[3];
  if (!mn_major) {
    dims[0] = k;
    dims[1] = rows_mn;
    box[0] = 64;
    box[1] = box_rows_kmajor;
  } else {
    dims[0] = rows_mn;
    dims[1] = k;
    box[0] = 64;
    box[1] = 64;
  }
  dims[2] = batch;
  box[2] = 1;
  strides[0] = static_cast<uint64_t>(ld) * 2;
  strides[1] = static_cast<uint64_t>(batch > 1 ? batch_stride : ld * dims[1]) * 2;
  if (strides[1] == 0) strides[1] = strides[0];
  return get_tensor_map(ptr, 2, 3, dims, strides, box, 1);
}

}  // namespace t5x

// C API -----------------------------------------------------------------------
// All pointers are device pointers; leading dimensions / strides are in elements.
// epilogue: 0 plain, 1 gated-GELU (B and B2 are wi_0 / wi_1; N is the width of each),
//           2 residual add (R bf16).
// Returns 0 on success; a negative value with t5x_last_error() set otherwise.
namespace t5x {
int launch_gemm_pair(int epilogue, const CUtensorMap* tA, const CUtensorMap* tB,
                     const CUtensorMap* tB2, GemmParams& p, int max_ctas, cudaStream_t stream,
                     const GemmTp* tp = nullptr, int tp_mode = 0);

// 0 = never use CTA pairs, 1 = when the shape suits them (default), 2 = always.
// Read once from T5X_GEMM_PAIR; t5x_gemm_set_pair_mode overrides it.
static int g_pair_mode = -1;
static int gemm_pair_mode() {
  if (g_pair_mode < 0) {
    const char* e = getenv("T5X_GEMM_PAIR");
    g_pair_mode = e ? atoi(e) : 1;
    if (g_pair_mode < 0 || g_pair_mode > 2) g_pair_mode = 1;
  }
  return g_pair_mode;
}
}  // namespace t5x

T5X_API int t5x_gemm_set_pair_mode(int mode) {
  if (mode < 0 || mode > 2) return t5x::set_error("gemm pair mode must be 0, 1 or 2");
  t5x::g_pair_mode = mode;
  return 0;
}

namespace t5x {
// What the cross-entropy epilogues need besides the GEMM itself.
struct GemmCe {
  const long long* targets;
  int vocab_start;
  float* part;
  int* arg;
  float* target_logit;
  const float* lse;
  const float* row_scale;
  float z, conf, low;
};
static thread_local const GemmCe* g_ce_extras = nullptr;  // set by the two entry points around gemm_impl

static int gemm_impl(const void* A, const void* B, const void* B2, void* C, int M, int N,
                     int K, int batch, long long lda, long long ldb, long long ldc,
                     long long a_batch_stride, long long b_batch_stride,
                     long long c_batch_stride, int a_mn_major, int b_mn_major, int out_fp32,
                     int accumulate, int epilogue, const void* R, long long ldr,
                     long long r_batch_stride, void* H0, void* H1, long long ldh, float alpha,
                     int max_ctas, void* stream, const GemmTp* tp, int tp_mode) {
  if (M <= 0 || N <= 0 || batch <= 0) return 0;
  if (K <= 0) return set_error("gemm: K must be positive");
  if (lda % 8 || ldb % 8) return set_error("gemm: lda/ldb must be multiples of 8 elements");
  if ((a_batch_stride % 8) || (b_batch_stride % 8))
    return set_error("gemm: batch strides must be multiples of 8 elements");
  GemmParams p;
  p.M = M;
  p.N = N;
  p.K = K;
  p.batch = batch;
  p.a_mn = a_mn_major;
  p.b_mn = b_mn_major;
  p.out_fp32 = out_fp32;
  p.accumulate = accumulate;
  p.C = C;
  p.ldc = ldc;
  p.c_batch_stride = c_batch_stride;
  p.R = static_cast<const __nv_bfloat16*>(R);
  p.ldr = ldr;
  p.r_batch_stride = r_batch_stride;
  p.H0 = static_cast<__nv_bfloat16*>(H0);
  p.H1 = static_cast<__nv_bfloat16*>(H1);
  p.ldh = ldh;
  p.alpha = alpha;
  p.status = device_status_buffer();
  p.tiles_m = (M + kBM - 1) / kBM;
  p.mt_rot = 0;
  p.b_constant = 0;
  p.trace = nullptr;
  p.ce_targets = nullptr;
  p.ce_part = nullptr;
  p.ce_arg = nullptr;
  p.ce_target_logit = nullptr;
  p.ce_lse = p.ce_row_scale = nullptr;
  p.ce_vocab_start = 0;
  p.ce_z = p.ce_conf = p.ce_low = 0.f;

  const CUtensorMap* tA = operand_map(A, a_mn_major, M, K, lda, a_batch_stride, batch, 128);
  const CUtensorMap* tB = operand_map(B, b_mn_major, N, K, ldb, b_batch_stride, batch, 128);
  if (!tA || !tB) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int sms = num_sms();
  auto waves_eff = [&](long long tiles, int units) {
    long long waves = (tiles + units - 1) / units;
    return static_cast<double>(tiles) / static_cast<double>(waves * units);
  };
  // CTA pairs (256 x 256 tiles, a third less shared-memory traffic per FLOP) when the problem
  // has at least one full pair tile and pairs fill the machine about as well as single CTAs.
  const int pair_tiles_m = (M + 2 * kBM - 1) / (2 * kBM);
  const int pair_mode = gemm_pair_mode();

  if (tp != nullptr) {
    // tensor-parallel kernels exist for CTA pairs only; the walk over row tiles is rotated so
    // that an all-gather starts with this rank's rows and a reduce-scatter ends with them
    if (batch != 1 || out_fp32 || accumulate)
      return set_error("tensor-parallel gemm: batch 1, bf16 output, no accumulate");
    if (epilogue == kEpiResidual && R == nullptr) return set_error("residual epilogue needs R");
    const CUtensorMap* tB2 = tB;
    if (epilogue == kEpiGatedGelu) {
      tB2 = operand_map(B2, b_mn_major, N, K, ldb, b_batch_stride, batch, 128);
      if (!tB2) return -1;
    }
    p.tiles_m = pair_tiles_m;
    p.tiles_n = epilogue == kEpiGatedGelu ? (N + 127) / 128 : (N + 255) / 256;
    const int first = tp_mode == kTpAllGather ? tp->rank : (tp->rank + 1) % tp->world;
    p.mt_rot = static_cast<int>((static_cast<long long>(first) * tp->rows_per_rank) / (2 * kBM));
    if (p.mt_rot >= p.tiles_m) p.mt_rot = 0;
    return launch_gemm_pair(epilogue, tA, tB, tB2, p, max_ctas, st, tp, tp_mode);
  }

  if (epilogue == kEpiCeStats || epilogue == kEpiCeGrad) {
    const GemmCe* ce = g_ce_extras;
    if (ce == nullptr || batch != 1) return set_error("cross-entropy epilogue: bad call");
    p.ce_targets = ce->targets;
    p.ce_vocab_start = ce->vocab_start;
    p.ce_part = ce->part;
    p.ce_arg = ce->arg;
    p.ce_target_logit = ce->target_logit;
    p.ce_lse = ce->lse;
    p.ce_row_scale = ce->row_scale;
    p.ce_z = ce->z;
    p.ce_conf = ce->conf;
    p.ce_low = ce->low;
    p.tiles_n = (N + 255) / 256;
    if (pair_mode != 0 && M >= 2 * kBM) {
      p.tiles_m = pair_tiles_m;
      return launch_gemm_pair(epilogue, tA, tB, tB, p, max_ctas, st);
    }
    return epilogue == kEpiCeStats ? launch_gemm<256, kEpiCeStats>(tA, tB, tB, p, max_ctas, st)
                                   : launch_gemm<256, kEpiCeGrad>(tA, tB, tB, p, max_ctas, st);
  }
  if (epilogue == kEpiGatedGelu) {
    if (out_fp32 || accumulate) return set_error("gated-GELU epilogue writes bf16 without accumulate");
    const CUtensorMap* tB2 = operand_map(B2, b_mn_major, N, K, ldb, b_batch_stride, batch, 128);
    if (!tB2) return -1;
    p.tiles_n = (N + 127) / 128;
    const double e1 = waves_eff(1ll * p.tiles_m * p.tiles_n * batch, sms);
    const double e2 = waves_eff(1ll * pair_tiles_m * p.tiles_n * batch, sms / 2);
    if (pair_mode == 2 || (pair_mode == 1 && M >= 2 * kBM && e2 * 1.2 >= e1)) {
      p.tiles_m = pair_tiles_m;
      return launch_gemm_pair(kEpiGatedGelu, tA, tB, tB2, p, max_ctas, st);
    }
    return launch_gemm<256, kEpiGatedGelu>(tA, tB, tB2, p, max_ctas, st);
  }
  // Tile width: 256 unless N is small or 128-wide tiles fill the SMs markedly better.
  const double e128 = waves_eff(1ll * p.tiles_m * ((N + 127) / 128) * batch, sms);
  const double e256 = waves_eff(1ll * p.tiles_m * ((N + 255) / 256) * batch, sms);
  int bn = 256;
  if (N <= 128 || e128 > e256 * 1.15) bn = 128;
  if (epilogue == kEpiResidual && R == nullptr) return set_error("residual epilogue needs R");
  {
    const double e1 = bn == 256 ? e256 : e128 / 1.15;
    const double e2 = waves_eff(1ll * pair_tiles_m * ((N + 255) / 256) * batch, sms / 2);
    if (pair_mode == 2 || (pair_mode == 1 && M >= 2 * kBM && N >= 256 && e2 * 1.2 >= e1)) {
      p.tiles_m = pair_tiles_m;
      p.tiles_n = (N + 255) / 256;
      return launch_gemm_pair(epilogue, tA, tB, tB, p, max_ctas, st);
    }
  }
  p.tiles_n = (N + bn - 1) / bn;
  if (epilogue == kEpiResidual) {
    return bn == 256 ? launch_gemm<256, kEpiResidual>(tA, tB, tB, p, max_ctas, st)
                     : launch_gemm<128, kEpiResidual>(tA, tB, tB, p, max_ctas, st);
  }
  return bn == 256 ? launch_gemm<256, kEpiPlain>(tA, tB, tB, p, max_ctas, st)
                   : launch_gemm<128, kEpiPlain>(tA, tB, tB, p, max_ctas, st);
}
}  // namespace t5x

// Phase trace of the one-CTA-per-tile GEMM for profiling: while `buffer` (device memory, 8
// int64 per CTA of the largest grid, i.e. 8 x the number of SMs) is set, every such GEMM
// launched from the calling thread records nanosecond timestamps of its first tile's phases
// (see GemmParams::trace). Null switches it off.
T5X_API int t5x_gemm_set_trace(void* buffer) {
  t5x::g_gemm_trace = static_cast<long long*>(buffer);
  return 0;
}

T5X_API int t5x_gemm_bf16(const void* A, const void* B, const void* B2, void* C, int M, int N,
                          int K, int batch, long long lda, long long ldb, long long ldc,
                          long long a_batch_stride, long long b_batch_stride,
                          long long c_batch_stride, int a_mn_major, int b_mn_major, int out_fp32,
                          int accumulate, int epilogue, const void* R, long long ldr,
                          long long r_batch_stride, void* H0, void* H1, long long ldh, float alpha,
                          int max_ctas, void* stream) {
  return t5x::gemm_impl(A, B, B2, C, M, N, K, batch, lda, ldb, ldc, a_batch_stride,
                        b_batch_stride, c_batch_stride, a_mn_major, b_mn_major, out_fp32,
                        accumulate, epilogue, R, ldr, r_batch_stride, H0, H1, ldh, alpha, max_ctas,
                        stream, nullptr, 0);
}

namespace t5x {
static int tp_signals(GemmTp& tp, void* sig_local, void* const* sig_peers, unsigned int epoch,
                      void* exit_count, const char* what) {
  if (sig_local == nullptr || sig_peers == nullptr || exit_count == nullptr)
    return set_error("%s: signal words are required", what);
  tp.sig_local = static_cast<unsigned int*>(sig_local);
  for (int r = 0; r < tp.world; ++r) tp.sig_peer[r] = static_cast<unsigned int*>(sig_peers[r]);
  tp.epoch = epoch;
  tp.exit_count = static_cast<unsigned int*>(exit_count);
  return 0;
}
}  // namespace t5x

// Number of arrival counters (uint32, zero before the first call) an all-gather GEMM over
// `world` ranks with `rows_per_rank` rows each uses.
T5X_API int t5x_gemm_allgather_flag_words(int world, int rows_per_rank) {
  return world * ((rows_per_rank + t5x::kTpGroupRows - 1) / t5x::kTpGroupRows);
}

// All-gather -> GEMM in one kernel. A is this rank's [M, K] bf16 buffer (row-major, lda == K)
// whose block `rank` (rows_per_rank rows) is already filled; a_peers[r] is rank r's buffer of
// the same layout as mapped into this process. The kernel pulls the other blocks over NVLink
// while it multiplies, so A is complete (and reusable) when it returns. No barrier is needed in
// front of the call: the kernel raises this rank's "rows ready" signal (epoch `epoch`, one
// more than in the previous call of either tensor-parallel GEMM on this group) and waits for
// each peer's before it reads from it. `flags`: t5x_gemm_allgather_flag_words counters of this
// GPU's memory, zero on entry and again on exit. sig_local / sig_peers: 32 uint32 per rank in
// memory every rank maps (zero at start); exit_count: one zeroed uint32 of this GPU.
// epilogue 0 (C = A @ B) or 1 (gated GELU). K must be a multiple of 32.
T5X_API int t5x_gemm_allgather_bf16(void* A, const void* const* a_peers, int world, int rank,
                                    int rows_per_rank, void* flags, const void* B, const void* B2,
                                    void* C, int M, int N, int K, long long ldb, long long ldc,
                                    int b_mn_major, int epilogue, void* H0, void* H1,
                                    long long ldh, void* sig_local, void* const* sig_peers,
                                    unsigned int epoch, void* exit_count, void* stream) {
  using namespace t5x;
  if (world < 1 || world > kTpMaxPeers || rank < 0 || rank >= world ||
      static_cast<long long>(rows_per_rank) * world != M || (K % 32))
    return set_error("gemm_allgather: bad world/rank/rows (%d/%d/%d for M=%d) or K=%d not a "
                     "multiple of 32", world, rank, rows_per_rank, M, K);
  GemmTp tp = {};
  tp.world = world;
  tp.rank = rank;
  tp.rows_per_rank = rows_per_rank;
  tp.block_bytes = static_cast<long long>(rows_per_rank) * K * 2;
  tp.group_bytes = static_cast<long long>(kTpGroupRows) * K * 2;
  tp.groups_per_block = (rows_per_rank + kTpGroupRows - 1) / kTpGroupRows;
  for (int r = 0; r < world; ++r) tp.a_src[r] = static_cast<const uint8_t*>(a_peers[r]);
  tp.a_dst = static_cast<uint8_t*>(A);
  tp.flags = static_cast<unsigned int*>(flags);
  if (int rc = tp_signals(tp, sig_local, sig_peers, epoch, exit_count, "gemm_allgather")) return rc;
  return gemm_impl(A, B, B2, C, M, N, K, 1, K, ldb, ldc, 0, 0, 0, 0, b_mn_major, 0, 0, epilogue,
                   nullptr, 0, 0, H0, H1, ldh, 1.f, 0, stream, &tp, kTpAllGather);
}

// GEMM -> reduce-scatter in one kernel: the bf16 partial product A @ B (+ R) of this rank is
// stored row block by row block into the owners' inboxes: c_peers[r] is this rank's slot
// ([rows_per_rank, ldc]) of rank r's inbox as mapped into this process. When its last store
// has been performed the kernel raises this rank's "scattered" signal (epoch `epoch`) on every
// peer; the owners sum their slots with t5x_slot_sum_wait_bf16, which waits for those signals.
// epilogue 0 or 2 (adds the local bf16 [M, N] matrix R first).
T5X_API int t5x_gemm_reducescatter_bf16(const void* A, const void* B, void* const* c_peers,
                                        int world, int rank, int rows_per_rank, int M, int N, int K,
                                        long long lda, long long ldb, long long ldc,
                                        int a_mn_major, int b_mn_major, const void* R,
                                        long long ldr, void* sig_local, void* const* sig_peers,
                                        unsigned int epoch, void* exit_count, void* stream) {
  using namespace t5x;
  if (world < 1 || world > kTpMaxPeers || rank < 0 || rank >= world ||
      static_cast<long long>(rows_per_rank) * world != M || (ldc % 8))
    return set_error("gemm_reducescatter: bad world/rank/rows (%d/%d/%d for M=%d)", world, rank,
                     rows_per_rank, M);
  GemmTp tp = {};
  tp.world = world;
  tp.rank = rank;
  tp.rows_per_rank = rows_per_rank;
  for (int r = 0; r < world; ++r) {
    if (reinterpret_cast<uintptr_t>(c_peers[r]) & 15)
      return set_error("gemm_reducescatter: inbox pointers must be 16-byte aligned");
    tp.c_dst[r] = static_cast<__nv_bfloat16*>(c_peers[r]);
  }
  if (int rc = tp_signals(tp, sig_local, sig_peers, epoch, exit_count, "gemm_reducescatter"))
    return rc;
  return gemm_impl(A, B, nullptr, nullptr, M, N, K, 1, lda, ldb, ldc, 0, 0, 0, a_mn_major,
                   b_mn_major, 0, 0, R ? kEpiResidual : kEpiPlain, R, ldr, 0, nullptr, nullptr, 0,
                   1.f, 0, stream, &tp, kTpReduceScatter);
}

// ---- logits projection fused with the cross-entropy: the [M, N] logits are never stored ----
// Number of column tiles (partials per row) the forward produces for a vocabulary slice of N.
T5X_API int t5x_gemm_ce_tiles(int N) { return (N + 255) / 256; }

// Forward: logits = alpha * A[M, K] @ B[K, N] are folded, tile by tile in the GEMM epilogue,
// into part[M, tiles, 4] (max, sum exp(x - max), sum x, largest x), arg[M, tiles] (vocabulary
// id of the largest x) and target_logit[M] (written only if the row's target lies in
// [vocab_start, vocab_start + N)). t5x_ce_merge turns the partials into per-row statistics.
T5X_API int t5x_gemm_ce_stats(const void* A, const void* B, int M, int N, int K, long long lda,
                              long long ldb, int a_mn_major, int b_mn_major, float alpha,
                              const void* targets, int vocab_start, void* part, void* arg,
                              void* target_logit, void* stream) {
  using namespace t5x;
  if (M <= 0 || N <= 0) return 0;
  if (targets == nullptr || part == nullptr || arg == nullptr || target_logit == nullptr)
    return set_error("gemm_ce_stats: null pointer");
  GemmCe ce = {};
  ce.targets = static_cast<const long long*>(targets);
  ce.vocab_start = vocab_start;
  ce.part = static_cast<float*>(part);
  ce.arg = static_cast<int*>(arg);
  ce.target_logit = static_cast<float*>(target_logit);
  g_ce_extras = &ce;
  const int rc = gemm_impl(A, B, nullptr, nullptr, M, N, K, 1, lda, ldb, 0, 0, 0, 0, a_mn_major,
                           b_mn_major, 0, 0, kEpiCeStats, nullptr, 0, 0, nullptr, nullptr, 0,
                           alpha, 0, stream, nullptr, 0);
  g_ce_extras = nullptr;
  return rc;
}

// Backward: recomputes the logits tiles and writes dlogits[M, N] (bf16, row stride ldd) =
// row_scale * ((1 + 2 z lse) * softmax - soft targets), with lse[M] over the whole vocabulary.
T5X_API int t5x_gemm_ce_grad(const void* A, const void* B, void* dlogits, long long ldd, int M,
                             int N, int K, long long lda, long long ldb, int a_mn_major,
                             int b_mn_major, float alpha, const void* targets, int vocab_start,
                             const void* lse, const void* row_scale, float z_loss,
                             float confidence, float low_confidence, void* stream) {
  using namespace t5x;
  if (M <= 0 || N <= 0) return 0;
  if (targets == nullptr || lse == nullptr || row_scale == nullptr || dlogits == nullptr)
    return set_error("gemm_ce_grad: null pointer");
  GemmCe ce = {};
  ce.targets = static_cast<const long long*>(targets);
  ce.vocab_start = vocab_start;
  ce.lse = static_cast<const float*>(lse);
  ce.row_scale = static_cast<const float*>(row_scale);
  ce.z = z_loss;
  ce.conf = confidence;
  ce.low = low_confidence;
  g_ce_extras = &ce;
  const int rc = gemm_impl(A, B, nullptr, dlogits, M, N, K, 1, lda, ldb, ldd, 0, 0, 0, a_mn_major,
                           b_mn_major, 0, 0, kEpiCeGrad, nullptr, 0, 0, nullptr, nullptr, 0,
                           alpha, 0, stream, nullptr, 0);
  g_ce_extras = nullptr;
  return rc;
}
