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

#include "common.cuh"

namespace t5x {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kGemmThreads = 192;
constexpr int kKernelIdGemm = 1;

enum GemmEpilogue : int { kEpiPlain = 0, kEpiGatedGelu = 1, kEpiResidual = 2 };

struct GemmParams {
  int M, N, K, batch;
  int a_mn, b_mn;
  int out_fp32, accumulate;
  void* C;
  long long ldc, c_batch_stride;  // elements
  const __nv_bfloat16* R;         // residual (bf16), same shape as C
  long long ldr, r_batch_stride;
  __nv_bfloat16* H0;  // gated-GELU: optional copies of the two pre-activations
  __nv_bfloat16* H1;
  long long ldh;
  float alpha;
  int tiles_m, tiles_n;
  int* status;
};

template <int BN>
struct GemmSmem {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kBarrierBytes = 1024;
  static constexpr int kTotal = kStages * kStageBytes + kBarrierBytes + 1024;  // +1024 align slack
};

__device__ __forceinline__ void store_row_bf16(__nv_bfloat16* dst, const float* v, int n_valid,
                                               bool vec_ok) {
  if (vec_ok && n_valid >= 32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 p0 = __floats2bfloat162_rn(v[i * 8 + 0], v[i * 8 + 1]);
      __nv_bfloat162 p1 = __floats2bfloat162_rn(v[i * 8 + 2], v[i * 8 + 3]);
      __nv_bfloat162 p2 = __floats2bfloat162_rn(v[i * 8 + 4], v[i * 8 + 5]);
      __nv_bfloat162 p3 = __floats2bfloat162_rn(v[i * 8 + 6], v[i * 8 + 7]);
      uint4 u;
      u.x = *reinterpret_cast<uint32_t*>(&p0);
      u.y = *reinterpret_cast<uint32_t*>(&p1);
      u.z = *reinterpret_cast<uint32_t*>(&p2);
      u.w = *reinterpret_cast<uint32_t*>(&p3);
      reinterpret_cast<uint4*>(dst)[i] = u;
    }
  } else {
    for (int i = 0; i < 32 && i < n_valid; ++i) dst[i] = __float2bfloat16(v[i]);
  }
}

__device__ __forceinline__ void load_row_bf16(const __nv_bfloat16* src, float* v, int n_valid,
                                              bool vec_ok) {
  if (vec_ok && n_valid >= 32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 u = reinterpret_cast<const uint4*>(src)[i];
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(p[j]);
        v[i * 8 + j * 2] = f.x;
        v[i * 8 + j * 2 + 1] = f.y;
      }
    }
  } else {
    for (int i = 0; i < 32; ++i) v[i] = (i < n_valid) ? __bfloat162float(src[i]) : 0.f;
  }
}

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

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
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

  const int num_kb = (p.K + kBK - 1) / kBK;
  const int tiles_per_batch = p.tiles_m * p.tiles_n;
  const int total_tiles = tiles_per_batch * p.batch;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int b = tile / tiles_per_batch;
        const int rem = tile - b * tiles_per_batch;
        const int m0 = (rem / p.tiles_n) * kBM;
        const int n0 = (rem % p.tiles_n) * kTileN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) {
            report_status(p.status, kStatusTimeoutProducer, kKernelIdGemm, tile, kb);
            *abort_flag = 1;
            ok = false;
            break;
          }
          mbar_expect_tx(&full[stage], S::kStageBytes);
          uint8_t* a_dst = sA + stage * S::kABytes;
          uint8_t* b_dst = sB + stage * S::kBBytes;
          const int k0 = kb * kBK;
          if (!p.a_mn) {
            tma_load_3d(a_dst, &tmA, &full[stage], k0, m0, b);  // box {64, 128, 1}
          } else {
#pragma unroll
            for (int j = 0; j < kBM / 64; ++j)  // box {64 (m), 64 (k), 1}
              tma_load_3d(a_dst + j * 8192, &tmA, &full[stage], m0 + 64 * j, k0, b);
          }
          if (EPI == kEpiGatedGelu) {
            constexpr int kHalf = BN / 2;  // 128 columns of each of wi_0 and wi_1
            if (!p.b_mn) {
              tma_load_3d(b_dst, &tmB, &full[stage], k0, n0, b);
              tma_load_3d(b_dst + kHalf * 128, &tmB2, &full[stage], k0, n0, b);
            } else {
#pragma unroll
              for (int j = 0; j < kHalf / 64; ++j) {
                tma_load_3d(b_dst + j * 8192, &tmB, &full[stage], n0 + 64 * j, k0, b);
                tma_load_3d(b_dst + (kHalf / 64 + j) * 8192, &tmB2, &full[stage], n0 + 64 * j, k0,
                            b);
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
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
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
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int q = warp & 3;  // TMEM lanes [32q, 32q+32) belong to warps with id % 4 == q
    int local = 0;
    bool ok = true;
    const bool c_vec_ok = (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      const int b = tile / tiles_per_batch;
      const int rem = tile - b * tiles_per_batch;
      const int m0 = (rem / p.tiles_n) * kBM;
      const int n0 = (rem % p.tiles_n) * kTileN;
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag)) {
        if (lane == 0) report_status(p.status, kStatusTimeoutEpilogue, kKernelIdGemm, tile, 0);
        *abort_flag = 1;
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;

      if (EPI == kEpiGatedGelu) {
        constexpr int kHalf = BN / 2;
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + b * p.c_batch_stride +
                             static_cast<long long>(row) * p.ldc;
#pragma unroll 1
        for (int c = 0; c < kHalf / 32; ++c) {
          uint32_t r0[32], r1[32];
          tmem_ld32(t_row + c * 32, r0);
          tmem_ld32(t_row + kHalf + c * 32, r1);
          tmem_ld_wait();
          const int col = n0 + c * 32;
          const int n_valid = p.N - col;
          if (row_ok && n_valid > 0) {
            float g[32], h0[32], h1[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              h0[i] = __uint_as_float(r0[i]);
              h1[i] = __uint_as_float(r1[i]);
              g[i] = gelu_tanh(h0[i]) * h1[i];
            }
            store_row_bf16(out + col, g, n_valid, c_vec_ok);
            if (p.H0 != nullptr) {
              const bool hv = (p.ldh % 8 == 0);
              store_row_bf16(p.H0 + static_cast<long long>(row) * p.ldh + col, h0, n_valid, hv);
              store_row_bf16(p.H1 + static_cast<long long>(row) * p.ldh + col, h1, n_valid, hv);
            }
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(t_row + c * 32, r);
          tmem_ld_wait();
          const int col = n0 + c * 32;
          const int n_valid = p.N - col;
          if (row_ok && n_valid > 0) {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
            if (EPI == kEpiResidual) {
              float rr[32];
              const bool rv = (p.ldr % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.R) & 15) == 0);
              load_row_bf16(p.R + b * p.r_batch_stride + static_cast<long long>(row) * p.ldr + col,
                            rr, n_valid, rv);
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] += rr[i];
            }
            if (p.out_fp32) {
              float* out = reinterpret_cast<float*>(p.C) + b * p.c_batch_stride +
                           static_cast<long long>(row) * p.ldc + col;
              const bool fv = (p.ldc % 4 == 0) && n_valid >= 32;
              if (fv) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  float4 o = make_float4(v[i * 4], v[i * 4 + 1], v[i * 4 + 2], v[i * 4 + 3]);
                  if (p.accumulate) {
                    float4 old = reinterpret_cast<float4*>(out)[i];
                    o.x += old.x;
                    o.y += old.y;
                    o.z += old.z;
                    o.w += old.w;
                  }
                  reinterpret_cast<float4*>(out)[i] = o;
                }
              } else {
                for (int i = 0; i < 32 && i < n_valid; ++i)
                  out[i] = p.accumulate ? out[i] + v[i] : v[i];
              }
            } else {
              __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + b * p.c_batch_stride +
                                   static_cast<long long>(row) * p.ldc + col;
              if (p.accumulate) {
                float old[32];
                load_row_bf16(out, old, n_valid, c_vec_ok);
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] += old[i];
              }
              store_row_bf16(out, v, n_valid, c_vec_ok);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
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
  gemm_bf16_kernel<BN, EPI><<<grid, kGemmThreads, S::kTotal, stream>>>(*tA, *tB, *tB2, p);
  count_launches(1);
  cudaError_t e = cudaGetLastError();
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
T5X_API int t5x_gemm_bf16(const void* A, const void* B, const void* B2, void* C, int M, int N,
                          int K, int batch, long long lda, long long ldb, long long ldc,
                          long long a_batch_stride, long long b_batch_stride,
                          long long c_batch_stride, int a_mn_major, int b_mn_major, int out_fp32,
                          int accumulate, int epilogue, const void* R, long long ldr,
                          long long r_batch_stride, void* H0, void* H1, long long ldh, float alpha,
                          int max_ctas, void* stream) {
  using namespace t5x;
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

  const CUtensorMap* tA = operand_map(A, a_mn_major, M, K, lda, a_batch_stride, batch, 128);
  const CUtensorMap* tB = operand_map(B, b_mn_major, N, K, ldb, b_batch_stride, batch, 128);
  if (!tA || !tB) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  if (epilogue == kEpiGatedGelu) {
    if (out_fp32 || accumulate) return set_error("gated-GELU epilogue writes bf16 without accumulate");
    const CUtensorMap* tB2 = operand_map(B2, b_mn_major, N, K, ldb, b_batch_stride, batch, 128);
    if (!tB2) return -1;
    p.tiles_n = (N + 127) / 128;
    return launch_gemm<256, kEpiGatedGelu>(tA, tB, tB2, p, max_ctas, st);
  }
  // Tile width: 256 unless N is small or 128-wide tiles fill the SMs markedly better.
  const int sms = num_sms();
  auto waves_eff = [&](int bn) {
    long long tiles = 1ll * p.tiles_m * ((N + bn - 1) / bn) * batch;
    long long waves = (tiles + sms - 1) / sms;
    return static_cast<double>(tiles) / static_cast<double>(waves * sms);
  };
  int bn = 256;
  if (N <= 128 || waves_eff(128) > waves_eff(256) * 1.15) bn = 128;
  p.tiles_n = (N + bn - 1) / bn;
  if (epilogue == kEpiResidual) {
    if (R == nullptr) return set_error("residual epilogue needs R");
    return bn == 256 ? launch_gemm<256, kEpiResidual>(tA, tB, tB, p, max_ctas, st)
                     : launch_gemm<128, kEpiResidual>(tA, tB, tB, p, max_ctas, st);
  }
  return bn == 256 ? launch_gemm<256, kEpiPlain>(tA, tB, tB, p, max_ctas, st)
                   : launch_gemm<128, kEpiPlain>(tA, tB, tB, p, max_ctas, st);
}
