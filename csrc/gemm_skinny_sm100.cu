// bf16 GEMM for few rows (decode steps: a few hundred rows against a weight matrix), with the
// K dimension split over the CTAs of a thread-block cluster and the partial products summed
// through distributed shared memory.
//
//   C[M, N] (bf16) = A[M, K] * B (+ R)        B: row-major [K, N] or [N, K]; R: residual, bf16
//
// Why: with M = 256 an output has only 2 x N/128 tiles, so one CTA per tile leaves most SMs
// idle while each busy one streams its whole K range (a latency chain of K/64 stages). Cutting
// K into slices puts more SMs on the weight stream, but the partial products then have to be
// added: through fp32 atomics into a workspace plus a finishing kernel that converts and
// clears it, the sum alone cost as much as the loads (4.5 us of a 9.8 us kernel, then a second
// launch). Here the S CTAs that share an output tile form a cluster. When its MMAs are done, a
// CTA parks its fp32 tile in its own operand ring (free by then) and sends each peer the rows
// that peer owns (rows [r * 128/S, (r+1) * 128/S) of the tile belong to cluster rank r) with
// one bulk shared-memory-to-shared-memory copy, counted on an mbarrier of the receiver; the
// receiver then sums the S contributions of its rows, adds the residual and stores bf16 rows:
// no workspace, no atomics, no second kernel. (Storing the rows into the peer with
// `st.shared::cluster` from registers, 16 bytes of 32 different rows per instruction, took
// 3.4 us for a 128 x 128 tile; the bulk copies are row-contiguous.)
//
// Roles per CTA (192 threads) as in the other GEMMs: warp 0 = TMA producer, warp 1 = MMA issuer
// and TMEM owner, warps 2..5 = epilogue (one TMEM lane quarter each). Every thread reaches both
// cluster barriers (one right after set-up, one before exit) whatever happened before (a wait that gave up raises the CTA's abort flag
// and a status word, and the CTA skips its work but still arrives), so a failure cannot leave
// the cluster waiting. No TMA load uses cluster multicast.
#include <algorithm>

#include "gemm_common.cuh"

namespace t5x {

constexpr int kSkBN = 128;
constexpr int kSkStages = 4;
constexpr int kSkABytes = kBM * kBK * 2;
constexpr int kSkBBytes = kSkBN * kBK * 2;
constexpr int kSkStageBytes = kSkABytes + kSkBBytes;
constexpr int kSkRingBytes = kSkStages * kSkStageBytes;
constexpr int kSkTileBytes = kBM * kSkBN * 4;  // one fp32 tile: S slots x (128 / S) rows x 128
constexpr int kSkSmemTotal = kSkRingBytes + kSkTileBytes + 1024 + 1024;
constexpr int kKernelIdGemmSkinny = 7;
static_assert(kSkTileBytes <= kSkRingBytes, "the outgoing tile is staged in the operand ring");

struct SkinnyParams {
  int M, N, K;
  int b_mn;
  int splits;         // cluster size S: 1, 2, 4 or 8
  int kb_per_split;   // 64-deep k blocks per CTA
  int tiles_n;
  __nv_bfloat16* C;
  long long ldc;
  const __nv_bfloat16* R;
  long long ldr;
  float alpha;
  int b_constant;
  int* status;
  // Optional phase trace (t5x_gemm_set_trace), 8 timestamps per CTA: entry, set-up done, first
  // loads issued, first operands landed, accumulator complete, tile parked in shared memory,
  // peers' rows received, rows stored.
  long long* trace;
};

// This CTA's shared memory -> another CTA's of the cluster; the bytes are counted on an
// mbarrier in the destination CTA. Both destination addresses are cluster-window addresses.
__device__ __forceinline__ void bulk_copy_to_cta(uint32_t dst_cluster_addr, const void* src_smem,
                                                 uint32_t bytes, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      :
      : "r"(dst_cluster_addr), "r"(smem_u32(src_smem)), "r"(bytes), "r"(bar_cluster_addr)
      : "memory");
}
__device__ __forceinline__ void epilogue_bar_sync() {  // the four epilogue warps (128 threads)
  asm volatile("bar.sync 1, 128;" ::: "memory");
}

__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmA,
                       const __grid_constant__ CUtensorMap tmB, const SkinnyParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + kSkStages * kSkABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kSkRingBytes + kSkTileBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + kSkStages;
  uint64_t* tmem_full = bars + 2 * kSkStages;
  uint64_t* recv_bar = bars + 2 * kSkStages + 1;  // counts the bytes of the peers' partial rows
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kSkStages + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // after the MMAs the ring holds this CTA's fp32 tile on its way out ([128 rows][128]); the
  // peers' contributions to this CTA's rows arrive in `recv` ([S slots][128 / S rows][128])
  float* staging = reinterpret_cast<float*>(smem);
  float* recv = reinterpret_cast<float*>(smem + kSkRingBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int S = p.splits;
  const int rank = S > 1 ? static_cast<int>(cluster_ctarank()) : 0;
  const int tile = blockIdx.x / S;
  const int mt = tile / p.tiles_n, nt = tile - mt * p.tiles_n;
  const int m0 = mt * kBM, n0 = nt * kSkBN;
  const int num_kb = p.kb_per_split;
  const int kb0 = rank * num_kb;

  chain_release();
  if (threadIdx.x == 0) {
    T5X_GEMM_TRACE(0);
    for (int s = 0; s < kSkStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(tmem_full, 1);
    mbar_init(recv_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
    if (S > 1) mbar_expect_tx(recv_bar, static_cast<uint32_t>((S - 1) * (kSkTileBytes / S)));
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kSkBN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  // every CTA of the cluster has initialised its barriers before any peer may signal them;
  // this early all CTAs are at the same point, so the barrier costs little
  if (S > 1) cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) T5X_GEMM_TRACE(1);

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      auto load_a = [&](int stage, int kb) {
        tma_load_3d(sA + stage * kSkABytes, &tmA, &full[stage], (kb0 + kb) * kBK, m0, 0);
      };
      auto load_b = [&](int stage, int kb) {
        uint8_t* b_dst = sB + stage * kSkBBytes;
        const int k0 = (kb0 + kb) * kBK;
        if (!p.b_mn) {
          tma_load_3d(b_dst, &tmB, &full[stage], k0, n0, 0);  // box {64 k, 128 n, 1}
        } else {
#pragma unroll
          for (int j = 0; j < kSkBN / 64; ++j)  // box {64 n, 64 k, 1}
            tma_load_3d(b_dst + j * 8192, &tmB, &full[stage], n0 + 64 * j, k0, 0);
        }
      };
      int stage = 0;
      uint32_t phase = 0;
      int first = 0;
      if (p.b_constant) {
        // constant weights: their first stages are requested before the wait for the
        // preceding kernel, the activations after it
        first = min(kSkStages, num_kb);
        for (int kb = 0; kb < first; ++kb) {
          mbar_expect_tx(&full[kb], kSkStageBytes);
          load_b(kb, kb);
        }
        chain_wait();
        for (int kb = 0; kb < first; ++kb) load_a(kb, kb);
        T5X_GEMM_TRACE(2);
        if (first == kSkStages) phase = 1;
        else stage = first;
      } else {
        chain_wait();
      }
      for (int kb = first; kb < num_kb; ++kb) {
        if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) {
          report_status(p.status, kStatusTimeoutProducer, kKernelIdGemmSkinny, tile, kb);
          *abort_flag = 1;
          break;
        }
        mbar_expect_tx(&full[stage], kSkStageBytes);
        load_a(stage, kb);
        load_b(stage, kb);
        if (kb == 0) T5X_GEMM_TRACE(2);
        if (++stage == kSkStages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(kBM, kSkBN, 0, p.b_mn);
      const uint32_t b_kstep = p.b_mn ? 2048u : 32u;
      const uint32_t b_lbo = p.b_mn ? 8192u : 16u;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait(&full[stage], phase, abort_flag)) {
          report_status(p.status, kStatusTimeoutMma, kKernelIdGemmSkinny, tile, kb);
          *abort_flag = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        if (kb == 0) T5X_GEMM_TRACE(3);
        const uint32_t a_addr = smem_u32(sA + stage * kSkABytes);
        const uint32_t b_addr = smem_u32(sB + stage * kSkBBytes);
#pragma unroll
        for (int s = 0; s < kBK / 16; ++s) {
          const uint64_t ad = make_smem_desc_sw128(a_addr + s * 32u, 16u, 1024);
          const uint64_t bd = make_smem_desc_sw128(b_addr + s * b_kstep, b_lbo, 1024);
          umma_bf16(tmem_base, ad, bd, idesc, (kb | s) != 0 ? 1u : 0u);
        }
        umma_commit(&empty[stage]);
        if (++stage == kSkStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok) umma_commit(tmem_full);
    }
  }
  __syncwarp();  // the idle lanes of warps 0 and 1 block here instead of polling beside lane 0

  // Everyone waits for this CTA's accumulator: once it is complete the tensor core has read
  // every operand stage, so the ring may be overwritten.
  bool acc_ok = mbar_wait(tmem_full, 0, abort_flag);
  if (!acc_ok && threadIdx.x == 64)
    report_status(p.status, kStatusTimeoutEpilogue, kKernelIdGemmSkinny, tile, 0);
  if (!acc_ok) *abort_flag = 1;
  tc_fence_after();
  if (threadIdx.x == 64) T5X_GEMM_TRACE(4);
  chain_wait();  // (epilogue threads) the residual read and the stores to C come after this

  const int rows_per = kBM / S;  // rows of the tile that one cluster rank finishes
  const int slot_bytes = kSkTileBytes / S;
  if (S > 1) {
    const int t = threadIdx.x - 64;  // epilogue threads: 0..127
    const int cg = t & 31;            // columns 4 cg .. 4 cg + 3 of the tile
    constexpr int kMaxIter = kBM / 2 / 4;  // rows per thread at S = 2
    uint2 res[kMaxIter];
    if (warp >= 2) {
      // the residual of the rows this CTA will finish is requested now, ahead of the exchange
#pragma unroll
      for (int it = 0; it < kMaxIter; ++it) {
        res[it] = make_uint2(0u, 0u);
        const int lrow = (t >> 5) + 4 * it;
        const int grow = m0 + rank * rows_per + lrow;
        if (p.R != nullptr && lrow < rows_per && grow < p.M)
          res[it] = *reinterpret_cast<const uint2*>(p.R + static_cast<long long>(grow) * p.ldr +
                                                    n0 + cg * 4);
      }
      if (acc_ok) {
        // TMEM -> the outgoing tile in this CTA's ring: lane = row, 16-byte chunks of a row
        // XOR-swizzled by the row so that the 32 lanes of a store hit 32 different banks
        const int q = warp & 3;
        const int row = q * 32 + lane;
        float* dst_row = staging + row * kSkBN;
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
        for (int c = 0; c < kSkBN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(t_row + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int chunk = (c * 8 + i) ^ (row & 31);
            *reinterpret_cast<float4*>(dst_row + chunk * 4) =
                make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                            __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
          }
        }
      }
      fence_proxy_async_smem();  // these stores, before the bulk copies read them
      epilogue_bar_sync();
      if (threadIdx.x == 64) T5X_GEMM_TRACE(5);
      // one bulk copy per peer: its rows of this CTA's tile -> slot `rank` of its `recv`
      if (t < S && t != rank && !*abort_flag) {
        const uint32_t dst = mapa_shared(smem_u32(recv), t) + static_cast<uint32_t>(rank * slot_bytes);
        bulk_copy_to_cta(dst, reinterpret_cast<const uint8_t*>(staging) + t * slot_bytes,
                         static_cast<uint32_t>(slot_bytes), mapa_shared(smem_u32(recv_bar), t));
      }
      // the peers' rows for this CTA
      const bool got = mbar_wait(recv_bar, 0, abort_flag);
      if (!got) {
        if (threadIdx.x == 64)
          report_status(p.status, kStatusTimeoutPeerFlag, kKernelIdGemmSkinny, tile, rank);
        *abort_flag = 1;
      }
      if (threadIdx.x == 64) T5X_GEMM_TRACE(6);
      // This CTA has everything that was sent to it: it arrives at the closing cluster barrier
      // now and waits for it only before leaving, so that the sum and the stores below do not
      // hold the other CTAs up.
      tc_fence_before();
      cluster_arrive();
      if (got && acc_ok) {
        const bool c_vec = (p.ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 7) == 0);
#pragma unroll
        for (int it = 0; it < kMaxIter; ++it) {
          const int lrow = (t >> 5) + 4 * it;
          const int grow = m0 + rank * rows_per + lrow;
          if (lrow >= rows_per || grow >= p.M) break;
          const int chunk = cg ^ ((rank * rows_per + lrow) & 31);
          float4 acc = *reinterpret_cast<const float4*>(
              staging + (rank * rows_per + lrow) * kSkBN + chunk * 4);  // this CTA's own part
          for (int sidx = 0; sidx < S; ++sidx) {
            if (sidx == rank) continue;
            const float4 v = *reinterpret_cast<const float4*>(
                recv + (sidx * rows_per + lrow) * kSkBN + chunk * 4);
            acc.x += v.x, acc.y += v.y, acc.z += v.z, acc.w += v.w;
          }
          float o[4] = {acc.x * p.alpha, acc.y * p.alpha, acc.z * p.alpha, acc.w * p.alpha};
          if (p.R != nullptr) {
            const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&res[it].x));
            const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&res[it].y));
            o[0] += a.x, o[1] += a.y, o[2] += b.x, o[3] += b.y;
          }
          __nv_bfloat16* cp = p.C + static_cast<long long>(grow) * p.ldc + n0 + cg * 4;
          if (c_vec) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]);
            __nv_bfloat162 hi = __floats2bfloat162_rn(o[2], o[3]);
            uint2 u;
            u.x = *reinterpret_cast<uint32_t*>(&lo);
            u.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(cp) = u;
          } else {
            for (int i = 0; i < 4; ++i) cp[i] = __float2bfloat16(o[i]);
          }
        }
      }
    }
    else {
      cluster_arrive();  // warps 0 and 1 take no part in the exchange
    }
    // No CTA leaves while a peer may still write into its `recv`, signal its barrier or read
    // its ring (the source of the outgoing copies): every CTA arrives only after it has all of
    // its incoming bytes, so once the barrier completes every copy is complete.
    cluster_wait();
  } else if (warp >= 2 && acc_ok) {
    // one CTA per tile: the ordinary epilogue, rows straight from TMEM through a staging
    // block in the (free) operand ring
    GemmParams gp;
    gp.M = p.M, gp.N = p.N, gp.K = p.K, gp.batch = 1;
    gp.out_fp32 = 0, gp.accumulate = 0;
    gp.C = p.C, gp.ldc = p.ldc, gp.c_batch_stride = 0;
    gp.R = p.R, gp.ldr = p.ldr, gp.r_batch_stride = 0;
    gp.alpha = p.alpha;
    const int q = warp & 3;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    float* stage = staging + (warp - 2) * (kEpiStageBytesPerWarp / 4);
    const bool c_vec16 = (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
    if (p.R != nullptr)
      gemm_epilogue_tile<kSkBN, kEpiResidual>(gp, t_row, m0, n0, 0, q, lane, c_vec16, stage);
    else
      gemm_epilogue_tile<kSkBN, kEpiPlain>(gp, t_row, m0, n0, 0, q, lane, c_vec16, stage);
  }

  // Teardown: loads still in flight after an abort get a bounded time to land.
  __syncwarp();
  if (threadIdx.x == 64) T5X_GEMM_TRACE(7);
  if (*abort_flag && warp == 0 && lane == 0) {
    for (int it = 0; it < 2000; ++it) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kSkBN);
  }
}

static const CUtensorMap* skinny_map(const void* ptr, int mn_major, long long rows_mn, long long k,
                                     long long ld) {
  uint64_t dims[3];
  uint64_t strides[2];
  uint32_t box[3];
  if (!mn_major) {
    dims[0] = k, dims[1] = rows_mn;
    box[0] = 64, box[1] = 128;
  } else {
    dims[0] = rows_mn, dims[1] = k;
    box[0] = 64, box[1] = 64;
  }
  dims[2] = 1;
  box[2] = 1;
  strides[0] = static_cast<uint64_t>(ld) * 2;
  strides[1] = strides[0] * dims[1];
  return get_tensor_map(ptr, 2, 3, dims, strides, box, 1);
}

}  // namespace t5x

// How many CTAs should share one 128 x 128 output tile of an [M, N] product with K input
// features: the largest cluster size in {1, 2, 4, 8} that divides K / 64 and keeps all
// clusters resident at once. 0 when the shape does not suit this kernel (N or K not a
// multiple of 128 / 64, too many tiles).
T5X_API int t5x_gemm_skinny_splits(int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0 || N % t5x::kSkBN || K % t5x::kBK) return 0;
  const int tiles = ((M + t5x::kBM - 1) / t5x::kBM) * (N / t5x::kSkBN);
  const int sms = t5x::num_sms();
  if (tiles > sms) return 0;
  const int kb = K / t5x::kBK;
  int best = 1;
  for (int s = 2; s <= 8; s *= 2)
    if (kb % s == 0 && tiles * s <= sms) best = s;
  return best;
}

// C[M, N] (bf16, row stride ldc) = alpha * A[M, K] (bf16, row stride lda) * B (+ R). B is
// row-major [K, N] (b_mn_major = 1, row stride ldb) or [N, K] (0). `splits` from
// t5x_gemm_skinny_splits (or any of 1, 2, 4, 8 that divides K / 64). All leading dimensions
// multiples of 8 elements, base pointers 16-byte aligned.
T5X_API int t5x_gemm_skinny_bf16(const void* A, const void* B, void* C, const void* R, int M, int N,
                                 int K, long long lda, long long ldb, long long ldc,
                                 long long ldr, int b_mn_major, int splits, float alpha,
                                 void* stream) {
  using namespace t5x;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % kBK || N % kSkBN) return set_error("gemm_skinny: K %% 64 or N %% 128 != 0");
  if (splits != 1 && splits != 2 && splits != 4 && splits != 8)
    return set_error("gemm_skinny: splits must be 1, 2, 4 or 8 (got %d)", splits);
  if ((K / kBK) % splits) return set_error("gemm_skinny: K / 64 must be a multiple of splits");
  if (lda % 8 || ldb % 8 || ldc % 4 || (R != nullptr && ldr % 4))
    return set_error("gemm_skinny: leading dimensions");
  if (R != nullptr && (reinterpret_cast<uintptr_t>(R) & 7))
    return set_error("gemm_skinny: the residual must be 8-byte aligned");
  SkinnyParams p;
  p.M = M, p.N = N, p.K = K;
  p.b_mn = b_mn_major;
  p.splits = splits;
  p.kb_per_split = K / kBK / splits;
  p.tiles_n = N / kSkBN;
  p.C = static_cast<__nv_bfloat16*>(C);
  p.ldc = ldc;
  p.R = static_cast<const __nv_bfloat16*>(R);
  p.ldr = ldr;
  p.alpha = alpha;
  p.b_constant = chained_launches_constant_b() ? 1 : 0;
  p.status = device_status_buffer();
  p.trace = gemm_trace_buffer();
  const CUtensorMap* tA = skinny_map(A, 0, M, K, lda);
  const CUtensorMap* tB = skinny_map(B, b_mn_major, N, K, ldb);
  if (!tA || !tB) return -1;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSkSmemTotal);
    if (e != cudaSuccess) return set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    attr_set[dev & 63] = true;
  }
  const int tiles = ((M + kBM - 1) / kBM) * p.tiles_n;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * splits);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = kSkSmemTotal;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if (splits > 1) {
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = splits;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
  }
  if (chained_launches()) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_skinny_kernel, *tA, *tB, p);
  count_launches(1);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("gemm_skinny launch: %s", cudaGetErrorString(e));
  return 0;
}
