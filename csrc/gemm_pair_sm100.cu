// bf16 GEMM on CTA pairs (tcgen05 cta_group::2): one 256 x 256 output tile per pair.
//
// Why pairs: with one CTA per tile a 128 x 256 tile stages (128 + 256) x 64 operand elements
// per 64-deep k block, and the shared memory of one SM has to absorb those TMA writes while the
// tensor core reads them back; that traffic, not the MMA rate, bounds the one-CTA kernel.
// A pair computes 256 x 256 with each CTA staging only its own 128 rows of A and its own 128
// columns of B (the tensor cores of both SMs read both B halves), a third less shared-memory
// traffic per FLOP.
//
// Roles per CTA (192 threads): warp 0 = TMA producer (both CTAs, own halves), warp 1 = MMA
// issuer (even CTA only; owns the TMEM allocation in both), warps 2..5 = epilogue of the
// CTA's own 128 accumulator rows. Barriers: `full` lives in the even CTA and counts the bytes
// of both CTAs' loads; `empty` and `tmem_full` exist in both CTAs and are signalled by one
// tcgen05.commit addressed to both; `tmem_empty` lives in the even CTA and collects the
// arrivals of all eight epilogue warps. Every wait is bounded and TMA loads never use
// cluster multicast.
#include <algorithm>

#include "gemm_common.cuh"

namespace t5x {

constexpr int kPairBN = 256;
constexpr int kPairStages = 6;
constexpr int kPairABytes = kBM * kBK * 2;           // 128 rows of A
constexpr int kPairBBytes = (kPairBN / 2) * kBK * 2;  // 128 columns of B
constexpr int kPairStageBytes = kPairABytes + kPairBBytes;
constexpr int kPairSmemTotal = kPairStages * kPairStageBytes + 1024 + 1024;
constexpr int kKernelIdGemmPair = 2;

// Tensor-parallel variants (MODE != kTpNone) of the same kernel:
//
//  kTpAllGather     A's row blocks live on `world` ranks. A seventh warp per CTA pulls the
//                   other ranks' blocks into this rank's A buffer with bulk copies staged
//                   through shared memory (peer memory -> shared -> local memory, never a
//                   multicast load) and counts landed pieces per group of 128 rows; the TMA
//                   producer waits (bounded) only for the row groups its tile reads. The
//                   row-tile walk starts at this rank's own block and follows the order in
//                   which the copy warps pull, so the tensor cores work while NVLink delivers.
//                   The kernel raises this rank's "rows ready" signal as it starts and the copy
//                   warps wait for a peer's signal before they read from it, so no barrier
//                   kernel is needed in front; the last CTA to leave clears the counters.
//  kTpReduceScatter the epilogue stores each bf16 row of the partial product into the inbox
//                   of the rank that owns the row (peer memory over NVLink); the walk starts
//                   at the next rank's block and ends with this rank's own. The last CTA to
//                   leave raises this rank's "scattered" signal on every peer, which the
//                   kernel that sums the inbox slots waits for.
constexpr int kTpPiece = 8192;   // bytes per bulk copy
constexpr int kTpSlots = 3;      // staging slots per CTA
constexpr int kTpStageBytes = kTpPiece * kTpSlots;
constexpr int kTpFlagLimit = 1 << 24;  // polls (>= 64 ns apart) before a flag wait gives up: 1-3 s

template <int MODE>
constexpr int pair_threads() { return MODE == kTpAllGather ? kGemmThreads + 32 : kGemmThreads; }
template <int MODE>
constexpr int pair_smem() {
  return MODE == kTpAllGather       ? kPairSmemTotal + kTpStageBytes
         : MODE == kTpReduceScatter ? kPairSmemTotal + 4 * kRsStageBytesPerWarp
                                    : kPairSmemTotal + 4 * kEpiStageBytesPerWarp;
}
static_assert(kPairSmemTotal + 4 * kRsStageBytesPerWarp <= 232448, "shared memory per CTA");

template <int EPI, int MODE = kTpNone>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(pair_threads<MODE>(), 1)
    gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmB2, const GemmParams p,
                     const __grid_constant__ GemmTp tp) {
  constexpr int BN = kPairBN;
  constexpr int kStages = kPairStages;
  constexpr int kTileN = (EPI == kEpiGatedGelu) ? BN / 2 : BN;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + kStages * kPairABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kPairStageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + kStages;
  uint64_t* tmem_full = bars + 2 * kStages;
  uint64_t* tmem_empty = bars + 2 * kStages + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint64_t* copy_full = bars + 2 * kStages + 8;                    // kTpSlots barriers
  uint8_t* staging = smem + kStages * kPairStageBytes + 1024;      // kTpSlots x kTpPiece

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0 = even CTA (issues the MMAs)
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  chain_release();  // the next kernel on the stream may set itself up behind this one
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 8);
    }
    if (MODE == kTpAllGather)
      for (int a = 0; a < kTpSlots; ++a) mbar_init(&copy_full[a], 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (EPI == kEpiGatedGelu) tma_prefetch_desc(&tmB2);
  }
  __syncthreads();
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_kb = (p.K + kBK - 1) / kBK;
  const int tiles_per_batch = p.tiles_m * p.tiles_n;  // tiles_m counts 256-row tiles here
  const int total_tiles = tiles_per_batch * p.batch;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      auto load_a = [&](int stage, int k0, int m0, int b) {
        const uint32_t bar = mapa_shared(smem_u32(&full[stage]), 0);
        uint8_t* a_dst = sA + stage * kPairABytes;
        if (!p.a_mn) {
          tma_load_3d_pair(a_dst, &tmA, bar, k0, m0, b);  // box {64 k, 128 m, 1}
        } else {
#pragma unroll
          for (int j = 0; j < kBM / 64; ++j)  // box {64 m, 64 k, 1}
            tma_load_3d_pair(a_dst + j * 8192, &tmA, bar, m0 + 64 * j, k0, b);
        }
      };
      auto load_b = [&](int stage, const CUtensorMap* tb, int k0, int n0, int b) {
        const uint32_t bar = mapa_shared(smem_u32(&full[stage]), 0);
        uint8_t* b_dst = sB + stage * kPairBBytes;
        if (!p.b_mn) {
          tma_load_3d_pair(b_dst, tb, bar, k0, n0, b);  // box {64 k, 128 n, 1}
        } else {
#pragma unroll
          for (int j = 0; j < (BN / 2) / 64; ++j)  // box {64 n, 64 k, 1}
            tma_load_3d_pair(b_dst + j * 8192, tb, bar, n0 + 64 * j, k0, b);
        }
      };
      // this CTA's 128 B columns of tile column nt: its half of the tile, or (gated) the same
      // 128 columns of wi_0 for the even CTA and of wi_1 for the odd one
      auto b_col = [&](int nt) {
        const int n_tile = nt * kTileN;
        return (EPI == kEpiGatedGelu) ? n_tile : n_tile + static_cast<int>(cta) * (BN / 2);
      };
      const CUtensorMap* tb = (EPI == kEpiGatedGelu && cta == 1) ? &tmB2 : &tmB;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // B is constant (weights that no kernel in flight writes): the B halves of the first
      // stages are requested before the wait for the preceding kernel, the A halves after it.
      int preloaded = 0;
      if (MODE == kTpNone && p.b_constant && pair < total_tiles) {
        int b, mt, nt;
        gemm_tile_coords(p, pair, tiles_per_batch, b, mt, nt);
        preloaded = min(kStages, num_kb);
        for (int kb = 0; kb < preloaded; ++kb) {
          if (cta == 0) mbar_expect_tx(&full[kb], 2 * kPairStageBytes);
          load_b(kb, tb, kb * kBK, b_col(nt), b);
        }
        chain_wait();
        for (int kb = 0; kb < preloaded; ++kb)
          load_a(kb, kb * kBK, mt * (2 * kBM) + static_cast<int>(cta) * kBM, b);
        if (preloaded == kStages) phase = 1;
        else stage = preloaded;
      } else {
        chain_wait();
      }
      for (int tile = pair; tile < total_tiles && ok; tile += num_pairs) {
        int b, mt, nt;
        gemm_tile_coords(p, tile, tiles_per_batch, b, mt, nt);
        const int m0 = mt * (2 * kBM) + static_cast<int>(cta) * kBM;
        const int n0 = b_col(nt);
        if (MODE == kTpAllGather && m0 < p.M) {
          // the rows of this CTA's A tile: wait for the row groups of other ranks among them
          const int m_end = min(m0 + kBM, p.M);  // exclusive
          const long long row_bytes = static_cast<long long>(p.K) * 2;
          const int r_lo = m0 / tp.rows_per_rank;
          const int r_hi = (m_end - 1) / tp.rows_per_rank;
          for (int r = r_lo; r <= r_hi && ok; ++r) {
            if (r == tp.rank) continue;
            const int b0 = r * tp.rows_per_rank;
            const long long lo = static_cast<long long>(max(m0, b0) - b0) * row_bytes;
            const long long hi =
                static_cast<long long>(min(m_end, b0 + tp.rows_per_rank) - b0) * row_bytes - 1;
            for (int g = static_cast<int>(lo / tp.group_bytes);
                 g <= static_cast<int>(hi / tp.group_bytes) && ok; ++g) {
              const long long gbytes = min(tp.group_bytes, tp.block_bytes - g * tp.group_bytes);
              const uint32_t need = static_cast<uint32_t>((gbytes + kTpPiece - 1) / kTpPiece);
              const unsigned int* flag = &tp.flags[r * tp.groups_per_block + g];
              bool here = false;
              for (int it = 0; it < kTpFlagLimit; ++it) {
                if (ld_acquire_gpu(flag) >= need) {
                  here = true;
                  break;
                }
                if (*abort_flag) break;
                __nanosleep(64);
              }
              if (!here) {
                report_status(p.status, kStatusTimeoutPeerFlag, kKernelIdGemmPair, tile, r);
                *abort_flag = 1;
                ok = false;
              }
            }
          }
          if (!ok) break;
          fence_proxy_async_all();  // the bulk stores that wrote A, before this TMA reads it
        }
        for (int kb = preloaded; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) {
            report_status(p.status, kStatusTimeoutProducer, kKernelIdGemmPair, tile, kb);
            *abort_flag = 1;
            ok = false;
            break;
          }
          if (cta == 0) mbar_expect_tx(&full[stage], 2 * kPairStageBytes);
          const int k0 = kb * kBK;
          load_a(stage, k0, m0, b);
          load_b(stage, tb, k0, n0, b);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        preloaded = 0;
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (even CTA) ------------------------------
    if (lane == 0 && cta == 0) {
      const uint32_t idesc = make_idesc_bf16(2 * kBM, BN, p.a_mn, p.b_mn);
      const uint32_t a_kstep = p.a_mn ? 2048u : 32u;
      const uint32_t b_kstep = p.b_mn ? 2048u : 32u;
      const uint32_t a_lbo = p.a_mn ? 8192u : 16u;
      const uint32_t b_lbo = p.b_mn ? 8192u : 16u;
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = pair; tile < total_tiles && ok; tile += num_pairs, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag)) {
          report_status(p.status, kStatusTimeoutMma, kKernelIdGemmPair, tile, -1);
          *abort_flag = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag)) {
            report_status(p.status, kStatusTimeoutMma, kKernelIdGemmPair, tile, kb);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + stage * kPairABytes);
          const uint32_t b_addr = smem_u32(sB + stage * kPairBBytes);
#pragma unroll
          for (int s = 0; s < kBK / 16; ++s) {
            const uint64_t ad = make_smem_desc_sw128(a_addr + s * a_kstep, a_lbo, 1024);
            const uint64_t bd = make_smem_desc_sw128(b_addr + s * b_kstep, b_lbo, 1024);
            umma_bf16_pair(d_tmem, ad, bd, idesc, (kb | s) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&empty[stage], 0x3);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit_pair(&tmem_full[acc], 0x3);
      }
    }
  } else if (MODE == kTpAllGather && warp == 6) {
    // ------------------------------ all-gather copy warp ------------------------------
    // Pieces of kTpPiece bytes of the other ranks' blocks, in ring order from the next rank,
    // are dealt round-robin to the CTAs. Each goes peer memory -> staging slot (bulk load on
    // an mbarrier) -> this rank's A (bulk store); flags[r] is raised once the stores of a few
    // pieces are complete.
    if (lane == 0 && tp.world > 1) {
      if (blockIdx.x == 0) {
        // this rank's own rows were written by the kernel before this one: tell the peers
        for (int r = 0; r < tp.world; ++r)
          if (r != tp.rank)
            st_release_sys_u32(tp.sig_peer[r] + kTpSigRowsReady * kTpMaxPeers + tp.rank, tp.epoch);
      }
      const long long ppb = (tp.block_bytes + kTpPiece - 1) / kTpPiece;
      const long long total = ppb * (tp.world - 1);
      long long g_issue = blockIdx.x, g_done = blockIdx.x;
      int n_issue = 0, n_done = 0;
      uint32_t ready = 1u << tp.rank;  // peers whose rows are known to be in place
      int pend_flag = -1;              // counter the stored-but-unpublished pieces belong to
      uint32_t pend_count = 0;
      bool ok = true;
      while (g_done < total && ok) {
        while (g_issue < total && n_issue - n_done < kTpSlots && ok) {
          const int r = (tp.rank + 1 + static_cast<int>(g_issue / ppb)) % tp.world;
          if (!((ready >> r) & 1u)) {
            const unsigned int* sig = tp.sig_local + kTpSigRowsReady * kTpMaxPeers + r;
            bool here = false;
            for (int it = 0; it < kTpFlagLimit; ++it) {
              if (static_cast<int32_t>(ld_acquire_sys_u32(sig) - tp.epoch) >= 0) {
                here = true;
                break;
              }
              if (*abort_flag) break;
              __nanosleep(64);
            }
            if (!here) {
              report_status(p.status, kStatusTimeoutPeerFlag, kKernelIdGemmPair, -3, r);
              *abort_flag = 1;
              ok = false;
              break;
            }
            ready |= 1u << r;
          }
          const long long off = (g_issue % ppb) * kTpPiece;
          const uint32_t bytes = static_cast<uint32_t>(min(static_cast<long long>(kTpPiece),
                                                           tp.block_bytes - off));
          const int slot = n_issue % kTpSlots;
          mbar_expect_tx(&copy_full[slot], bytes);
          bulk_load(staging + slot * kTpPiece, tp.a_src[r] + r * tp.block_bytes + off, bytes,
                    &copy_full[slot]);
          ++n_issue;
          g_issue += gridDim.x;
        }
        if (!ok || n_done == n_issue) break;
        const int r = (tp.rank + 1 + static_cast<int>(g_done / ppb)) % tp.world;
        const long long off = (g_done % ppb) * kTpPiece;
        const uint32_t bytes = static_cast<uint32_t>(min(static_cast<long long>(kTpPiece),
                                                         tp.block_bytes - off));
        const int slot = n_done % kTpSlots;
        if (!mbar_wait(&copy_full[slot], (n_done / kTpSlots) & 1, abort_flag)) {
          report_status(p.status, kStatusTimeoutPeerFlag, kKernelIdGemmPair, -2, r);
          *abort_flag = 1;
          ok = false;
          break;
        }
        bulk_store(tp.a_dst + r * tp.block_bytes + off, staging + slot * kTpPiece, bytes);
        bulk_store_wait_read();  // the slot may be refilled
        const int flag = r * tp.groups_per_block + static_cast<int>(off / tp.group_bytes);
        if (pend_count && pend_flag != flag) {
          // pieces of another row group: publish them once all stores but the one just issued
          // are complete
          bulk_store_wait_all_but_last();
          fence_proxy_async_all();
          red_release_gpu_add(&tp.flags[pend_flag], pend_count);
          pend_count = 0;
        }
        pend_flag = flag;
        ++pend_count;
        ++n_done;
        g_done += gridDim.x;
        if (pend_count == 4) {
          bulk_store_wait_all();
          fence_proxy_async_all();
          red_release_gpu_add(&tp.flags[pend_flag], pend_count);
          pend_count = 0;
        }
      }
      if (pend_count) {
        bulk_store_wait_all();
        fence_proxy_async_all();
        red_release_gpu_add(&tp.flags[pend_flag], pend_count);
      }
      if (!ok) {
        // loads still in flight target this CTA's shared memory: give them time to land
        for (int it = 0; it < 2000; ++it) __nanosleep(1000);
      }
    }
  } else {
    // ------------------------------ epilogue (own 128 rows) ------------------------------
    const int q = warp & 3;
    int local = 0;
    bool ok = true;
    chain_wait();  // the epilogue reads residuals and writes C
    const bool c_vec_ok = (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
    const uint32_t drained = mapa_shared(smem_u32(&tmem_empty[0]), 0);
    for (int tile = pair; tile < total_tiles && ok; tile += num_pairs, ++local) {
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      int b, mt, nt;
      gemm_tile_coords(p, tile, tiles_per_batch, b, mt, nt);
      const int m0 = mt * (2 * kBM) + static_cast<int>(cta) * kBM;
      const int n0 = nt * kTileN;
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag)) {
        if (lane == 0) report_status(p.status, kStatusTimeoutEpilogue, kKernelIdGemmPair, tile, 0);
        *abort_flag = 1;
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      if (MODE == kTpReduceScatter)
        gemm_epilogue_tile_rs<BN, EPI>(p, tp, t_row, m0, n0, q, lane,
                                       staging + (warp - 2) * kRsStageBytesPerWarp);
      else if (EPI == kEpiCeStats)
        gemm_epilogue_ce_stats<BN>(p, t_row, m0, n0, nt, q, lane);
      else if (EPI == kEpiCeGrad)
        gemm_epilogue_ce_grad<BN>(p, t_row, m0, n0, q, lane, c_vec_ok);
      else
        gemm_epilogue_tile<BN, EPI>(
            p, t_row, m0, n0, b, q, lane, c_vec_ok,
            MODE == kTpNone
                ? reinterpret_cast<float*>(staging + (warp - 2) * kEpiStageBytesPerWarp)
                : nullptr);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(drained + acc * 8);
    }
    if (MODE == kTpReduceScatter) __threadfence_system();  // this thread's inbox stores
  }

  // Teardown: neither CTA may leave (or free TMEM) while its partner can still read its
  // shared memory, signal its barriers or write its accumulators.
  __syncwarp();
  if (*abort_flag && warp == 0 && lane == 0) {
    for (int it = 0; it < 2000; ++it) __nanosleep(1000);  // ~2 ms for copies in flight to land
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (MODE != kTpNone && threadIdx.x == 0 && tp.world > 1) {
    // The last CTA to get here speaks for the whole kernel: it clears the arrival counters
    // for the next all-gather, or tells the peers that this rank's scatter is complete.
    __threadfence_system();
    const unsigned int arrived = atomicAdd(tp.exit_count, 1u);
    if (arrived == gridDim.x - 1) {
      __threadfence_system();
      if (MODE == kTpAllGather) {
        const int n = tp.world * tp.groups_per_block;
        for (int i = 0; i < n; ++i) tp.flags[i] = 0u;
      } else {
        for (int r = 0; r < tp.world; ++r)
          if (r != tp.rank)
            st_release_sys_u32(tp.sig_peer[r] + kTpSigScattered * kTpMaxPeers + tp.rank, tp.epoch);
      }
      *tp.exit_count = 0u;
      __threadfence();
    }
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

template <int EPI, int MODE>
static int launch_pair(const CUtensorMap* tA, const CUtensorMap* tB, const CUtensorMap* tB2,
                       GemmParams& p, const GemmTp& tp, int max_ctas, cudaStream_t stream) {
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<EPI, MODE>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         pair_smem<MODE>());
    if (e != cudaSuccess) return set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    attr_set[dev] = true;
  }
  const int total = p.tiles_m * p.tiles_n * p.batch;
  int pairs = num_sms() / 2;
  if (max_ctas > 0) pairs = std::min(pairs, std::max(1, max_ctas / 2));
  pairs = std::max(1, std::min(pairs, total));
  cudaError_t e;
  if (MODE == kTpNone) {
    p.b_constant = chained_launches_constant_b() ? 1 : 0;
    e = launch_chained(gemm_pair_kernel<EPI, MODE>, dim3(2 * pairs), dim3(pair_threads<MODE>()),
                       pair_smem<MODE>(), stream, *tA, *tB, *tB2, p, tp);
  } else {
    // kernels that wait for other ranks are launched the ordinary way
    gemm_pair_kernel<EPI, MODE><<<2 * pairs, pair_threads<MODE>(), pair_smem<MODE>(), stream>>>(
        *tA, *tB, *tB2, p, tp);
    e = cudaSuccess;
  }
  count_launches(1);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("gemm_pair launch: %s", cudaGetErrorString(e));
  return 0;
}

template <int MODE>
static int launch_pair_mode(int epilogue, const CUtensorMap* tA, const CUtensorMap* tB,
                            const CUtensorMap* tB2, GemmParams& p, const GemmTp& tp, int max_ctas,
                            cudaStream_t stream) {
  switch (epilogue) {
    case kEpiPlain:
      return launch_pair<kEpiPlain, MODE>(tA, tB, tB2, p, tp, max_ctas, stream);
    case kEpiGatedGelu:
      if (MODE == kTpReduceScatter) break;
      return launch_pair<kEpiGatedGelu, MODE == kTpReduceScatter ? kTpNone : MODE>(
          tA, tB, tB2, p, tp, max_ctas, stream);
    case kEpiResidual:
      if (MODE == kTpAllGather) break;
      return launch_pair<kEpiResidual, MODE == kTpAllGather ? kTpNone : MODE>(
          tA, tB, tB2, p, tp, max_ctas, stream);
    case kEpiCeStats:
      if (MODE != kTpNone) break;
      return launch_pair<kEpiCeStats, kTpNone>(tA, tB, tB2, p, tp, max_ctas, stream);
    case kEpiCeGrad:
      if (MODE != kTpNone) break;
      return launch_pair<kEpiCeGrad, kTpNone>(tA, tB, tB2, p, tp, max_ctas, stream);
    default:
      break;
  }
  return set_error("gemm_pair: epilogue %d is not available in tensor-parallel mode %d", epilogue,
                   MODE);
}

// Called by t5x_gemm_bf16 for problems large enough to fill CTA pairs. `p.tiles_m` must count
// 256-row tiles; the tensor maps are the same as for the one-CTA kernel with BN = 128-column
// (K-major) or 64-column (MN-major) B boxes. `tp` is null for a plain GEMM.
int launch_gemm_pair(int epilogue, const CUtensorMap* tA, const CUtensorMap* tB,
                     const CUtensorMap* tB2, GemmParams& p, int max_ctas, cudaStream_t stream,
                     const GemmTp* tp, int tp_mode) {
  static const GemmTp none = {};
  switch (tp == nullptr ? kTpNone : tp_mode) {
    case kTpNone:
      return launch_pair_mode<kTpNone>(epilogue, tA, tB, tB2, p, none, max_ctas, stream);
    case kTpAllGather:
      return launch_pair_mode<kTpAllGather>(epilogue, tA, tB, tB2, p, *tp, max_ctas, stream);
    case kTpReduceScatter:
      return launch_pair_mode<kTpReduceScatter>(epilogue, tA, tB, tB2, p, *tp, max_ctas, stream);
    default:
      return set_error("gemm_pair: unknown tensor-parallel mode %d", tp_mode);
  }
}

}  // namespace t5x
