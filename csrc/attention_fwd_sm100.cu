// Streaming flash-attention forward for sm_100a: softmax(Q K^T + bias(k - q) + mask) V for any
// key length, head_dim 64 or 128, same bias / mask semantics as attention_sm100.cu (masked
// logits take the value -1e10; no 1/sqrt(d) scaling).
//
// One CTA per (query tile group, head, batch). The CTA walks the key range in blocks of 128
// keys that arrive by TMA through a ring of shared-memory stages, keeps a running row maximum
// and row sum (online softmax) and accumulates O in TMEM, so neither the key length nor the
// query length is bounded by on-chip memory.
//
// Roles (head_dim 64: two query tiles of 128 rows per CTA, head_dim 128: one):
//   warps 0-3 / 4-7  softmax group of tile 0 / 1: one thread per query row. The thread reads its
//                    128 scores of the block from TMEM into registers (which frees the score
//                    columns for the next block's MMA at once), adds the bias, takes the row
//                    maximum, writes exp2 of the shifted scores as bf16 into the swizzled
//                    shared-memory tile that the P V MMA reads, and keeps the row sum. No value
//                    is exchanged between threads.
//   warp 8           issues the MMAs (one elected thread): S_t = Q_t K_j^T, O_t += P_t V_j.
//                    While the softmax group of one tile works, the tensor cores serve the other.
//   warp 9           TMA producer: Q once, then K_j / V_j into the ring.
//
// Each block is read from TMEM twice, in chunks of 32 columns (once for the row maximum, once
// for the exponentials), which keeps the thread's registers free. The running maximum is only
// raised when a block exceeds it by more than 2^8 (the stale maximum keeps every exponential
// below 256, exact in fp32 sums and harmless in bf16): O then needs rescaling only for such
// blocks, and the softmax warps do it themselves in TMEM at a point where the previous P V MMA
// has completed anyway (the P tile is single-buffered).
//
// The bias by relative position is staged per (tile, block) as a 255-entry window, pre-scaled
// by log2(e) and stored four times with shifts 0..3, so that every thread reads its 128
// consecutive entries with aligned 16-byte loads whatever its row.
#include "attention_common.cuh"

namespace t5x {
namespace {

constexpr int kFsGroupThreads = 128;
constexpr int kFsMaxTiles = 2;
constexpr int kFsCtrlWarp = 8;
constexpr int kFsLoadWarp = 9;
constexpr int kFsThreads = 320;
constexpr int kFsPanel = 128 * 128;       // bytes of a [128 x 64] bf16 panel
constexpr int kFsRelCopy = 260;           // floats per shifted copy of the bias window
constexpr float kFsMasked2 = kMaskValue * kLog2e;  // the masked logit in the log2 domain
constexpr float kFsRescaleGap = 8.f;

template <int D, int kTiles>
struct FsCfg {
  static constexpr int kPanels = D / 64;
  static constexpr int kStages = (D == 64) ? 3 : 2;
  static constexpr int kQ = 0;                                        // kTiles x kPanels panels
  static constexpr int kKV = kQ + kTiles * kPanels * kFsPanel;        // kStages x (K, V) x kPanels
  static constexpr int kP = kKV + kStages * 2 * kPanels * kFsPanel;   // kTiles x 2 panels
  static constexpr int kRel = kP + kTiles * 2 * kFsPanel;             // kTiles x 2 x 4 copies
  static constexpr int kKey = kRel + kTiles * 2 * 4 * kFsRelCopy * 4; // kTiles x 2 x (128 seg + 4 words)
  static constexpr int kBars = kKey + kTiles * 2 * 132 * 4;
  static constexpr int kTotal = kBars + 256 + 1024;
  static constexpr int kColS = 0;                  // tile t: columns t * 128
  static constexpr int kColO = kTiles * 128;       // tile t: columns kColO + t * D
  static constexpr int kTmemCols = (kTiles * (128 + D) <= 256) ? 256 : 512;
};

__device__ __forceinline__ void group_bar_sync(int tile) {
  asm volatile("bar.sync %0, %1;" ::"r"(1 + tile), "n"(kFsGroupThreads) : "memory");
}

__device__ __forceinline__ uint32_t low_bits(int n) {  // n leading ones, n clamped to 0..32
  return n >= 32 ? 0xffffffffu : (n <= 0 ? 0u : ((1u << n) - 1u));
}

template <int D, int kTiles>
__global__ void __launch_bounds__(kFsThreads, 1)
    attn_fwd_stream_kernel(const __grid_constant__ CUtensorMap tmQ,
                           const __grid_constant__ CUtensorMap tmK,
                           const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  using Cfg = FsCfg<D, kTiles>;
  constexpr int kPanels = Cfg::kPanels;
  constexpr int kStages = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem + Cfg::kQ;
  uint8_t* sKV = smem + Cfg::kKV;
  uint8_t* sP = smem + Cfg::kP;
  float* sRel = reinterpret_cast<float*>(smem + Cfg::kRel);
  int* sKey = reinterpret_cast<int*>(smem + Cfg::kKey);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kBars);
  uint64_t* bar_q = bars;                    // Q landed
  uint64_t* bar_full = bars + 1;             // kStages: K_j and V_j landed
  uint64_t* bar_free = bar_full + kStages;   // kStages: every MMA that reads the stage is done
  uint64_t* bar_s = bar_free + kStages;      // kTiles: S_t of the current block is in TMEM
  uint64_t* bar_p = bar_s + kFsMaxTiles;     // kTiles: P_t is in shared memory, S_t consumed
  uint64_t* bar_pv = bar_p + kFsMaxTiles;    // kTiles: O_t += P_t V_j finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_pv + kFsMaxTiles);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, b = blockIdx.z;
  const int q_base = blockIdx.x * (128 * kTiles);
  const int tiles_here = min(kTiles, (p.Lq - q_base + 127) / 128);  // >= 1
  int nblk = (p.Lk + 127) / 128;
  if (p.causal && p.key_mask == nullptr && p.kv_seg == nullptr) {
    // every row sees key 0, so blocks beyond the last visible key of the CTA's last row
    // contribute exact zeros and are skipped
    const int last_q = min(p.Lq, q_base + 128 * kTiles) - 1;
    const long long last_k = static_cast<long long>(last_q) + p.causal_off;
    if (last_k >= 0 && last_k / 128 + 1 < nblk) nblk = static_cast<int>(last_k / 128) + 1;
  }

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_free[s], 1);
    }
    for (int t = 0; t < kFsMaxTiles; ++t) {
      mbar_init(&bar_s[t], 1);
      mbar_init(&bar_p[t], 4);
      mbar_init(&bar_pv[t], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kFsCtrlWarp) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t kStageBytes = 2 * kPanels * kFsPanel;

  if (warp == kFsLoadWarp) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      bool ok = true;
      mbar_expect_tx(bar_q, tiles_here * kPanels * kFsPanel);
      for (int t = 0; t < tiles_here; ++t)
        for (int c = 0; c < kPanels; ++c)
          tma_load_4d(sQ + (t * kPanels + c) * kFsPanel, &tmQ, bar_q, c * 64, h,
                      q_base + t * 128, b);
      for (int j = 0; j < nblk && ok; ++j) {
        const int s = j % kStages;
        if (j >= kStages) ok = mbar_wait(&bar_free[s], ((j / kStages) - 1) & 1, abort_flag);
        if (!ok) break;
        uint8_t* st = sKV + s * kStageBytes;
        mbar_expect_tx(&bar_full[s], kStageBytes);
        for (int c = 0; c < kPanels; ++c) {
          tma_load_4d(st + c * kFsPanel, &tmK, &bar_full[s], c * 64, h, j * 128, b);
          tma_load_4d(st + (kPanels + c) * kFsPanel, &tmV, &bar_full[s], c * 64, h, j * 128, b);
        }
      }
      if (!ok) {
        report_status(p.status, kStatusTimeoutMma, kKernelIdAttnFwd, blockIdx.x, 100 + blockIdx.y);
        *abort_flag = 1;
      }
    }
  } else if (warp == kFsCtrlWarp) {
    // ------------------------------ MMA issue ------------------------------
    if (lane == 0) {
      bool ok = true;
      const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_o = make_idesc_bf16(128, D, 0, 1);
      auto issue_scores = [&](int t, int j) {
        const uint32_t qa = smem_u32(sQ + t * kPanels * kFsPanel);
        const uint32_t ka = smem_u32(sKV + (j % kStages) * kStageBytes);
#pragma unroll
        for (int s = 0; s < D / 16; ++s)
          umma_bf16(tmem_base + Cfg::kColS + t * 128,
                    make_smem_desc_sw128(qa + (s >> 2) * kFsPanel + (s & 3) * 32, 16, 1024),
                    make_smem_desc_sw128(ka + (s >> 2) * kFsPanel + (s & 3) * 32, 16, 1024),
                    idesc_s, s != 0);
        umma_commit(&bar_s[t]);
      };
      ok = mbar_wait(bar_q, 0, abort_flag) && mbar_wait(&bar_full[0], 0, abort_flag);
      if (ok) {
        tc_fence_after();
        for (int t = 0; t < tiles_here; ++t) issue_scores(t, 0);
      }
      for (int j = 0; j < nblk && ok; ++j) {
        const uint32_t ph = j & 1;
        const uint32_t va = smem_u32(sKV + (j % kStages) * kStageBytes + kPanels * kFsPanel);
        for (int t = 0; t < tiles_here && ok; ++t) {
          ok = mbar_wait(&bar_p[t], ph, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t pa = smem_u32(sP + t * 2 * kFsPanel);
          // A = P_t [128 q x 128 keys] (two key panels), B = V_j [128 keys x D], channels
          // contiguous: 64-channel groups are one panel apart, 16 keys = 2048 bytes per step.
#pragma unroll
          for (int s = 0; s < 8; ++s)
            umma_bf16(tmem_base + Cfg::kColO + t * D,
                      make_smem_desc_sw128(pa + (s >> 2) * kFsPanel + (s & 3) * 32, 16, 1024),
                      make_smem_desc_sw128(va + s * 2048, kFsPanel, 1024), idesc_o, (j | s) != 0);
          umma_commit(&bar_pv[t]);
          if (t == tiles_here - 1) umma_commit(&bar_free[j % kStages]);
          if (j + 1 < nblk) {
            // S_t's columns were consumed before bar_p fired
            ok = mbar_wait(&bar_full[(j + 1) % kStages], ((j + 1) / kStages) & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            issue_scores(t, j + 1);
          }
        }
      }
      if (!ok) {
        report_status(p.status, kStatusTimeoutMma, kKernelIdAttnFwd, blockIdx.x, blockIdx.y);
        *abort_flag = 1;
      }
    }
  } else if (warp < 4 * tiles_here) {
    // ------------------------------ softmax groups ------------------------------
    const int t = warp >> 2;
    const int r = (warp & 3) * 32 + lane;  // row of the tile == TMEM lane
    const int g = threadIdx.x & 127;       // index within the group (== r)
    const int q0 = q_base + t * 128;
    const int q = q0 + r;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const uint32_t t_s = t_row + Cfg::kColS + t * 128;
    const uint32_t t_o = t_row + Cfg::kColO + t * D;
    const bool has_bias = p.rel_bias != nullptr;
    const bool key_only = !p.causal && p.kv_seg == nullptr;
    // causal == 2: prefix LM. Segment codes then carry "inside the prefix" in bit 30, and a key
    // inside the prefix is visible to every query inside the prefix, whatever their order.
    const bool prefix_lm = p.causal == 2;
    const int seg_mask = prefix_lm ? 0x3fffffff : -1;
    const int qcode = (p.q_seg != nullptr && q < p.Lq) ? p.q_seg[static_cast<long long>(b) * p.Lq + q] : 0;
    const int qseg = qcode & seg_mask;
    const bool q_pre = prefix_lm && ((qcode >> 30) & 1);
    const long long kmax = p.causal ? static_cast<long long>(q) + p.causal_off : (1ll << 40);
    float* rel_stage = sRel + t * 2 * 4 * kFsRelCopy;
    int* key_stage = sKey + t * 2 * 132;
    uint8_t* p_tile = sP + t * 2 * kFsPanel;
    const float* tab = has_bias ? p.rel_bias + static_cast<long long>(h) * p.nrel : nullptr;
    const int shift = (127 - r) & 3;
    bool ok = true;

    // Per-block metadata is fetched one block ahead into registers and published to the other
    // shared-memory stage after the arithmetic of the current block.
    float pf_rel0 = 0.f, pf_rel1 = 0.f;
    int pf_seg = -1;
    auto fetch_meta = [&](int j) {
      if (has_bias) {
        const int base = j * 128 - q0 - 127 + p.rel_off;  // index of window entry 0
        const int i0 = base + g, i1 = base + g + 128;
        // raw values only: anything computed from them here would wait for the loads at once
        pf_rel0 = (i0 >= 0 && i0 < p.nrel) ? __ldg(tab + i0) : 0.f;
        pf_rel1 = (g < 127 && i1 >= 0 && i1 < p.nrel) ? __ldg(tab + i1) : 0.f;
      }
      const int k = j * 128 + g;
      pf_seg = -1;
      if (k < p.Lk) {
        const long long off = static_cast<long long>(b) * p.Lk + k;
        pf_seg = p.kv_seg ? p.kv_seg[off] : 0;
        if (p.key_mask && p.key_mask[off] == 0) pf_seg = -1;
      }
    };
    auto publish_meta = [&](int j) {
      float* rs = rel_stage + (j & 1) * 4 * kFsRelCopy;
      int* ks = key_stage + (j & 1) * 132;
      if (has_bias) {
        const float r0 = pf_rel0 * kLog2e, r1 = pf_rel1 * kLog2e;
#pragma unroll
        for (int m = 0; m < 4; ++m) {  // copy m holds window[i + m] at i
          if (g - m >= 0) rs[m * kFsRelCopy + g - m] = r0;
          rs[m * kFsRelCopy + g + 128 - m] = r1;
        }
      }
      ks[g] = pf_seg;
      const uint32_t word = __ballot_sync(0xffffffffu, pf_seg >= 0);
      if (lane == 0) ks[128 + (warp & 3)] = static_cast<int>(word);
    };

    fetch_meta(0);
    publish_meta(0);
    group_bar_sync(t);

    float m_used = 0.f, l = 0.f;
    // One key block. Returns false when a wait gave up; the result is made uniform over the
    // warp, and the caller keeps every thread of the group on the same sequence of group
    // barriers whatever the outcome.
    auto process_block = [&](int j) -> bool {
      const uint32_t ph = j & 1;
      if (j + 1 < nblk) fetch_meta(j + 1);
      const float* rs = rel_stage + (j & 1) * 4 * kFsRelCopy + shift * kFsRelCopy + (127 - r - shift);
      const int* ks = key_stage + (j & 1) * 132;
      // visibility words of this row: bit x of word w <-> key j*128 + w*32 + x
      uint32_t vis[4], inr[4];
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const int k0 = j * 128 + w * 32;
        inr[w] = low_bits(p.Lk - k0);
        uint32_t mv = static_cast<uint32_t>(ks[128 + w]);
        if (!key_only) {
          uint32_t pre_w = 0;
          if (p.kv_seg != nullptr) {
            uint32_t ms = 0;
#pragma unroll
            for (int x4 = 0; x4 < 8; ++x4) {
              const int4 sg = reinterpret_cast<const int4*>(ks + w * 32)[x4];
              const int sgv[4] = {sg.x, sg.y, sg.z, sg.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                ms |= ((sgv[e] & seg_mask) == qseg ? 1u : 0u) << (x4 * 4 + e);
                pre_w |= static_cast<uint32_t>((sgv[e] >> 30) & 1) << (x4 * 4 + e);
              }
            }
            mv &= ms;
          }
          if (p.causal) {
            const long long n = kmax - k0 + 1;
            const uint32_t cw = low_bits(n > 32 ? 32 : (n < 0 ? 0 : static_cast<int>(n)));
            mv &= q_pre ? (cw | pre_w) : cw;
          }
        }
        vis[w] = mv;
      }
      if (!__all_sync(0xffffffffu, mbar_wait_relaxed(&bar_s[t], ph, abort_flag))) return false;
      tc_fence_after();
      // 32 scores of the row -> log2 domain with bias and masks (in place); returns their
      // maximum over the keys that exist.
      auto load_chunk = [&](int w, uint32_t (&sv)[32]) -> float {
        tmem_ld32(t_s + w * 32, sv);
        tmem_ld_wait();
        float cmax = -3.0e38f;
        const bool plain = vis[w] == 0xffffffffu && inr[w] == 0xffffffffu;
#pragma unroll
        for (int x4 = 0; x4 < 8; ++x4) {
          float4 rb = make_float4(0.f, 0.f, 0.f, 0.f);
          if (has_bias) rb = reinterpret_cast<const float4*>(rs + w * 32)[x4];
          const float rbv[4] = {rb.x, rb.y, rb.z, rb.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int x = x4 * 4 + e;
            float sc = fmaf(__uint_as_float(sv[x]), kLog2e, rbv[e]);
            if (!plain) {
              sc = ((vis[w] >> x) & 1u) ? sc : kFsMasked2;
              if ((inr[w] >> x) & 1u) {
                cmax = fmaxf(cmax, sc);
              } else {
                sc = -3.0e38f;  // beyond the last key: contributes exactly zero
              }
            } else {
              cmax = fmaxf(cmax, sc);
            }
            sv[x] = __float_as_uint(sc);
          }
        }
        return cmax;
      };
      // pass 1: the block's maximum
      float bmax = -3.0e38f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        uint32_t sv[32];
        bmax = fmaxf(bmax, load_chunk(w, sv));
      }
      // The maximum in use only moves when the block exceeds it by more than 2^8; O and the
      // row sum are then rescaled. The P tile and O are free once the previous P V MMA is done.
      if (j == 0) {
        m_used = bmax;
      } else {
        float fix = 1.f;
        if (bmax > m_used + kFsRescaleGap) {
          fix = exp2f(m_used - bmax);
          m_used = bmax;
          l *= fix;
        }
        if (!__all_sync(0xffffffffu, mbar_wait_relaxed(&bar_pv[t], ph ^ 1, abort_flag)))
          return false;
        if (__any_sync(0xffffffffu, fix != 1.f)) {
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t ov[32];
            tmem_ld32(t_o + c * 32, ov);
            tmem_ld_wait();
#pragma unroll
            for (int x = 0; x < 32; ++x) ov[x] = __float_as_uint(__uint_as_float(ov[x]) * fix);
            tmem_st32(t_o + c * 32, ov);
          }
          tmem_st_wait();
        }
      }
      // pass 2: probabilities -> shared memory (bf16), row sum
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        uint32_t sv[32];
        load_chunk(w, sv);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float pr[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            pr[e] = exp2f(__uint_as_float(sv[c * 8 + e]) - m_used);
            l += pr[e];
          }
          store_swizzled_chunk(p_tile + (w >> 1) * kFsPanel, r, (w & 1) * 4 + c, pr);
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_p[t]);  // P_t written, S_t read, O_t rescaled
      if (j + 1 < nblk) publish_meta(j + 1);
      return true;
    };
    for (int j = 0; j < nblk; ++j) {
      if (ok) ok = process_block(j);
      group_bar_sync(t);  // metadata of block j + 1 complete; that of block j no longer read
    }
    // ---- epilogue: O / l ----
    if (ok)
      ok = __all_sync(0xffffffffu, mbar_wait_relaxed(&bar_pv[t], (nblk - 1) & 1, abort_flag));
    if (ok) {
      tc_fence_after();
      const float inv = 1.f / l;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t ov[32];
        tmem_ld32(t_o + c * 32, ov);
        tmem_ld_wait();
        if (q < p.Lq) {
          __nv_bfloat16* dst =
              p.O + b * p.o_sb + static_cast<long long>(q) * p.o_sl + h * p.o_sh + c * 32;
#pragma unroll
          for (int x = 0; x < 32; x += 8) {
            uint4 u;
            u.x = pack_bf16x2(__uint_as_float(ov[x]) * inv, __uint_as_float(ov[x + 1]) * inv);
            u.y = pack_bf16x2(__uint_as_float(ov[x + 2]) * inv, __uint_as_float(ov[x + 3]) * inv);
            u.z = pack_bf16x2(__uint_as_float(ov[x + 4]) * inv, __uint_as_float(ov[x + 5]) * inv);
            u.w = pack_bf16x2(__uint_as_float(ov[x + 6]) * inv, __uint_as_float(ov[x + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + x) = u;
          }
        }
      }
      if (q < p.Lq && p.lse != nullptr)
        p.lse[(static_cast<long long>(b) * p.H + h) * p.Lq + q] =
            (m_used + log2f(l)) * 0.6931471805599453f;
    } else if (lane == 0) {
      report_status(p.status, kStatusTimeoutEpilogue, kKernelIdAttnFwd, blockIdx.x, blockIdx.y);
      *abort_flag = 1;
    }
  }
  if (*abort_flag && threadIdx.x == 0)
    for (int it = 0; it < 2000; ++it) __nanosleep(1000);
  tc_fence_before();
  __syncthreads();
  if (warp == kFsCtrlWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int D, int kTiles>
int launch_stream(const CUtensorMap* tq, const CUtensorMap* tk, const CUtensorMap* tv,
                  const AttnParams& p, cudaStream_t st) {
  using Cfg = FsCfg<D, kTiles>;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_stream_kernel<D, kTiles>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kTotal);
    if (e != cudaSuccess) return set_error("attention_fwd_stream attr: %s", cudaGetErrorString(e));
    attr_set[dev] = true;
  }
  dim3 grid((p.Lq + 128 * kTiles - 1) / (128 * kTiles), p.H, p.B);
  attn_fwd_stream_kernel<D, kTiles><<<grid, kFsThreads, Cfg::kTotal, st>>>(*tq, *tk, *tv, p);
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("attention_fwd_stream: %s", cudaGetErrorString(e));
  return 0;
}

}  // namespace
}  // namespace t5x

using namespace t5x;

// q [B,Lq,H,D], k/v [B,Lk,H,D] bf16 with element strides (sb, sl, sh), innermost contiguous,
// D = 64 or 128, any Lq and Lk. rel_bias [H, nrel] fp32 or null: bias = rel_bias[h][(k - q) +
// rel_off]. lse [B,H,Lq] fp32 or null.
T5X_API int t5x_attention_fwd_stream(const void* q, const void* k, const void* v, void* o,
                                     void* lse, int B, int H, int Lq, int Lk, int D,
                                     long long q_sb, long long q_sl, long long q_sh,
                                     long long k_sb, long long k_sl, long long k_sh,
                                     long long v_sb, long long v_sl, long long v_sh,
                                     long long o_sb, long long o_sl, long long o_sh,
                                     const void* rel_bias, int nrel, int rel_off,
                                     const void* key_mask, const void* q_seg, const void* kv_seg,
                                     int causal, int causal_off, void* stream) {
  if (B <= 0 || H <= 0 || Lq <= 0 || Lk <= 0) return 0;
  if (D != 64 && D != 128) return set_error("attention_fwd_stream: head_dim %d not in {64, 128}", D);
  if (B > 65535 || H > 65535) return set_error("attention_fwd_stream: B or H beyond the grid limit");
  if ((o_sb | o_sl | o_sh) & 7 || (reinterpret_cast<uintptr_t>(o) & 15))
    return set_error("attention_fwd_stream: output rows must be 16-byte aligned");
  const CUtensorMap* tq = bhld_map(q, B, Lq, H, q_sb, q_sl, q_sh, D);
  const CUtensorMap* tk = bhld_map(k, B, Lk, H, k_sb, k_sl, k_sh, D);
  const CUtensorMap* tv = bhld_map(v, B, Lk, H, v_sb, v_sl, v_sh, D);
  if (!tq || !tk || !tv) return -1;
  AttnParams p = {};
  p.B = B; p.H = H; p.Lq = Lq; p.Lk = Lk;
  p.rel_bias = static_cast<const float*>(rel_bias);
  p.nrel = nrel; p.rel_off = rel_off;
  p.key_mask = static_cast<const uint8_t*>(key_mask);
  p.q_seg = static_cast<const int*>(q_seg);
  p.kv_seg = static_cast<const int*>(kv_seg);
  p.causal = causal; p.causal_off = causal_off;
  p.O = static_cast<__nv_bfloat16*>(o);
  p.o_sb = o_sb; p.o_sl = o_sl; p.o_sh = o_sh;
  p.lse = static_cast<float*>(lse);
  p.status = device_status_buffer();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (D == 128) return launch_stream<128, 1>(tq, tk, tv, p, st);
  if (Lq > 128) return launch_stream<64, 2>(tq, tk, tv, p, st);
  return launch_stream<64, 1>(tq, tk, tv, p, st);
}
