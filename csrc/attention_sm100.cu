// Flash attention for T5 on sm_100a: softmax(Q K^T + bias(k - q) + mask) V, head_dim 64,
// no 1/sqrt(d) scaling (T5 folds it into the query initialiser).
//
// Both GEMMs of the forward pass and all five of the backward pass run on tcgen05 with
// accumulators in TMEM; Q/K/V/dO tiles arrive by TMA (128-byte swizzle, no multicast) and the
// probability / dS tiles are written by the softmax warps straight into the swizzled shared
// layout that the next MMA reads as its A operand. The [b,h,q,k] score matrix never exists in
// global memory. Bias and masks are generated in-kernel from per-token metadata:
//   bias      : rel_bias[h][(k - q) + rel_off]  (the T5 bucket table expanded by relative
//               offset on the host, so the bucket arithmetic is bit-identical to the oracle)
//   masks     : key padding [B,Lk], causal (k <= q + causal_off), packed-segment ids.
// Masked logits take the value -1e10 (not -inf): a fully masked row gives a uniform
// distribution, exactly like the additive-mask formulation of the reference.
//
// Forward : one CTA per (head, batch); K and V stay in shared memory while the CTA walks the
//           128-query blocks; S = Q K^T for the whole key range sits in TMEM (Lk <= 512), the
//           S MMAs of the next query block are issued as soon as the softmax warps release
//           the columns. 16 softmax warps (4 threads per row) + 1 warp for TMA and MMA issue.
// Backward: one CTA per (128-key block, head, batch), looping over query blocks; dK/dV
//           accumulate in TMEM, dQ partial tiles are added to an fp32 buffer with vector
//           red.global.add.
#include "attention_common.cuh"

namespace t5x {

// ---------------------------------------------------------------------------------------
// Forward
// ---------------------------------------------------------------------------------------
struct FwdSmem {
  static constexpr int kTile = 128 * 128;  // bytes of a [128 x 64] bf16 tile
  static constexpr int kQ = 0;
  static constexpr int kK = kTile;              // up to 4 tiles
  static constexpr int kV = kK + 4 * kTile;     // up to 4 tiles
  static constexpr int kP = kV + 4 * kTile;     // 2 buffers x 2 tiles
  static constexpr int kRel = kP + 4 * kTile;   // bias by (k - q): up to 512 + 512 floats
  static constexpr int kStat = kRel + 1024 * 4; // 128 x 4 floats (row max parts), then sums
  static constexpr int kKeySeg = kStat + 128 * 4 * 4 * 2;  // 512 ints: segment id of key k, -1 = hidden
  static constexpr int kBars = kKeySeg + 512 * 4;
  static constexpr int kTotal = kBars + 256 + 1024;
};
constexpr int kFwdMaxLq = 512;  // sRel covers (k - q) for Lq, Lk <= 512

__global__ void __launch_bounds__(kAttnThreads, 1)
    attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem + FwdSmem::kQ;
  uint8_t* sK = smem + FwdSmem::kK;
  uint8_t* sV = smem + FwdSmem::kV;
  uint8_t* sP = smem + FwdSmem::kP;
  float* sRel = reinterpret_cast<float*>(smem + FwdSmem::kRel);
  float* sStat = reinterpret_cast<float*>(smem + FwdSmem::kStat);
  int* sKeySeg = reinterpret_cast<int*>(smem + FwdSmem::kKeySeg);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + FwdSmem::kBars);
  uint64_t* bar_q = bars;           // Q tile landed (once per query block)
  uint64_t* bar_kv = bars + 1;      // 4: K_j and V_j landed (once per CTA)
  uint64_t* bar_s = bars + 5;       // 4: S block j ready in TMEM (once per query block)
  uint64_t* bar_p = bars + 9;       // 4: P block j written to smem, S block j released
  uint64_t* bar_pv = bars + 13;     // 4: PV MMA of block j finished (P buffer reusable)
  uint64_t* bar_qfree = bars + 17;  // all S MMAs of this query block done: Q smem reusable
  uint64_t* bar_oread = bars + 18;  // O accumulator of this query block has been read out
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x, b = blockIdx.y;
  const int nblk = (p.Lk + 127) / 128;
  const int nq = (p.Lq + 127) / 128;
  const int lq_pad = nq * 128;
  const int o_col = (nblk * 128) & 511;  // TMEM column of O (reuses S block 0 when Lk fills TMEM)

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    mbar_init(bar_qfree, 1);
    mbar_init(bar_oread, kSoftmaxWarps);
    for (int j = 0; j < 4; ++j) {
      mbar_init(&bar_kv[j], 1);
      mbar_init(&bar_s[j], 1);
      mbar_init(&bar_p[j], kSoftmaxWarps);
      mbar_init(&bar_pv[j], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kCtrlWarp) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  // Bias by relative offset for this head: sRel[u], u = (k - q) + lq_pad - 1.
  if (p.rel_bias != nullptr) {
    const float* tab = p.rel_bias + static_cast<long long>(h) * p.nrel;
    for (int u = threadIdx.x; u < lq_pad + nblk * 128; u += kAttnThreads) {
      const int idx = u - (lq_pad - 1) + p.rel_off;
      sRel[u] = (idx >= 0 && idx < p.nrel) ? tab[idx] : 0.f;
    }
  }
  // Per-key metadata: segment id (0 when unpacked), -1 for padded / out-of-range keys.
  for (int k = threadIdx.x; k < 512; k += kAttnThreads) {
    int sgm = -1;
    if (k < p.Lk) {
      const long long off = static_cast<long long>(b) * p.Lk + k;
      sgm = p.kv_seg ? p.kv_seg[off] : 0;
      if (p.key_mask && p.key_mask[off] == 0) sgm = -1;
    }
    sKeySeg[k] = sgm;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == kCtrlWarp) {
    if (lane == 0) {
      bool ok = true;
      mbar_expect_tx(bar_q, FwdSmem::kTile);
      tma_load_4d(sQ, &tmQ, bar_q, 0, h, 0, b);
      for (int j = 0; j < nblk; ++j) {
        mbar_expect_tx(&bar_kv[j], 2 * FwdSmem::kTile);
        tma_load_4d(sK + j * FwdSmem::kTile, &tmK, &bar_kv[j], 0, h, j * 128, b);
        tma_load_4d(sV + j * FwdSmem::kTile, &tmV, &bar_kv[j], 0, h, j * 128, b);
      }
      const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_o = make_idesc_bf16(128, 64, 0, 1);
      const uint32_t qa = smem_u32(sQ);
      for (int i = 0; i < nq && ok; ++i) {
        const uint32_t ph = i & 1;
        // ---- S_j = Q_i K_j^T, as soon as the previous query block released the columns ----
        ok = mbar_wait(bar_q, ph, abort_flag);
        for (int j = 0; j < nblk && ok; ++j) {
          if (i == 0) ok = mbar_wait(&bar_kv[j], 0, abort_flag);
          if (ok && i > 0) {
            ok = mbar_wait(&bar_p[j], ph ^ 1, abort_flag);
            // the O accumulator of the previous block may live in S block 0's columns
            if (ok && j * 128 == o_col) ok = mbar_wait(bar_oread, ph ^ 1, abort_flag);
          }
          if (!ok) break;
          tc_fence_after();
          const uint32_t ka = smem_u32(sK + j * FwdSmem::kTile);
#pragma unroll
          for (int s = 0; s < 4; ++s)
            umma_bf16(tmem_base + j * 128, make_smem_desc_sw128(qa + s * 32, 16, 1024),
                      make_smem_desc_sw128(ka + s * 32, 16, 1024), idesc_s, s != 0);
          umma_commit(&bar_s[j]);
        }
        if (!ok) break;
        // Q smem is free once the S MMAs are done: prefetch the next query block.
        if (i + 1 < nq) {
          umma_commit(bar_qfree);
          ok = mbar_wait(bar_qfree, ph, abort_flag);
          if (!ok) break;
          mbar_expect_tx(bar_q, FwdSmem::kTile);
          tma_load_4d(sQ, &tmQ, bar_q, 0, h, (i + 1) * 128, b);
        }
        // ---- O_i += P_j V_j ----
        if (i > 0 && o_col >= nblk * 128) {
          // O has its own columns: they must have been read out before being overwritten
          ok = mbar_wait(bar_oread, ph ^ 1, abort_flag);
          if (!ok) break;
        }
        for (int j = 0; j < nblk && ok; ++j) {
          ok = mbar_wait(&bar_p[j], ph, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t pa = smem_u32(sP + (j & 1) * 2 * FwdSmem::kTile);
          const uint32_t va = smem_u32(sV + j * FwdSmem::kTile);
#pragma unroll
          for (int s = 0; s < 8; ++s)
            umma_bf16(tmem_base + o_col,
                      make_smem_desc_sw128(pa + (s >> 2) * FwdSmem::kTile + (s & 3) * 32, 16, 1024),
                      make_smem_desc_sw128(va + s * 2048, 8192, 1024), idesc_o, (j | s) != 0);
          umma_commit(&bar_pv[j]);
        }
      }
      if (!ok) {
        report_status(p.status, kStatusTimeoutMma, kKernelIdAttnFwd, blockIdx.x, blockIdx.y);
        *abort_flag = 1;
      }
    }
  } else {
    // ------------------------------ softmax warps ------------------------------
    const int quarter = warp & 3, part = warp >> 2;  // 4 threads per row, 32 columns each
    const int r = quarter * 32 + lane;               // row of the tile == TMEM lane
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const bool has_bias = p.rel_bias != nullptr;
    bool ok = true;
    // Key-only visibility (padding / key mask) and in-range bits, fixed for the whole CTA.
    uint32_t kvis[4], inr[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t m_vis = 0, m_in = 0;
      if (j < nblk) {
        for (int x = 0; x < 32; ++x) {
          const int kk = j * 128 + part * 32 + x;
          m_vis |= (sKeySeg[kk] >= 0 ? 1u : 0u) << x;
          m_in |= (kk < p.Lk ? 1u : 0u) << x;
        }
      }
      kvis[j] = m_vis;
      inr[j] = m_in;
    }
    for (int i = 0; i < nq && ok; ++i) {
      const uint32_t ph = i & 1;
      const int q = i * 128 + r;
      const int qseg = (p.q_seg != nullptr && q < p.Lq) ? p.q_seg[b * p.Lq + q] : 0;
      const int kmax = p.causal ? q + p.causal_off : 0x7fffffff;
      // Visibility bits of this thread's keys: chunk j covers keys j*128 + part*32 .. +31.
      uint32_t vis[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t mvis = kvis[j];
        if (p.causal) {
          const int n = kmax - (j * 128 + part * 32) + 1;  // number of leading visible keys
          mvis &= n >= 32 ? 0xffffffffu : (n <= 0 ? 0u : ((1u << n) - 1u));
        }
        if (p.kv_seg != nullptr && j < nblk) {
          uint32_t ms = 0;
          for (int x = 0; x < 32; ++x)
            ms |= (sKeySeg[j * 128 + part * 32 + x] == qseg ? 1u : 0u) << x;
          mvis &= ms;
        }
        vis[j] = mvis;
      }
      // ---- pass 1: row max ----
      float m = -3.0e38f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (j >= nblk || !ok) break;
        ok = mbar_wait_relaxed(&bar_s[j], ph, abort_flag);
        if (!ok) break;
        tc_fence_after();
        uint32_t v[32];
        const int col0 = j * 128 + part * 32;
        tmem_ld32(t_row + col0, v);
        tmem_ld_wait();
        const float* rel = sRel + (col0 - q + lq_pad - 1);
        if (vis[j] == 0xffffffffu) {
#pragma unroll
          for (int x = 0; x < 32; ++x) {
            float sc = __uint_as_float(v[x]);
            if (has_bias) sc += rel[x];
            m = fmaxf(m, sc);
          }
        } else {
          const uint32_t mv = vis[j], mi = inr[j];
#pragma unroll
          for (int x = 0; x < 32; ++x) {
            float sc = __uint_as_float(v[x]);
            if (has_bias) sc += rel[x];
            sc = ((mv >> x) & 1u) ? sc : kMaskValue;
            if ((mi >> x) & 1u) m = fmaxf(m, sc);
          }
        }
      }
      sStat[r * 4 + part] = m;
      softmax_bar_sync();
      m = fmaxf(fmaxf(sStat[r * 4], sStat[r * 4 + 1]), fmaxf(sStat[r * 4 + 2], sStat[r * 4 + 3]));
      const float m2 = m * kLog2e;
      // ---- pass 2: probabilities -> smem (bf16), row sums ----
      float l = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (j >= nblk || !ok) break;
        // P buffer (j & 1) was last read by the PV MMA of block j-2 (this query block) or of
        // the last block with the same parity of the previous query block.
        if (j >= 2) {
          ok = mbar_wait_relaxed(&bar_pv[j - 2], ph, abort_flag);
        } else if (i > 0) {
          const int jp = ((nblk - 1 - j) & ~1) + j;  // last block index with parity j
          if (jp < nblk) ok = mbar_wait_relaxed(&bar_pv[jp], ph ^ 1, abort_flag);
        }
        if (!ok) break;
        uint8_t* ptile = sP + (j & 1) * 2 * FwdSmem::kTile + (part >> 1) * FwdSmem::kTile;
        uint32_t v[32];
        const int col0 = j * 128 + part * 32;
        tmem_ld32(t_row + col0, v);
        tmem_ld_wait();
        const float* rel = sRel + (col0 - q + lq_pad - 1);
        float pr[32];
        if (vis[j] == 0xffffffffu) {
#pragma unroll
          for (int x = 0; x < 32; ++x) {
            float sc = __uint_as_float(v[x]);
            if (has_bias) sc += rel[x];
            const float e = exp2f(fmaf(sc, kLog2e, -m2));
            pr[x] = e;
            l += e;
          }
        } else {
          const uint32_t mv = vis[j], mi = inr[j];
#pragma unroll
          for (int x = 0; x < 32; ++x) {
            float sc = __uint_as_float(v[x]);
            if (has_bias) sc += rel[x];
            sc = ((mv >> x) & 1u) ? sc : kMaskValue;
            // subtract first: a fully masked row has sc == m == -1e10 and must give exp2(0)
            const float e = ((mi >> x) & 1u) ? exp2f((sc - m) * kLog2e) : 0.f;
            pr[x] = e;
            l += e;
          }
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) store_swizzled_chunk(ptile, r, (part & 1) * 4 + g, pr + g * 8);
        tc_fence_before();
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_p[j]);
      }
      sStat[512 + r * 4 + part] = l;
      softmax_bar_sync();
      l = (sStat[512 + r * 4] + sStat[512 + r * 4 + 1]) + (sStat[512 + r * 4 + 2] + sStat[512 + r * 4 + 3]);
      // ---- epilogue: O / l (each of the 4 threads of a row writes 16 of the 64 columns) ----
      if (ok) ok = mbar_wait_relaxed(&bar_pv[nblk - 1], ph, abort_flag);
      if (!ok) break;
      tc_fence_after();
      {
        uint32_t v[16];
        tmem_ld16(t_row + o_col + part * 16, v);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_oread);
        if (q < p.Lq) {
          __nv_bfloat16* dst =
              p.O + b * p.o_sb + static_cast<long long>(q) * p.o_sl + h * p.o_sh + part * 16;
          store16_bf16(dst, v, 1.f / l);
          if (part == 0 && p.lse != nullptr)
            p.lse[(static_cast<long long>(b) * p.H + h) * p.Lq + q] = m + __logf(l);
        }
      }
      // sStat is rewritten by the next query block only after everyone read the sums
      softmax_bar_sync();
    }
    if (!ok && lane == 0) {
      report_status(p.status, kStatusTimeoutEpilogue, kKernelIdAttnFwd, blockIdx.x, blockIdx.y);
      *abort_flag = 1;
    }
  }
  if (*abort_flag && threadIdx.x == 0)
    for (int it = 0; it < 2000; ++it) __nanosleep(1000);
  tc_fence_before();
  __syncthreads();
  if (warp == kCtrlWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------
// Backward
// ---------------------------------------------------------------------------------------
// delta[b,h,q] = sum_d dO[b,q,h,d] * O[b,q,h,d]
template <int D>
__global__ void __launch_bounds__(256)
    attn_delta_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O,
                      float* __restrict__ delta, int B, int H, int Lq, long long do_sb,
                      long long do_sl, long long do_sh, long long o_sb, long long o_sl,
                      long long o_sh) {
  // D / 8 lanes per (b, q, h): one 16-byte load per lane and tensor; four items in flight per
  // thread. Requires 16-byte aligned rows (strides multiples of 8 elements).
  constexpr int kLanes = D / 8;           // 8 or 16
  constexpr int kShift = (D == 64) ? 3 : 4;
  const long long total = static_cast<long long>(B) * Lq * H;
  const int sub = threadIdx.x & (kLanes - 1);
  const long long first = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> kShift;
  const long long stride = (static_cast<long long>(gridDim.x) * blockDim.x) >> kShift;
  // the lane groups of a warp leave the loop together (the shuffles use the full mask)
  const int group = (threadIdx.x & 31) >> kShift;
  for (long long w0 = first; w0 - group < total; w0 += 4 * stride) {
    uint4 a[4], c[4];
    long long out[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long w = w0 + u * stride;
      out[u] = -1;
      if (w < total) {
        const int hh = static_cast<int>(w % H);
        const long long t = w / H;
        const int q = static_cast<int>(t % Lq);
        const int bb = static_cast<int>(t / Lq);
        a[u] = *reinterpret_cast<const uint4*>(dO + bb * do_sb + static_cast<long long>(q) * do_sl +
                                               hh * do_sh + sub * 8);
        c[u] = *reinterpret_cast<const uint4*>(O + bb * o_sb + static_cast<long long>(q) * o_sl +
                                               hh * o_sh + sub * 8);
        out[u] = (static_cast<long long>(bb) * H + hh) * Lq + q;
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float s = 0.f;
      if (out[u] >= 0) {
        const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a[u]);
        const __nv_bfloat162* pc = reinterpret_cast<const __nv_bfloat162*>(&c[u]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 fa = __bfloat1622float2(pa[j]), fc = __bfloat1622float2(pc[j]);
          s += fa.x * fc.x + fa.y * fc.y;
        }
      }
      if (kLanes == 16) s += __shfl_xor_sync(0xffffffffu, s, 8);
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      if (sub == 0 && out[u] >= 0) delta[out[u]] = s;
    }
  }
}

// head_dim 64: Q / dO double-buffered, the scores of the next query block are issued while the
// softmax warps work, dQ partial tiles alternate between two TMEM buffers. head_dim 128: operand
// tiles are twice as large and dK, dV take twice the TMEM columns, so Q / dO have one stage, dQ
// reuses the columns of S^T and the query blocks run one after the other.
template <int D>
struct BwdSmem {
  static constexpr int kTile = 128 * 128;  // bytes of a [128 x 64] bf16 panel
  static constexpr int kPanels = D / 64;
  static constexpr int kStages = (D == 64) ? 2 : 1;
  static constexpr int kK = 0;
  static constexpr int kV = kK + kPanels * kTile;
  static constexpr int kQ = kV + kPanels * kTile;                 // kStages x kPanels
  static constexpr int kDO = kQ + kStages * kPanels * kTile;      // kStages x kPanels
  static constexpr int kPT = kDO + kStages * kPanels * kTile;     // P^T : 2 panels (128 keys x 128 queries)
  static constexpr int kDST = kPT + 2 * kTile;                    // dS^T: 2 panels
  static constexpr int kVec = kDST + 2 * kTile;     // 2 stages x {lse[128], delta[128], qseg[128]}
  static constexpr int kRel = kVec + 2 * 3 * 128 * 4;   // bias by rel for the (i, j) pair: 2 x 256 floats
  static constexpr int kDRel = kRel + 2 * 256 * 4;      // d bias by rel accumulators: (Lq_pad + 128) floats
  static constexpr int kBars = kDRel + (4096 + 128) * 4;
  static constexpr int kTotal = kBars + 256 + 1024;
};

template <int D>
__global__ void __launch_bounds__(kAttnThreads, 1)
    attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                    const AttnParams p) {
  using Smem = BwdSmem<D>;
  constexpr int kPanels = Smem::kPanels;
  constexpr int kStageBytes = kPanels * Smem::kTile;  // one Q (or dO) stage
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem + Smem::kK;
  uint8_t* sV = smem + Smem::kV;
  uint8_t* sQ = smem + Smem::kQ;
  uint8_t* sDO = smem + Smem::kDO;
  uint8_t* sPT = smem + Smem::kPT;
  uint8_t* sDST = smem + Smem::kDST;
  float* sVec = reinterpret_cast<float*>(smem + Smem::kVec);
  float* sRelAll = reinterpret_cast<float*>(smem + Smem::kRel);
  float* sDRel = reinterpret_cast<float*>(smem + Smem::kDRel);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Smem::kBars);
  uint64_t* bar_kv = bars;          // 1
  uint64_t* bar_qdo = bars + 1;     // 2 (full, per stage)
  uint64_t* bar_free = bars + 3;    // 2 (stage consumed by the MMAs)
  uint64_t* bar_s = bars + 5;       // S^T and dP^T ready
  uint64_t* bar_p = bars + 6;       // P^T / dS^T written, S^T / dP^T released
  uint64_t* bar_dq = bars + 7;      // dQ partial ready (also: P^T/dS^T smem consumed)
  uint64_t* bar_dq_read = bars + 8; // dQ partial consumed
  uint64_t* bar_sfree = bars + 9;   // S^T / dP^T columns read into registers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k0 = blockIdx.x * 128, h = blockIdx.y, b = blockIdx.z;
  const int nq = (p.Lq + 127) / 128;
  const int lq_pad = nq * 128;
  // TMEM columns
  // dQ partial tiles alternate between two 64-column buffers, so that the tile of query block
  // i is read out while the MMAs of block i + 1 run.
  constexpr int cS = 0, cDP = 128;
  constexpr int cDQ = (D == 64) ? 256 : 0;     // head_dim 128: dQ takes over the columns of S^T
  constexpr int cDK = (D == 64) ? 384 : 256;
  constexpr int cDV = (D == 64) ? 448 : 384;
  constexpr int kColsPerPart = D / 4;          // output columns per thread of a row

  if (threadIdx.x == 0) {
    mbar_init(bar_kv, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bar_qdo[s], 1);
      mbar_init(&bar_free[s], 1);
    }
    mbar_init(bar_s, 1);
    mbar_init(bar_p, kSoftmaxWarps);
    mbar_init(bar_dq, 1);
    mbar_init(bar_dq_read, kSoftmaxWarps);
    mbar_init(bar_sfree, kSoftmaxWarps);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kCtrlWarp) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if (p.d_rel_bias != nullptr)
    for (int t = threadIdx.x; t < lq_pad + 128; t += kAttnThreads) sDRel[t] = 0.f;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == kCtrlWarp) {
    if (lane == 0) {
      bool ok = true;
      mbar_expect_tx(bar_kv, 2 * kStageBytes);
      for (int c = 0; c < kPanels; ++c) {
        tma_load_4d(sK + c * Smem::kTile, &tmK, bar_kv, c * 64, h, k0, b);
        tma_load_4d(sV + c * Smem::kTile, &tmV, bar_kv, c * 64, h, k0, b);
      }
      auto load_qdo = [&](int i, int st) {
        mbar_expect_tx(&bar_qdo[st], 2 * kStageBytes);
        for (int c = 0; c < kPanels; ++c) {
          tma_load_4d(sQ + st * kStageBytes + c * Smem::kTile, &tmQ, &bar_qdo[st], c * 64, h,
                      i * 128, b);
          tma_load_4d(sDO + st * kStageBytes + c * Smem::kTile, &tmDO, &bar_qdo[st], c * 64, h,
                      i * 128, b);
        }
      };
      for (int i = 0; i < nq && i < Smem::kStages; ++i) load_qdo(i, i);
      const uint32_t idesc_kq = make_idesc_bf16(128, 128, 0, 0);  // [keys x queries], K = d
      const uint32_t idesc_kd = make_idesc_bf16(128, D, 0, 1);    // [keys x d], K = queries (B MN-major)
      const uint32_t idesc_qd = make_idesc_bf16(128, D, 1, 1);    // [queries x d], A and B MN-major
      const uint32_t ka = smem_u32(sK), va = smem_u32(sV);
      const uint32_t pta = smem_u32(sPT), dsta = smem_u32(sDST);

      auto issue_scores = [&](int st) {  // S^T = K Q_i^T ; dP^T = V dO_i^T
        const uint32_t qa = smem_u32(sQ + st * kStageBytes);
        const uint32_t doa = smem_u32(sDO + st * kStageBytes);
#pragma unroll
        for (int s = 0; s < D / 16; ++s)
          umma_bf16(tmem_base + cS,
                    make_smem_desc_sw128(ka + (s >> 2) * Smem::kTile + (s & 3) * 32, 16, 1024),
                    make_smem_desc_sw128(qa + (s >> 2) * Smem::kTile + (s & 3) * 32, 16, 1024),
                    idesc_kq, s != 0);
#pragma unroll
        for (int s = 0; s < D / 16; ++s)
          umma_bf16(tmem_base + cDP,
                    make_smem_desc_sw128(va + (s >> 2) * Smem::kTile + (s & 3) * 32, 16, 1024),
                    make_smem_desc_sw128(doa + (s >> 2) * Smem::kTile + (s & 3) * 32, 16, 1024),
                    idesc_kq, s != 0);
        umma_commit(bar_s);
      };
      // dV += P^T dO ; dK += dS^T Q ; dQ_i = dS K. The B operands hold d contiguous (MN-major):
      // 64-channel groups are one panel apart, 16 rows of the K dimension 2048 bytes.
      auto issue_grads = [&](int i, int st, int dq_col) {
        const uint32_t qa = smem_u32(sQ + st * kStageBytes);
        const uint32_t doa = smem_u32(sDO + st * kStageBytes);
#pragma unroll
        for (int s = 0; s < 8; ++s)
          umma_bf16(tmem_base + cDV,
                    make_smem_desc_sw128(pta + (s >> 2) * Smem::kTile + (s & 3) * 32, 16, 1024),
                    make_smem_desc_sw128(doa + s * 2048, Smem::kTile, 1024), idesc_kd, (i | s) != 0);
#pragma unroll
        for (int s = 0; s < 8; ++s)
          umma_bf16(tmem_base + cDK,
                    make_smem_desc_sw128(dsta + (s >> 2) * Smem::kTile + (s & 3) * 32, 16, 1024),
                    make_smem_desc_sw128(qa + s * 2048, Smem::kTile, 1024), idesc_kd, (i | s) != 0);
        // A = dS (M = queries) read from the dS^T tiles as an MN-major operand: 64-query groups
        // are kTile apart (LBO), 8-key groups 1024 B apart (SBO); K advances 16 keys = 2048 B.
#pragma unroll
        for (int s = 0; s < 8; ++s)
          umma_bf16(tmem_base + dq_col,
                    make_smem_desc_sw128(dsta + s * 2048, Smem::kTile, 1024),
                    make_smem_desc_sw128(ka + s * 2048, Smem::kTile, 1024), idesc_qd, s != 0);
        umma_commit(bar_dq);
      };

      ok = mbar_wait(bar_kv, 0, abort_flag) && mbar_wait(&bar_qdo[0], 0, abort_flag);
      if (ok) {
        tc_fence_after();
        issue_scores(0);
      }
      if constexpr (D == 64) {
        // Order per query block i: the scores of block i + 1 are issued as soon as the softmax
        // warps hold those of block i in registers (bar_sfree), so they are computed while the
        // warps do their arithmetic; the gradient MMAs of block i follow when P^T / dS^T are
        // in shared memory (bar_p).
        for (int i = 0; i < nq && ok; ++i) {
          const int st = i & 1;
          const uint32_t ph = (i >> 1) & 1;
          ok = mbar_wait(bar_sfree, i & 1, abort_flag);
          if (ok && i + 1 < nq) {
            ok = mbar_wait(&bar_qdo[(i + 1) & 1], ((i + 1) >> 1) & 1, abort_flag);
            if (ok) {
              tc_fence_after();
              issue_scores((i + 1) & 1);
            }
          }
          if (ok) ok = mbar_wait(bar_p, i & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          issue_grads(i, st, cDQ + (i & 1) * 64);
          umma_commit(&bar_free[st]);
          // The softmax warps read dQ_{i-1} right after they signalled bar_p for block i; once
          // they have, its buffer is free for dQ_{i+1}. (Waiting here, not before the next
          // block's MMAs, keeps at most one completion of bar_dq_read ahead of this wait.)
          if (i >= 1 && i + 1 < nq) {
            ok = mbar_wait(bar_dq_read, (i - 1) & 1, abort_flag);
            if (!ok) break;
          }
          // refill this stage with query block i + 2
          if (i + 2 < nq) {
            ok = mbar_wait(&bar_free[st], ph, abort_flag);
            if (!ok) break;
            load_qdo(i + 2, st);
          }
        }
      } else {
        // One query block at a time: scores, softmax, gradient MMAs, dQ read-out (from the
        // columns of S^T), then the next block's operands and scores.
        for (int i = 0; i < nq && ok; ++i) {
          ok = mbar_wait(bar_p, i & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          issue_grads(i, 0, cDQ);
          umma_commit(&bar_free[0]);
          if (i + 1 < nq) {
            ok = mbar_wait(&bar_free[0], i & 1, abort_flag);
            if (!ok) break;
            load_qdo(i + 1, 0);
            ok = mbar_wait(bar_dq_read, i & 1, abort_flag) &&
                 mbar_wait(&bar_qdo[0], (i + 1) & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            issue_scores(0);
          }
        }
      }
      if (!ok) {
        report_status(p.status, kStatusTimeoutMma, kKernelIdAttnBwd, blockIdx.x, blockIdx.y);
        *abort_flag = 1;
      }
    }
  } else {
    // ------------------------------ softmax / gradient warps ------------------------------
    const int quarter = warp & 3, part = warp >> 2;  // 4 threads per key row, 32 queries each
    const int r = quarter * 32 + lane;               // key row of the tile == TMEM lane
    const int k = k0 + r;
    const bool k_ok = k < p.Lk;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    bool kvis = k_ok;
    if (p.key_mask && k_ok) kvis = p.key_mask[static_cast<long long>(b) * p.Lk + k] != 0;
    // causal == 2: prefix LM (segment codes carry "inside the prefix" in bit 30; a key inside
    // the prefix is visible to every query inside the prefix)
    const bool prefix_lm = p.causal == 2;
    const int seg_mask = prefix_lm ? 0x3fffffff : -1;
    const int kcode = (p.kv_seg && k_ok) ? p.kv_seg[static_cast<long long>(b) * p.Lk + k] : 0;
    const int kseg = kcode & seg_mask;
    const bool k_pre = prefix_lm && ((kcode >> 30) & 1);
    const float inv_lk = 1.f / static_cast<float>(p.Lk);
    const bool has_bias = p.rel_bias != nullptr;
    const bool simple_mask = !p.causal && p.kv_seg == nullptr;
    bool ok = true;

    // Per-query vectors of block i go to stage (i & 1) of shared memory; all softmax threads
    // cooperate (thread t < 128: lse, delta and segment id of query t; the next 255 threads:
    // the bias by relative position over the (key block, query block) pair, index
    // u = r - c + 127). `fetch` issues the global loads early, `publish` stores them after the
    // arithmetic of the current block, so their latency is off the critical path.
    float pf_a = 0.f, pf_b = 0.f;
    int pf_c = 0;
    auto fetch_vectors = [&](int i) {
      const int qb = i * 128;
      const int t = threadIdx.x;
      if (t < 128) {
        const int q = qb + t;
        const long long off = (static_cast<long long>(b) * p.H + h) * p.Lq + q;
        pf_a = (q < p.Lq) ? p.lse[off] * kLog2e : 0.f;
        pf_b = (q < p.Lq) ? p.delta[off] : 0.f;
        pf_c = (p.q_seg && q < p.Lq) ? p.q_seg[static_cast<long long>(b) * p.Lq + q] : 0;
      } else if (t < 128 + 255 && has_bias) {
        const int u = t - 128;
        const float* tab = p.rel_bias + static_cast<long long>(h) * p.nrel;
        const int idx = (k0 - qb) + (u - 127) + p.rel_off;
        pf_a = (idx >= 0 && idx < p.nrel) ? tab[idx] : 0.f;
      }
    };
    auto publish_vectors = [&](int i) {
      float* sLse = sVec + (i & 1) * 384;
      float* sDelta = sLse + 128;
      int* sQseg = reinterpret_cast<int*>(sDelta + 128);
      float* sRel = sRelAll + (i & 1) * 256;
      const int t = threadIdx.x;
      if (t < 128) {
        sLse[t] = pf_a;
        sDelta[t] = pf_b;
        sQseg[t] = pf_c;
      } else if (t < 128 + 255 && has_bias) {
        sRel[t - 128] = pf_a;
      }
    };

    auto read_dq = [&](int blk, bool release) {
      uint32_t v[kColsPerPart];
      if constexpr (D == 64) {
        tmem_ld16(t_row + cDQ + (blk & 1) * 64 + part * 16, v);
      } else {
        tmem_ld32(t_row + cDQ + part * 32, v);
      }
      tmem_ld_wait();
      if (release) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_dq_read);
      }
      const int q = blk * 128 + r;
      if (q < p.Lq) {
        float* dst = p.dQ + ((static_cast<long long>(b) * p.Lq + q) * p.H + h) * D +
                     part * kColsPerPart;
#pragma unroll
        for (int x = 0; x < kColsPerPart; x += 4)
          asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + x),
                       "f"(__uint_as_float(v[x])), "f"(__uint_as_float(v[x + 1])),
                       "f"(__uint_as_float(v[x + 2])), "f"(__uint_as_float(v[x + 3]))
                       : "memory");
      }
    };

    fetch_vectors(0);
    publish_vectors(0);
    softmax_bar_sync();
    for (int i = 0; i < nq && ok; ++i) {
      const int qb = i * 128;
      const float* sLse = sVec + (i & 1) * 384;
      const float* sDelta = sLse + 128;
      const int* sQseg = reinterpret_cast<const int*>(sDelta + 128);
      const float* sRel = sRelAll + (i & 1) * 256;
      if (i + 1 < nq) fetch_vectors(i + 1);  // published before the sync at the loop end
      const int col0 = part * 32;  // query column within the block
      // visibility of (this key, queries col0..col0+31)
      uint32_t mv;
      if (simple_mask) {
        mv = kvis ? 0xffffffffu : 0u;
      } else {
        mv = 0;
        for (int x = 0; x < 32; ++x) {
          const int q = qb + col0 + x;
          bool v = kvis;
          const int qcode = sQseg[col0 + x];
          if (p.causal) v = v && (k <= q + p.causal_off || (k_pre && ((qcode >> 30) & 1)));
          if (p.kv_seg) v = v && (kseg == (qcode & seg_mask));
          mv |= (v ? 1u : 0u) << x;
        }
      }
      ok = mbar_wait_relaxed(bar_s, i & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      // 16 columns (queries) at a time keeps the working set in registers: scores and dP of
      // the chunk, its per-query statistics, and the packed bf16 results.
      const float* rel = sRel + (r - col0 + 127);
      const bool interior = simple_mask && k0 + 128 <= p.Lk && qb + 128 <= p.Lq;
      // interior tile with a key-only mask: the mask is one additive constant per thread
      // (-1e10 absorbs any score: |s| is far below the fp32 spacing at 1e10)
      const float madd = kvis ? 0.f : kMaskValue;
      uint8_t* pt_tile = sPT + (part >> 1) * Smem::kTile;
      uint8_t* dst_tile = sDST + (part >> 1) * Smem::kTile;
      // Bias gradient: dS[key r][query c] belongs to bin (r - c). Within the warp's 32 x 32
      // block (lane = key row, x = query column) lane L collects diagonal L and diagonal L - 32:
      // at column x it fetches the value of lane (L + x) mod 32, which lies on diagonal L when
      // L + x < 32 and on diagonal L - 32 otherwise. The 32 shuffles are independent of each
      // other, and the block costs two shared-memory atomics per lane instead of 32. (Masks
      // are additive, so the bias receives dS everywhere.)
      const bool want_drel = p.d_rel_bias != nullptr;
      float* bins = sDRel + (quarter * 32 - qb - col0 + lq_pad);  // bins[lane - x]
      float diag_pos = 0.f, diag_neg = 0.f;
#pragma unroll
      for (int hc = 0; hc < 2; ++hc) {
        uint32_t sv[16], dpv[16];
        tmem_ld16(t_row + cS + col0 + hc * 16, sv);
        tmem_ld16(t_row + cDP + col0 + hc * 16, dpv);
        tmem_ld_wait();
        if (hc == 1) {
          // all of S^T / dP^T of this block is in registers: the scores of the next block may
          // overwrite the columns while the arithmetic below runs
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_sfree);
        }
        float lse_c[16], del_c[16];
#pragma unroll
        for (int g = 0; g < 4; ++g) {  // 16-byte broadcast loads of the per-query statistics
          const float4 a = reinterpret_cast<const float4*>(sLse + col0 + hc * 16)[g];
          const float4 d = reinterpret_cast<const float4*>(sDelta + col0 + hc * 16)[g];
          lse_c[4 * g] = a.x, lse_c[4 * g + 1] = a.y, lse_c[4 * g + 2] = a.z, lse_c[4 * g + 3] = a.w;
          del_c[4 * g] = d.x, del_c[4 * g + 1] = d.y, del_c[4 * g + 2] = d.z, del_c[4 * g + 3] = d.w;
        }
        float pr[16], ds[16];
#pragma unroll
        for (int x = 0; x < 16; ++x) {
          const int xx = hc * 16 + x;
          float s = __uint_as_float(sv[x]);
          if (has_bias) s += rel[-xx];
          if (interior) {
            s = fmaxf(s + madd, kMaskValue);
          } else {
            s = ((mv >> xx) & 1u) ? s : kMaskValue;
          }
          float e = exp2f(fmaf(s, kLog2e, -lse_c[x]));
          // A row with every key masked has lse = -1e10 + log(Lk), which fp32 rounds to -1e10:
          // its probabilities are uniform over the Lk keys.
          if (lse_c[x] < -5e9f) e = inv_lk;
          if (!interior && (!k_ok || qb + col0 + xx >= p.Lq)) e = 0.f;
          pr[x] = e;
          ds[x] = e * (__uint_as_float(dpv[x]) - del_c[x]);
        }
        if (want_drel) {
#pragma unroll
          for (int x = 0; x < 16; ++x) {
            const int xx = hc * 16 + x;
            const float v = __shfl_sync(0xffffffffu, ds[x], (lane + xx) & 31);
            if (lane + xx < 32) {
              diag_pos += v;
            } else {
              diag_neg += v;
            }
          }
        }
        if (D == 64 && hc == 0 && i > 0) {
          // the gradient MMAs of block i - 1 still read P^T / dS^T; they also produce dQ_{i-1}
          // (head_dim 128 has waited for them already, at the end of block i - 1)
          ok = mbar_wait_relaxed(bar_dq, (i - 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
        }
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          store_swizzled_chunk(pt_tile, r, (part & 1) * 4 + hc * 2 + g, pr + g * 8);
          store_swizzled_chunk(dst_tile, r, (part & 1) * 4 + hc * 2 + g, ds + g * 8);
        }
      }
      if (want_drel) {
        atomicAdd(bins + lane, diag_pos);
        if (lane != 0) atomicAdd(bins + (lane - 32), diag_neg);
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p);
      if (!ok) break;
      // dQ partial of the previous block (its MMAs were waited for above), while the MMAs of
      // this block run: rows are queries here (TMEM lane = query within the block), 16 columns
      // per thread.
      if constexpr (D == 64) {
        if (i > 0) read_dq(i - 1, true);
      } else {
        // dQ_i sits in the columns of S^T: out before the next block's scores may be issued
        ok = mbar_wait_relaxed(bar_dq, i & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        read_dq(i, true);
      }
      if (i + 1 < nq) publish_vectors(i + 1);  // other stage than the one block i used
      softmax_bar_sync();  // the vectors of block i+1 are complete; those of block i are dead
    }
    if (D == 64 && ok) {
      ok = mbar_wait_relaxed(bar_dq, (nq - 1) & 1, abort_flag);
      if (ok) {
        tc_fence_after();
        read_dq(nq - 1, false);
      }
    }
    if (ok) {
      // dK, dV accumulators are complete once the last bar_dq fired (same commit group).
#pragma unroll
      for (int c = 0; c < kColsPerPart / 16; ++c) {
        uint32_t vk[16], vv[16];
        tmem_ld16(t_row + cDK + part * kColsPerPart + c * 16, vk);
        tmem_ld16(t_row + cDV + part * kColsPerPart + c * 16, vv);
        tmem_ld_wait();
        if (k_ok) {
          const long long off = b * p.dk_sb + static_cast<long long>(k) * p.dk_sl + h * p.dk_sh +
                                part * kColsPerPart + c * 16;
          store16_bf16(p.dK + off, vk, 1.f);
          store16_bf16(p.dV + off, vv, 1.f);
        }
      }
      softmax_bar_sync();
      if (p.d_rel_bias != nullptr) {
        // sDRel[t] holds sum dS over (k - q) = k0 + t - lq_pad for this key block
        float* out = p.d_rel_bias + static_cast<long long>(h) * p.nrel;
        for (int t = threadIdx.x; t < lq_pad + 128; t += kSoftmaxThreads) {
          const float g = sDRel[t];
          if (g != 0.f) {
            const int idx = k0 + (t - lq_pad) + p.rel_off;  // (k - q) + rel_off
            if (idx >= 0 && idx < p.nrel) atomicAdd(out + idx, g);
          }
        }
      }
    } else if (lane == 0) {
      report_status(p.status, kStatusTimeoutEpilogue, kKernelIdAttnBwd, blockIdx.x, blockIdx.y);
      *abort_flag = 1;
    }
  }
  if (*abort_flag && threadIdx.x == 0)
    for (int it = 0; it < 2000; ++it) __nanosleep(1000);
  tc_fence_before();
  __syncthreads();
  if (warp == kCtrlWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace t5x

using namespace t5x;

// q [B,Lq,H,64], k/v [B,Lk,H,64] bf16 with element strides (sb, sl, sh), innermost contiguous.
// rel_bias [H, nrel] fp32 or null: bias = rel_bias[h][(k - q) + rel_off].
T5X_API int t5x_attention_fwd(const void* q, const void* k, const void* v, void* o, void* lse, int B,
                              int H, int Lq, int Lk, long long q_sb, long long q_sl, long long q_sh,
                              long long k_sb, long long k_sl, long long k_sh, long long v_sb,
                              long long v_sl, long long v_sh, long long o_sb, long long o_sl,
                              long long o_sh, const void* rel_bias, int nrel, int rel_off,
                              const void* key_mask, const void* q_seg, const void* kv_seg,
                              int causal, int causal_off, void* stream) {
  if (B <= 0 || H <= 0 || Lq <= 0 || Lk <= 0) return 0;
  if (Lk > 512) return set_error("attention_fwd: Lk=%d > 512 is not covered by this kernel", Lk);
  if (causal == 2) return set_error("attention_fwd: prefix-LM masks need the streaming kernel");
  if (Lq > kFwdMaxLq && rel_bias != nullptr)
    return set_error("attention_fwd: Lq=%d > %d with a relative bias is not covered", Lq, kFwdMaxLq);
  const CUtensorMap* tq = bhld_map(q, B, Lq, H, q_sb, q_sl, q_sh);
  const CUtensorMap* tk = bhld_map(k, B, Lk, H, k_sb, k_sl, k_sh);
  const CUtensorMap* tv = bhld_map(v, B, Lk, H, v_sb, v_sl, v_sh);
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
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         FwdSmem::kTotal);
    if (e != cudaSuccess) return set_error("attention_fwd attr: %s", cudaGetErrorString(e));
    attr_set[dev] = true;
  }
  dim3 grid(H, B);
  attn_fwd_kernel<<<grid, kAttnThreads, FwdSmem::kTotal, static_cast<cudaStream_t>(stream)>>>(
      *tq, *tk, *tv, p);
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("attention_fwd: %s", cudaGetErrorString(e));
  return 0;
}

namespace t5x {
template <int D>
static int launch_attention_bwd(const void* d_o, const void* o, void* delta, const CUtensorMap* tq,
                                const CUtensorMap* tk, const CUtensorMap* tv,
                                const CUtensorMap* tdo, const AttnParams& p, long long do_sb,
                                long long do_sl, long long do_sh, long long o_sb, long long o_sl,
                                long long o_sh, cudaStream_t st) {
  long long items = static_cast<long long>(p.B) * p.Lq * p.H;
  long long blocks = (items * (D / 8) / 4 + 255) / 256;
  long long cap = static_cast<long long>(num_sms()) * 8;
  attn_delta_kernel<D><<<static_cast<int>(blocks > cap ? cap : blocks), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(d_o), static_cast<const __nv_bfloat16*>(o),
      static_cast<float*>(delta), p.B, p.H, p.Lq, do_sb, do_sl, do_sh, o_sb, o_sl, o_sh);
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_kernel<D>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         BwdSmem<D>::kTotal);
    if (e != cudaSuccess) return set_error("attention_bwd attr: %s", cudaGetErrorString(e));
    attr_set[dev] = true;
  }
  dim3 grid((p.Lk + 127) / 128, p.H, p.B);
  attn_bwd_kernel<D><<<grid, kAttnThreads, BwdSmem<D>::kTotal, st>>>(*tq, *tk, *tv, *tdo, p);
  count_launches(2);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("attention_bwd: %s", cudaGetErrorString(e));
  return 0;
}
}  // namespace t5x

// dq_f32 [B,Lq,H,D] fp32 contiguous, zero on entry. delta [B,H,Lq] fp32 scratch. D = 64 or 128.
T5X_API int t5x_attention_bwd(const void* q, const void* k, const void* v, const void* o,
                              const void* d_o, const void* lse, void* delta, void* dq_f32, void* dk,
                              void* dv, int B, int H, int Lq, int Lk, int D, long long q_sb,
                              long long q_sl, long long q_sh, long long k_sb, long long k_sl,
                              long long k_sh, long long v_sb, long long v_sl, long long v_sh,
                              long long o_sb, long long o_sl, long long o_sh, long long do_sb,
                              long long do_sl, long long do_sh, long long dk_sb, long long dk_sl,
                              long long dk_sh, const void* rel_bias, void* d_rel_bias, int nrel,
                              int rel_off, const void* key_mask, const void* q_seg,
                              const void* kv_seg, int causal, int causal_off, void* stream) {
  if (B <= 0 || H <= 0 || Lq <= 0 || Lk <= 0) return 0;
  if (D != 64 && D != 128) return set_error("attention_bwd: head_dim %d not in {64, 128}", D);
  if (Lq > 4096) return set_error("attention_bwd: Lq=%d > 4096 is not covered by this kernel", Lq);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const CUtensorMap* tq = bhld_map(q, B, Lq, H, q_sb, q_sl, q_sh, D);
  const CUtensorMap* tk = bhld_map(k, B, Lk, H, k_sb, k_sl, k_sh, D);
  const CUtensorMap* tv = bhld_map(v, B, Lk, H, v_sb, v_sl, v_sh, D);
  const CUtensorMap* tdo = bhld_map(d_o, B, Lq, H, do_sb, do_sl, do_sh, D);
  if (!tq || !tk || !tv || !tdo) return -1;
  if ((do_sb | do_sl | do_sh | o_sb | o_sl | o_sh | dk_sb | dk_sl | dk_sh) & 7)
    return set_error("attention_bwd: dO / O / dK strides must be multiples of 8 elements");
  AttnParams p = {};
  p.B = B; p.H = H; p.Lq = Lq; p.Lk = Lk;
  p.rel_bias = static_cast<const float*>(rel_bias);
  p.d_rel_bias = static_cast<float*>(d_rel_bias);
  p.nrel = nrel; p.rel_off = rel_off;
  p.key_mask = static_cast<const uint8_t*>(key_mask);
  p.q_seg = static_cast<const int*>(q_seg);
  p.kv_seg = static_cast<const int*>(kv_seg);
  p.causal = causal; p.causal_off = causal_off;
  p.lse = const_cast<float*>(static_cast<const float*>(lse));
  p.delta = static_cast<const float*>(delta);
  p.dQ = static_cast<float*>(dq_f32);
  p.dK = static_cast<__nv_bfloat16*>(dk);
  p.dV = static_cast<__nv_bfloat16*>(dv);
  p.dk_sb = dk_sb; p.dk_sl = dk_sl; p.dk_sh = dk_sh;
  p.status = device_status_buffer();
  if (D == 128)
    return launch_attention_bwd<128>(d_o, o, delta, tq, tk, tv, tdo, p, do_sb, do_sl, do_sh, o_sb,
                                     o_sl, o_sh, st);
  return launch_attention_bwd<64>(d_o, o, delta, tq, tk, tv, tdo, p, do_sb, do_sl, do_sh, o_sb,
                                  o_sl, o_sh, st);
}
