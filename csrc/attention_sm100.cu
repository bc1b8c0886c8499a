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
// Forward : one CTA per (128-query block, head, batch). Lk <= 512 (S fills TMEM's 512 columns).
// Backward: one CTA per (128-key block, head, batch), looping over query blocks; dQ partial
//           tiles are added to an fp32 buffer with red.global.add.
#include "common.cuh"

namespace t5x {

constexpr int kAttnD = 64;
constexpr int kAttnThreads = 288;  // warps 0-7 softmax/epilogue, warp 8 TMA + MMA issue
constexpr int kKernelIdAttnFwd = 2;
constexpr int kKernelIdAttnBwd = 3;
constexpr float kMaskValue = -1e10f;

struct AttnParams {
  int B, H, Lq, Lk;
  const float* rel_bias;  // [H, nrel] or null
  int nrel, rel_off;
  const uint8_t* key_mask;  // [B, Lk] (1 = attend) or null
  const int* q_seg;         // [B, Lq] or null
  const int* kv_seg;        // [B, Lk] or null
  int causal, causal_off;
  __nv_bfloat16* O;         // forward output [B, Lq, H, D]
  long long o_sb, o_sl, o_sh;
  float* lse;               // [B, H, Lq]
  // backward
  const float* delta;       // [B, H, Lq] rowsum(dO * O)
  float* dQ;                // fp32 [B, Lq, H, D] (contiguous), accumulated atomically
  __nv_bfloat16* dK;        // [B, Lk, H, D]
  __nv_bfloat16* dV;
  long long dk_sb, dk_sl, dk_sh;
  float* d_rel_bias;        // [H, nrel] or null
  int* status;
};

__device__ __forceinline__ void softmax_bar_sync() {
  asm volatile("bar.sync 1, 256;" ::: "memory");
}

// Writes 8 consecutive bf16 (one 16-byte chunk) of row r, chunk c (0..7) of a [128 x 64] K-major
// 128B-swizzled tile.
__device__ __forceinline__ void store_swizzled_chunk(uint8_t* tile, int r, int c, const float* v) {
  __nv_bfloat162 p0 = __floats2bfloat162_rn(v[0], v[1]);
  __nv_bfloat162 p1 = __floats2bfloat162_rn(v[2], v[3]);
  __nv_bfloat162 p2 = __floats2bfloat162_rn(v[4], v[5]);
  __nv_bfloat162 p3 = __floats2bfloat162_rn(v[6], v[7]);
  uint4 u;
  u.x = *reinterpret_cast<uint32_t*>(&p0);
  u.y = *reinterpret_cast<uint32_t*>(&p1);
  u.z = *reinterpret_cast<uint32_t*>(&p2);
  u.w = *reinterpret_cast<uint32_t*>(&p3);
  *reinterpret_cast<uint4*>(tile + r * 128 + ((c ^ (r & 7)) << 4)) = u;
}

// ---------------------------------------------------------------------------------------
// Forward
// ---------------------------------------------------------------------------------------
struct FwdSmem {
  static constexpr int kTile = 128 * 128;  // bytes of a [128 x 64] bf16 tile
  static constexpr int kQ = 0;
  static constexpr int kK = kTile;              // up to 4 tiles
  static constexpr int kV = kK + 4 * kTile;     // up to 4 tiles
  static constexpr int kP = kV + 4 * kTile;     // 2 buffers x 2 tiles
  static constexpr int kRel = kP + 4 * kTile;   // (512 + 128) floats
  static constexpr int kStat = kRel + 640 * 4;  // 128 x 2 floats (row max halves), then sums
  static constexpr int kKeySeg = kStat + 128 * 4 * 4;  // 512 ints: segment id of key k, -1 = hidden
  static constexpr int kBars = kKeySeg + 512 * 4;
  static constexpr int kTotal = kBars + 256 + 1024;
};

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
  uint64_t* bar_q = bars;           // 1
  uint64_t* bar_k = bars + 1;       // 4
  uint64_t* bar_v = bars + 5;       // 4
  uint64_t* bar_s = bars + 9;       // 4  S block ready in TMEM
  uint64_t* bar_p = bars + 13;      // 4  P block written to smem (8 warp arrivals)
  uint64_t* bar_pv = bars + 17;     // 4  PV MMA of block j finished (P buffer reusable)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * 128, h = blockIdx.y, b = blockIdx.z;
  const int nblk = (p.Lk + 127) / 128;
  const int o_col = (nblk * 128) & 511;  // TMEM column of the O accumulator (reuses S block 0 when full)

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    for (int j = 0; j < 4; ++j) {
      mbar_init(&bar_k[j], 1);
      mbar_init(&bar_v[j], 1);
      mbar_init(&bar_s[j], 1);
      mbar_init(&bar_p[j], 8);
      mbar_init(&bar_pv[j], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 8) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  // Relative-position bias for this tile: sRel[t], t = k - r + 127  (r = row within the tile).
  if (p.rel_bias != nullptr) {
    const float* tab = p.rel_bias + static_cast<long long>(h) * p.nrel;
    for (int t = threadIdx.x; t < nblk * 128 + 128; t += kAttnThreads) {
      const int idx = t - 127 - q0 + p.rel_off;
      sRel[t] = (idx >= 0 && idx < p.nrel) ? tab[idx] : 0.f;
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

  if (warp == 8) {
    if (lane == 0) {
      bool ok = true;
      // ---- loads ----
      mbar_expect_tx(bar_q, FwdSmem::kTile);
      tma_load_4d(sQ, &tmQ, bar_q, 0, h, q0, b);
      for (int j = 0; j < nblk; ++j) {
        mbar_expect_tx(&bar_k[j], FwdSmem::kTile);
        tma_load_4d(sK + j * FwdSmem::kTile, &tmK, &bar_k[j], 0, h, j * 128, b);
      }
      for (int j = 0; j < nblk; ++j) {
        mbar_expect_tx(&bar_v[j], FwdSmem::kTile);
        tma_load_4d(sV + j * FwdSmem::kTile, &tmV, &bar_v[j], 0, h, j * 128, b);
      }
      // ---- S_j = Q K_j^T ----
      const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      ok = mbar_wait(bar_q, 0, abort_flag);
      for (int j = 0; j < nblk && ok; ++j) {
        ok = mbar_wait(&bar_k[j], 0, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK + j * FwdSmem::kTile);
#pragma unroll
        for (int s = 0; s < 4; ++s)
          umma_bf16(tmem_base + j * 128, make_smem_desc_sw128(qa + s * 32, 16, 1024),
                    make_smem_desc_sw128(ka + s * 32, 16, 1024), idesc_s, s != 0);
        umma_commit(&bar_s[j]);
      }
      // ---- O += P_j V_j ----
      const uint32_t idesc_o = make_idesc_bf16(128, 64, 0, 1);
      for (int j = 0; j < nblk && ok; ++j) {
        ok = mbar_wait(&bar_p[j], 0, abort_flag) && mbar_wait(&bar_v[j], 0, abort_flag);
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
      if (!ok) {
        report_status(p.status, kStatusTimeoutMma, kKernelIdAttnFwd, blockIdx.x, blockIdx.y);
        *abort_flag = 1;
      }
    }
  } else {
    // ------------------------------ softmax warps ------------------------------
    const int quarter = warp & 3, half = warp >> 2;
    const int r = quarter * 32 + lane;  // row of the tile == TMEM lane
    const int q = q0 + r;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const int qseg = (p.q_seg != nullptr && q < p.Lq) ? p.q_seg[b * p.Lq + q] : 0;
    const int kmax = p.causal ? q + p.causal_off : 0x7fffffff;
    const bool has_bias = p.rel_bias != nullptr;
    bool ok = true;
    // Visibility of this thread's keys, one bit per key: chunk (j, c) covers keys
    // j*128 + half*64 + c*32 .. +31.  bit set = attend; `inr` = key index < Lk.
    uint32_t vis[8], inr[8];
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) {
      const int col0 = (ch >> 1) * 128 + half * 64 + (ch & 1) * 32;
      uint32_t m_vis = 0, m_in = 0;
      if (col0 < nblk * 128) {
        for (int i = 0; i < 32; ++i) {
          const int kk = col0 + i;
          const int sgm = sKeySeg[kk];
          const bool in_range = kk < p.Lk;
          const bool v = (sgm >= 0) && (p.kv_seg == nullptr || sgm == qseg) && (kk <= kmax);
          m_vis |= (v ? 1u : 0u) << i;
          m_in |= (in_range ? 1u : 0u) << i;
        }
      }
      vis[ch] = m_vis;
      inr[ch] = m_in;
    }

    // pass 1: row max
    float m = -3.0e38f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (j >= nblk || !ok) break;
      ok = mbar_wait(&bar_s[j], 0, abort_flag);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        const int col0 = j * 128 + half * 64 + c * 32;
        tmem_ld32(t_row + col0, v);
        tmem_ld_wait();
        const uint32_t mv = vis[(j << 1) | c], mi = inr[(j << 1) | c];
        const float* rel = sRel + (col0 - r + 127);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float sc = __uint_as_float(v[i]);
          if (has_bias) sc += rel[i];
          sc = ((mv >> i) & 1u) ? sc : kMaskValue;
          if ((mi >> i) & 1u) m = fmaxf(m, sc);
        }
      }
    }
    sStat[r * 2 + half] = m;
    softmax_bar_sync();
    m = fmaxf(sStat[r * 2], sStat[r * 2 + 1]);
    // pass 2: probabilities -> smem (bf16), row sums
    float l = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (j >= nblk || !ok) break;
      if (j >= 2) {
        ok = mbar_wait(&bar_pv[j - 2], 0, abort_flag);  // P buffer (j&1) is free again
        if (!ok) break;
      }
      uint8_t* ptile = sP + (j & 1) * 2 * FwdSmem::kTile + half * FwdSmem::kTile;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        const int col0 = j * 128 + half * 64 + c * 32;
        tmem_ld32(t_row + col0, v);
        tmem_ld_wait();
        const uint32_t mv = vis[(j << 1) | c], mi = inr[(j << 1) | c];
        const float* rel = sRel + (col0 - r + 127);
        float pr[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float sc = __uint_as_float(v[i]);
          if (has_bias) sc += rel[i];
          sc = ((mv >> i) & 1u) ? sc : kMaskValue;
          float e = ((mi >> i) & 1u) ? __expf(sc - m) : 0.f;
          // the PV MMA consumes bf16 probabilities: sum what it will actually see
          e = __bfloat162float(__float2bfloat16(e));
          pr[i] = e;
          l += e;
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) store_swizzled_chunk(ptile, r, c * 4 + g, pr + g * 8);
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_p[j]);
    }
    sStat[256 + r * 2 + half] = l;
    softmax_bar_sync();
    l = sStat[256 + r * 2] + sStat[256 + r * 2 + 1];
    // epilogue: O / l
    if (ok) ok = mbar_wait(&bar_pv[nblk - 1], 0, abort_flag);
    if (ok) {
      tc_fence_after();
      uint32_t v[32];
      tmem_ld32(t_row + o_col + half * 32, v);
      tmem_ld_wait();
      if (q < p.Lq) {
        const float inv = 1.f / l;
        float o[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = __uint_as_float(v[i]) * inv;
        __nv_bfloat16* dst = p.O + b * p.o_sb + static_cast<long long>(q) * p.o_sl + h * p.o_sh + half * 32;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          __nv_bfloat162 a0 = __floats2bfloat162_rn(o[g * 8], o[g * 8 + 1]);
          __nv_bfloat162 a1 = __floats2bfloat162_rn(o[g * 8 + 2], o[g * 8 + 3]);
          __nv_bfloat162 a2 = __floats2bfloat162_rn(o[g * 8 + 4], o[g * 8 + 5]);
          __nv_bfloat162 a3 = __floats2bfloat162_rn(o[g * 8 + 6], o[g * 8 + 7]);
          uint4 u;
          u.x = *reinterpret_cast<uint32_t*>(&a0);
          u.y = *reinterpret_cast<uint32_t*>(&a1);
          u.z = *reinterpret_cast<uint32_t*>(&a2);
          u.w = *reinterpret_cast<uint32_t*>(&a3);
          reinterpret_cast<uint4*>(dst)[g] = u;
        }
        if (half == 0 && p.lse != nullptr)
          p.lse[(static_cast<long long>(b) * p.H + h) * p.Lq + q] = m + __logf(l);
      }
    } else if (lane == 0) {
      report_status(p.status, kStatusTimeoutEpilogue, kKernelIdAttnFwd, blockIdx.x, blockIdx.y);
      *abort_flag = 1;
    }
  }
  if (*abort_flag && threadIdx.x == 0)
    for (int it = 0; it < 2000; ++it) __nanosleep(1000);
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------
// Backward
// ---------------------------------------------------------------------------------------
// delta[b,h,q] = sum_d dO[b,q,h,d] * O[b,q,h,d]
__global__ void __launch_bounds__(256)
    attn_delta_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O,
                      float* __restrict__ delta, int B, int H, int Lq, long long do_sb,
                      long long do_sl, long long do_sh, long long o_sb, long long o_sl,
                      long long o_sh) {
  // one warp per (b, q, h): 64 elements -> 2 per lane
  const long long total = static_cast<long long>(B) * Lq * H;
  const int lane = threadIdx.x & 31;
  for (long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5; w < total;
       w += (static_cast<long long>(gridDim.x) * blockDim.x) >> 5) {
    const int hh = static_cast<int>(w % H);
    const long long t = w / H;
    const int q = static_cast<int>(t % Lq);
    const int bb = static_cast<int>(t / Lq);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(
        dO + bb * do_sb + static_cast<long long>(q) * do_sl + hh * do_sh + lane * 2);
    const __nv_bfloat162 c = *reinterpret_cast<const __nv_bfloat162*>(
        O + bb * o_sb + static_cast<long long>(q) * o_sl + hh * o_sh + lane * 2);
    const float2 fa = __bfloat1622float2(a), fc = __bfloat1622float2(c);
    float s = warp_sum(fa.x * fc.x + fa.y * fc.y);
    if (lane == 0) delta[(static_cast<long long>(bb) * H + hh) * Lq + q] = s;
  }
}

struct BwdSmem {
  static constexpr int kTile = 128 * 128;
  static constexpr int kK = 0;
  static constexpr int kV = kTile;
  static constexpr int kQ = 2 * kTile;        // 2 stages
  static constexpr int kDO = 4 * kTile;       // 2 stages
  static constexpr int kPT = 6 * kTile;       // P^T : 2 tiles (128 keys x 128 queries)
  static constexpr int kDST = 8 * kTile;      // dS^T: 2 tiles
  static constexpr int kVec = 10 * kTile;     // lse[128], delta[128], qseg[128] (ints)
  static constexpr int kRel = kVec + 3 * 128 * 4;   // bias by rel for the (i, j) pair: 256 floats
  static constexpr int kDRel = kRel + 256 * 4;      // d bias by rel accumulators: (Lq_pad + 128) floats
  static constexpr int kBars = kDRel + (4096 + 128) * 4;
  static constexpr int kTotal = kBars + 256 + 1024;
};

__global__ void __launch_bounds__(kAttnThreads, 1)
    attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                    const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem + BwdSmem::kK;
  uint8_t* sV = smem + BwdSmem::kV;
  uint8_t* sQ = smem + BwdSmem::kQ;
  uint8_t* sDO = smem + BwdSmem::kDO;
  uint8_t* sPT = smem + BwdSmem::kPT;
  uint8_t* sDST = smem + BwdSmem::kDST;
  float* sLse = reinterpret_cast<float*>(smem + BwdSmem::kVec);
  float* sDelta = sLse + 128;
  int* sQseg = reinterpret_cast<int*>(sDelta + 128);
  float* sRel = reinterpret_cast<float*>(smem + BwdSmem::kRel);
  float* sDRel = reinterpret_cast<float*>(smem + BwdSmem::kDRel);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + BwdSmem::kBars);
  uint64_t* bar_kv = bars;          // 1
  uint64_t* bar_qdo = bars + 1;     // 2 (full, per stage)
  uint64_t* bar_free = bars + 3;    // 2 (stage consumed by the MMAs)
  uint64_t* bar_s = bars + 5;       // S^T and dP^T ready
  uint64_t* bar_p = bars + 6;       // P^T / dS^T written (8 warp arrivals)
  uint64_t* bar_dq = bars + 7;      // dQ partial ready (also: P^T/dS^T smem and stage are free)
  uint64_t* bar_dq_read = bars + 8; // dQ partial consumed (8 warp arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k0 = blockIdx.x * 128, h = blockIdx.y, b = blockIdx.z;
  const int nq = (p.Lq + 127) / 128;
  const int lq_pad = nq * 128;
  // TMEM columns
  constexpr int cS = 0, cDP = 128, cDQ = 256, cDK = 320, cDV = 384;

  if (threadIdx.x == 0) {
    mbar_init(bar_kv, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bar_qdo[s], 1);
      mbar_init(&bar_free[s], 1);
    }
    mbar_init(bar_s, 1);
    mbar_init(bar_p, 8);
    mbar_init(bar_dq, 1);
    mbar_init(bar_dq_read, 8);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 8) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if (p.d_rel_bias != nullptr)
    for (int t = threadIdx.x; t < lq_pad + 128; t += kAttnThreads) sDRel[t] = 0.f;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    if (lane == 0) {
      bool ok = true;
      mbar_expect_tx(bar_kv, 2 * BwdSmem::kTile);
      tma_load_4d(sK, &tmK, bar_kv, 0, h, k0, b);
      tma_load_4d(sV, &tmV, bar_kv, 0, h, k0, b);
      // prefetch the first two query blocks
      for (int i = 0; i < nq && i < 2; ++i) {
        mbar_expect_tx(&bar_qdo[i], 2 * BwdSmem::kTile);
        tma_load_4d(sQ + i * BwdSmem::kTile, &tmQ, &bar_qdo[i], 0, h, i * 128, b);
        tma_load_4d(sDO + i * BwdSmem::kTile, &tmDO, &bar_qdo[i], 0, h, i * 128, b);
      }
      ok = mbar_wait(bar_kv, 0, abort_flag);
      const uint32_t idesc_kq = make_idesc_bf16(128, 128, 0, 0);   // [keys x queries], K = d
      const uint32_t idesc_kd = make_idesc_bf16(128, 64, 0, 1);    // [keys x d], K = queries (B MN-major)
      const uint32_t idesc_qd = make_idesc_bf16(128, 64, 1, 1);    // [queries x d], A and B MN-major
      const uint32_t ka = smem_u32(sK), va = smem_u32(sV);
      const uint32_t pta = smem_u32(sPT), dsta = smem_u32(sDST);
      for (int i = 0; i < nq && ok; ++i) {
        const int st = i & 1;
        const uint32_t ph = (i >> 1) & 1;
        ok = mbar_wait(&bar_qdo[st], ph, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ + st * BwdSmem::kTile);
        const uint32_t doa = smem_u32(sDO + st * BwdSmem::kTile);
        // S^T = K Q^T ; dP^T = V dO^T
#pragma unroll
        for (int s = 0; s < 4; ++s)
          umma_bf16(tmem_base + cS, make_smem_desc_sw128(ka + s * 32, 16, 1024),
                    make_smem_desc_sw128(qa + s * 32, 16, 1024), idesc_kq, s != 0);
#pragma unroll
        for (int s = 0; s < 4; ++s)
          umma_bf16(tmem_base + cDP, make_smem_desc_sw128(va + s * 32, 16, 1024),
                    make_smem_desc_sw128(doa + s * 32, 16, 1024), idesc_kq, s != 0);
        umma_commit(bar_s);
        // wait for P^T / dS^T
        ok = mbar_wait(bar_p, i & 1, abort_flag);
        if (!ok) break;
        if (i > 0) {
          ok = mbar_wait(bar_dq_read, (i - 1) & 1, abort_flag);  // previous dQ tile has been read
          if (!ok) break;
        }
        tc_fence_after();
        // dV += P^T dO ; dK += dS^T Q ; dQ_i = dS K
#pragma unroll
        for (int s = 0; s < 8; ++s)
          umma_bf16(tmem_base + cDV,
                    make_smem_desc_sw128(pta + (s >> 2) * BwdSmem::kTile + (s & 3) * 32, 16, 1024),
                    make_smem_desc_sw128(doa + s * 2048, 8192, 1024), idesc_kd, (i | s) != 0);
#pragma unroll
        for (int s = 0; s < 8; ++s)
          umma_bf16(tmem_base + cDK,
                    make_smem_desc_sw128(dsta + (s >> 2) * BwdSmem::kTile + (s & 3) * 32, 16, 1024),
                    make_smem_desc_sw128(qa + s * 2048, 8192, 1024), idesc_kd, (i | s) != 0);
        // A = dS (M = queries) read from the dS^T tiles as an MN-major operand: 64-query groups
        // are kTile apart (LBO), 8-key groups 1024 B apart (SBO); K advances 16 keys = 2048 B.
#pragma unroll
        for (int s = 0; s < 8; ++s)
          umma_bf16(tmem_base + cDQ, make_smem_desc_sw128(dsta + s * 2048, BwdSmem::kTile, 1024),
                    make_smem_desc_sw128(ka + s * 2048, 8192, 1024), idesc_qd, s != 0);
        umma_commit(bar_dq);
        umma_commit(&bar_free[st]);
        // refill this stage with query block i + 2
        if (i + 2 < nq) {
          ok = mbar_wait(&bar_free[st], ph, abort_flag);
          if (!ok) break;
          mbar_expect_tx(&bar_qdo[st], 2 * BwdSmem::kTile);
          tma_load_4d(sQ + st * BwdSmem::kTile, &tmQ, &bar_qdo[st], 0, h, (i + 2) * 128, b);
          tma_load_4d(sDO + st * BwdSmem::kTile, &tmDO, &bar_qdo[st], 0, h, (i + 2) * 128, b);
        }
      }
      if (!ok) {
        report_status(p.status, kStatusTimeoutMma, kKernelIdAttnBwd, blockIdx.x, blockIdx.y);
        *abort_flag = 1;
      }
    }
  } else {
    // ------------------------------ softmax / gradient warps ------------------------------
    const int quarter = warp & 3, half = warp >> 2;
    const int r = quarter * 32 + lane;  // key row of the tile == TMEM lane
    const int k = k0 + r;
    const bool k_ok = k < p.Lk;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    bool kvis = k_ok;
    if (p.key_mask && k_ok) kvis = p.key_mask[static_cast<long long>(b) * p.Lk + k] != 0;
    const int kseg = (p.kv_seg && k_ok) ? p.kv_seg[static_cast<long long>(b) * p.Lk + k] : 0;
    const float inv_lk = 1.f / static_cast<float>(p.Lk);
    bool ok = true;
    for (int i = 0; i < nq && ok; ++i) {
      const int qb = i * 128;
      // per-query vectors for this block (all 256 threads cooperate)
      {
        const int t = threadIdx.x;
        if (t < 128) {
          const int q = qb + t;
          const long long off = (static_cast<long long>(b) * p.H + h) * p.Lq + q;
          sLse[t] = (q < p.Lq) ? p.lse[off] : 0.f;
          sDelta[t] = (q < p.Lq) ? p.delta[off] : 0.f;
          sQseg[t] = (p.q_seg && q < p.Lq) ? p.q_seg[static_cast<long long>(b) * p.Lq + q] : 0;
        }
        if (p.rel_bias != nullptr) {
          // rel = k - q over the pair: index u = r - c + 127 in [0, 255)
          const float* tab = p.rel_bias + static_cast<long long>(h) * p.nrel;
          if (t < 255) {
            const int idx = (k0 - qb) + (t - 127) + p.rel_off;
            sRel[t] = (idx >= 0 && idx < p.nrel) ? tab[idx] : 0.f;
          }
        }
      }
      softmax_bar_sync();
      ok = mbar_wait(bar_s, i & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      uint8_t* pt_tile = sPT + half * BwdSmem::kTile;
      uint8_t* dst_tile = sDST + half * BwdSmem::kTile;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t sv[32], dpv[32];
        const int col0 = half * 64 + c * 32;  // query column within the block
        tmem_ld32(t_row + cS + col0, sv);
        tmem_ld32(t_row + cDP + col0, dpv);
        tmem_ld_wait();
        float pr[32], ds[32];
#pragma unroll
        for (int x = 0; x < 32; ++x) {
          const int cq = col0 + x;
          const int q = qb + cq;
          float s = __uint_as_float(sv[x]);
          if (p.rel_bias != nullptr) s += sRel[r - cq + 127];
          bool vis = kvis;
          if (p.causal) vis = vis && (k <= q + p.causal_off);
          if (p.kv_seg) vis = vis && (kseg == sQseg[cq]);
          s = vis ? s : kMaskValue;
          float e = (k_ok && q < p.Lq) ? __expf(s - sLse[cq]) : 0.f;
          // A row with every key masked has lse = -1e10 + log(Lk), which fp32 rounds to -1e10:
          // its probabilities are uniform over the Lk keys.
          if (sLse[cq] < -5e9f && k_ok && q < p.Lq) e = inv_lk;
          const float g = e * (__uint_as_float(dpv[x]) - sDelta[cq]);
          pr[x] = e;
          ds[x] = g;
          // masks are additive, so the bias term receives the softmax gradient everywhere
          if (p.d_rel_bias != nullptr && g != 0.f) atomicAdd(&sDRel[r - q + lq_pad], g);
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          store_swizzled_chunk(pt_tile, r, c * 4 + g, pr + g * 8);
          store_swizzled_chunk(dst_tile, r, c * 4 + g, ds + g * 8);
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p);
      // dQ partial: rows are queries here (TMEM lane = query within the block)
      ok = mbar_wait(bar_dq, i & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      {
        uint32_t v[32];
        tmem_ld32(t_row + cDQ + half * 32, v);
        tmem_ld_wait();
        const int q = qb + r;
        if (q < p.Lq) {
          float* dst = p.dQ + ((static_cast<long long>(b) * p.Lq + q) * p.H + h) * kAttnD + half * 32;
#pragma unroll
          for (int x = 0; x < 32; x += 4)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + x),
                         "f"(__uint_as_float(v[x])), "f"(__uint_as_float(v[x + 1])),
                         "f"(__uint_as_float(v[x + 2])), "f"(__uint_as_float(v[x + 3]))
                         : "memory");
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_dq_read);
      softmax_bar_sync();  // sLse/sDelta/sRel are rewritten at the top of the next iteration
    }
    if (ok) {
      // dK, dV accumulators are complete once the last bar_dq fired (same commit group).
      uint32_t vk[32], vv[32];
      tmem_ld32(t_row + cDK + half * 32, vk);
      tmem_ld32(t_row + cDV + half * 32, vv);
      tmem_ld_wait();
      if (k_ok) {
        __nv_bfloat16* dk = p.dK + b * p.dk_sb + static_cast<long long>(k) * p.dk_sl + h * p.dk_sh + half * 32;
        __nv_bfloat16* dv = p.dV + b * p.dk_sb + static_cast<long long>(k) * p.dk_sl + h * p.dk_sh + half * 32;
#pragma unroll
        for (int x = 0; x < 32; x += 2) {
          *reinterpret_cast<__nv_bfloat162*>(dk + x) =
              __floats2bfloat162_rn(__uint_as_float(vk[x]), __uint_as_float(vk[x + 1]));
          *reinterpret_cast<__nv_bfloat162*>(dv + x) =
              __floats2bfloat162_rn(__uint_as_float(vv[x]), __uint_as_float(vv[x + 1]));
        }
      }
      softmax_bar_sync();
      if (p.d_rel_bias != nullptr) {
        // sDRel[t] holds sum dS over (k - q) = k0 + t - lq_pad for this key block
        float* out = p.d_rel_bias + static_cast<long long>(h) * p.nrel;
        for (int t = threadIdx.x; t < lq_pad + 128; t += 256) {
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
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

static const CUtensorMap* bhld_map(const void* ptr, int B, int L, int H, long long sb, long long sl,
                                   long long sh) {
  uint64_t dims[4] = {static_cast<uint64_t>(kAttnD), static_cast<uint64_t>(H),
                      static_cast<uint64_t>(L), static_cast<uint64_t>(B)};
  uint64_t strides[3] = {static_cast<uint64_t>(sh) * 2, static_cast<uint64_t>(sl) * 2,
                         static_cast<uint64_t>(sb) * 2};
  uint32_t box[4] = {64, 1, 128, 1};
  return get_tensor_map(ptr, 2, 4, dims, strides, box, 1);
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
  dim3 grid((Lq + 127) / 128, H, B);
  attn_fwd_kernel<<<grid, kAttnThreads, FwdSmem::kTotal, static_cast<cudaStream_t>(stream)>>>(
      *tq, *tk, *tv, p);
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("attention_fwd: %s", cudaGetErrorString(e));
  return 0;
}

// dq_f32 [B,Lq,H,64] fp32 contiguous, zero on entry. delta [B,H,Lq] fp32 scratch.
T5X_API int t5x_attention_bwd(const void* q, const void* k, const void* v, const void* o,
                              const void* d_o, const void* lse, void* delta, void* dq_f32, void* dk,
                              void* dv, int B, int H, int Lq, int Lk, long long q_sb, long long q_sl,
                              long long q_sh, long long k_sb, long long k_sl, long long k_sh,
                              long long v_sb, long long v_sl, long long v_sh, long long o_sb,
                              long long o_sl, long long o_sh, long long do_sb, long long do_sl,
                              long long do_sh, long long dk_sb, long long dk_sl, long long dk_sh,
                              const void* rel_bias, void* d_rel_bias, int nrel, int rel_off,
                              const void* key_mask, const void* q_seg, const void* kv_seg,
                              int causal, int causal_off, void* stream) {
  if (B <= 0 || H <= 0 || Lq <= 0 || Lk <= 0) return 0;
  if (Lq > 4096) return set_error("attention_bwd: Lq=%d > 4096 is not covered by this kernel", Lq);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const CUtensorMap* tq = bhld_map(q, B, Lq, H, q_sb, q_sl, q_sh);
  const CUtensorMap* tk = bhld_map(k, B, Lk, H, k_sb, k_sl, k_sh);
  const CUtensorMap* tv = bhld_map(v, B, Lk, H, v_sb, v_sl, v_sh);
  const CUtensorMap* tdo = bhld_map(d_o, B, Lq, H, do_sb, do_sl, do_sh);
  if (!tq || !tk || !tv || !tdo) return -1;
  {
    long long warps = static_cast<long long>(B) * Lq * H;
    long long blocks = (warps * 32 + 255) / 256;
    long long cap = static_cast<long long>(num_sms()) * 8;
    attn_delta_kernel<<<static_cast<int>(blocks > cap ? cap : blocks), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(d_o), static_cast<const __nv_bfloat16*>(o),
        static_cast<float*>(delta), B, H, Lq, do_sb, do_sl, do_sh, o_sb, o_sl, o_sh);
  }
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
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         BwdSmem::kTotal);
    if (e != cudaSuccess) return set_error("attention_bwd attr: %s", cudaGetErrorString(e));
    attr_set[dev] = true;
  }
  dim3 grid((Lk + 127) / 128, H, B);
  attn_bwd_kernel<<<grid, kAttnThreads, BwdSmem::kTotal, st>>>(*tq, *tk, *tv, *tdo, p);
  count_launches(2);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("attention_bwd: %s", cudaGetErrorString(e));
  return 0;
}
