// Pieces shared by the one-CTA and the CTA-pair GEMM kernels: problem description, row
// load/store helpers and the epilogue of one accumulator tile.
#pragma once
#include "common.cuh"

namespace t5x {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kGemmThreads = 192;
constexpr int kKernelIdGemm = 1;
constexpr int kGemmTraceSlots = 8;
long long* gemm_trace_buffer();  // host: the calling thread's trace buffer, or null
#define T5X_GEMM_TRACE(slot)                                                              \
  do {                                                                                    \
    if (p.trace != nullptr) p.trace[blockIdx.x * kGemmTraceSlots + (slot)] = global_timer_ns(); \
  } while (0)

enum GemmEpilogue : int {
  kEpiPlain = 0,
  kEpiGatedGelu = 1,
  kEpiResidual = 2,
  // The product is a logits matrix that is consumed in the epilogue and never stored:
  kEpiCeStats = 3,  // per (row, column tile) softmax partials for the cross-entropy forward
  kEpiCeGrad = 4,   // gradient of the cross-entropy w.r.t. the logits, written as bf16
};

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
  int mt_rot;  // the row-tile walk starts at this tile (tensor-parallel kernels); 0 otherwise
  int b_constant;  // B is not written by any kernel in flight: it may be loaded before chain_wait()
  // Optional phase trace (t5x_gemm_set_trace): 8 timestamps per CTA for its first tile: entry,
  // set-up done, first loads issued, first operands landed, last MMA issued, accumulator
  // complete, epilogue done, exit. Null in normal use.
  long long* trace;
  int* status;
  // Cross-entropy epilogues. Column c of the product is vocabulary entry ce_vocab_start + c.
  const long long* ce_targets;  // [M] target ids
  int ce_vocab_start;
  float* ce_part;          // kEpiCeStats: [M, tiles_n, 4] = max, sum exp(x - max), sum x, largest x
  int* ce_arg;             // kEpiCeStats: [M, tiles_n] column of the largest x
  float* ce_target_logit;  // kEpiCeStats: [M], written by the tile that holds the target
  const float* ce_lse;     // kEpiCeGrad: [M] log-sum-exp of the row over the whole vocabulary
  const float* ce_row_scale;  // kEpiCeGrad: [M] upstream gradient of the row's loss
  float ce_z, ce_conf, ce_low;  // z-loss factor, label-smoothing confidences
};

// Tensor-parallel extensions of the CTA-pair GEMM. The rows of A (all-gather) or of C
// (reduce-scatter) are split evenly over `world` ranks, `rows_per_rank` consecutive rows each.
//
// Ordering between ranks needs no separate barrier kernel. Every rank owns a small array of
// signal words in memory that all ranks map; word [kind][r] is written only by rank r, with an
// epoch number that grows by one per call (all ranks make the same calls in the same order).
//   kTpSigRowsReady  rank r's own rows of the A buffer are in place (written by the kernel that
//                    precedes the all-gather GEMM on r's stream). Raised by r's all-gather GEMM
//                    as it starts; awaited by the copy warps before they pull from r.
//   kTpSigScattered  every store of rank r's reduce-scatter GEMM into the inboxes has been
//                    performed. Raised by the last CTA of that GEMM; awaited by the kernel that
//                    sums the inbox slots.
// Waits compare epochs by signed distance (wrap-safe), are bounded, and report a status.
enum GemmTpMode : int { kTpNone = 0, kTpAllGather = 1, kTpReduceScatter = 2 };
constexpr int kTpMaxPeers = 16;
constexpr int kTpSigRowsReady = 0;
constexpr int kTpSigScattered = 1;
constexpr int kTpSigWords = 2 * kTpMaxPeers;
constexpr int kTpGroupRows = 128;  // rows of A whose arrival is tracked by one counter
struct GemmTp {
  int world, rank, rows_per_rank;
  // all-gather -> GEMM: A is this rank's [M, K] buffer; block r of it is pulled from
  // a_src[r] (rank r's buffer as mapped here, same layout) by the copy warps while the tensor
  // cores work on blocks that are already here. flags[r * groups_per_block + g] counts the
  // pieces landed in row group g (kTpGroupRows rows) of block r; the last CTA to leave the
  // kernel clears them again.
  const uint8_t* a_src[kTpMaxPeers];
  uint8_t* a_dst;
  long long block_bytes;
  long long group_bytes;
  int groups_per_block;
  unsigned int* flags;
  // GEMM -> reduce-scatter: rows of block r are stored to c_dst[r] ([rows_per_rank, ldc] bf16,
  // this rank's slot of rank r's inbox as mapped here) instead of C.
  __nv_bfloat16* c_dst[kTpMaxPeers];
  // signal words: this rank's own array and the peers' arrays as mapped here; `epoch` is what
  // this call raises and waits for; `exit_count` counts CTAs that have finished (device word).
  unsigned int* sig_local;
  unsigned int* sig_peer[kTpMaxPeers];
  unsigned int epoch;
  unsigned int* exit_count;
};

__device__ __forceinline__ void st_release_sys_u32(unsigned int* addr, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys_u32(const unsigned int* addr) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

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

// Coalesced epilogue stores. A lane holds 32 consecutive columns of ONE accumulator row, so a
// store straight from registers sends 16-byte pieces of 32 different rows per warp
// instruction: 32 separate 128-byte lines each time, which the load/store unit serialises (a
// 128 x 128 fp32 tile of split-K atomics took 7 us that way). Instead the warp parks its
// 32 x 32 block in shared memory (`stage`: 4 KB of this warp, 16-byte chunks XOR-swizzled by
// row so that neither side has bank conflicts) and writes it out as whole row segments:
// four rows of 128 bytes (fp32) or eight rows of 64 bytes (bf16) per instruction.
constexpr int kEpiStageBytesPerWarp = 32 * 128;

// v: this lane's row (32 floats). out: &C[first row of the warp's block][first column], fp32.
// MODE 0: plain store, 1: add to what is there (one writer per element), 2: atomic add; a
// template argument so that every variant is straight-line code (with the mode as a run-time
// value the atomic variant ran almost four times slower). Rows >= rows_valid are skipped. All
// lanes must call it.
template <int MODE>
__device__ __forceinline__ void staged_store_f32(float* stage, const float (&v)[32], float* out,
                                                 long long ldc, int rows_valid, int lane) {
#pragma unroll
  for (int c = 0; c < 8; ++c)
    *reinterpret_cast<float4*>(stage + lane * 32 + ((c ^ (lane & 7)) * 4)) =
        make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
  __syncwarp();
  const int c = lane & 7;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int row = j * 4 + (lane >> 3);
    const float4 o = *reinterpret_cast<const float4*>(stage + row * 32 + ((c ^ (row & 7)) * 4));
    if (row < rows_valid) {
      float4* dst = reinterpret_cast<float4*>(out + static_cast<long long>(row) * ldc + c * 4);
      if (MODE == 2) {
        atomicAdd(dst, o);
      } else if (MODE == 1) {
        const float4 old = *dst;
        *dst = make_float4(o.x + old.x, o.y + old.y, o.z + old.z, o.w + old.w);
      } else {
        *dst = o;
      }
    }
  }
  __syncwarp();
}

// The same for a bf16 output: the staged block is 32 rows x 64 bytes (the first half of each
// 128-byte staging row), written out as eight 64-byte row segments per instruction.
__device__ __forceinline__ void staged_store_bf16(float* stage, const float (&v)[32],
                                                  __nv_bfloat16* out, long long ldc,
                                                  int rows_valid, int lane) {
  uint4* st4 = reinterpret_cast<uint4*>(stage);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    __nv_bfloat162 p0 = __floats2bfloat162_rn(v[c * 8 + 0], v[c * 8 + 1]);
    __nv_bfloat162 p1 = __floats2bfloat162_rn(v[c * 8 + 2], v[c * 8 + 3]);
    __nv_bfloat162 p2 = __floats2bfloat162_rn(v[c * 8 + 4], v[c * 8 + 5]);
    __nv_bfloat162 p3 = __floats2bfloat162_rn(v[c * 8 + 6], v[c * 8 + 7]);
    uint4 u;
    u.x = *reinterpret_cast<uint32_t*>(&p0);
    u.y = *reinterpret_cast<uint32_t*>(&p1);
    u.z = *reinterpret_cast<uint32_t*>(&p2);
    u.w = *reinterpret_cast<uint32_t*>(&p3);
    // row `lane`, 16-byte chunk c of 4, swizzled over the 8 chunk slots of the 128-byte row
    st4[lane * 8 + ((c ^ (lane & 7)))] = u;
  }
  __syncwarp();
  const int c = lane & 3;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int row = j * 8 + (lane >> 2);
    const uint4 u = st4[row * 8 + (c ^ (row & 7))];
    if (row < rows_valid)
      *reinterpret_cast<uint4*>(out + static_cast<long long>(row) * ldc + c * 8) = u;
  }
  __syncwarp();
}

// Tile order: groups of kRasterGroup row tiles are walked column by column, so that the tiles
// in flight at one time (one per SM or SM pair) share a few A row blocks and a few B column
// blocks instead of one A block and every B block; the operands of a wave then fit in L2.
constexpr int kRasterGroup = 8;
__device__ __forceinline__ void gemm_tile_coords(const GemmParams& p, int tile, int tiles_per_batch,
                                                 int& b, int& mt, int& nt) {
  b = tile / tiles_per_batch;
  const int rem = tile - b * tiles_per_batch;
  const int per_group = kRasterGroup * p.tiles_n;
  const int g = rem / per_group;
  const int first_m = g * kRasterGroup;
  const int gsz = min(kRasterGroup, p.tiles_m - first_m);
  const int r = rem - g * per_group;
  nt = r / gsz;
  mt = first_m + (r - nt * gsz);
  if (p.mt_rot) {
    mt += p.mt_rot;
    if (mt >= p.tiles_m) mt -= p.tiles_m;
  }
}

// Epilogue of one 128-row accumulator tile held in TMEM columns [t_cols, t_cols + BN): the
// calling warp owns lane quarter q (rows m0 + 32q .. +31), `c_vec_ok` says whether 16-byte
// stores to C are legal.
template <int BN, int EPI>
__device__ __forceinline__ void gemm_epilogue_tile(const GemmParams& p, uint32_t t_row, int m0,
                                                   int n0, int b, int q, int lane,
                                                   bool c_vec_ok, float* stage = nullptr) {
  const int row = m0 + q * 32 + lane;
  const bool row_ok = row < p.M;
  const int rows_valid = p.M - (m0 + q * 32);  // of this warp's 32 rows (may exceed 32 or be <= 0)

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
      const bool hv16 = p.H0 == nullptr ||
                        ((p.ldh % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.H0) |
                                               reinterpret_cast<uintptr_t>(p.H1)) & 15) == 0);
      if (stage != nullptr && n_valid >= 32 && rows_valid > 0 && c_vec_ok && hv16) {
        // whole 32-column blocks: row-contiguous stores through the staging block
        float g[32], h0[32], h1[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          h0[i] = __uint_as_float(r0[i]);
          h1[i] = __uint_as_float(r1[i]);
          g[i] = gelu_tanh(h0[i]) * h1[i];
        }
        const long long first_row = m0 + q * 32;
        staged_store_bf16(stage, g,
                          reinterpret_cast<__nv_bfloat16*>(p.C) + b * p.c_batch_stride +
                              first_row * p.ldc + col,
                          p.ldc, rows_valid, lane);
        if (p.H0 != nullptr) {
          staged_store_bf16(stage, h0, p.H0 + first_row * p.ldh + col, p.ldh, rows_valid, lane);
          staged_store_bf16(stage, h1, p.H1 + first_row * p.ldh + col, p.ldh, rows_valid, lane);
        }
        continue;
      }
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
      // whole 32-column blocks go out through the staging buffer (warp-uniform condition)
      const bool staged = stage != nullptr && n_valid >= 32 && rows_valid > 0 &&
                          (p.out_fp32 ? (p.ldc % 4 == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0)
                                      : (c_vec_ok && p.accumulate == 0));
      if (staged) {
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
        if (EPI == kEpiResidual && row_ok) {
          float rr[32];
          const bool rv = (p.ldr % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.R) & 15) == 0);
          load_row_bf16(p.R + b * p.r_batch_stride + static_cast<long long>(row) * p.ldr + col,
                        rr, n_valid, rv);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] += rr[i];
        }
        const long long first = b * p.c_batch_stride +
                                static_cast<long long>(m0 + q * 32) * p.ldc + col;
        if (p.out_fp32) {
          float* dst = reinterpret_cast<float*>(p.C) + first;
          if (p.accumulate == 2)
            staged_store_f32<2>(stage, v, dst, p.ldc, rows_valid, lane);
          else if (p.accumulate == 1)
            staged_store_f32<1>(stage, v, dst, p.ldc, rows_valid, lane);
          else
            staged_store_f32<0>(stage, v, dst, p.ldc, rows_valid, lane);
        } else
          staged_store_bf16(stage, v, reinterpret_cast<__nv_bfloat16*>(p.C) + first, p.ldc,
                            rows_valid, lane);
        continue;
      }
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
              if (p.accumulate == 2) {  // several CTAs (split K) add into the same tile
                atomicAdd(reinterpret_cast<float4*>(out) + i, o);
                continue;
              }
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
            for (int i = 0; i < 32 && i < n_valid; ++i) {
              if (p.accumulate == 2)
                atomicAdd(out + i, v[i]);
              else
                out[i] = p.accumulate ? out[i] + v[i] : v[i];
            }
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
}

// Cross-entropy forward epilogue of one accumulator tile: the calling thread owns one row of
// logits x = alpha * acc and folds the tile's BN columns into (max, sum exp(x - max), sum x,
// largest x and its column), which a small kernel merges over the column tiles afterwards.
// The logits themselves are never stored.
template <int BN>
__device__ __forceinline__ void gemm_epilogue_ce_stats(const GemmParams& p, uint32_t t_row, int m0,
                                                       int n0, int nt, int q, int lane) {
  const int row = m0 + q * 32 + lane;
  const bool row_ok = row < p.M;
  const long long tgt = row_ok ? p.ce_targets[row] - p.ce_vocab_start : -1;
  float mx = -3.0e38f, se = 0.f, sx = 0.f, best = -3.0e38f;
  int best_col = 0;
#pragma unroll 1
  for (int c = 0; c < BN / 32; ++c) {
    uint32_t r[32];
    tmem_ld32(t_row + c * 32, r);
    tmem_ld_wait();
    const int col = n0 + c * 32;
    const int n_valid = p.N - col;
    if (!row_ok || n_valid <= 0) continue;
    float v[32];
    float cm = -3.0e38f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      v[i] = __uint_as_float(r[i]) * p.alpha;
      if (i < n_valid) {
        cm = fmaxf(cm, v[i]);
        sx += v[i];
        if (v[i] > best) {
          best = v[i];
          best_col = col + i;
        }
        if (col + i == tgt) p.ce_target_logit[row] = v[i];
      }
    }
    const float nm = fmaxf(mx, cm);
    float add = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < n_valid) add += __expf(v[i] - nm);
    se = se * __expf(mx - nm) + add;
    mx = nm;
  }
  if (row_ok) {
    float4* out = reinterpret_cast<float4*>(p.ce_part) + static_cast<long long>(row) * p.tiles_n + nt;
    *out = make_float4(mx, se, sx, best);
    p.ce_arg[static_cast<long long>(row) * p.tiles_n + nt] = best_col + p.ce_vocab_start;
  }
}

// Cross-entropy backward epilogue: the logits tile is recomputed by the GEMM and turned into
//   dlogits = row_scale * ((1 + 2 z lse) * exp(x - lse) - soft_target)        (bf16)
// which the two gradient GEMMs of the projection read next. C is the bf16 [M, N] output.
template <int BN>
__device__ __forceinline__ void gemm_epilogue_ce_grad(const GemmParams& p, uint32_t t_row, int m0,
                                                      int n0, int q, int lane, bool c_vec_ok) {
  const int row = m0 + q * 32 + lane;
  const bool row_ok = row < p.M;
  const float lse = row_ok ? p.ce_lse[row] : 0.f;
  const float g = row_ok ? p.ce_row_scale[row] : 0.f;
  const float zf = 1.f + 2.f * p.ce_z * lse;
  const long long tgt = row_ok ? p.ce_targets[row] - p.ce_vocab_start : -1;
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc;
#pragma unroll 1
  for (int c = 0; c < BN / 32; ++c) {
    uint32_t r[32];
    tmem_ld32(t_row + c * 32, r);
    tmem_ld_wait();
    const int col = n0 + c * 32;
    const int n_valid = p.N - col;
    if (!row_ok || n_valid <= 0) continue;
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float x = __uint_as_float(r[i]) * p.alpha;
      const float soft = (col + i == tgt) ? p.ce_conf : p.ce_low;
      v[i] = g == 0.f ? 0.f : g * (zf * __expf(x - lse) - soft);
    }
    store_row_bf16(out + col, v, n_valid, c_vec_ok);
  }
}

// Reduce-scatter epilogue of one 128-row accumulator tile: each row of the bf16 partial product
// (+ local residual) goes to the inbox of the rank that owns the row, mostly peer memory. A
// lane holds one row of the accumulator, so storing straight from registers would send 16-byte
// pieces of 32 different rows per instruction; over NVLink that is one small packet each.
// Instead 128 columns at a time are staged in shared memory (`stage`: 8 KB of this warp, 16-byte
// chunks XOR-swizzled by row so that neither side has bank conflicts) and written out as
// 256-byte row segments, two rows per warp instruction. Requires N % 8 == 0 and ldc % 8 == 0.
constexpr int kRsGroupCols = 128;
constexpr int kRsStageBytesPerWarp = 32 * kRsGroupCols * 2;
template <int BN, int EPI>
__device__ __forceinline__ void gemm_epilogue_tile_rs(const GemmParams& p, const GemmTp& tp,
                                                      uint32_t t_row, int m0, int n0, int q,
                                                      int lane, uint8_t* stage) {
  const int row = m0 + q * 32 + lane;
  const bool row_ok = row < p.M;
#pragma unroll 1
  for (int g = 0; g < BN / kRsGroupCols; ++g) {
    const int gcol = n0 + g * kRsGroupCols;
#pragma unroll 1
    for (int c = 0; c < kRsGroupCols / 32; ++c) {
      uint32_t r[32];
      tmem_ld32(t_row + g * kRsGroupCols + c * 32, r);
      tmem_ld_wait();
      const int col = gcol + c * 32;
      const int n_valid = p.N - col;
      float v[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
      if (EPI == kEpiResidual && row_ok && n_valid > 0) {
        float rr[32];
        const bool rv = (p.ldr % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.R) & 15) == 0);
        load_row_bf16(p.R + static_cast<long long>(row) * p.ldr + col, rr, n_valid, rv);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] += rr[i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {  // four 16-byte chunks of this lane's row
        __nv_bfloat162 p0 = __floats2bfloat162_rn(v[i * 8 + 0], v[i * 8 + 1]);
        __nv_bfloat162 p1 = __floats2bfloat162_rn(v[i * 8 + 2], v[i * 8 + 3]);
        __nv_bfloat162 p2 = __floats2bfloat162_rn(v[i * 8 + 4], v[i * 8 + 5]);
        __nv_bfloat162 p3 = __floats2bfloat162_rn(v[i * 8 + 6], v[i * 8 + 7]);
        uint4 u;
        u.x = *reinterpret_cast<uint32_t*>(&p0);
        u.y = *reinterpret_cast<uint32_t*>(&p1);
        u.z = *reinterpret_cast<uint32_t*>(&p2);
        u.w = *reinterpret_cast<uint32_t*>(&p3);
        const int chunk = (c * 4 + i) ^ (lane & 15);
        *reinterpret_cast<uint4*>(stage + lane * (kRsGroupCols * 2) + chunk * 16) = u;
      }
    }
    __syncwarp();
    // 16 instructions, each: lanes 0-15 one row, lanes 16-31 the next, 16 bytes per lane
    const int chunk = lane & 15;
    const int ccol = gcol + chunk * 8;
#pragma unroll 4
    for (int it = 0; it < 16; ++it) {
      const int rloc = it * 2 + (lane >> 4);
      const int grow = m0 + q * 32 + rloc;
      if (grow < p.M && ccol < p.N) {
        const uint4 u = *reinterpret_cast<const uint4*>(stage + rloc * (kRsGroupCols * 2) +
                                                        ((chunk ^ (rloc & 15)) * 16));
        const int owner = grow / tp.rows_per_rank;
        __nv_bfloat16* dst = tp.c_dst[owner] +
                             static_cast<long long>(grow - owner * tp.rows_per_rank) * p.ldc + ccol;
        *reinterpret_cast<uint4*>(dst) = u;
      }
    }
    __syncwarp();
  }
}

}  // namespace t5x
