// Attention kernels of the autoregressive decode step (one new token per row).
//
// decode_self_attention: each (batch, beam) row attends over that beam's key/value history.
// The cache is written once per step and never reordered: row (b, j) stores the key/value it
// computed at position t in cache[b][j][t], and `ancestry[b][j][t]` names the slot that holds
// beam j's key/value for position t (beam search rewrites the small ancestry table when beams
// are reselected, instead of gathering every layer's cache). Fused in one launch: the cache
// write of the new key/value, the T5 relative-position bias (a [heads, max_len] row prepared
// once per step), the softmax and the value sum. One warp per (row, head).
//
// decode_cross_attention: the `beams` rows of one example attend over that example's encoder
// keys/values, stored once per example. One CTA per (example, head): every key / value row is
// read once and used for all beams.
//
// Memory layout of the work, both kernels (head_dim = 64, bf16): 8 adjacent lanes read one
// 128-byte key or value row with one 16-byte load each, so a warp instruction fetches four
// rows; partial dot products are combined with three shuffles, partial value sums with two.
#include "common.cuh"
#include "t5x_b200.h"

namespace t5x {

constexpr int kDecHeadDim = 64;
constexpr int kDecWarps = 4;
constexpr int kDecMaxLen = 1024;  // probabilities of one row are staged in shared memory

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 t = __bfloat1622float2(p2[e]);
    f[2 * e] = t.x;
    f[2 * e + 1] = t.y;
  }
}
__device__ __forceinline__ float sum_over_row_lanes(float x) {  // the 8 lanes of one row
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  x += __shfl_xor_sync(0xffffffffu, x, 4);
  return x;
}
__device__ __forceinline__ float sum_over_row_groups(float x) {  // the 4 row groups of a warp
  x += __shfl_xor_sync(0xffffffffu, x, 8);
  x += __shfl_xor_sync(0xffffffffu, x, 16);
  return x;
}

__global__ void __launch_bounds__(kDecWarps * 32)
    decode_self_attention_kernel(const __nv_bfloat16* __restrict__ q,      // [rows, H, 64]
                                 const __nv_bfloat16* __restrict__ k_new,  // [rows, H, 64]
                                 const __nv_bfloat16* __restrict__ v_new,
                                 __nv_bfloat16* __restrict__ cache_k,  // [B, beams, H, L, 64]
                                 __nv_bfloat16* __restrict__ cache_v,
                                 const int* __restrict__ ancestry,     // [B, beams, L]
                                 const float* __restrict__ bias_row,   // [H, L] or null
                                 const int* __restrict__ cur_index,    // device scalar
                                 __nv_bfloat16* __restrict__ out,      // [rows, H, 64]
                                 long long in_ld,  // row stride of q / k_new / v_new (elements)
                                 int rows, int beams, int H, int L) {
  __shared__ float sprob[kDecWarps][kDecMaxLen];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int item = blockIdx.x * kDecWarps + warp;  // (row, head)
  chain_release();
  chain_wait();  // q / k / v, the ancestry table and the position come from earlier kernels
  if (item >= rows * H) return;
  const int row = item / H, h = item - row * H;
  const int b = row / beams;
  const int cur = min(max(*cur_index, 0), L - 1);
  const int g = lane >> 3, part = lane & 7;
  const long long rh = static_cast<long long>(row) * in_ld + h * kDecHeadDim;  // inputs
  const long long oh = (static_cast<long long>(row) * H + h) * kDecHeadDim;   // output
  // cache layout [B, beams, H, L, 64]: the history of one (slot, head) is contiguous
  const long long tstride = kDecHeadDim;
  const long long slot_stride = static_cast<long long>(H) * L * kDecHeadDim;
  const long long batch_base = static_cast<long long>(b) * beams * slot_stride +
                               static_cast<long long>(h) * L * kDecHeadDim;
  const int* anc = ancestry + static_cast<long long>(row) * L;

  // 1. this step's query / key / value (8 dims per lane); append key / value at position
  //    `cur` of the row's own slot
  const uint4 qu = reinterpret_cast<const uint4*>(q + rh)[part];
  const uint4 kn = reinterpret_cast<const uint4*>(k_new + rh)[part];
  const uint4 vn = reinterpret_cast<const uint4*>(v_new + rh)[part];
  if (g == 0) {
    const long long dst = batch_base + (row - b * beams) * slot_stride + cur * tstride;
    reinterpret_cast<uint4*>(cache_k + dst)[part] = kn;
    reinterpret_cast<uint4*>(cache_v + dst)[part] = vn;
  }
  float qf[8];
  unpack8(qu, qf);

  // 2. scores over positions 0..cur (no 1/sqrt(d): T5 folds it into the query init)
  float mx = -INFINITY;
  constexpr int kU = 4;  // positions in flight per lane group
  for (int t0 = 0; t0 <= cur; t0 += 4 * kU) {
    uint4 ku[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int t = t0 + u * 4 + g;
      ku[u] = kn;
      if (t < cur)
        ku[u] = reinterpret_cast<const uint4*>(cache_k + batch_base + anc[t] * slot_stride +
                                               t * tstride)[part];
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int t = t0 + u * 4 + g;
      float kf[8];
      unpack8(ku[u], kf);
      float s = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) s = fmaf(qf[e], kf[e], s);
      s = sum_over_row_lanes(s);
      if (t <= cur) {
        if (bias_row != nullptr) s += bias_row[static_cast<long long>(h) * L + t];
        if (part == 0) sprob[warp][t] = s;
        mx = fmaxf(mx, s);
      }
    }
  }
  mx = warp_max(mx);
  __syncwarp();
  float sum = 0.f;
  for (int t = lane; t <= cur; t += 32) {
    const float e = __expf(sprob[warp][t] - mx);
    sprob[warp][t] = e;
    sum += e;
  }
  sum = warp_sum(sum);
  __syncwarp();

  // 3. out = sum_t p_t * V[t]; lane accumulates its 8 dims over its row group's positions
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  for (int t0 = 0; t0 <= cur; t0 += 4 * kU) {
    uint4 vu[kU];
    float pt[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int t = t0 + u * 4 + g;
      pt[u] = 0.f;
      vu[u] = vn;
      if (t <= cur) {
        pt[u] = sprob[warp][t];
        if (t < cur)
          vu[u] = reinterpret_cast<const uint4*>(cache_v + batch_base + anc[t] * slot_stride +
                                                 t * tstride)[part];
      }
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      float vf[8];
      unpack8(vu[u], vf);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = fmaf(pt[u], vf[e], acc[e]);
    }
  }
  const float inv = 1.f / sum;
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = sum_over_row_groups(acc[e]) * inv;
  if (g == 0) {
    uint4 o;
    __nv_bfloat162 p0 = __floats2bfloat162_rn(acc[0], acc[1]);
    __nv_bfloat162 p1 = __floats2bfloat162_rn(acc[2], acc[3]);
    __nv_bfloat162 p2 = __floats2bfloat162_rn(acc[4], acc[5]);
    __nv_bfloat162 p3 = __floats2bfloat162_rn(acc[6], acc[7]);
    o.x = *reinterpret_cast<uint32_t*>(&p0);
    o.y = *reinterpret_cast<uint32_t*>(&p1);
    o.z = *reinterpret_cast<uint32_t*>(&p2);
    o.w = *reinterpret_cast<uint32_t*>(&p3);
    reinterpret_cast<uint4*>(out + oh)[part] = o;
  }
}

constexpr int kCrossWarps = 8;
constexpr int kCrossThreads = kCrossWarps * 32;
constexpr int kCrossMaxKeys = 1024;

template <int BEAMS>
__global__ void __launch_bounds__(kCrossThreads, BEAMS <= 4 ? 4 : 2)
    decode_cross_attention_kernel(const __nv_bfloat16* __restrict__ q,  // [B*beams, H, 64]
                                  const __nv_bfloat16* __restrict__ k,  // [B, H, Lk, 64]
                                  const __nv_bfloat16* __restrict__ v,
                                  const uint8_t* __restrict__ key_mask,  // [B, Lk] or null
                                  __nv_bfloat16* __restrict__ out,       // [B*beams, H, 64]
                                  long long q_ld, int H, int Lk) {
  __shared__ float sp[BEAMS][kCrossMaxKeys];
  __shared__ float sred[BEAMS][kCrossWarps];
  // per-warp partial outputs reuse the probability buffer once every warp is done with it
  float (*sout)[BEAMS][kDecHeadDim] = reinterpret_cast<float (*)[BEAMS][kDecHeadDim]>(&sp[0][0]);
  static_assert(kCrossWarps * kDecHeadDim <= kCrossMaxKeys, "sout must fit in sp");
  const int b = blockIdx.x / H, h = blockIdx.x - b * H;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 3, part = lane & 7;
  constexpr int kRowsPerIter = kCrossWarps * 4;
  float qf[BEAMS][8];
#pragma unroll
  for (int j = 0; j < BEAMS; ++j) {
    const uint4 qu = reinterpret_cast<const uint4*>(
        q + (static_cast<long long>(b) * BEAMS + j) * q_ld + h * kDecHeadDim)[part];
    unpack8(qu, qf[j]);
  }
  // key / value layout [B, H, Lk, 64]: one (example, head) is a contiguous 128 * Lk bytes
  const long long kv_stride = kDecHeadDim;
  const long long kv_base = (static_cast<long long>(b) * H + h) * Lk * kDecHeadDim;
  const uint8_t* km = key_mask == nullptr ? nullptr : key_mask + static_cast<long long>(b) * Lk;

  // scores
  float mx[BEAMS];
#pragma unroll
  for (int j = 0; j < BEAMS; ++j) mx[j] = -INFINITY;
  constexpr int kU = 4;  // key rows in flight per lane group
  for (int t0 = 0; t0 < Lk; t0 += kU * kRowsPerIter) {
    uint4 ku[kU];
    int tt[kU];
    bool valid[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      tt[u] = t0 + u * kRowsPerIter + warp * 4 + g;
      valid[u] = tt[u] < Lk && (km == nullptr || km[tt[u]] != 0);
      ku[u] = make_uint4(0, 0, 0, 0);
      if (valid[u]) ku[u] = reinterpret_cast<const uint4*>(k + kv_base + tt[u] * kv_stride)[part];
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      float kf[8];
      unpack8(ku[u], kf);
#pragma unroll
      for (int j = 0; j < BEAMS; ++j) {
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) s = fmaf(qf[j][e], kf[e], s);
        float sv = sum_over_row_lanes(s);
        if (tt[u] < Lk) {
          if (!valid[u]) sv = -1e10f;  // additive mask value of the reference
          if (part == 0) sp[j][tt[u]] = sv;
          mx[j] = fmaxf(mx[j], sv);
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < BEAMS; ++j) {
    const float m = warp_max(mx[j]);
    if (lane == 0) sred[j][warp] = m;
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < BEAMS; ++j) {
    float m = sred[j][0];
#pragma unroll
    for (int w = 1; w < kCrossWarps; ++w) m = fmaxf(m, sred[j][w]);
    mx[j] = m;
  }
  __syncthreads();
  float sum[BEAMS];
#pragma unroll
  for (int j = 0; j < BEAMS; ++j) sum[j] = 0.f;
  for (int t = tid; t < Lk; t += kCrossThreads) {
#pragma unroll
    for (int j = 0; j < BEAMS; ++j) {
      const float e = __expf(sp[j][t] - mx[j]);
      sp[j][t] = e;
      sum[j] += e;
    }
  }
#pragma unroll
  for (int j = 0; j < BEAMS; ++j) {
    const float sj = warp_sum(sum[j]);
    if (lane == 0) sred[j][warp] = sj;
  }
  __syncthreads();

  // values
  float acc[BEAMS][8];
#pragma unroll
  for (int j = 0; j < BEAMS; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[j][e] = 0.f;
  for (int t0 = 0; t0 < Lk; t0 += kU * kRowsPerIter) {
    uint4 vu[kU];
    int tt[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      tt[u] = t0 + u * kRowsPerIter + warp * 4 + g;
      vu[u] = make_uint4(0, 0, 0, 0);
      if (tt[u] < Lk) vu[u] = reinterpret_cast<const uint4*>(v + kv_base + tt[u] * kv_stride)[part];
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      if (tt[u] < Lk) {
        float vf[8];
        unpack8(vu[u], vf);
#pragma unroll
        for (int j = 0; j < BEAMS; ++j) {
          const float pt = sp[j][tt[u]];
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[j][e] = fmaf(pt, vf[e], acc[j][e]);
        }
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < BEAMS; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float tot = sum_over_row_groups(acc[j][e]);
      if (g == 0) sout[warp][j][part * 8 + e] = tot;
    }
  __syncthreads();
  for (int i = tid; i < BEAMS * kDecHeadDim; i += kCrossThreads) {
    const int j = i / kDecHeadDim, d = i - j * kDecHeadDim;
    float tot = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < kCrossWarps; ++w) {
      tot += sout[w][j][d];
      den += sred[j][w];
    }
    out[((static_cast<long long>(b) * BEAMS + j) * H + h) * kDecHeadDim + d] =
        __float2bfloat16(tot / den);
  }
}

}  // namespace t5x

using namespace t5x;

// q, k_new, v_new: [rows, heads, 64] bf16 with row stride `in_ld` elements (views into one
// fused projection are fine; 16-byte aligned), out: [rows, heads, 64] contiguous; rows =
// batch * beams; cache_k / cache_v: [batch, beams, heads, max_len, 64] bf16; ancestry:
// [batch, beams, max_len] int32; bias_row: [heads, max_len] fp32 or null; cur_index: device
// int32 (position being decoded).
T5X_API int t5x_decode_self_attention(const void* q, const void* k_new, const void* v_new,
                                      void* cache_k, void* cache_v, const void* ancestry,
                                      const void* bias_row, const void* cur_index, void* out,
                                      long long in_ld, int rows, int beams, int heads,
                                      int head_dim, int max_len, void* stream) {
  if (rows <= 0) return 0;
  if (head_dim != kDecHeadDim) return set_error("decode_self_attention: head_dim must be 64");
  if (max_len > kDecMaxLen) return set_error("decode_self_attention: max_len > %d", kDecMaxLen);
  if (beams <= 0 || rows % beams) return set_error("decode_self_attention: rows %% beams != 0");
  if (in_ld % 8) return set_error("decode_self_attention: input row stride must be a multiple of 8");
  const int items = rows * heads;
  cudaError_t e = launch_chained(
      decode_self_attention_kernel, dim3((items + kDecWarps - 1) / kDecWarps), dim3(kDecWarps * 32),
      0, static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(q),
      static_cast<const __nv_bfloat16*>(k_new), static_cast<const __nv_bfloat16*>(v_new),
      static_cast<__nv_bfloat16*>(cache_k), static_cast<__nv_bfloat16*>(cache_v),
      static_cast<const int*>(ancestry), static_cast<const float*>(bias_row),
      static_cast<const int*>(cur_index), static_cast<__nv_bfloat16*>(out), in_ld, rows, beams,
      heads, max_len);
  count_launches(1);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("decode_self_attention: %s", cudaGetErrorString(e));
  return 0;
}

// q: [batch * beams, heads, 64] bf16 with row stride q_ld; k, v: [batch, heads, Lk, 64] bf16
// contiguous; key_mask: [batch, Lk] uint8 (0 = padding) or null; out: [batch * beams, heads, 64].
// beams must be 1, 2, 4 or 8.
T5X_API int t5x_decode_cross_attention(const void* q, const void* k, const void* v,
                                       const void* key_mask, void* out, long long q_ld, int batch,
                                       int beams, int heads, int head_dim, int Lk, void* stream) {
  if (batch <= 0) return 0;
  if (head_dim != kDecHeadDim) return set_error("decode_cross_attention: head_dim must be 64");
  if (Lk < 1 || Lk > kCrossMaxKeys)
    return set_error("decode_cross_attention: Lk must be in [1, %d]", kCrossMaxKeys);
  if (q_ld % 8) return set_error("decode_cross_attention: q row stride must be a multiple of 8");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid(batch * heads);
  auto qp = static_cast<const __nv_bfloat16*>(q);
  auto kp = static_cast<const __nv_bfloat16*>(k);
  auto vp = static_cast<const __nv_bfloat16*>(v);
  auto mp = static_cast<const uint8_t*>(key_mask);
  auto op = static_cast<__nv_bfloat16*>(out);
  switch (beams) {
    case 1:
      decode_cross_attention_kernel<1><<<grid, kCrossThreads, 0, st>>>(qp, kp, vp, mp, op, q_ld, heads, Lk);
      break;
    case 2:
      decode_cross_attention_kernel<2><<<grid, kCrossThreads, 0, st>>>(qp, kp, vp, mp, op, q_ld, heads, Lk);
      break;
    case 4:
      decode_cross_attention_kernel<4><<<grid, kCrossThreads, 0, st>>>(qp, kp, vp, mp, op, q_ld, heads, Lk);
      break;
    case 8:
      decode_cross_attention_kernel<8><<<grid, kCrossThreads, 0, st>>>(qp, kp, vp, mp, op, q_ld, heads, Lk);
      break;
    default:
      return set_error("decode_cross_attention: beams must be 1, 2, 4 or 8 (got %d)", beams);
  }
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("decode_cross_attention: %s", cudaGetErrorString(e));
  return 0;
}
