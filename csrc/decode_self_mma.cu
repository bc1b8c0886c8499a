// Decode-step self attention on the tensor cores, one CTA per (example, head).
//
// The cache is never reordered: beam j writes the key / value of the position it decodes into
// its own slot, and `ancestry[b][j][t]` names the slot that holds beam j's history at position
// t. Seen from one example, the beams are the rows of a small query matrix and every
// (slot, position) pair is a key; beam j may attend to key (s, t) iff t < cur and
// ancestry[b][j][t] == s, or t == cur and s == j (its own new key). So the kernel multiplies
// the [beams x 64] queries with ALL cached keys of the example (every cache row is read once,
// whatever the beams share) and masks what a beam does not own: the operand layouts, the
// permuted channel / key order and the transposed value cache are those of the cross-attention
// kernel (decode_cross_mma.cu), which explains them.
//
//   keys    cache_k  [B, beams, H, Lc, 64]   Lc = cache length, a multiple of 32
//   values  cache_vt [B, beams, H, 64, Lc]   transposed: one key position is a column
//
// The new key row is stored as it comes; the new value is scattered into its column (64
// two-byte stores per beam and head), which costs about a tenth of the bytes the step reads.
// Both are written by this CTA before it reads the cache; the T5 relative-position bias is one
// [H, Lc] row prepared once per step.
#include "common.cuh"
#include "t5x_b200.h"

namespace t5x {
namespace {

constexpr int kSmWarps = 8;
constexpr int kSmThreads = kSmWarps * 32;
constexpr int kSmMaxChunksPerWarp = 4;   // 32-key chunks per warp
constexpr int kSmMaxLen = 1024;

__device__ __forceinline__ void sm_mma(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0,
                                       uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t sm_pack2(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}

// position of column n of score tile (half u, tile) within a 32-position chunk
__device__ __forceinline__ int sm_pos_of_column(int u, int tile, int n) {
  return 8 * (n >> 1) + 4 * u + 2 * tile + (n & 1);
}

template <int BEAMS>
__global__ void __launch_bounds__(kSmThreads, 2)
    decode_self_mma_kernel(const __nv_bfloat16* __restrict__ q,      // [B*beams, H, 64], stride in_ld
                           const __nv_bfloat16* __restrict__ k_new,  // same layout
                           const __nv_bfloat16* __restrict__ v_new,
                           __nv_bfloat16* cache_k,                   // [B, beams, H, Lc, 64]
                           __nv_bfloat16* cache_vt,                  // [B, beams, H, 64, Lc]
                           const int* __restrict__ ancestry,         // [B, beams, L]
                           const float* __restrict__ bias_row,       // [H, L] or null
                           const int* __restrict__ cur_index,
                           __nv_bfloat16* __restrict__ out,          // [B*beams, H, 64]
                           long long in_ld, int H, int L, int Lc) {
  // positions per beam are bounded by the chunk budget: beams * ceil(L / 32) <= 32 chunks
  constexpr int kAncStride = kSmWarps * kSmMaxChunksPerWarp * 32 / BEAMS;
  __shared__ int s_anc[kSmWarps * kSmMaxChunksPerWarp * 32];
  __shared__ float s_max[kSmWarps][8];
  __shared__ float s_sum[kSmWarps][8];
  __shared__ float s_out[kSmWarps][8][64];
  const int b = blockIdx.x / H, h = blockIdx.x - b * H;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int cur = min(max(*cur_index, 0), L - 1);
  const long long slot_k = static_cast<long long>(H) * Lc * 64;  // elements between slots
  __nv_bfloat16* kb = cache_k + (static_cast<long long>(b) * BEAMS * H + h) * Lc * 64;
  __nv_bfloat16* vb = cache_vt + (static_cast<long long>(b) * BEAMS * H + h) * 64 * Lc;

  // ---- append this step's key rows and value columns; stage the ancestry table ----
  if (tid < BEAMS * 8) {  // 16 bytes of one beam's key row
    const int j = tid >> 3, part = tid & 7;
    const uint4 kn = reinterpret_cast<const uint4*>(
        k_new + (static_cast<long long>(b) * BEAMS + j) * in_ld + h * 64)[part];
    reinterpret_cast<uint4*>(kb + j * slot_k + static_cast<long long>(cur) * 64)[part] = kn;
  }
  for (int i = tid; i < BEAMS * 64; i += kSmThreads) {
    const int j = i >> 6, ch = i & 63;
    vb[j * slot_k + static_cast<long long>(ch) * Lc + cur] =
        v_new[(static_cast<long long>(b) * BEAMS + j) * in_ld + h * 64 + ch];
  }
  const int npos = cur + 1;
  for (int i = tid; i < BEAMS * npos; i += kSmThreads) {
    const int j = i / npos, p = i - j * npos;
    s_anc[j * kAncStride + p] = ancestry[(static_cast<long long>(b) * BEAMS + j) * L + p];
  }
  // A operand: this lane's 16 channels of beam g
  uint32_t qa[8];
#pragma unroll
  for (int r = 0; r < 8; ++r) qa[r] = 0u;
  if (g < BEAMS) {
    const uint4* src = reinterpret_cast<const uint4*>(
        q + (static_cast<long long>(b) * BEAMS + g) * in_ld + h * 64 + 16 * t);
    const uint4 lo = src[0], hi = src[1];
    qa[0] = lo.x, qa[1] = lo.y, qa[2] = lo.z, qa[3] = lo.w;
    qa[4] = hi.x, qa[5] = hi.y, qa[6] = hi.z, qa[7] = hi.w;
  }
  __syncthreads();  // the appended rows / columns are visible to the whole CTA

  // ---- scores: (slot, 32-position chunk) pairs dealt to the warps round robin ----
  const int pos_chunks = cur / 32 + 1;
  const int nchunks = BEAMS * pos_chunks;
  float sc[kSmMaxChunksPerWarp][2][4];
  float mx = -3.0e38f;
  const float* bias = bias_row == nullptr ? nullptr : bias_row + static_cast<long long>(h) * L;
#pragma unroll
  for (int i = 0; i < kSmMaxChunksPerWarp; ++i) {
    const int chunk = warp + i * kSmWarps;
    if (chunk >= nchunks) break;
    const int s = chunk / pos_chunks, base = (chunk - s * pos_chunks) * 32;
    const __nv_bfloat16* ks = kb + s * slot_k;
    uint4 kr[4][2];
#pragma unroll
    for (int ut = 0; ut < 4; ++ut) {
      const int pos = base + sm_pos_of_column(ut >> 1, ut & 1, g);
      const uint4* src = reinterpret_cast<const uint4*>(ks + static_cast<long long>(pos) * 64 + 16 * t);
      kr[ut][0] = src[0];
      kr[ut][1] = src[1];
    }
#pragma unroll
    for (int ut = 0; ut < 4; ++ut) {
      const int u = ut >> 1, tile = ut & 1;
      const uint4 lo = kr[ut][0], hi = kr[ut][1];
      const uint32_t r[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
      float c4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int st = 0; st < 4; ++st) sm_mma(c4, qa[2 * st], qa[2 * st + 1], r[2 * st], r[2 * st + 1]);
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int pos = base + sm_pos_of_column(u, tile, 2 * t + e);
        // beam g owns key (s, pos) iff its history at pos lives in slot s
        bool mine = false;
        if (g < BEAMS && pos <= cur)
          mine = pos == cur ? (s == g) : (s_anc[(g < BEAMS ? g : 0) * kAncStride + pos] == s);
        float v = -3.0e38f;
        if (mine) {
          v = c4[e] + (bias != nullptr ? bias[pos] : 0.f);
          mx = fmaxf(mx, v);
        }
        sc[i][u][2 * tile + e] = v;
      }
    }
  }
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
  if (t == 0) s_max[warp][g] = mx;
  __syncthreads();
  mx = s_max[0][g];
#pragma unroll
  for (int w = 1; w < kSmWarps; ++w) mx = fmaxf(mx, s_max[w][g]);

  // ---- probabilities and the value product ----
  float acc[8][4];
#pragma unroll
  for (int n = 0; n < 8; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[n][e] = 0.f;
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kSmMaxChunksPerWarp; ++i) {
    const int chunk = warp + i * kSmWarps;
    if (chunk >= nchunks) break;
    const int s = chunk / pos_chunks, base = (chunk - s * pos_chunks) * 32;
    const __nv_bfloat16* vs = vb + s * slot_k;
    uint4 vv[8];
#pragma unroll
    for (int n = 0; n < 8; ++n)
      vv[n] = *reinterpret_cast<const uint4*>(vs + static_cast<long long>(n * 8 + g) * Lc + base + 8 * t);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      float pr[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        // keys a beam does not own have weight exactly zero (also when the beam owns nothing
        // in this warp's chunks and mx is still the sentinel)
        pr[e] = sc[i][u][e] > -1.0e38f ? __expf(sc[i][u][e] - mx) : 0.f;
        sum += pr[e];
      }
      const uint32_t pa0 = sm_pack2(pr[0], pr[1]), pa2 = sm_pack2(pr[2], pr[3]);
#pragma unroll
      for (int n = 0; n < 8; ++n)
        sm_mma(acc[n], pa0, pa2, u == 0 ? vv[n].x : vv[n].z, u == 0 ? vv[n].y : vv[n].w);
    }
  }
  sum += __shfl_xor_sync(0xffffffffu, sum, 1);
  sum += __shfl_xor_sync(0xffffffffu, sum, 2);
  if (t == 0) s_sum[warp][g] = sum;
#pragma unroll
  for (int n = 0; n < 8; ++n) {
    s_out[warp][g][8 * n + 2 * t] = acc[n][0];
    s_out[warp][g][8 * n + 2 * t + 1] = acc[n][1];
  }
  __syncthreads();
  for (int i = tid; i < BEAMS * 64; i += kSmThreads) {
    const int j = i >> 6, d = i & 63;
    float tot = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < kSmWarps; ++w) {
      tot += s_out[w][j][d];
      den += s_sum[w][j];
    }
    out[((static_cast<long long>(b) * BEAMS + j) * H + h) * 64 + d] = __float2bfloat16(tot / den);
  }
}

}  // namespace
}  // namespace t5x

using namespace t5x;

// q, k_new, v_new: [batch * beams, heads, 64] bf16 with row stride in_ld; cache_k: [batch,
// beams, heads, Lc, 64]; cache_vt: [batch, beams, heads, 64, Lc] (values transposed), both
// zero-initialised, Lc a multiple of 32 and >= max_len; ancestry: [batch, beams, max_len]
// int32; bias_row: [heads, max_len] fp32 or null; cur_index: device int32. beams in
// {1, 2, 4, 8} with beams * ceil(max_len / 32) <= 32 chunks.
T5X_API int t5x_decode_self_attention_mma(const void* q, const void* k_new, const void* v_new,
                                          void* cache_k, void* cache_vt, const void* ancestry,
                                          const void* bias_row, const void* cur_index, void* out,
                                          long long in_ld, int batch, int beams, int heads,
                                          int head_dim, int max_len, int cache_len, void* stream) {
  if (batch <= 0) return 0;
  if (head_dim != 64) return set_error("decode_self_attention_mma: head_dim must be 64");
  if (max_len < 1 || max_len > kSmMaxLen || cache_len < max_len || cache_len % 32)
    return set_error("decode_self_attention_mma: need 1 <= max_len <= cache_len, cache_len %% 32 == 0");
  if (beams * ((max_len + 31) / 32) > kSmWarps * kSmMaxChunksPerWarp)
    return set_error("decode_self_attention_mma: beams x positions beyond %d chunks",
                     kSmWarps * kSmMaxChunksPerWarp);
  if (in_ld % 8) return set_error("decode_self_attention_mma: input row stride must be a multiple of 8");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid(batch * heads);
#define T5X_LAUNCH_SELF_MMA(B_)                                                                   \
  decode_self_mma_kernel<B_><<<grid, kSmThreads, 0, st>>>(                                        \
      static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k_new),            \
      static_cast<const __nv_bfloat16*>(v_new), static_cast<__nv_bfloat16*>(cache_k),            \
      static_cast<__nv_bfloat16*>(cache_vt), static_cast<const int*>(ancestry),                  \
      static_cast<const float*>(bias_row), static_cast<const int*>(cur_index),                   \
      static_cast<__nv_bfloat16*>(out), in_ld, heads, max_len, cache_len)
  switch (beams) {
    case 1: T5X_LAUNCH_SELF_MMA(1); break;
    case 2: T5X_LAUNCH_SELF_MMA(2); break;
    case 4: T5X_LAUNCH_SELF_MMA(4); break;
    case 8: T5X_LAUNCH_SELF_MMA(8); break;
    default:
      return set_error("decode_self_attention_mma: beams must be 1, 2, 4 or 8 (got %d)", beams);
  }
#undef T5X_LAUNCH_SELF_MMA
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("decode_self_attention_mma: %s", cudaGetErrorString(e));
  return 0;
}
