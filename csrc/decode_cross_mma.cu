// Decode-step cross attention on the tensor cores: the `beams` query rows of one example
// against that example's encoder keys and values, one CTA per (example, head).
//
// The work is a [beams x 64] x [64 x Lk] product, a softmax over Lk and a [beams x Lk] x
// [Lk x 64] product, with beams <= 8: far too few rows for a tcgen05 tile (64 or 128 rows of one
// operand), and the CUDA-core form spends its time in shuffles and scalar FMAs instead of
// waiting for memory. `mma.sync.m16n8k16` fits: rows 0..beams-1 of the 16-row A operand are the
// beams, the rest is zero, and one warp instruction covers 8 keys x 16 channels.
//
// Loads are arranged so that every lane reads whole 16- or 8-byte pieces straight from global
// memory into the registers the MMA wants, with no shared-memory staging:
//   * a dot product does not care in which order its terms are added, so the channel index is
//     permuted: lane (g, t) (g = lane / 4, t = lane % 4) holds channels 16t .. 16t+15 of "its"
//     key row (two 16-byte loads) and of its beam's query, and MMA step s uses channels
//     16t + 4s .. 16t + 4s + 3 as its k positions {2t, 2t+1, 2t+8, 2t+9};
//   * which key sits in which column of a score tile is free too: a chunk of 32 keys is four
//     score tiles (half u = 0, 1; tile = 0, 1), and column n of tile (u, tile) holds key
//     8(n/2) + 4u + 2 tile + n%2, so the four probabilities that lane t carries into the second
//     product of half u (k positions 2t, 2t+1, 2t+8, 2t+9) belong to the adjacent keys
//     8t + 4u .. 8t + 4u + 3;
//   * the values are stored transposed ([example, head, channel, key]), so the eight keys
//     8t .. 8t+7 of channel g are one 16-byte load: a warp instruction reads 64 contiguous
//     bytes of each of 8 channel rows.
// Key rows are requested two chunks (64 keys) ahead of their use, so that enough bytes are in
// flight. Scores stay in registers between the two products (Lk <=
// 1024: 32 values per lane), the row
// maximum and sum cross the eight warps through shared memory, and the partial outputs of the
// warps are added there at the end. Masked keys take the additive -1e10 of the reference.
#include "common.cuh"
#include "t5x_b200.h"

namespace t5x {
namespace {

constexpr int kXmWarps = 8;
constexpr int kXmThreads = kXmWarps * 32;
constexpr int kXmMaxKeys = 1024;
constexpr int kXmMaxChunks = kXmMaxKeys / 32 / kXmWarps;  // 32-key chunks per warp
constexpr float kXmMasked = -1e10f;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}

// key of column n of score tile (half u, tile) within a 32-key chunk
__device__ __forceinline__ int key_of_column(int u, int tile, int n) {
  return 8 * (n >> 1) + 4 * u + 2 * tile + (n & 1);
}

template <int BEAMS>
__global__ void __launch_bounds__(kXmThreads)
    decode_cross_mma_kernel(const __nv_bfloat16* __restrict__ q,   // [B*beams, H, 64], row stride q_ld
                            const __nv_bfloat16* __restrict__ k,   // [B, H, Lp, 64]
                            const __nv_bfloat16* __restrict__ vt,  // [B, H, 64, Lp]
                            const uint8_t* __restrict__ key_mask,  // [B, Lk] or null
                            __nv_bfloat16* __restrict__ out,       // [B*beams, H, 64]
                            long long q_ld, int H, int Lk, int Lp) {
  __shared__ float s_max[kXmWarps][8];
  __shared__ float s_sum[kXmWarps][8];
  __shared__ float s_out[kXmWarps][8][64];
  const int b = blockIdx.x / H, h = blockIdx.x - b * H;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const long long bh = static_cast<long long>(b) * H + h;
  const __nv_bfloat16* kb = k + bh * Lp * 64;
  const __nv_bfloat16* vb = vt + bh * 64 * Lp;
  const uint8_t* km = key_mask == nullptr ? nullptr : key_mask + static_cast<long long>(b) * Lk;

  // Keys and values are encoder products, constant while decoding: this CTA's part of them is
  // pulled toward L2 while the kernel before this one (which produces q) may still be running.
  chain_release();
  for (int line = threadIdx.x; line < Lp; line += kXmThreads) {  // Lp x 128 bytes each
    prefetch_l2(reinterpret_cast<const char*>(kb) + static_cast<long long>(line) * 128);
    prefetch_l2(reinterpret_cast<const char*>(vb) + static_cast<long long>(line) * 128);
  }
  chain_wait();

  // A operand of the score product: this lane's 16 channels of beam g (zero rows beyond the beams)
  uint32_t qa[8];
#pragma unroll
  for (int r = 0; r < 8; ++r) qa[r] = 0u;
  if (g < BEAMS) {
    const uint4* src = reinterpret_cast<const uint4*>(
        q + (static_cast<long long>(b) * BEAMS + g) * q_ld + h * 64 + 16 * t);
    const uint4 lo = src[0], hi = src[1];
    qa[0] = lo.x, qa[1] = lo.y, qa[2] = lo.z, qa[3] = lo.w;
    qa[4] = hi.x, qa[5] = hi.y, qa[6] = hi.z, qa[7] = hi.w;
  }

  // ---- scores: chunks of 32 keys; every warp takes a contiguous run of chunks ----
  const int nchunks = Lp / 32;
  const int per_warp = (nchunks + kXmWarps - 1) / kXmWarps;
  const int first = warp * per_warp;
  const int mine = max(0, min(per_warp, nchunks - first));
  float sc[kXmMaxChunks][2][4];  // [chunk][half]: tile 0 columns (2t, 2t+1), tile 1 columns (2t, 2t+1)
  float mx = -3.0e38f;
  constexpr int kBatch = 2;  // chunks whose key rows are requested before any is used
#pragma unroll
  for (int i0 = 0; i0 < kXmMaxChunks; i0 += kBatch) {
    if (i0 >= mine) break;
    uint4 kr[kBatch][4][2];
#pragma unroll
    for (int c = 0; c < kBatch; ++c) {
      const int base = (first + min(i0 + c, mine - 1)) * 32;
#pragma unroll
      for (int ut = 0; ut < 4; ++ut) {
        const int key = base + key_of_column(ut >> 1, ut & 1, g);  // the row this lane group loads
        const uint4* src =
            reinterpret_cast<const uint4*>(kb + static_cast<long long>(key) * 64 + 16 * t);
        kr[c][ut][0] = src[0];
        kr[c][ut][1] = src[1];
      }
    }
#pragma unroll
    for (int c = 0; c < kBatch; ++c) {
      const int i = i0 + c;
      if (i >= mine) break;
      const int base = (first + i) * 32;
#pragma unroll
      for (int ut = 0; ut < 4; ++ut) {
        const int u = ut >> 1, tile = ut & 1;
        const uint4 lo = kr[c][ut][0], hi = kr[c][ut][1];
        const uint32_t r[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        float acc4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int s_ = 0; s_ < 4; ++s_)
          mma_bf16_16816(acc4, qa[2 * s_], 0u, qa[2 * s_ + 1], 0u, r[2 * s_], r[2 * s_ + 1]);
        // acc4[0], acc4[1]: beam g, columns 2t and 2t+1 of this tile
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int kk = base + key_of_column(u, tile, 2 * t + e);
          float v = acc4[e];
          const bool exists = kk < Lk;
          if (exists && km != nullptr && km[kk] == 0) v = kXmMasked;
          if (!exists) v = -3.0e38f;  // padding of the key range: weight exactly zero
          sc[i][u][2 * tile + e] = v;
          if (exists) mx = fmaxf(mx, v);
        }
      }
    }
  }
  // row maximum: over the four lanes of a row, then over the warps
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
  if (t == 0) s_max[warp][g] = mx;
  __syncthreads();
  mx = s_max[0][g];
#pragma unroll
  for (int w = 1; w < kXmWarps; ++w) mx = fmaxf(mx, s_max[w][g]);

  // ---- probabilities and the value product ----
  float acc[8][4];
#pragma unroll
  for (int n = 0; n < 8; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[n][e] = 0.f;
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kXmMaxChunks; ++i) {
    if (i >= mine) break;
    const int base = (first + i) * 32;
    uint4 vv[8];
#pragma unroll
    for (int n = 0; n < 8; ++n)
      vv[n] = *reinterpret_cast<const uint4*>(
          vb + static_cast<long long>(n * 8 + g) * Lp + base + 8 * t);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      float pr[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        pr[e] = __expf(sc[i][u][e] - mx);
        sum += pr[e];
      }
      // A operand of half u: k positions (2t, 2t+1) <- tile 0, (2t+8, 2t+9) <- tile 1, i.e. keys
      // base + 8t + 4u .. + 3: the low (u = 0) or high (u = 1) half of the 16 bytes loaded
      const uint32_t pa0 = pack2(pr[0], pr[1]), pa2 = pack2(pr[2], pr[3]);
#pragma unroll
      for (int n = 0; n < 8; ++n)
        mma_bf16_16816(acc[n], pa0, 0u, pa2, 0u, u == 0 ? vv[n].x : vv[n].z,
                       u == 0 ? vv[n].y : vv[n].w);
    }
  }
  sum += __shfl_xor_sync(0xffffffffu, sum, 1);
  sum += __shfl_xor_sync(0xffffffffu, sum, 2);
  if (t == 0) s_sum[warp][g] = sum;
  // acc[n][0], acc[n][1]: beam g, channels 8n + 2t, 8n + 2t + 1
#pragma unroll
  for (int n = 0; n < 8; ++n) {
    s_out[warp][g][8 * n + 2 * t] = acc[n][0];
    s_out[warp][g][8 * n + 2 * t + 1] = acc[n][1];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < BEAMS * 64; i += kXmThreads) {
    const int j = i >> 6, d = i & 63;
    float tot = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < kXmWarps; ++w) {
      tot += s_out[w][j][d];
      den += s_sum[w][j];
    }
    out[((static_cast<long long>(b) * BEAMS + j) * H + h) * 64 + d] = __float2bfloat16(tot / den);
  }
}

}  // namespace
}  // namespace t5x

using namespace t5x;

// q: [batch * beams, heads, 64] bf16 with row stride q_ld; k: [batch, heads, Lp, 64] bf16;
// vt: [batch, heads, 64, Lp] bf16 (values transposed); Lp = Lk rounded up to a multiple of 32
// (the padding may hold anything finite); key_mask: [batch, Lk] uint8 (0 = padding) or null;
// out: [batch * beams, heads, 64] contiguous. beams in {1, 2, 4, 8}, Lk <= 1024.
T5X_API int t5x_decode_cross_attention_mma(const void* q, const void* k, const void* vt,
                                           const void* key_mask, void* out, long long q_ld,
                                           int batch, int beams, int heads, int head_dim, int Lk,
                                           int Lp, void* stream) {
  if (batch <= 0) return 0;
  if (head_dim != 64) return set_error("decode_cross_attention_mma: head_dim must be 64");
  if (Lk < 1 || Lk > kXmMaxKeys || Lp < Lk || Lp % 32 || Lp > kXmMaxKeys)
    return set_error("decode_cross_attention_mma: need 1 <= Lk <= Lp <= %d, Lp %% 32 == 0",
                     kXmMaxKeys);
  if (q_ld % 8 || (reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k)) & 15 ||
      (reinterpret_cast<uintptr_t>(vt) & 15))
    return set_error("decode_cross_attention_mma: misaligned operand");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid(batch * heads);
  auto qp = static_cast<const __nv_bfloat16*>(q);
  auto kp = static_cast<const __nv_bfloat16*>(k);
  auto vp = static_cast<const __nv_bfloat16*>(vt);
  auto mp = static_cast<const uint8_t*>(key_mask);
  auto op = static_cast<__nv_bfloat16*>(out);
  cudaError_t le = cudaSuccess;
  switch (beams) {
    case 1:
      le = launch_chained(decode_cross_mma_kernel<1>, grid, dim3(kXmThreads), 0, st, qp, kp, vp, mp, op, q_ld, heads, Lk, Lp);
      break;
    case 2:
      le = launch_chained(decode_cross_mma_kernel<2>, grid, dim3(kXmThreads), 0, st, qp, kp, vp, mp, op, q_ld, heads, Lk, Lp);
      break;
    case 4:
      le = launch_chained(decode_cross_mma_kernel<4>, grid, dim3(kXmThreads), 0, st, qp, kp, vp, mp, op, q_ld, heads, Lk, Lp);
      break;
    case 8:
      le = launch_chained(decode_cross_mma_kernel<8>, grid, dim3(kXmThreads), 0, st, qp, kp, vp, mp, op, q_ld, heads, Lk, Lp);
      break;
    default:
      return set_error("decode_cross_attention_mma: beams must be 1, 2, 4 or 8 (got %d)", beams);
  }
  count_launches(1);
  cudaError_t e = le != cudaSuccess ? le : cudaGetLastError();
  if (e != cudaSuccess) return set_error("decode_cross_attention_mma: %s", cudaGetErrorString(e));
  return 0;
}
