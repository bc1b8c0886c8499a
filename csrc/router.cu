// Mixture-of-experts router ("tokens choose") as three forward and two backward kernels.
//
// The reference takes its router from Flaxformer; its own code fixes the contract: fp32 router
// logits, softmax, top-k experts per token, a fixed per-expert capacity filled in token order
// with every first choice placed before any second choice, the router z-loss and the
// load-balancing loss, and the metrics auxiliary_loss / router_z_loss /
// fraction_tokens_left_behind / expert_usage / router_confidence
// (t5x/contrib/moe/models.py:40-46).
//
//   router_token_kernel   a warp per token: logits = x . W (fp32, W transposed in shared memory),
//                         softmax, top-k (value, then lowest expert index); per-CTA partial sums
//                         of lse^2 and of the probabilities per expert (written, not added
//                         atomically: results do not depend on scheduling).
//   router_slot_kernel    a CTA per expert: ordered scan over the choice-major list of
//                         (choice, token) pairs that picked this expert -> position in the expert,
//                         capacity cut, gate of dropped choices zeroed, row index in the dispatch
//                         buffer; per-expert counts.
//   router_final_kernel   one CTA: the two losses and the three usage metrics.
//   router_bwd_kernel     a warp per token: gradient of the logits from the gate gradients and
//                         the two losses, and of the tokens (dlogits . W^T).
//   router_dw_*_kernel    gradient of W: per-tile partial sums, then a fixed-order sum over tiles.
#include <float.h>

#include "common.cuh"

namespace t5x {
namespace {

constexpr int kRtWarps = 8;
constexpr int kRtThreads = kRtWarps * 32;
constexpr int kRtMaxExperts = 64;
constexpr int kRtMaxChoices = 4;

struct RouterDims {
  int T, d, E, k, capacity;
};

// logits of one token in the warp: lane l holds experts l and l + 32.
__device__ __forceinline__ void token_logits(const float* xs, const float* wt, int d, int E,
                                             int lane, float& l0, float& l1) {
  l0 = l1 = -FLT_MAX;
  for (int e = 0; e < E; ++e) {
    const float* w = wt + static_cast<long long>(e) * d;
    float acc = 0.f;
    for (int c = lane; c < d; c += 32) acc = fmaf(xs[c], w[c], acc);
    acc = warp_sum(acc);
    if ((e & 31) == lane) {
      if (e < 32) l0 = acc; else l1 = acc;
    }
  }
}

__global__ void __launch_bounds__(kRtThreads)
    router_token_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                        const float* __restrict__ w /* [d, E] */, const RouterDims dm,
                        float* __restrict__ probs /* [T, E] */, float* __restrict__ lse /* [T] */,
                        int* __restrict__ index /* [T, k] */, float* __restrict__ gate /* [T, k] */,
                        float* __restrict__ part /* [grid, 1 + E]: sum lse^2, sum probs[e] */) {
  extern __shared__ float rsm[];
  float* wt = rsm;                                  // [E, d]
  float* xs = rsm + static_cast<long long>(dm.E) * dm.d;  // [warps, d]
  float* acc_p = xs + kRtWarps * dm.d;              // [warps, E]
  float* acc_z = acc_p + kRtWarps * dm.E;           // [warps]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < dm.d * dm.E; i += kRtThreads) {
    const int c = i / dm.E, e = i - c * dm.E;
    wt[static_cast<long long>(e) * dm.d + c] = w[i];
  }
  for (int i = threadIdx.x; i < kRtWarps * dm.E; i += kRtThreads) acc_p[i] = 0.f;
  if (threadIdx.x < kRtWarps) acc_z[threadIdx.x] = 0.f;
  __syncthreads();
  float* my_x = xs + warp * dm.d;
  float zsum = 0.f;
  for (int t = blockIdx.x * kRtWarps + warp; t < dm.T; t += gridDim.x * kRtWarps) {
    const __nv_bfloat16* row = x + static_cast<long long>(t) * ldx;
    for (int c = lane; c < dm.d; c += 32) my_x[c] = __bfloat162float(row[c]);
    __syncwarp();
    float l0, l1;
    token_logits(my_x, wt, dm.d, dm.E, lane, l0, l1);
    const float m = warp_max(fmaxf(l0, l1));
    const float e0 = lane < dm.E ? expf(l0 - m) : 0.f;
    const float e1 = lane + 32 < dm.E ? expf(l1 - m) : 0.f;
    const float s = warp_sum(e0 + e1);
    const float p0 = e0 / s, p1 = e1 / s;
    const float ls = m + logf(s);
    if (lane < dm.E) probs[static_cast<long long>(t) * dm.E + lane] = p0;
    if (lane + 32 < dm.E) probs[static_cast<long long>(t) * dm.E + lane + 32] = p1;
    if (lane < dm.E) acc_p[warp * dm.E + lane] += p0;
    if (lane + 32 < dm.E) acc_p[warp * dm.E + lane + 32] += p1;
    if (lane == 0) {
      lse[t] = ls;
      zsum += ls * ls;
    }
    // top-k: k rounds of (probability desc, expert asc)
    float q0 = lane < dm.E ? p0 : -1.f, q1 = lane + 32 < dm.E ? p1 : -1.f;
    for (int c = 0; c < dm.k; ++c) {
      float v = q0;
      int e = lane;
      if (q1 > v) v = q1, e = lane + 32;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oe = __shfl_xor_sync(0xffffffffu, e, o);
        if (ov > v || (ov == v && oe < e)) v = ov, e = oe;
      }
      if (lane == 0) {
        index[static_cast<long long>(t) * dm.k + c] = e;
        gate[static_cast<long long>(t) * dm.k + c] = v;
      }
      if (e == lane) q0 = -1.f;
      if (e == lane + 32) q1 = -1.f;
    }
    __syncwarp();
  }
  if (lane == 0) acc_z[warp] = zsum;
  __syncthreads();
  float* out = part + static_cast<long long>(blockIdx.x) * (1 + dm.E);
  if (threadIdx.x == 0) {
    float z = 0.f;
    for (int wq = 0; wq < kRtWarps; ++wq) z += acc_z[wq];
    out[0] = z;
  }
  for (int e = threadIdx.x; e < dm.E; e += kRtThreads) {
    float p = 0.f;
    for (int wq = 0; wq < kRtWarps; ++wq) p += acc_p[wq * dm.E + e];
    out[1 + e] = p;
  }
}

// stats[e] = {choices that picked e, of those kept, sum of kept gates, sum of probs[:, e]}
__global__ void __launch_bounds__(1024)
    router_slot_kernel(const int* __restrict__ index, float* __restrict__ gate,
                       int* __restrict__ flat_slot, const float* __restrict__ part, int num_parts,
                       const RouterDims dm, float* __restrict__ stats) {
  __shared__ int warp_tot[32];
  __shared__ int running;
  __shared__ float red[32];
  const int e = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) running = 0;
  __syncthreads();
  const long long n = static_cast<long long>(dm.T) * dm.k;  // choice-major: j = c * T + t
  float kept_gate = 0.f;
  int kept = 0;
  for (long long base = 0; base < n; base += blockDim.x) {
    const long long j = base + threadIdx.x;
    int c = 0, t = 0;
    bool hit = false;
    if (j < n) {
      c = static_cast<int>(j / dm.T);
      t = static_cast<int>(j - static_cast<long long>(c) * dm.T);
      hit = index[static_cast<long long>(t) * dm.k + c] == e;
    }
    const unsigned int ballot = __ballot_sync(0xffffffffu, hit);
    const int before = __popc(ballot & ((1u << lane) - 1u));
    if (lane == 0) warp_tot[warp] = __popc(ballot);
    __syncthreads();
    int offset = running;
    for (int wq = 0; wq < warp; ++wq) offset += warp_tot[wq];
    if (hit) {
      const int pos = offset + before;
      const long long o = static_cast<long long>(t) * dm.k + c;
      if (pos < dm.capacity) {
        flat_slot[o] = e * dm.capacity + pos;
        kept_gate += gate[o];
        ++kept;
      } else {
        flat_slot[o] = -1;
        gate[o] = 0.f;
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int tot = 0;
      for (int wq = 0; wq < (blockDim.x >> 5); ++wq) tot += warp_tot[wq];
      running += tot;
    }
    __syncthreads();
  }
  // fixed-order block sums
  float v = warp_sum(kept_gate);
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float gate_sum = 0.f;
  if (threadIdx.x == 0)
    for (int wq = 0; wq < (blockDim.x >> 5); ++wq) gate_sum += red[wq];
  __syncthreads();
  v = warp_sum(static_cast<float>(kept));
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float kept_sum = 0.f;
    for (int wq = 0; wq < (blockDim.x >> 5); ++wq) kept_sum += red[wq];
    float psum = 0.f;
    for (int b = 0; b < num_parts; ++b) psum += part[static_cast<long long>(b) * (1 + dm.E) + 1 + e];
    stats[e * 4 + 0] = static_cast<float>(running);
    stats[e * 4 + 1] = kept_sum;
    stats[e * 4 + 2] = gate_sum;
    stats[e * 4 + 3] = psum;
  }
}

// out[0..6] = auxiliary_loss, router_z_loss, fraction_tokens_left_behind, expert_usage,
// router_confidence, tokens dispatched somewhere, (unused)
__global__ void __launch_bounds__(1024)
    router_final_kernel(const int* __restrict__ flat_slot, const float* __restrict__ part,
                        int num_parts, const float* __restrict__ stats, const RouterDims dm,
                        float* __restrict__ out) {
  __shared__ float red[32];
  int any = 0;
  for (int t = threadIdx.x; t < dm.T; t += blockDim.x) {
    bool a = false;
    for (int c = 0; c < dm.k; ++c) a = a || flat_slot[static_cast<long long>(t) * dm.k + c] >= 0;
    any += a ? 1 : 0;
  }
  float v = warp_sum(static_cast<float>(any));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float dispatched = 0.f;
    for (int wq = 0; wq < (blockDim.x >> 5); ++wq) dispatched += red[wq];
    float z = 0.f;
    for (int b = 0; b < num_parts; ++b) z += part[static_cast<long long>(b) * (1 + dm.E)];
    const float T = static_cast<float>(dm.T);
    float aux = 0.f, kept = 0.f, gates = 0.f;
    for (int e = 0; e < dm.E; ++e) {
      aux += (stats[e * 4 + 0] / T) * (stats[e * 4 + 3] / T);
      kept += stats[e * 4 + 1];
      gates += stats[e * 4 + 2];
    }
    out[0] = aux * static_cast<float>(dm.E);
    out[1] = z / T;
    out[2] = 1.f - dispatched / T;
    out[3] = kept / (static_cast<float>(dm.E) * static_cast<float>(dm.capacity));
    out[4] = gates / fmaxf(dispatched, 1.f);
    out[5] = dispatched;
  }
}

// dlogits [T, E] (fp32) and dx [T, d] (bf16). coef[0] = d(loss)/d(auxiliary_loss),
// coef[1] = d(loss)/d(router_z_loss) (device scalars).
__global__ void __launch_bounds__(kRtThreads)
    router_bwd_kernel(const float* __restrict__ probs, const float* __restrict__ lse,
                      const int* __restrict__ index, const int* __restrict__ flat_slot,
                      const float* __restrict__ dgate, const float* __restrict__ stats,
                      const float* __restrict__ coef, const float* __restrict__ w /* [d, E] */,
                      const RouterDims dm, float* __restrict__ dlogits,
                      __nv_bfloat16* __restrict__ dx, long long lddx) {
  extern __shared__ float rsm[];
  float* wt = rsm;                                        // [E, d]
  float* dls = rsm + static_cast<long long>(dm.E) * dm.d;  // [warps, E]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < dm.d * dm.E; i += kRtThreads) {
    const int c = i / dm.E, e = i - c * dm.E;
    wt[static_cast<long long>(e) * dm.d + c] = w[i];
  }
  __syncthreads();
  const float T = static_cast<float>(dm.T);
  const float d_aux = coef[0], d_z = coef[1];
  float* my = dls + warp * dm.E;
  for (int t = blockIdx.x * kRtWarps + warp; t < dm.T; t += gridDim.x * kRtWarps) {
    float dp[2], p[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int e = lane + 32 * h;
      p[h] = dp[h] = 0.f;
      if (e < dm.E) {
        p[h] = probs[static_cast<long long>(t) * dm.E + e];
        dp[h] = d_aux * static_cast<float>(dm.E) * (stats[e * 4 + 0] / T) / T;
        for (int c = 0; c < dm.k; ++c) {
          const long long o = static_cast<long long>(t) * dm.k + c;
          if (index[o] == e && flat_slot[o] >= 0) dp[h] += dgate[o];
        }
      }
    }
    const float dot = warp_sum(p[0] * dp[0] + p[1] * dp[1]);
    const float zc = d_z * 2.f * lse[t] / T;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int e = lane + 32 * h;
      if (e < dm.E) {
        const float dl = p[h] * (dp[h] - dot) + zc * p[h];
        dlogits[static_cast<long long>(t) * dm.E + e] = dl;
        my[e] = dl;
      }
    }
    __syncwarp();
    if (dx != nullptr) {
      for (int c = lane; c < dm.d; c += 32) {
        float acc = 0.f;
        for (int e = 0; e < dm.E; ++e) acc = fmaf(my[e], wt[static_cast<long long>(e) * dm.d + c], acc);
        dx[static_cast<long long>(t) * lddx + c] = __float2bfloat16(acc);
      }
    }
    __syncwarp();
  }
}

// dw[c, e] = sum_t x[t, c] * dlogits[t, e] in two deterministic stages: every CTA reduces a
// tile of kDwTile tokens into part[tile, c, e] (a thread owns feature columns, the tile's dlogits
// sit in shared memory), then a second kernel adds the tiles in order.
constexpr int kDwTile = 512;
constexpr int kDwThreads = 256;
constexpr int kDwMaxColsPerThread = 4;  // d <= 1024 per pass over the tile

__global__ void __launch_bounds__(kDwThreads)
    router_dw_partial_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                             const float* __restrict__ dlogits, const RouterDims dm,
                             float* __restrict__ part /* [tiles, d, E] */) {
  __shared__ __align__(16) float dl[kDwTile * 8];
  const int tile = blockIdx.x;
  const int t0 = tile * kDwTile, nt = min(kDwTile, dm.T - t0);
  float* out = part + static_cast<long long>(tile) * dm.d * dm.E;
  for (int e0 = 0; e0 < dm.E; e0 += 8) {
    const int ne = min(8, dm.E - e0);
    __syncthreads();
    for (int i = threadIdx.x; i < nt * 8; i += kDwThreads) {
      const int t = i >> 3, j = i & 7;
      dl[i] = j < ne ? dlogits[static_cast<long long>(t0 + t) * dm.E + e0 + j] : 0.f;
    }
    __syncthreads();
    for (int c0 = 0; c0 < dm.d; c0 += kDwThreads * kDwMaxColsPerThread) {
      float acc[kDwMaxColsPerThread][8];
#pragma unroll
      for (int q = 0; q < kDwMaxColsPerThread; ++q)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[q][j] = 0.f;
      for (int t = 0; t < nt; ++t) {
        const __nv_bfloat16* row = x + static_cast<long long>(t0 + t) * ldx + c0;
        const float4 a = *reinterpret_cast<const float4*>(dl + t * 8);
        const float4 b = *reinterpret_cast<const float4*>(dl + t * 8 + 4);
#pragma unroll
        for (int q = 0; q < kDwMaxColsPerThread; ++q) {
          const int c = c0 + q * kDwThreads + threadIdx.x;
          const float xv = c < dm.d ? __bfloat162float(row[q * kDwThreads + threadIdx.x]) : 0.f;
          acc[q][0] = fmaf(xv, a.x, acc[q][0]);
          acc[q][1] = fmaf(xv, a.y, acc[q][1]);
          acc[q][2] = fmaf(xv, a.z, acc[q][2]);
          acc[q][3] = fmaf(xv, a.w, acc[q][3]);
          acc[q][4] = fmaf(xv, b.x, acc[q][4]);
          acc[q][5] = fmaf(xv, b.y, acc[q][5]);
          acc[q][6] = fmaf(xv, b.z, acc[q][6]);
          acc[q][7] = fmaf(xv, b.w, acc[q][7]);
        }
      }
#pragma unroll
      for (int q = 0; q < kDwMaxColsPerThread; ++q) {
        const int c = c0 + q * kDwThreads + threadIdx.x;
        if (c < dm.d)
          for (int j = 0; j < ne; ++j) out[static_cast<long long>(c) * dm.E + e0 + j] = acc[q][j];
      }
    }
  }
}

__global__ void __launch_bounds__(256)
    router_dw_reduce_kernel(const float* __restrict__ part, int tiles, int n,
                            float* __restrict__ dw) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = 0.f;
  for (int t = 0; t < tiles; ++t) s += part[static_cast<long long>(t) * n + i];
  dw[i] = s;
}

static int router_check(const RouterDims& dm, size_t smem) {
  if (dm.T <= 0 || dm.d <= 0) return set_error("router: empty input");
  if (dm.E < 1 || dm.E > kRtMaxExperts) return set_error("router: 1..%d experts (got %d)", kRtMaxExperts, dm.E);
  if (dm.k < 1 || dm.k > kRtMaxChoices || dm.k > dm.E)
    return set_error("router: 1..%d choices per token (got %d)", kRtMaxChoices, dm.k);
  if (smem > 200 * 1024) return set_error("router: d=%d x experts=%d does not fit shared memory", dm.d, dm.E);
  return 0;
}

}  // namespace
}  // namespace t5x

// Number of per-CTA partial records (1 + E floats each) the forward writes.
T5X_API int t5x_moe_router_parts(int T) {
  const int want = (T + t5x::kRtWarps - 1) / t5x::kRtWarps;
  const int cap = 2 * t5x::num_sms();
  return want < cap ? (want < 1 ? 1 : want) : cap;
}

T5X_API int t5x_moe_router_dw_tiles(int T) { return (T + t5x::kDwTile - 1) / t5x::kDwTile; }

// Forward. x [T, d] bf16 (row stride ldx), w [d, E] fp32. Outputs: probs [T, E], lse [T],
// index [T, k] int32, gate [T, k] fp32 (zero where the choice lost its slot), flat_slot [T, k]
// int32 (expert * capacity + position, or -1), stats [E, 4], metrics [8], part [parts, 1 + E].
T5X_API int t5x_moe_router_fwd(const void* x, long long ldx, const void* w, int T, int d, int E,
                               int k, int capacity, void* probs, void* lse, void* index,
                               void* gate, void* flat_slot, void* stats, void* metrics, void* part,
                               void* stream) {
  using namespace t5x;
  RouterDims dm = {T, d, E, k, capacity};
  const size_t smem = (static_cast<size_t>(E) * d + kRtWarps * d + kRtWarps * E + kRtWarps) * 4;
  if (int rc = router_check(dm, smem)) return rc;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(router_token_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(router_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               200 * 1024);
    if (e != cudaSuccess) return set_error("router: %s", cudaGetErrorString(e));
    attr_set[dev & 63] = true;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int parts = t5x_moe_router_parts(T);
  router_token_kernel<<<parts, kRtThreads, smem, st>>>(
      static_cast<const __nv_bfloat16*>(x), ldx, static_cast<const float*>(w), dm,
      static_cast<float*>(probs), static_cast<float*>(lse), static_cast<int*>(index),
      static_cast<float*>(gate), static_cast<float*>(part));
  router_slot_kernel<<<E, 1024, 0, st>>>(static_cast<const int*>(index), static_cast<float*>(gate),
                                         static_cast<int*>(flat_slot),
                                         static_cast<const float*>(part), parts, dm,
                                         static_cast<float*>(stats));
  router_final_kernel<<<1, 1024, 0, st>>>(static_cast<const int*>(flat_slot),
                                          static_cast<const float*>(part), parts,
                                          static_cast<const float*>(stats), dm,
                                          static_cast<float*>(metrics));
  count_launches(3);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("router_fwd launch: %s", cudaGetErrorString(e));
  return 0;
}

// Backward. dgate [T, k] (gradient of the returned gates), coef [2] device floats (gradients of
// the auxiliary and z losses). Writes dlogits [T, E] (scratch), dx [T, d] bf16 (may be null)
// and dw [d, E] fp32; dw_part: scratch of t5x_moe_router_dw_tiles(T) * d * E floats.
T5X_API int t5x_moe_router_bwd(const void* x, long long ldx, const void* w, int T, int d, int E,
                               int k, int capacity, const void* probs, const void* lse,
                               const void* index, const void* flat_slot, const void* dgate,
                               const void* stats, const void* coef, void* dlogits, void* dx,
                               long long lddx, void* dw, void* dw_part, void* stream) {
  using namespace t5x;
  RouterDims dm = {T, d, E, k, capacity};
  const size_t smem = (static_cast<size_t>(E) * d + kRtWarps * E) * 4;
  if (int rc = router_check(dm, smem)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = t5x_moe_router_parts(T);
  router_bwd_kernel<<<grid, kRtThreads, smem, st>>>(
      static_cast<const float*>(probs), static_cast<const float*>(lse),
      static_cast<const int*>(index), static_cast<const int*>(flat_slot),
      static_cast<const float*>(dgate), static_cast<const float*>(stats),
      static_cast<const float*>(coef), static_cast<const float*>(w), dm,
      static_cast<float*>(dlogits), static_cast<__nv_bfloat16*>(dx), lddx);
  const int tiles = (T + kDwTile - 1) / kDwTile;
  router_dw_partial_kernel<<<tiles, kDwThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(x), ldx,
                                                        static_cast<const float*>(dlogits), dm,
                                                        static_cast<float*>(dw_part));
  router_dw_reduce_kernel<<<(d * E + 255) / 256, 256, 0, st>>>(
      static_cast<const float*>(dw_part), tiles, d * E, static_cast<float*>(dw));
  count_launches(3);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("router_bwd launch: %s", cudaGetErrorString(e));
  return 0;
}
