// z-loss cross-entropy over a (possibly vocab-sharded) logits matrix.
//
// Two kernels so that the vocabulary may be split across tensor-parallel ranks:
//   stats : per row and per local vocab slice -> running max, sum exp(l - max),
//           the target's logit (if it falls in the slice), sum of logits (label
//           smoothing), and the local argmax (accuracy metric).
//   grad  : given the globally combined log-sum-exp per row,
//           dlogits = row_scale * ((1 + 2 z lse) softmax - soft_targets)     (bf16 out)
// The combine between them is a handful of floats per token (host wrapper / NVLink).
#include <cfloat>

#include "common.cuh"

namespace t5x {

constexpr int kCeThreads = 256;

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) {
  return v;
}
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}

// stats[row] = {max, sumexp, target_logit, sum_logits}; arg_val/arg_idx = local argmax.
template <typename T>
__global__ void __launch_bounds__(kCeThreads)
    ce_stats_kernel(const T* __restrict__ logits, const long long* __restrict__ targets,
                    float4* __restrict__ stats, float* __restrict__ arg_val,
                    int* __restrict__ arg_idx, int rows, int vocab_local, long long ld,
                    int vocab_start) {
  __shared__ float s_max[kCeThreads / 32], s_sum[kCeThreads / 32], s_tot[kCeThreads / 32];
  __shared__ float s_av[kCeThreads / 32];
  __shared__ int s_ai[kCeThreads / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* lr = logits + static_cast<long long>(row) * ld;
    float m = -FLT_MAX, s = 0.f, tot = 0.f, av = -FLT_MAX;
    int ai = 0x7fffffff;
    for (int v = threadIdx.x; v < vocab_local; v += kCeThreads) {
      const float x = to_f32<T>(lr[v]);
      tot += x;
      if (x > av) {  // strict: the lowest index wins ties within a thread's ascending scan
        av = x;
        ai = v;
      }
      if (x > m) {
        s = s * __expf(m - x) + 1.f;
        m = x;
      } else {
        s += __expf(x - m);
      }
    }
    // warp combine
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
      const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
      const float av2 = __shfl_xor_sync(0xffffffffu, av, o);
      const int ai2 = __shfl_xor_sync(0xffffffffu, ai, o);
      tot += __shfl_xor_sync(0xffffffffu, tot, o);
      const float mn = fmaxf(m, m2);
      s = s * __expf(m - mn) + s2 * __expf(m2 - mn);
      m = mn;
      if (av2 > av || (av2 == av && ai2 < ai)) {
        av = av2;
        ai = ai2;
      }
    }
    __syncthreads();
    if (lane == 0) {
      s_max[warp] = m;
      s_sum[warp] = s;
      s_tot[warp] = tot;
      s_av[warp] = av;
      s_ai[warp] = ai;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float M = s_max[0], S = s_sum[0], TT = s_tot[0], AV = s_av[0];
      int AI = s_ai[0];
      for (int w = 1; w < kCeThreads / 32; ++w) {
        const float mn = fmaxf(M, s_max[w]);
        S = S * __expf(M - mn) + s_sum[w] * __expf(s_max[w] - mn);
        M = mn;
        TT += s_tot[w];
        if (s_av[w] > AV || (s_av[w] == AV && s_ai[w] < AI)) {
          AV = s_av[w];
          AI = s_ai[w];
        }
      }
      const long long t = targets[row] - vocab_start;
      const float tl = (t >= 0 && t < vocab_local) ? to_f32<T>(lr[t]) : 0.f;
      stats[row] = make_float4(M, S, tl, TT);
      arg_val[row] = AV;
      arg_idx[row] = AI + vocab_start;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kCeThreads)
    ce_grad_kernel(const T* __restrict__ logits, const long long* __restrict__ targets,
                   const float* __restrict__ lse, const float* __restrict__ row_scale,
                   __nv_bfloat16* __restrict__ dlogits, int rows, int vocab_local, long long ld,
                   long long ldd, int vocab_start, float z_loss, float confidence,
                   float low_confidence) {
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* lr = logits + static_cast<long long>(row) * ld;
    __nv_bfloat16* dr = dlogits + static_cast<long long>(row) * ldd;
    const float l = lse[row];
    const float g = row_scale[row];
    const float zf = 1.f + 2.f * z_loss * l;
    const long long t = targets[row] - vocab_start;
    if (g == 0.f) {
      for (int v = threadIdx.x; v < vocab_local; v += kCeThreads) dr[v] = __float2bfloat16(0.f);
      continue;
    }
    for (int v = threadIdx.x; v < vocab_local; v += kCeThreads) {
      const float p = __expf(to_f32<T>(lr[v]) - l);
      const float soft = (v == t) ? confidence : low_confidence;
      dr[v] = __float2bfloat16(g * (zf * p - soft));
    }
  }
}

// Merges the per-tile partials of the fused projection + cross-entropy forward
// (t5x_gemm_ce_stats) into the per-row statistics t5x_ce_stats produces: one warp per row.
__global__ void __launch_bounds__(256)
    ce_merge_kernel(const float4* __restrict__ part, const int* __restrict__ arg,
                    const float* __restrict__ target_logit, const long long* __restrict__ targets,
                    float4* __restrict__ stats, float* __restrict__ arg_val,
                    int* __restrict__ arg_idx, int rows, int tiles, int vocab_start,
                    int vocab_local) {
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (row >= rows) return;
  float mx = -3.0e38f, se = 0.f, sx = 0.f, best = -3.0e38f;
  int best_idx = 0x7fffffff;
  for (int t = lane; t < tiles; t += 32) {
    const float4 v = part[static_cast<long long>(row) * tiles + t];
    const float nm = fmaxf(mx, v.x);
    se = se * __expf(mx - nm) + v.y * __expf(v.x - nm);
    mx = nm;
    sx += v.z;
    const int idx = arg[static_cast<long long>(row) * tiles + t];
    if (v.w > best || (v.w == best && idx < best_idx)) {
      best = v.w;
      best_idx = idx;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, mx, o);
    const float os = __shfl_xor_sync(0xffffffffu, se, o);
    const float nm = fmaxf(mx, om);
    se = se * __expf(mx - nm) + os * __expf(om - nm);
    mx = nm;
    sx += __shfl_xor_sync(0xffffffffu, sx, o);
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_idx, o);
    if (ob > best || (ob == best && oi < best_idx)) {
      best = ob;
      best_idx = oi;
    }
  }
  if (lane == 0) {
    const long long t = targets[row] - vocab_start;
    const float tl = (t >= 0 && t < vocab_local) ? target_logit[row] : 0.f;
    stats[row] = make_float4(mx, se, tl, sx);
    arg_val[row] = best;
    arg_idx[row] = best_idx;
  }
}

}  // namespace t5x

using namespace t5x;

// stats[rows] = (max, sum exp(x - max), target logit, sum x), arg_val / arg_idx = largest logit
// and its vocabulary id, from the partials of t5x_gemm_ce_stats.
T5X_API int t5x_ce_merge(const void* part, const void* arg, const void* target_logit,
                         const void* targets, void* stats, void* arg_val, void* arg_idx, int rows,
                         int tiles, int vocab_start, int vocab_local, void* stream) {
  if (rows <= 0) return 0;
  ce_merge_kernel<<<(rows + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float4*>(part), static_cast<const int*>(arg),
      static_cast<const float*>(target_logit), static_cast<const long long*>(targets),
      static_cast<float4*>(stats), static_cast<float*>(arg_val), static_cast<int*>(arg_idx), rows,
      tiles, vocab_start, vocab_local);
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("ce_merge: %s", cudaGetErrorString(e));
  return 0;
}

T5X_API int t5x_ce_stats(const void* logits, int logits_fp32, const void* targets, void* stats,
                         void* arg_val, void* arg_idx, int rows, int vocab_local, long long ld,
                         int vocab_start, void* stream) {
  if (rows <= 0) return 0;
  int grid = rows < num_sms() * 8 ? rows : num_sms() * 8;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (logits_fp32)
    ce_stats_kernel<float><<<grid, kCeThreads, 0, st>>>(
        static_cast<const float*>(logits), static_cast<const long long*>(targets),
        static_cast<float4*>(stats), static_cast<float*>(arg_val), static_cast<int*>(arg_idx), rows,
        vocab_local, ld, vocab_start);
  else
    ce_stats_kernel<__nv_bfloat16><<<grid, kCeThreads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(logits), static_cast<const long long*>(targets),
        static_cast<float4*>(stats), static_cast<float*>(arg_val), static_cast<int*>(arg_idx), rows,
        vocab_local, ld, vocab_start);
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("ce_stats: %s", cudaGetErrorString(e));
  return 0;
}

T5X_API int t5x_ce_grad(const void* logits, int logits_fp32, const void* targets, const void* lse,
                        const void* row_scale, void* dlogits, int rows, int vocab_local,
                        long long ld, long long ldd, int vocab_start, float z_loss,
                        float confidence, float low_confidence, void* stream) {
  if (rows <= 0) return 0;
  int grid = rows < num_sms() * 8 ? rows : num_sms() * 8;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (logits_fp32)
    ce_grad_kernel<float><<<grid, kCeThreads, 0, st>>>(
        static_cast<const float*>(logits), static_cast<const long long*>(targets),
        static_cast<const float*>(lse), static_cast<const float*>(row_scale),
        static_cast<__nv_bfloat16*>(dlogits), rows, vocab_local, ld, ldd, vocab_start, z_loss,
        confidence, low_confidence);
  else
    ce_grad_kernel<__nv_bfloat16><<<grid, kCeThreads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(logits), static_cast<const long long*>(targets),
        static_cast<const float*>(lse), static_cast<const float*>(row_scale),
        static_cast<__nv_bfloat16*>(dlogits), rows, vocab_local, ld, ldd, vocab_start, z_loss,
        confidence, low_confidence);
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("ce_grad: %s", cudaGetErrorString(e));
  return 0;
}
