// Factored Adafactor update (the T5X variant) as a short chain of bandwidth-bound
// kernels over one parameter [batch, R, C] (batch = stacked-layer / expert dims that the
// optimizer treats independently):
//
//   stats   : rowsum[R] = sum_j (g^2 + eps1), colsum[C] = sum_i (g^2 + eps1), sum p^2
//   factors : EMA of the two second-moment vectors, then the two factor vectors
//             (v_row / mean(v_row))^-1/2 and v_col^-1/2
//   usq     : sum (g * rf_i * cf_j)^2                        (for RMS update clipping)
//   apply   : p <- (1 - wd) p - lr * scale(p) * u / max(1, rms(u)/thr)   (+ momentum),
//             also writing the bf16 working copy that the next forward pass reads.
//
// The unfactored form (vectors, small matrices) keeps a full second moment and needs
// two kernels. Scratch (rowsum/colsum/factor vectors/scalars) is provided by the caller
// and must be zero on entry to `stats`.
#include <mutex>

#include "adafactor_common.cuh"
#include "common.cuh"
#include "t5x_b200.h"

namespace t5x {

constexpr int kAfThreads = 256;
constexpr int kAfTileR = 64;
constexpr int kAfTileC = 512;

template <bool VEC>
__global__ void __launch_bounds__(kAfThreads)
    af_stats_kernel(const float* __restrict__ g, const float* __restrict__ p,
                    float* __restrict__ rowsum, float* __restrict__ colsum,
                    AdafactorScalars* __restrict__ scal, int R, int C, float eps1) {
  __shared__ float scol[kAfTileC];
  __shared__ float red[32];
  const int b = blockIdx.z;
  const long long base = static_cast<long long>(b) * R * C;
  g += base;
  p += base;
  rowsum += static_cast<long long>(b) * R;
  colsum += static_cast<long long>(b) * C;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int tile_r = blockIdx.y * kAfTileR, tile_c = blockIdx.x * kAfTileC;
  for (int i = threadIdx.x; i < kAfTileC; i += kAfThreads) scol[i] = 0.f;
  __syncthreads();
  float cacc[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int k = 0; k < 4; ++k) cacc[a][k] = 0.f;
  float psq = 0.f;
  if (VEC && tile_r + kAfTileR <= R && tile_c + kAfTileC <= C) {
    // interior tile: two rows per trip, their sixteen 16-byte loads issued before the first use
    for (int rr = 0; rr < kAfTileR / 8; rr += 2) {
      const int row = tile_r + warp * (kAfTileR / 8) + rr;
      float4 gq[2][4], pq[2][4];
#pragma unroll
      for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const long long off = static_cast<long long>(row + u) * C + tile_c + ch * 128 + lane * 4;
          gq[u][ch] = *reinterpret_cast<const float4*>(g + off);
          pq[u][ch] = *reinterpret_cast<const float4*>(p + off);
        }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        float rs = 0.f;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const float4 gv = gq[u][ch], pv = pq[u][ch];
          const float s0 = gv.x * gv.x + eps1, s1 = gv.y * gv.y + eps1, s2 = gv.z * gv.z + eps1,
                      s3 = gv.w * gv.w + eps1;
          rs += (s0 + s1) + (s2 + s3);
          cacc[ch][0] += s0;
          cacc[ch][1] += s1;
          cacc[ch][2] += s2;
          cacc[ch][3] += s3;
          psq += pv.x * pv.x + pv.y * pv.y + pv.z * pv.z + pv.w * pv.w;
        }
        rs = warp_sum(rs);
        if (lane == 0) atomicAdd(&rowsum[row + u], rs);
      }
    }
  } else
  for (int rr = 0; rr < kAfTileR / 8; ++rr) {
    const int row = tile_r + warp * (kAfTileR / 8) + rr;
    if (row >= R) break;
    float rs = 0.f;
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
      const int col = tile_c + ch * 128 + lane * 4;
      if (VEC) {
        if (col < C) {
          const float4 gv = *reinterpret_cast<const float4*>(g + static_cast<long long>(row) * C + col);
          const float4 pv = *reinterpret_cast<const float4*>(p + static_cast<long long>(row) * C + col);
          const float s0 = gv.x * gv.x + eps1, s1 = gv.y * gv.y + eps1, s2 = gv.z * gv.z + eps1,
                      s3 = gv.w * gv.w + eps1;
          rs += (s0 + s1) + (s2 + s3);
          cacc[ch][0] += s0;
          cacc[ch][1] += s1;
          cacc[ch][2] += s2;
          cacc[ch][3] += s3;
          psq += pv.x * pv.x + pv.y * pv.y + pv.z * pv.z + pv.w * pv.w;
        }
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (col + k < C) {
            const float gv = g[static_cast<long long>(row) * C + col + k];
            const float pv = p[static_cast<long long>(row) * C + col + k];
            const float s = gv * gv + eps1;
            rs += s;
            cacc[ch][k] += s;
            psq += pv * pv;
          }
        }
      }
    }
    rs = warp_sum(rs);
    if (lane == 0) atomicAdd(&rowsum[row], rs);
  }
#pragma unroll
  for (int ch = 0; ch < 4; ++ch)
#pragma unroll
    for (int k = 0; k < 4; ++k) atomicAdd(&scol[ch * 128 + lane * 4 + k], cacc[ch][k]);
  __syncthreads();
  for (int i = threadIdx.x; i < kAfTileC; i += kAfThreads)
    if (tile_c + i < C) atomicAdd(&colsum[tile_c + i], scol[i]);
  psq = warp_sum(psq);
  if (lane == 0) red[warp] = psq;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < kAfThreads / 32; ++w) t += red[w];
    atomicAdd(&scal[b].psq, t);
  }
}

// EMA of the two second-moment vectors; one CTA per batch element. `row_is_normalized`: the
// vector indexed by matrix rows is the one divided by its mean (T5X "v_row"); otherwise the
// column-indexed vector is. row_div / col_div are the GLOBAL column / row counts (the means are
// over the unsharded dims); the local sums were combined across ranks beforehand if needed.
__global__ void __launch_bounds__(1024)
    af_ema_kernel(float* __restrict__ v_rvec, float* __restrict__ v_cvec,
                  const float* __restrict__ rowsum, const float* __restrict__ colsum,
                  AdafactorScalars* __restrict__ scal, int R, int C, float row_div, float col_div,
                  float decay, int row_is_normalized, int skip_nan) {
  __shared__ float red[32];
  const int b = blockIdx.x;
  v_rvec += static_cast<long long>(b) * R;
  v_cvec += static_cast<long long>(b) * C;
  rowsum += static_cast<long long>(b) * R;
  colsum += static_cast<long long>(b) * C;
  const float mix = 1.f - decay;
  float acc = 0.f;
  for (int i = threadIdx.x; i < R; i += blockDim.x) {
    const float old = v_rvec[i];
    float nv = decay * old + mix * (rowsum[i] / row_div);
    if (skip_nan && isnan(nv)) nv = old;
    v_rvec[i] = nv;
    if (row_is_normalized) acc += nv;
  }
  for (int i = threadIdx.x; i < C; i += blockDim.x) {
    const float old = v_cvec[i];
    float nv = decay * old + mix * (colsum[i] / col_div);
    if (skip_nan && isnan(nv)) nv = old;
    v_cvec[i] = nv;
    if (!row_is_normalized) acc += nv;
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) tot += red[w];
    scal[b].vsum = tot;
  }
}

// Factor vectors from the updated moments: (v_row / mean(v_row))^-1/2 and v_col^-1/2.
// norm_count = GLOBAL length of the normalised vector.
__global__ void __launch_bounds__(1024)
    af_finalize_kernel(const float* __restrict__ v_rvec, const float* __restrict__ v_cvec,
                       float* __restrict__ rf, float* __restrict__ cf,
                       const AdafactorScalars* __restrict__ scal, int R, int C, float norm_count,
                       int row_is_normalized) {
  const int b = blockIdx.x;
  v_rvec += static_cast<long long>(b) * R;
  v_cvec += static_cast<long long>(b) * C;
  rf += static_cast<long long>(b) * R;
  cf += static_cast<long long>(b) * C;
  const float mean = scal[b].vsum / norm_count;
  for (int i = threadIdx.x; i < R; i += blockDim.x)
    rf[i] = row_is_normalized ? rsqrtf(v_rvec[i] / mean) : rsqrtf(v_rvec[i]);
  for (int i = threadIdx.x; i < C; i += blockDim.x)
    cf[i] = row_is_normalized ? rsqrtf(v_cvec[i]) : rsqrtf(v_cvec[i] / mean);
}

__global__ void __launch_bounds__(kAfThreads)
    af_usq_kernel(const float* __restrict__ g, const float* __restrict__ rf,
                  const float* __restrict__ cf, AdafactorScalars* __restrict__ scal, int R, int C) {
  __shared__ float red[32];
  const int b = blockIdx.y;
  g += static_cast<long long>(b) * R * C;
  rf += static_cast<long long>(b) * R;
  cf += static_cast<long long>(b) * C;
  const long long n = static_cast<long long>(R) * C;
  float acc = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(kAfThreads) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * kAfThreads) {
    const int r = static_cast<int>(i / C), c = static_cast<int>(i - static_cast<long long>(r) * C);
    const float u = g[i] * rf[r] * cf[c];
    acc += u * u;
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < kAfThreads / 32; ++w) t += red[w];
    atomicAdd(&scal[b].usq, t);
  }
}

// FACTORED: u = g * rf[r] * cf[c].  !FACTORED: u = g * rsqrt(v) with v already updated.
template <bool FACTORED>
__global__ void __launch_bounds__(kAfThreads)
    af_apply_kernel(float* __restrict__ p, const float* __restrict__ g, const float* __restrict__ rf,
                    const float* __restrict__ cf, const float* __restrict__ v, float* __restrict__ m,
                    __nv_bfloat16* __restrict__ p_bf16, long long ld_bf16, long long bf16_batch_stride,
                    const AdafactorScalars* __restrict__ scal, int R, int C, float n_global,
                    AfHyper h) {
  const int b = blockIdx.y;
  const long long n = static_cast<long long>(R) * C;
  const long long base = static_cast<long long>(b) * n;
  const float scale = af_update_scale(scal[b], n_global, h);
  if (FACTORED) {
    rf += static_cast<long long>(b) * R;
    cf += static_cast<long long>(b) * C;
  }
  for (long long i = blockIdx.x * static_cast<long long>(kAfThreads) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * kAfThreads) {
    const int r = static_cast<int>(i / C), c = static_cast<int>(i - static_cast<long long>(r) * C);
    const float gv = g[base + i];
    const float u = FACTORED ? gv * rf[r] * cf[c] : gv * rsqrtf(v[base + i]);
    float sub = scale * u;
    if (h.use_momentum) {
      const float old_m = m[base + i];
      float nm = h.beta1 * old_m + (1.f - h.beta1) * sub;
      sub = nm;
      if (h.skip_nan && isnan(nm)) nm = old_m;
      m[base + i] = nm;
    }
    const float old = p[base + i];
    float np = (h.use_wd ? (1.f - h.weight_decay) * old : old) - sub;
    if (h.skip_nan && isnan(np)) np = old;
    p[base + i] = np;
    if (p_bf16) p_bf16[b * bf16_batch_stride + static_cast<long long>(r) * ld_bf16 + c] = __float2bfloat16(np);
  }
}

// Unfactored pass 1: v <- decay v + (1-decay)(g^2+eps1); accumulates sum u^2 and sum p^2.
__global__ void __launch_bounds__(kAfThreads)
    af_unfactored_stats_kernel(const float* __restrict__ g, const float* __restrict__ p,
                               float* __restrict__ v, AdafactorScalars* __restrict__ scal,
                               long long n, float decay, float eps1, int skip_nan) {
  __shared__ float red[2][32];
  const int b = blockIdx.y;
  const long long base = static_cast<long long>(b) * n;
  float usq = 0.f, psq = 0.f;
  const float mix = 1.f - decay;
  for (long long i = blockIdx.x * static_cast<long long>(kAfThreads) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * kAfThreads) {
    const float gv = g[base + i], pv = p[base + i], old = v[base + i];
    float nv = decay * old + mix * (gv * gv + eps1);
    if (skip_nan && isnan(nv)) nv = old;
    v[base + i] = nv;
    const float u = gv * rsqrtf(nv);
    usq += u * u;
    psq += pv * pv;
  }
  usq = warp_sum(usq);
  psq = warp_sum(psq);
  if ((threadIdx.x & 31) == 0) {
    red[0][threadIdx.x >> 5] = usq;
    red[1][threadIdx.x >> 5] = psq;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.f, c = 0.f;
    for (int w = 0; w < kAfThreads / 32; ++w) {
      a += red[0][w];
      c += red[1][w];
    }
    atomicAdd(&scal[b].usq, a);
    atomicAdd(&scal[b].psq, c);
  }
}

// Tiled forms of the two element-wise factored passes: a CTA covers kAfRowsPerCta rows x 1024
// columns, a thread 4 adjacent columns of each row, so the row / column factors are indexed
// without a division per element and loads are 16 bytes wide when C % 4 == 0.
constexpr int kAfRowsPerCta = 32;
constexpr int kAfColsPerCta = kAfThreads * 4;

template <bool VEC>
__global__ void __launch_bounds__(kAfThreads)
    af_usq_tiled_kernel(const float* __restrict__ g, const float* __restrict__ rf,
                        const float* __restrict__ cf, AdafactorScalars* __restrict__ scal, int R,
                        int C) {
  __shared__ float red[kAfThreads / 32];
  const int b = blockIdx.z;
  g += static_cast<long long>(b) * R * C;
  rf += static_cast<long long>(b) * R;
  cf += static_cast<long long>(b) * C;
  const int r0 = blockIdx.y * kAfRowsPerCta;
  const int col = blockIdx.x * kAfColsPerCta + threadIdx.x * 4;
  const int rows = min(kAfRowsPerCta, R - r0);
  float acc = 0.f;
  if (col < C) {
    float c[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) c[k] = (col + k < C) ? cf[col + k] : 0.f;
    for (int rr = 0; rr < rows; ++rr) {
      const float* gp = g + static_cast<long long>(r0 + rr) * C + col;
      const float rv = rf[r0 + rr];
      float v[4];
      if (VEC) {
        const float4 t = *reinterpret_cast<const float4*>(gp);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = (col + k < C) ? gp[k] : 0.f;
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float u = v[k] * rv * c[k];
        acc += u * u;
      }
    }
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < kAfThreads / 32; ++w) t += red[w];
    atomicAdd(&scal[b].usq, t);
  }
}

template <bool VEC>
__global__ void __launch_bounds__(kAfThreads)
    af_apply_tiled_kernel(float* __restrict__ p, const float* __restrict__ g,
                          const float* __restrict__ rf, const float* __restrict__ cf,
                          float* __restrict__ m, __nv_bfloat16* __restrict__ p_bf16,
                          long long ld_bf16, long long bf16_batch_stride,
                          const AdafactorScalars* __restrict__ scal, int R, int C, float n_global,
                          AfHyper h) {
  const int b = blockIdx.z;
  const long long base = static_cast<long long>(b) * R * C;
  const int r0 = blockIdx.y * kAfRowsPerCta;
  const int col = blockIdx.x * kAfColsPerCta + threadIdx.x * 4;
  if (col >= C) return;
  const float scale = af_update_scale(scal[b], n_global, h);
  rf += static_cast<long long>(b) * R;
  cf += static_cast<long long>(b) * C;
  float c[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) c[k] = (col + k < C) ? cf[col + k] : 0.f;
  const int nk = min(4, C - col);
  const int rows = min(kAfRowsPerCta, R - r0);
  const bool bf_vec = VEC && p_bf16 != nullptr && (ld_bf16 % 4 == 0) &&
                      (bf16_batch_stride % 4 == 0) &&
                      ((reinterpret_cast<uintptr_t>(p_bf16) & 7) == 0);
  // Four rows per trip with all eight 16-byte loads issued before the first use: the kernel
  // is bound by how many bytes each thread keeps in flight.
  constexpr int kRowUnroll = 4;
  for (int r4 = 0; r4 < rows; r4 += kRowUnroll) {
    float4 tg[kRowUnroll], to[kRowUnroll];
    if (VEC) {
#pragma unroll
      for (int u = 0; u < kRowUnroll; ++u) {
        if (r4 + u < rows) {
          const long long off = base + static_cast<long long>(r0 + r4 + u) * C + col;
          tg[u] = *reinterpret_cast<const float4*>(g + off);
          to[u] = *reinterpret_cast<const float4*>(p + off);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kRowUnroll; ++u) {
    const int rr = r4 + u;
    if (rr >= rows) break;
    const long long off = base + static_cast<long long>(r0 + rr) * C + col;
    const float rv = rf[r0 + rr] * scale;
    float gv[4], ov[4], nv[4];
    if (VEC) {
      const float4 t = tg[u];
      const float4 o = to[u];
      gv[0] = t.x; gv[1] = t.y; gv[2] = t.z; gv[3] = t.w;
      ov[0] = o.x; ov[1] = o.y; ov[2] = o.z; ov[3] = o.w;
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        gv[k] = k < nk ? g[off + k] : 0.f;
        ov[k] = k < nk ? p[off + k] : 0.f;
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float sub = gv[k] * rv * c[k];
      if (h.use_momentum && k < nk) {
        const float old_m = m[off + k];
        float nm = h.beta1 * old_m + (1.f - h.beta1) * sub;
        sub = nm;
        if (h.skip_nan && isnan(nm)) nm = old_m;
        m[off + k] = nm;
      }
      float np = (h.use_wd ? (1.f - h.weight_decay) * ov[k] : ov[k]) - sub;
      if (h.skip_nan && isnan(np)) np = ov[k];
      nv[k] = np;
    }
    if (VEC) {
      *reinterpret_cast<float4*>(p + off) = make_float4(nv[0], nv[1], nv[2], nv[3]);
    } else {
      for (int k = 0; k < nk; ++k) p[off + k] = nv[k];
    }
    if (p_bf16 != nullptr) {
      __nv_bfloat16* o = p_bf16 + b * bf16_batch_stride +
                         static_cast<long long>(r0 + rr) * ld_bf16 + col;
      if (bf_vec) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(nv[0], nv[1]);
        __nv_bfloat162 hi = __floats2bfloat162_rn(nv[2], nv[3]);
        uint2 packed;
        packed.x = *reinterpret_cast<uint32_t*>(&lo);
        packed.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(o) = packed;
      } else {
        for (int k = 0; k < nk; ++k) o[k] = __float2bfloat16(nv[k]);
      }
    }
    }
  }
}

static inline dim3 af_tiled_grid(int batch, int R, int C) {
  return dim3((C + kAfColsPerCta - 1) / kAfColsPerCta, (R + kAfRowsPerCta - 1) / kAfRowsPerCta,
              batch);
}

static inline int af_grid(long long n) {
  long long blocks = (n + kAfThreads * 4 - 1) / (kAfThreads * 4);
  long long cap = static_cast<long long>(num_sms()) * 8;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace t5x

using namespace t5x;

// Scratch layout (floats): [batch*R rowsum][batch*C colsum][batch*R rf][batch*C cf][batch*4 scalars]
T5X_API long long t5x_adafactor_scratch_floats(int batch, int R, int C) {
  return 2ll * batch * (static_cast<long long>(R) + C) + 4ll * batch;
}

namespace {
struct AfScratch {
  float *rowsum, *colsum, *rf, *cf;
  AdafactorScalars* scal;
};
AfScratch af_split(void* scratch, int batch, int R, int C) {
  AfScratch a;
  float* s = static_cast<float*>(scratch);
  a.rowsum = s;
  a.colsum = a.rowsum + static_cast<long long>(batch) * R;
  a.rf = a.colsum + static_cast<long long>(batch) * C;
  a.cf = a.rf + static_cast<long long>(batch) * R;
  a.scal = reinterpret_cast<AdafactorScalars*>(a.cf + static_cast<long long>(batch) * C);
  return a;
}
int af_check(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("%s: %s", what, cudaGetErrorString(e));
  return 0;
}
// 16-byte loads of the statistics kernel need p and g on 16-byte boundaries as well as C % 4 == 0.
static bool af_stats_vec_ok(const void* p, const void* g, int C) {
  return C % 4 == 0 && ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g)) & 15) == 0;
}

// Pointers every factored update dereferences on the device; `m` only with the momentum flag.
static int af_validate(const char* what, const void* p, const void* g, const void* v_rvec,
                       const void* v_cvec, const void* m, int flags) {
  if (p == nullptr || g == nullptr) return set_error("%s: p and g must not be null", what);
  if (v_rvec == nullptr || v_cvec == nullptr)
    return set_error("%s: v_rvec and v_cvec must not be null", what);
  if ((flags & 8) && m == nullptr)
    return set_error("%s: the momentum flag (8) is set but m is null", what);
  if (((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g)) & 3) != 0)
    return set_error("%s: p and g must be 4-byte aligned", what);
  return 0;
}
}  // namespace

// The factored update is split in phases so that a tensor-parallel caller can sum the
// partial statistics across ranks between them (row sums when columns are sharded, column
// sums when rows are sharded, and the three scalars). A single-GPU caller uses
// t5x_adafactor_factored, which runs the phases back to back.

// Phase 1: clears the scratch and accumulates rowsum / colsum / sum p^2 of the local shard.
T5X_API int t5x_adafactor_stats(const void* p, const void* g, void* scratch, int batch, int R,
                                int C, float eps1, void* stream) {
  if (batch <= 0 || R <= 0 || C <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  AfScratch a = af_split(scratch, batch, R, C);
  cudaMemsetAsync(scratch, 0, t5x_adafactor_scratch_floats(batch, R, C) * sizeof(float), st);
  dim3 sgrid((C + kAfTileC - 1) / kAfTileC, (R + kAfTileR - 1) / kAfTileR, batch);
  if (p == nullptr || g == nullptr) return set_error("adafactor_stats: p and g must not be null");
  if (af_stats_vec_ok(p, g, C))
    af_stats_kernel<true><<<sgrid, kAfThreads, 0, st>>>(static_cast<const float*>(g),
                                                        static_cast<const float*>(p), a.rowsum,
                                                        a.colsum, a.scal, R, C, eps1);
  else
    af_stats_kernel<false><<<sgrid, kAfThreads, 0, st>>>(static_cast<const float*>(g),
                                                         static_cast<const float*>(p), a.rowsum,
                                                         a.colsum, a.scal, R, C, eps1);
  count_launches(1);
  return af_check("adafactor_stats");
}

// Phase 2: EMA of both vectors (global_R / global_C = unsharded dims); leaves the local sum of
// the normalised vector in scal.vsum.
T5X_API int t5x_adafactor_ema(void* v_rvec, void* v_cvec, void* scratch, int batch, int R, int C,
                              int global_R, int global_C, int row_is_normalized, float decay,
                              int skip_nan, void* stream) {
  if (batch <= 0) return 0;
  AfScratch a = af_split(scratch, batch, R, C);
  af_ema_kernel<<<batch, 1024, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<float*>(v_rvec), static_cast<float*>(v_cvec), a.rowsum, a.colsum, a.scal, R, C,
      static_cast<float>(global_C), static_cast<float>(global_R), decay, row_is_normalized,
      skip_nan);
  count_launches(1);
  return af_check("adafactor_ema");
}

// Phase 3: factor vectors, then sum u^2 of the local shard (when clipping is on).
T5X_API int t5x_adafactor_usq(const void* g, const void* v_rvec, const void* v_cvec, void* scratch,
                              int batch, int R, int C, int global_R, int global_C,
                              int row_is_normalized, int use_clip, void* stream) {
  if (batch <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  AfScratch a = af_split(scratch, batch, R, C);
  af_finalize_kernel<<<batch, 1024, 0, st>>>(
      static_cast<const float*>(v_rvec), static_cast<const float*>(v_cvec), a.rf, a.cf, a.scal, R,
      C, static_cast<float>(row_is_normalized ? global_R : global_C), row_is_normalized);
  if (use_clip) {
    const dim3 tgrid = af_tiled_grid(batch, R, C);
    if (C % 4 == 0 && (reinterpret_cast<uintptr_t>(g) & 15) == 0)
      af_usq_tiled_kernel<true><<<tgrid, kAfThreads, 0, st>>>(static_cast<const float*>(g), a.rf,
                                                              a.cf, a.scal, R, C);
    else
      af_usq_tiled_kernel<false><<<tgrid, kAfThreads, 0, st>>>(static_cast<const float*>(g), a.rf,
                                                               a.cf, a.scal, R, C);
  }
  count_launches(use_clip ? 2 : 1);
  return af_check("adafactor_usq");
}

// Phase 4: the parameter update. n_global = number of elements of the unsharded parameter
// (per batch element) over which the two RMS values are taken.
T5X_API int t5x_adafactor_apply(void* p, const void* g, void* m, void* p_bf16, long long ld_bf16,
                                long long bf16_batch_stride, void* scratch, int batch, int R, int C,
                                long long n_global, float lr, float eps2, float clip_threshold,
                                float weight_decay, float beta1, float max_param_scale, int flags,
                                void* stream) {
  if (batch <= 0) return 0;
  AfScratch a = af_split(scratch, batch, R, C);
  AfHyper h = af_hyper(lr, eps2, clip_threshold, weight_decay, beta1, max_param_scale, flags);
  const dim3 tgrid = af_tiled_grid(batch, R, C);
  const bool vec = C % 4 == 0 && (reinterpret_cast<uintptr_t>(p) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(g) & 15) == 0;
  if (vec)
    af_apply_tiled_kernel<true><<<tgrid, kAfThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<float*>(p), static_cast<const float*>(g), a.rf, a.cf, static_cast<float*>(m),
        static_cast<__nv_bfloat16*>(p_bf16), ld_bf16, bf16_batch_stride, a.scal, R, C,
        static_cast<float>(n_global), h);
  else
    af_apply_tiled_kernel<false><<<tgrid, kAfThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<float*>(p), static_cast<const float*>(g), a.rf, a.cf, static_cast<float*>(m),
        static_cast<__nv_bfloat16*>(p_bf16), ld_bf16, bf16_batch_stride, a.scal, R, C,
        static_cast<float>(n_global), h);
  count_launches(1);
  return af_check("adafactor_apply");
}

// Factored update of p[batch,R,C] on one GPU. v_rvec[batch,R] is the second-moment vector
// indexed by matrix rows (mean over columns), v_cvec[batch,C] the one indexed by columns.
T5X_API int t5x_adafactor_factored(void* p, const void* g, void* v_rvec, void* v_cvec, void* m,
                                   void* p_bf16, long long ld_bf16, long long bf16_batch_stride,
                                   void* scratch, int batch, int R, int C, int row_is_normalized,
                                   float lr, float decay, float eps1, float eps2,
                                   float clip_threshold, float weight_decay, float beta1,
                                   float max_param_scale, int flags, void* stream) {
  if (batch <= 0 || R <= 0 || C <= 0) return 0;
  int rc = af_validate("adafactor_factored", p, g, v_rvec, v_cvec, m, flags);
  if (rc) return rc;
  if (scratch == nullptr) return set_error("adafactor_factored: scratch must not be null");
  rc = t5x_adafactor_stats(p, g, scratch, batch, R, C, eps1, stream);
  if (rc) return rc;
  rc = t5x_adafactor_ema(v_rvec, v_cvec, scratch, batch, R, C, R, C, row_is_normalized, decay,
                         (flags >> 5) & 1, stream);
  if (rc) return rc;
  rc = t5x_adafactor_usq(g, v_rvec, v_cvec, scratch, batch, R, C, R, C, row_is_normalized,
                         (flags >> 1) & 1, stream);
  if (rc) return rc;
  return t5x_adafactor_apply(p, g, m, p_bf16, ld_bf16, bf16_batch_stride, scratch, batch, R, C,
                             static_cast<long long>(R) * C, lr, eps2, clip_threshold, weight_decay,
                             beta1, max_param_scale, flags, stream);
}

// Unfactored: phase 1 (v update, sum u^2, sum p^2 into scratch[batch*4]) and phase 2 (apply).
T5X_API int t5x_adafactor_unfactored_stats(const void* p, const void* g, void* v, void* scratch,
                                           int batch, long long n, float decay, float eps1,
                                           int skip_nan, void* stream) {
  if (batch <= 0 || n <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaMemsetAsync(scratch, 0, sizeof(AdafactorScalars) * batch, st);
  dim3 egrid(af_grid(n), batch);
  af_unfactored_stats_kernel<<<egrid, kAfThreads, 0, st>>>(
      static_cast<const float*>(g), static_cast<const float*>(p), static_cast<float*>(v),
      static_cast<AdafactorScalars*>(scratch), n, decay, eps1, skip_nan);
  count_launches(1);
  return af_check("adafactor_unfactored_stats");
}

T5X_API int t5x_adafactor_unfactored_apply(void* p, const void* g, const void* v, void* m,
                                           void* p_bf16, long long ld_bf16,
                                           long long bf16_batch_stride, void* scratch, int batch,
                                           int R, int C, long long n_global, float lr, float eps2,
                                           float clip_threshold, float weight_decay, float beta1,
                                           float max_param_scale, int flags, void* stream) {
  if (batch <= 0) return 0;
  AfHyper h = af_hyper(lr, eps2, clip_threshold, weight_decay, beta1, max_param_scale, flags);
  dim3 egrid(af_grid(static_cast<long long>(R) * C), batch);
  af_apply_kernel<false><<<egrid, kAfThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<float*>(p), static_cast<const float*>(g), nullptr, nullptr,
      static_cast<const float*>(v), static_cast<float*>(m), static_cast<__nv_bfloat16*>(p_bf16),
      ld_bf16, bf16_batch_stride, static_cast<const AdafactorScalars*>(scratch), R, C,
      static_cast<float>(n_global), h);
  count_launches(1);
  return af_check("adafactor_unfactored_apply");
}

// Unfactored update of p[batch, R, C] on one GPU (C = row width of the bf16 copy).
T5X_API int t5x_adafactor_unfactored(void* p, const void* g, void* v, void* m, void* p_bf16,
                                     long long ld_bf16, long long bf16_batch_stride, void* scratch,
                                     int batch, int R, int C, float lr, float decay, float eps1,
                                     float eps2, float clip_threshold, float weight_decay,
                                     float beta1, float max_param_scale, int flags, void* stream) {
  const long long n = static_cast<long long>(R) * C;
  int rc = t5x_adafactor_unfactored_stats(p, g, v, scratch, batch, n, decay, eps1, (flags >> 5) & 1,
                                          stream);
  if (rc) return rc;
  return t5x_adafactor_unfactored_apply(p, g, v, m, p_bf16, ld_bf16, bf16_batch_stride, scratch,
                                        batch, R, C, n, lr, eps2, clip_threshold, weight_decay,
                                        beta1, max_param_scale, flags, stream);
}

// ---------------------------------------------------------------------------------------
// Allocation-free variant of t5x_adafactor_factored (declared in t5x_b200.h).
//
// Some hosts of this library may not allocate device memory at the point where they step the
// optimizer: a caller that has handed the whole device heap to its own pool or arena, one that
// runs the update from a callback in which cudaMalloc is off limits (it synchronises the
// device), or a plain C program that links this .so without any tensor library to allocate
// with. For them the scratch (row/column sums, factor vectors, three scalars per batch
// element) lives in the fixed device array below instead of a caller-provided buffer.
// ---------------------------------------------------------------------------------------
namespace t5x {

constexpr long long kAfStaticScratchFloats = 1ll << 20;  // 4 MiB per GPU that loads this library
static __device__ __align__(256) float g_af_static_scratch[kAfStaticScratchFloats];

struct AfStaticDevice {
  float* scratch = nullptr;  // device address of g_af_static_scratch on this device
  int sms = 0;
};
static AfStaticDevice g_af_static[64];
static std::mutex g_af_static_mu;

// Looks up (once per device, with that device current) the device address of the static array.
// In host code the array's name is only a handle for the runtime, never a pointer a kernel may
// receive, so the address has to come from cudaGetSymbolAddress.
static int af_static_setup(AfStaticDevice** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return set_error("adafactor_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return set_error("adafactor_static: device %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_af_static_mu);
  AfStaticDevice& d = g_af_static[dev];
  if (d.scratch == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_af_static_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return set_error("adafactor_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    int sms = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess || sms <= 0)
      return set_error("adafactor_static: SM count query: %s", cudaGetErrorString(e));
    d.sms = sms;
    d.scratch = static_cast<float*>(ptr);
  }
  *out = &d;
  return 0;
}

}  // namespace t5x

T5X_API long long t5x_adafactor_factored_static_max_floats() { return t5x::kAfStaticScratchFloats; }

T5X_API int t5x_adafactor_factored_static(void* p, const void* g, void* v_rvec, void* v_cvec,
                                          void* m, void* p_bf16, long long ld_bf16,
                                          long long bf16_batch_stride, int batch, int R, int C,
                                          int row_is_normalized, float lr, float decay, float eps1,
                                          float eps2, float clip_threshold, float weight_decay,
                                          float beta1, float max_param_scale, int flags,
                                          void* stream) {
  if (batch <= 0 || R <= 0 || C <= 0) return 0;
  const long long need = t5x_adafactor_scratch_floats(batch, R, C);
  if (need > kAfStaticScratchFloats)
    return set_error(
        "adafactor_static: batch=%d rows=%d cols=%d needs %lld scratch floats but the built-in "
        "scratch holds %lld; use t5x_adafactor_factored with a caller-provided buffer",
        batch, R, C, need, kAfStaticScratchFloats);
  if (int rc = af_validate("adafactor_static", p, g, v_rvec, v_cvec, m, flags)) return rc;
  AfStaticDevice* d = nullptr;
  if (int rc = af_static_setup(&d)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  AfScratch a = af_split(d->scratch, batch, R, C);
  AfHyper h = af_hyper(lr, eps2, clip_threshold, weight_decay, beta1, max_param_scale, flags);
  // The array keeps whatever the previous call left: the sums and scalars must start at zero.
  cudaError_t e = cudaMemsetAsync(d->scratch, 0, need * sizeof(float), st);
  if (e != cudaSuccess) return set_error("adafactor_static: memset: %s", cudaGetErrorString(e));
  dim3 sgrid((C + kAfTileC - 1) / kAfTileC, (R + kAfTileR - 1) / kAfTileR, batch);
  if (af_stats_vec_ok(p, g, C))
    af_stats_kernel<true><<<sgrid, kAfThreads, 0, st>>>(static_cast<const float*>(g),
                                                        static_cast<const float*>(p), a.rowsum,
                                                        a.colsum, a.scal, R, C, eps1);
  else
    af_stats_kernel<false><<<sgrid, kAfThreads, 0, st>>>(static_cast<const float*>(g),
                                                         static_cast<const float*>(p), a.rowsum,
                                                         a.colsum, a.scal, R, C, eps1);
  af_ema_kernel<<<batch, 1024, 0, st>>>(static_cast<float*>(v_rvec), static_cast<float*>(v_cvec),
                                        a.rowsum, a.colsum, a.scal, R, C, static_cast<float>(C),
                                        static_cast<float>(R), decay, row_is_normalized, h.skip_nan);
  af_finalize_kernel<<<batch, 1024, 0, st>>>(
      static_cast<const float*>(v_rvec), static_cast<const float*>(v_cvec), a.rf, a.cf, a.scal, R,
      C, static_cast<float>(row_is_normalized ? R : C), row_is_normalized);
  const long long n = static_cast<long long>(R) * C;
  long long blocks = (n + kAfThreads * 4 - 1) / (kAfThreads * 4);
  const long long cap = static_cast<long long>(d->sms) * 8;
  blocks = blocks < 1 ? 1 : (blocks > cap ? cap : blocks);
  dim3 egrid(static_cast<unsigned>(blocks), batch);
  int launched = 3;
  if (h.use_clip) {
    af_usq_kernel<<<egrid, kAfThreads, 0, st>>>(static_cast<const float*>(g), a.rf, a.cf, a.scal,
                                                R, C);
    ++launched;
  }
  af_apply_kernel<true><<<egrid, kAfThreads, 0, st>>>(
      static_cast<float*>(p), static_cast<const float*>(g), a.rf, a.cf, nullptr,
      static_cast<float*>(m), static_cast<__nv_bfloat16*>(p_bf16), ld_bf16, bf16_batch_stride,
      a.scal, R, C, static_cast<float>(n), h);
  count_launches(launched + 1);
  return af_check("adafactor_factored_static");
}
