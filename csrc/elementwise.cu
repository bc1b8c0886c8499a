// Bandwidth-bound kernels of the T5 block: RMSNorm forward/backward (with the
// residual gradient folded in), gated-GELU backward, embedding gather and its
// scatter-add backward, and fp32->bf16 casts. All are written as grid-stride /
// persistent loops sized from the SM count, with 16-byte vector accesses.
#include "common.cuh"

namespace t5x {

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.f;
  if (warp == 0) {
    t = warp_sum(t);
    if (lane == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}

struct alignas(16) Bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void unpack8(const Bf16x8& p, float* f) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ Bf16x8 pack8(const float* f) {
  Bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}

// ---------------------------------------------------------------------------
// RMSNorm forward: y = x * rsqrt(mean(x^2) + eps) * scale      (fp32 statistics)
// One CTA per row at a time (grid-stride over rows). d % 8 == 0.
// ---------------------------------------------------------------------------
constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 4;  // up to 256*8*4 = 8192 features kept in registers

__global__ void __launch_bounds__(kNormThreads)
    rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ scale,
                       __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out, int rows, int d,
                       float eps) {
  __shared__ float red[32];
  const int nvec = d / 8;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const Bf16x8* xr = reinterpret_cast<const Bf16x8*>(x + static_cast<long long>(row) * d);
    float vals[kNormMaxVec][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        unpack8(xr[v], vals[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
      }
    }
    const float tot = block_sum(ss, red);
    const float rstd = rsqrtf(tot / static_cast<float>(d) + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
    Bf16x8* yr = reinterpret_cast<Bf16x8*>(y + static_cast<long long>(row) * d);
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        const float4 s0 = reinterpret_cast<const float4*>(scale)[2 * v];
        const float4 s1 = reinterpret_cast<const float4*>(scale)[2 * v + 1];
        const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * rstd * sc[j];
        yr[v] = pack8(o);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// RMSNorm backward.
//   g = dy * scale ;  dx = rstd * (g - x * rstd^2 * mean(g * x)) (+ dres)
//   dscale[j] += sum_rows dy * x * rstd            (per-CTA partial sums, then one reduction)
// ---------------------------------------------------------------------------
// NV = 16-byte vectors per thread (d <= 2048 * NV). Operands stay packed (bf16) in registers
// between the two passes over a row and the scale is re-read from L1, so that four CTAs fit an
// SM for d <= 4096: the kernel is bound by how many rows are in flight. The per-feature sums
// for dscale are kept in registers over the CTA's rows and written to `partial`
// ([gridDim.x, d], plain stores); rmsnorm_dscale_reduce_kernel adds them up.
template <int NV>
__global__ void __launch_bounds__(kNormThreads, NV <= 2 ? 4 : 2)
    rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                       const float* __restrict__ scale, const float* __restrict__ rstd_in,
                       const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                       float* __restrict__ partial, int rows, int d) {
  __shared__ float red[32];
  const int nvec = d / 8;
  float ds_acc[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) ds_acc[i][j] = 0.f;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const long long off = static_cast<long long>(row) * d;
    const Bf16x8* xr = reinterpret_cast<const Bf16x8*>(x + off);
    const Bf16x8* dyr = reinterpret_cast<const Bf16x8*>(dy + off);
    Bf16x8 xp[NV], dyp[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {  // all loads of the row before the first use
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        xp[i] = xr[v];
        dyp[i] = dyr[v];
      }
    }
    const float rstd = rstd_in[row];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float xv[8], dyv[8];
        unpack8(xp[i], xv);
        unpack8(dyp[i], dyv);
        const float4 s0 = reinterpret_cast<const float4*>(scale)[2 * v];
        const float4 s1 = reinterpret_cast<const float4*>(scale)[2 * v + 1];
        const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float t = dyv[j] * xv[j];
          ds_acc[i][j] += t * rstd;
          dot += t * sc[j];
        }
      }
    }
    const float tot = block_sum(dot, red);
    const float c = tot / static_cast<float>(d) * rstd * rstd;
    Bf16x8* dxr = reinterpret_cast<Bf16x8*>(dx + off);
    const Bf16x8* rr = dres ? reinterpret_cast<const Bf16x8*>(dres + off) : nullptr;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float xv[8], dyv[8], o[8];
        unpack8(xp[i], xv);
        unpack8(dyp[i], dyv);
        const float4 s0 = reinterpret_cast<const float4*>(scale)[2 * v];
        const float4 s1 = reinterpret_cast<const float4*>(scale)[2 * v + 1];
        const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (dyv[j] * sc[j] - xv[j] * c);
        if (rr) {
          float r8[8];
          unpack8(rr[v], r8);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r8[j];
        }
        dxr[v] = pack8(o);
      }
    }
  }
  if (partial) {
    float* out = partial + static_cast<long long>(blockIdx.x) * d;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        reinterpret_cast<float4*>(out)[2 * v] =
            make_float4(ds_acc[i][0], ds_acc[i][1], ds_acc[i][2], ds_acc[i][3]);
        reinterpret_cast<float4*>(out)[2 * v + 1] =
            make_float4(ds_acc[i][4], ds_acc[i][5], ds_acc[i][6], ds_acc[i][7]);
      }
    }
  }
}

// dscale[j] += sum over the CTAs of partial[cta][j]. One CTA per 32 features: 8 warps split the
// `parts` rows between them (each load is one 128-byte line), then add up through shared memory.
__global__ void __launch_bounds__(256)
    rmsnorm_dscale_reduce_kernel(const float* __restrict__ partial, int parts, int d,
                                 float* __restrict__ dscale) {
  __shared__ float red[8][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int j = blockIdx.x * 32 + lane;
  float a0 = 0.f, a1 = 0.f;
  if (j < d) {
    int p = warp;
    for (; p + 8 < parts; p += 16) {
      a0 += partial[static_cast<long long>(p) * d + j];
      a1 += partial[static_cast<long long>(p + 8) * d + j];
    }
    if (p < parts) a0 += partial[static_cast<long long>(p) * d + j];
  }
  red[warp][lane] = a0 + a1;
  __syncthreads();
  if (warp == 0 && j < d) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[w][lane];
    dscale[j] += t;
  }
}

// ---------------------------------------------------------------------------
// RMSNorm for narrow rows (d <= 1024): one warp per row, eight rows per CTA, reductions by
// shuffles only. With one CTA per row most of its 256 threads would idle (d = 768 is 96
// 16-byte vectors) and every row would cost three block barriers.
// ---------------------------------------------------------------------------
constexpr int kNormWarpMaxVec = 4;  // 32 lanes x 4 vectors x 8 = 1024 features

__global__ void __launch_bounds__(kNormThreads)
    rmsnorm_fwd_warp_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ scale,
                            __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out, int rows,
                            int d, float eps) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = d / 8;
  const int wpb = kNormThreads / 32;
  for (int row = blockIdx.x * wpb + warp; row < rows; row += gridDim.x * wpb) {
    const Bf16x8* xr = reinterpret_cast<const Bf16x8*>(x + static_cast<long long>(row) * d);
    float vals[kNormWarpMaxVec][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kNormWarpMaxVec; ++i) {
      const int v = lane + i * 32;
      if (v < nvec) {
        unpack8(xr[v], vals[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
      }
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / static_cast<float>(d) + eps);
    if (lane == 0 && rstd_out) rstd_out[row] = rstd;
    Bf16x8* yr = reinterpret_cast<Bf16x8*>(y + static_cast<long long>(row) * d);
#pragma unroll
    for (int i = 0; i < kNormWarpMaxVec; ++i) {
      const int v = lane + i * 32;
      if (v < nvec) {
        const float4 s0 = reinterpret_cast<const float4*>(scale)[2 * v];
        const float4 s1 = reinterpret_cast<const float4*>(scale)[2 * v + 1];
        const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * rstd * sc[j];
        yr[v] = pack8(o);
      }
    }
  }
}

__global__ void __launch_bounds__(kNormThreads)
    rmsnorm_bwd_warp_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                            const float* __restrict__ scale, const float* __restrict__ rstd_in,
                            const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                            float* __restrict__ partial, int rows, int d) {
  __shared__ float sacc[kNormThreads / 32][kNormWarpMaxVec * 32 * 8 / 4];  // one quarter at a time
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = d / 8;
  const int wpb = kNormThreads / 32;
  float ds_acc[kNormWarpMaxVec][8];
#pragma unroll
  for (int i = 0; i < kNormWarpMaxVec; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) ds_acc[i][j] = 0.f;
  for (int row = blockIdx.x * wpb + warp; row < rows; row += gridDim.x * wpb) {
    const long long off = static_cast<long long>(row) * d;
    const Bf16x8* xr = reinterpret_cast<const Bf16x8*>(x + off);
    const Bf16x8* dyr = reinterpret_cast<const Bf16x8*>(dy + off);
    Bf16x8 xp[kNormWarpMaxVec], dyp[kNormWarpMaxVec];
#pragma unroll
    for (int i = 0; i < kNormWarpMaxVec; ++i) {
      const int v = lane + i * 32;
      if (v < nvec) {
        xp[i] = xr[v];
        dyp[i] = dyr[v];
      }
    }
    const float rstd = rstd_in[row];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kNormWarpMaxVec; ++i) {
      const int v = lane + i * 32;
      if (v < nvec) {
        float xv[8], dyv[8];
        unpack8(xp[i], xv);
        unpack8(dyp[i], dyv);
        const float4 s0 = reinterpret_cast<const float4*>(scale)[2 * v];
        const float4 s1 = reinterpret_cast<const float4*>(scale)[2 * v + 1];
        const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float t = dyv[j] * xv[j];
          ds_acc[i][j] += t * rstd;
          dot += t * sc[j];
        }
      }
    }
    dot = warp_sum(dot);
    const float c = dot / static_cast<float>(d) * rstd * rstd;
    Bf16x8* dxr = reinterpret_cast<Bf16x8*>(dx + off);
    const Bf16x8* rr = dres ? reinterpret_cast<const Bf16x8*>(dres + off) : nullptr;
#pragma unroll
    for (int i = 0; i < kNormWarpMaxVec; ++i) {
      const int v = lane + i * 32;
      if (v < nvec) {
        float xv[8], dyv[8], o[8];
        unpack8(xp[i], xv);
        unpack8(dyp[i], dyv);
        const float4 s0 = reinterpret_cast<const float4*>(scale)[2 * v];
        const float4 s1 = reinterpret_cast<const float4*>(scale)[2 * v + 1];
        const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (dyv[j] * sc[j] - xv[j] * c);
        if (rr) {
          float r8[8];
          unpack8(rr[v], r8);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r8[j];
        }
        dxr[v] = pack8(o);
      }
    }
  }
  if (partial) {
    // the eight warps hold sums for the same features: add them through shared memory, one
    // vector slot (32 lanes x 8 features) at a time
    float* out = partial + static_cast<long long>(blockIdx.x) * d;
#pragma unroll
    for (int i = 0; i < kNormWarpMaxVec; ++i) {
      __syncthreads();
#pragma unroll
      for (int j = 0; j < 8; ++j) sacc[warp][lane * 8 + j] = ds_acc[i][j];
      __syncthreads();
      const int f = threadIdx.x;  // feature within the slot: 256 per slot
      const int col = i * 256 + f;
      if (col < d) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < kNormThreads / 32; ++w) t += sacc[w][f];
        out[col] = t;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Gated-GELU backward. h = [h0 | h1] with row stride ldh (h1 at column offset `dff`).
//   in : dg [T, dff] (grad of g = gelu(h0) * h1)
//   out: h0 <- dg * h1 * gelu'(h0) ; h1 <- dg * gelu(h0) ; dg <- g  (recomputed activation,
//        needed by the wgrad of the following projection) when write_g is set
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
    gated_gelu_bwd_kernel(__nv_bfloat16* __restrict__ dg, __nv_bfloat16* __restrict__ h, long long rows,
                          int dff, long long ldh, long long ldg, int write_g) {
  const int nvec = dff / 8;
  const long long total = rows * nvec;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / nvec;
    const int v = static_cast<int>(i - r * nvec);
    Bf16x8* p0 = reinterpret_cast<Bf16x8*>(h + r * ldh) + v;
    Bf16x8* p1 = reinterpret_cast<Bf16x8*>(h + r * ldh + dff) + v;
    Bf16x8* pg = reinterpret_cast<Bf16x8*>(dg + r * ldg) + v;
    float a[8], b[8], g[8], o0[8], o1[8], og[8];
    unpack8(*p0, a);
    unpack8(*p1, b);
    unpack8(*pg, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float ge = gelu_tanh(a[j]);
      o0[j] = g[j] * b[j] * gelu_tanh_grad(a[j]);
      o1[j] = g[j] * ge;
      og[j] = ge * b[j];
    }
    *p0 = pack8(o0);
    *p1 = pack8(o1);
    if (write_g) *pg = pack8(og);
  }
}

// Gated-GELU forward on separate pre-activations (used when the GEMM epilogue is not).
__global__ void __launch_bounds__(256)
    gated_gelu_fwd_kernel(const __nv_bfloat16* __restrict__ h, __nv_bfloat16* __restrict__ g,
                          long long rows, int dff, long long ldh, long long ldg) {
  const int nvec = dff / 8;
  const long long total = rows * nvec;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / nvec;
    const int v = static_cast<int>(i - r * nvec);
    float a[8], b[8], o[8];
    unpack8(reinterpret_cast<const Bf16x8*>(h + r * ldh)[v], a);
    unpack8(reinterpret_cast<const Bf16x8*>(h + r * ldh + dff)[v], b);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = gelu_tanh(a[j]) * b[j];
    reinterpret_cast<Bf16x8*>(g + r * ldg)[v] = pack8(o);
  }
}

// ---------------------------------------------------------------------------
// Embedding gather (bf16 table) and scatter-add backward into an fp32 gradient.
// Ids outside [vocab_start, vocab_start + vocab_rows) produce zeros / are skipped:
// that is the vocab-parallel form (each rank owns a slice of the table).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
    embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                         __nv_bfloat16* __restrict__ out, long long tokens, int d, int vocab_start,
                         int vocab_rows) {
  const int nvec = d / 8;
  const long long total = tokens * nvec;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / nvec;
    const int v = static_cast<int>(i - t * nvec);
    const long long id = ids[t] - vocab_start;
    Bf16x8 val;
    if (id >= 0 && id < vocab_rows) {
      val = reinterpret_cast<const Bf16x8*>(table + id * d)[v];
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) val.v[j] = __floats2bfloat162_rn(0.f, 0.f);
    }
    reinterpret_cast<Bf16x8*>(out + t * d)[v] = val;
  }
}

__global__ void __launch_bounds__(256)
    embedding_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dout,
                         float* __restrict__ dtable, long long tokens, int d, int vocab_start,
                         int vocab_rows) {
  const int nvec = d / 8;
  const long long total = tokens * nvec;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / nvec;
    const int v = static_cast<int>(i - t * nvec);
    const long long id = ids[t] - vocab_start;
    if (id < 0 || id >= vocab_rows) continue;
    float f[8];
    unpack8(reinterpret_cast<const Bf16x8*>(dout + t * d)[v], f);
    float* dst = dtable + id * d + v * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(dst + j, f[j]);
  }
}

// fp32 -> bf16 cast with independent leading dimensions (to fill slices of fused weights).
__global__ void __launch_bounds__(256)
    cast_f32_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long rows,
                         int cols, long long lds, long long ldd) {
  const int nvec = cols / 4;
  const long long total = rows * nvec;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / nvec;
    const int v = static_cast<int>(i - r * nvec);
    const float4 f = reinterpret_cast<const float4*>(src + r * lds)[v];
    __nv_bfloat162 a = __floats2bfloat162_rn(f.x, f.y), b = __floats2bfloat162_rn(f.z, f.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&b);
    reinterpret_cast<uint2*>(dst + r * ldd)[v] = u;
  }
}

static inline int ew_grid(long long work_items, int threads) {
  long long blocks = (work_items + threads - 1) / threads;
  long long cap = static_cast<long long>(num_sms()) * 8;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace t5x

using namespace t5x;

#define CHECK_LAUNCH(name)                                                           \
  do {                                                                               \
    count_launches(1);                                                               \
    cudaError_t e__ = cudaGetLastError();                                            \
    if (e__ != cudaSuccess) return set_error(name ": %s", cudaGetErrorString(e__)); \
  } while (0)

T5X_API int t5x_rmsnorm_fwd(const void* x, const void* scale, void* y, void* rstd, int rows, int d,
                            float eps, void* stream) {
  if (rows <= 0) return 0;
  if (d % 8 || d > kNormThreads * 8 * kNormMaxVec)
    return set_error("rmsnorm: d=%d must be a multiple of 8 and <= %d", d,
                     kNormThreads * 8 * kNormMaxVec);
  if (d <= kNormWarpMaxVec * 32 * 8) {  // narrow rows: one warp per row
    const int wpb = kNormThreads / 32;
    int blocks = (rows + wpb - 1) / wpb;
    if (blocks > num_sms() * 8) blocks = num_sms() * 8;
    rmsnorm_fwd_warp_kernel<<<blocks, kNormThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<const float*>(scale),
        static_cast<__nv_bfloat16*>(y), static_cast<float*>(rstd), rows, d, eps);
    CHECK_LAUNCH("rmsnorm_fwd");
    return 0;
  }
  int grid = rows < num_sms() * 8 ? rows : num_sms() * 8;
  rmsnorm_fwd_kernel<<<grid, kNormThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const float*>(scale),
      static_cast<__nv_bfloat16*>(y), static_cast<float*>(rstd), rows, d, eps);
  CHECK_LAUNCH("rmsnorm_fwd");
  return 0;
}

T5X_API int t5x_rmsnorm_bwd(const void* dy, const void* x, const void* scale, const void* rstd,
                            const void* dres, void* dx, void* dscale, int rows, int d,
                            void* stream) {
  if (rows <= 0) return 0;
  if (d % 8 || d > kNormThreads * 8 * kNormMaxVec)
    return set_error("rmsnorm: d=%d must be a multiple of 8 and <= %d", d,
                     kNormThreads * 8 * kNormMaxVec);
  // Workspace for the per-CTA dscale sums: one buffer per device, allocated at the first call
  // (so not under stream capture) and shared by all calls: backward passes on one stream.
  constexpr int kMaxParts = 1024;
  static float* ws[64] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dscale != nullptr && ws[dev] == nullptr) {
    if (cudaMalloc(&ws[dev], sizeof(float) * kMaxParts * kNormThreads * 8 * kNormMaxVec) !=
        cudaSuccess)
      return set_error("rmsnorm_bwd: workspace allocation failed");
  }
  const int nv = d <= 2048 ? 1 : (d <= 4096 ? 2 : 4);
  int grid = num_sms() * (nv <= 2 ? 4 : 2);
  if (grid > rows) grid = rows;
  if (grid > kMaxParts) grid = kMaxParts;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* partial = dscale != nullptr ? ws[dev] : nullptr;
  auto launch = [&](auto kernel) {
    kernel<<<grid, kNormThreads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
        static_cast<const float*>(scale), static_cast<const float*>(rstd),
        static_cast<const __nv_bfloat16*>(dres), static_cast<__nv_bfloat16*>(dx), partial, rows, d);
  };
  if (d <= kNormWarpMaxVec * 32 * 8) {  // narrow rows: one warp per row, eight rows per CTA
    const int wpb = kNormThreads / 32;
    grid = (rows + wpb - 1) / wpb;
    if (grid > num_sms() * 4) grid = num_sms() * 4;
    if (grid > kMaxParts) grid = kMaxParts;
    launch(rmsnorm_bwd_warp_kernel);
  } else if (nv == 1) launch(rmsnorm_bwd_kernel<1>);
  else if (nv == 2) launch(rmsnorm_bwd_kernel<2>);
  else launch(rmsnorm_bwd_kernel<4>);
  if (dscale != nullptr) {
    count_launches(1);
    rmsnorm_dscale_reduce_kernel<<<(d + 31) / 32, 256, 0, st>>>(partial, grid, d,
                                                                  static_cast<float*>(dscale));
  }
  CHECK_LAUNCH("rmsnorm_bwd");
  return 0;
}

T5X_API int t5x_gated_gelu_bwd(void* dg, void* h, long long rows, int dff, long long ldh,
                               long long ldg, int write_g, void* stream) {
  if (rows <= 0) return 0;
  if (dff % 8 || ldh % 8 || ldg % 8) return set_error("gated_gelu: sizes must be multiples of 8");
  gated_gelu_bwd_kernel<<<ew_grid(rows * (dff / 8), 256), 256, 0,
                          static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(dg), static_cast<__nv_bfloat16*>(h), rows, dff, ldh, ldg, write_g);
  CHECK_LAUNCH("gated_gelu_bwd");
  return 0;
}

T5X_API int t5x_gated_gelu_fwd(const void* h, void* g, long long rows, int dff, long long ldh,
                               long long ldg, void* stream) {
  if (rows <= 0) return 0;
  if (dff % 8 || ldh % 8 || ldg % 8) return set_error("gated_gelu: sizes must be multiples of 8");
  gated_gelu_fwd_kernel<<<ew_grid(rows * (dff / 8), 256), 256, 0,
                          static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(h), static_cast<__nv_bfloat16*>(g), rows, dff, ldh, ldg);
  CHECK_LAUNCH("gated_gelu_fwd");
  return 0;
}

T5X_API int t5x_embedding_fwd(const void* ids, const void* table, void* out, long long tokens, int d,
                              int vocab_start, int vocab_rows, void* stream) {
  if (tokens <= 0) return 0;
  if (d % 8) return set_error("embedding: d must be a multiple of 8");
  embedding_fwd_kernel<<<ew_grid(tokens * (d / 8), 256), 256, 0,
                         static_cast<cudaStream_t>(stream)>>>(
      static_cast<const long long*>(ids), static_cast<const __nv_bfloat16*>(table),
      static_cast<__nv_bfloat16*>(out), tokens, d, vocab_start, vocab_rows);
  CHECK_LAUNCH("embedding_fwd");
  return 0;
}

T5X_API int t5x_embedding_bwd(const void* ids, const void* dout, void* dtable, long long tokens,
                              int d, int vocab_start, int vocab_rows, void* stream) {
  if (tokens <= 0) return 0;
  if (d % 8) return set_error("embedding: d must be a multiple of 8");
  embedding_bwd_kernel<<<ew_grid(tokens * (d / 8), 256), 256, 0,
                         static_cast<cudaStream_t>(stream)>>>(
      static_cast<const long long*>(ids), static_cast<const __nv_bfloat16*>(dout),
      static_cast<float*>(dtable), tokens, d, vocab_start, vocab_rows);
  CHECK_LAUNCH("embedding_bwd");
  return 0;
}

T5X_API int t5x_cast_f32_bf16(const void* src, void* dst, long long rows, int cols, long long lds,
                              long long ldd, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (cols % 4 || lds % 4 || ldd % 4) return set_error("cast: sizes must be multiples of 4");
  cast_f32_bf16_kernel<<<ew_grid(rows * (cols / 4), 256), 256, 0,
                         static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(src), static_cast<__nv_bfloat16*>(dst), rows, cols, lds, ldd);
  CHECK_LAUNCH("cast");
  return 0;
}


// dst[i] = bf16(src[i] (+ residual[i])): finishes a split-K GEMM whose partial products were
// added into an fp32 workspace. With kClear the workspace is left zero, ready for the next GEMM
// that accumulates into it (no separate fill kernel).
namespace t5x {
template <bool kClear>
__global__ void __launch_bounds__(256)
    f32_to_bf16_residual_kernel(float* __restrict__ src, const __nv_bfloat16* __restrict__ res,
                                __nv_bfloat16* __restrict__ dst, long long n4) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  chain_release();
  chain_wait();  // the sums in src come from the kernel before this one
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += stride) {
    float4 a = reinterpret_cast<const float4*>(src)[i];
    if (kClear) reinterpret_cast<float4*>(src)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (res != nullptr) {
      const uint2 r = reinterpret_cast<const uint2*>(res)[i];
      const float2 r0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
      const float2 r1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
      a.x += r0.x;
      a.y += r0.y;
      a.z += r1.x;
      a.w += r1.y;
    }
    __nv_bfloat162 lo = __floats2bfloat162_rn(a.x, a.y), hi = __floats2bfloat162_rn(a.z, a.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&lo);
    o.y = *reinterpret_cast<uint32_t*>(&hi);
    reinterpret_cast<uint2*>(dst)[i] = o;
  }
}
}  // namespace t5x

// n must be a multiple of 4; all pointers 16-byte (src) / 8-byte (res, dst) aligned.
T5X_API int t5x_f32_to_bf16_residual(const void* src, const void* residual, void* dst,
                                     long long n, void* stream) {
  if (n <= 0) return 0;
  if (n % 4) return t5x::set_error("f32_to_bf16_residual: n must be a multiple of 4");
  const long long n4 = n / 4;
  long long blocks = (n4 + 255) / 256;
  const long long cap = static_cast<long long>(t5x::num_sms()) * 8;
  if (blocks > cap) blocks = cap;
  cudaError_t e = t5x::launch_chained(
      t5x::f32_to_bf16_residual_kernel<false>, dim3(static_cast<int>(blocks)), dim3(256), 0,
      static_cast<cudaStream_t>(stream), static_cast<float*>(const_cast<void*>(src)),
      static_cast<const __nv_bfloat16*>(residual), static_cast<__nv_bfloat16*>(dst), n4);
  t5x::count_launches(1);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return t5x::set_error("f32_to_bf16_residual: %s", cudaGetErrorString(e));
  return 0;
}

// The same, and src[0..n) is zero afterwards.
T5X_API int t5x_f32_to_bf16_residual_clear(void* src, const void* residual, void* dst, long long n,
                                           void* stream) {
  if (n <= 0) return 0;
  if (n % 4) return t5x::set_error("f32_to_bf16_residual_clear: n must be a multiple of 4");
  const long long n4 = n / 4;
  long long blocks = (n4 + 255) / 256;
  const long long cap = static_cast<long long>(t5x::num_sms()) * 8;
  if (blocks > cap) blocks = cap;
  cudaError_t e = t5x::launch_chained(
      t5x::f32_to_bf16_residual_kernel<true>, dim3(static_cast<int>(blocks)), dim3(256), 0,
      static_cast<cudaStream_t>(stream), static_cast<float*>(src),
      static_cast<const __nv_bfloat16*>(residual), static_cast<__nv_bfloat16*>(dst), n4);
  t5x::count_launches(1);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess)
    return t5x::set_error("f32_to_bf16_residual_clear: %s", cudaGetErrorString(e));
  return 0;
}

// Finishes a split-K GEMM and applies the RMSNorm that follows it, one CTA per row:
//   x[row] = bf16(ws[row] + residual[row]);  ws[row] = 0;  h[row] = x[row] * rstd * scale
// with rstd taken from the rounded x, exactly as the separate norm kernel would see it. For the
// decode step, where every residual projection is followed by a norm: one launch instead of two.
namespace t5x {
__global__ void __launch_bounds__(kNormThreads)
    finish_residual_rmsnorm_kernel(float* __restrict__ ws, const __nv_bfloat16* __restrict__ res,
                                   const float* __restrict__ scale, __nv_bfloat16* __restrict__ x,
                                   __nv_bfloat16* __restrict__ h, int d, float eps) {
  __shared__ float red[32];
  const int nvec = d / 8;
  const long long row = blockIdx.x;
  float vals[kNormMaxVec][8];
  float ss = 0.f;
  chain_release();
  chain_wait();  // the sums in ws come from the kernel before this one
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
      float4* src = reinterpret_cast<float4*>(ws + row * d) + 2 * v;
      const float4 a = src[0], b = src[1];
      src[0] = make_float4(0.f, 0.f, 0.f, 0.f);
      src[1] = make_float4(0.f, 0.f, 0.f, 0.f);
      float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
      if (res != nullptr) {
        float r[8];
        unpack8(reinterpret_cast<const Bf16x8*>(res + row * d)[v], r);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += r[j];
      }
      const Bf16x8 packed = pack8(f);
      reinterpret_cast<Bf16x8*>(x + row * d)[v] = packed;
      unpack8(packed, vals[i]);  // the norm sees the rounded values
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
    }
  }
  const float tot = block_sum(ss, red);
  const float rstd = rsqrtf(tot / static_cast<float>(d) + eps);
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
      const float4 s0 = reinterpret_cast<const float4*>(scale)[2 * v];
      const float4 s1 = reinterpret_cast<const float4*>(scale)[2 * v + 1];
      const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * rstd * sc[j];
      reinterpret_cast<Bf16x8*>(h + row * d)[v] = pack8(o);
    }
  }
}
}  // namespace t5x

// ws [rows, d] fp32 (cleared on return), residual [rows, d] bf16 or null, scale [d] fp32 ->
// x [rows, d] bf16 and h = rmsnorm(x) [rows, d] bf16. d a multiple of 8, d <= 8192.
T5X_API int t5x_finish_residual_rmsnorm(void* ws, const void* residual, const void* scale,
                                        void* x, void* h, int rows, int d, float eps,
                                        void* stream) {
  using namespace t5x;
  if (rows <= 0) return 0;
  if (d % 8 || d > kNormThreads * 8 * kNormMaxVec)
    return set_error("finish_residual_rmsnorm: d=%d must be a multiple of 8 and <= %d", d,
                     kNormThreads * 8 * kNormMaxVec);
  if (ws == nullptr || scale == nullptr || x == nullptr || h == nullptr)
    return set_error("finish_residual_rmsnorm: null pointer");
  cudaError_t e = launch_chained(
      finish_residual_rmsnorm_kernel, dim3(rows), dim3(kNormThreads), 0,
      static_cast<cudaStream_t>(stream), static_cast<float*>(ws),
      static_cast<const __nv_bfloat16*>(residual), static_cast<const float*>(scale),
      static_cast<__nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(h), d, eps);
  count_launches(1);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("finish_residual_rmsnorm: %s", cudaGetErrorString(e));
  return 0;
}

// dst[i] = bf16(sum over s of slots[s * n + i] (+ residual[i])) with fp32 accumulation: the
// owner's side of the tensor-parallel reduce-scatter (`slots` is its inbox, one slot per rank).
namespace t5x {
struct SlotSumWait {
  const unsigned int* sig;  // this rank's "scattered" words, one per rank; null: no wait
  int world, rank;
  unsigned int epoch;
  int* status;
};
constexpr int kSlotSumSpinLimit = 1 << 24;  // polls >= 64 ns apart: 1-3 s

__global__ void __launch_bounds__(256)
    slot_sum_bf16_kernel(const __nv_bfloat16* __restrict__ slots, int num_slots, long long n8,
                         const __nv_bfloat16* __restrict__ res, __nv_bfloat16* __restrict__ dst,
                         const SlotSumWait w) {
  if (w.sig != nullptr) {
    // every peer's reduce-scatter GEMM has performed all its stores into this rank's inbox
    if (threadIdx.x < w.world && threadIdx.x != w.rank) {
      const unsigned int* word = w.sig + threadIdx.x;
      bool here = false;
      for (int it = 0; it < kSlotSumSpinLimit; ++it) {
        unsigned int v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(word) : "memory");
        if (static_cast<int>(v - w.epoch) >= 0) {
          here = true;
          break;
        }
        __nanosleep(64);
      }
      if (!here) report_status(w.status, kStatusTimeoutPeerFlag, 41, threadIdx.x,
                               static_cast<int>(w.epoch));
    }
    __syncthreads();
  }
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += stride) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    if (res != nullptr) {
      const uint4 u = reinterpret_cast<const uint4*>(res)[i];
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(p[j]);
        acc[2 * j] = f.x;
        acc[2 * j + 1] = f.y;
      }
    }
    for (int s = 0; s < num_slots; ++s) {
      const uint4 u = reinterpret_cast<const uint4*>(slots)[s * n8 + i];
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(p[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) q[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    reinterpret_cast<uint4*>(dst)[i] = o;
  }
}
}  // namespace t5x

// n (elements per slot) must be a multiple of 8; pointers 16-byte aligned.
T5X_API int t5x_slot_sum_bf16(const void* slots, int num_slots, long long n, const void* residual,
                              void* dst, void* stream) {
  using namespace t5x;
  if (n <= 0) return 0;
  if (n % 8 || num_slots < 1) return set_error("slot_sum_bf16: n must be a multiple of 8");
  const long long n8 = n / 8;
  long long blocks = (n8 + 255) / 256;
  const long long cap = static_cast<long long>(num_sms()) * 8;
  if (blocks > cap) blocks = cap;
  slot_sum_bf16_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(slots), num_slots, n8,
      static_cast<const __nv_bfloat16*>(residual), static_cast<__nv_bfloat16*>(dst),
      SlotSumWait{nullptr, 0, 0, 0u, nullptr});
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("slot_sum_bf16: %s", cudaGetErrorString(e));
  return 0;
}

// The same sum, preceded (inside the kernel) by a bounded wait until every other rank's
// reduce-scatter GEMM of epoch `epoch` has raised its "scattered" signal: `sig` points at this
// rank's `world` signal words of that kind. Takes the place of a barrier kernel between the
// GEMM and the sum.
T5X_API int t5x_slot_sum_wait_bf16(const void* slots, int num_slots, long long n,
                                   const void* residual, void* dst, const void* sig, int world,
                                   int rank, unsigned int epoch, void* stream) {
  using namespace t5x;
  if (n <= 0) return 0;
  if (n % 8 || num_slots < 1) return set_error("slot_sum_wait_bf16: n must be a multiple of 8");
  if (sig == nullptr || world < 1 || world > 256 || rank < 0 || rank >= world)
    return set_error("slot_sum_wait_bf16: bad signal arguments");
  const long long n8 = n / 8;
  long long blocks = (n8 + 255) / 256;
  const long long cap = static_cast<long long>(num_sms()) * 8;
  if (blocks > cap) blocks = cap;
  slot_sum_bf16_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(slots), num_slots, n8,
      static_cast<const __nv_bfloat16*>(residual), static_cast<__nv_bfloat16*>(dst),
      SlotSumWait{static_cast<const unsigned int*>(sig), world, rank, epoch,
                  device_status_buffer()});
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("slot_sum_wait_bf16: %s", cudaGetErrorString(e));
  return 0;
}
