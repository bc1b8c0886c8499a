// Expert-parallel token exchange of a mixture-of-experts layer over NVLink peer memory.
//
// Every rank routes its own T tokens; (token, choice) pairs that won a slot carry
// `flat_slot = expert * capacity + position` (or -1 when dropped). Expert e lives on rank
// e / E_local, whose exchange buffer is laid out [E_local][EP source ranks][capacity][d].
//
//   moe_scatter : rows (optionally scaled per choice) are stored straight into the owning
//                 rank's buffer - the dispatch all-to-all fused with the routing decision
//                 (forward), or the combine's gradient fused with the gate scaling (backward);
//   moe_gather  : out[t] = sum_choices w * owner_buffer[slot] read straight from the owning
//                 ranks - the combine all-to-all fused with the gate-weighted sum (forward),
//                 or the dispatch's gradient (backward). With `dout` given it instead returns
//                 the gate gradients dot(dout[t], row).
//
// Plain 16-byte loads / stores on peer mappings; callers separate phases with the bounded
// barrier of csrc/comm.cu.
#include "common.cuh"
#include "t5x_b200.h"

namespace t5x {

constexpr int kMoeMaxPeers = 16;
struct MoePeers {
  __nv_bfloat16* p[kMoeMaxPeers];
};

__device__ __forceinline__ long long moe_slot_offset(int flat_slot, int capacity, int e_local,
                                                     int ep, int my_rank, int d, int& owner) {
  const int e = flat_slot / capacity, c = flat_slot - e * capacity;
  owner = e / e_local;
  const int el = e - owner * e_local;
  return ((static_cast<long long>(el) * ep + my_rank) * capacity + c) * d;
}

// One warp per (token, choice); d % 8 == 0.
__global__ void __launch_bounds__(256)
    moe_scatter_kernel(const __nv_bfloat16* __restrict__ rows, const float* __restrict__ scale,
                       const int* __restrict__ flat_slot, MoePeers dst, int T, int k, int capacity,
                       int e_local, int ep, int my_rank, int d) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= T * k) return;
  const int fs = flat_slot[warp];
  if (fs < 0) return;
  const int t = warp / k;
  int owner;
  const long long off = moe_slot_offset(fs, capacity, e_local, ep, my_rank, d, owner);
  const uint4* src = reinterpret_cast<const uint4*>(rows + static_cast<long long>(t) * d);
  uint4* out = reinterpret_cast<uint4*>(dst.p[owner] + off);
  const float s = scale != nullptr ? scale[warp] : 1.f;
  for (int i = lane; i < d / 8; i += 32) {
    uint4 u = src[i];
    if (scale != nullptr) {
      __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 f = __bfloat1622float2(p2[e]);
        p2[e] = __floats2bfloat162_rn(f.x * s, f.y * s);
      }
    }
    out[i] = u;
  }
}

// One warp per token. out (bf16 [T, d]) = sum_j w[t][j] * row_j, or, when `dout` is given,
// dw[t][j] = dot(dout[t], row_j) and `out` is not written.
__global__ void __launch_bounds__(256)
    moe_gather_kernel(__nv_bfloat16* __restrict__ out, float* __restrict__ dw,
                      const __nv_bfloat16* __restrict__ dout, const float* __restrict__ w,
                      const int* __restrict__ flat_slot, MoePeers src, int T, int k, int capacity,
                      int e_local, int ep, int my_rank, int d) {
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (t >= T) return;
  for (int i0 = 0; i0 < d / 8; i0 += 32) {
    const int i = i0 + lane;
    const bool in = i < d / 8;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    float dvec[8];
    if (dout != nullptr && in) {
      const uint4 u = reinterpret_cast<const uint4*>(dout + static_cast<long long>(t) * d)[i];
      const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(p2[e]);
        dvec[2 * e] = f.x;
        dvec[2 * e + 1] = f.y;
      }
    }
    for (int j = 0; j < k; ++j) {
      const int fs = flat_slot[t * k + j];
      float part = 0.f;
      if (fs >= 0 && in) {
        int owner;
        const long long off = moe_slot_offset(fs, capacity, e_local, ep, my_rank, d, owner);
        const uint4 u = reinterpret_cast<const uint4*>(src.p[owner] + off)[i];
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&u);
        const float wj = (w != nullptr) ? w[t * k + j] : 1.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(p2[e]);
          if (dout != nullptr) {
            part = fmaf(dvec[2 * e], f.x, part);
            part = fmaf(dvec[2 * e + 1], f.y, part);
          } else {
            acc[2 * e] = fmaf(wj, f.x, acc[2 * e]);
            acc[2 * e + 1] = fmaf(wj, f.y, acc[2 * e + 1]);
          }
        }
      }
      if (dout != nullptr) {
        part = warp_sum(part);
        if (lane == 0) {
          if (i0 == 0)
            dw[t * k + j] = part;
          else
            dw[t * k + j] += part;
        }
      }
    }
    if (dout == nullptr && in) {
      uint4 o;
      __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) p2[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
      reinterpret_cast<uint4*>(out + static_cast<long long>(t) * d)[i] = o;
    }
  }
}

}  // namespace t5x

using namespace t5x;

static int moe_args_ok(const char* what, int T, int k, int capacity, int e_local, int ep,
                       int my_rank, int d) {
  if (ep < 1 || ep > kMoeMaxPeers || my_rank < 0 || my_rank >= ep)
    return set_error("%s: bad expert-parallel rank %d of %d", what, my_rank, ep);
  if (d % 8 || T < 0 || k < 1 || capacity < 1 || e_local < 1)
    return set_error("%s: bad shape (T=%d k=%d C=%d E_local=%d d=%d; d must be a multiple of 8)",
                     what, T, k, capacity, e_local, d);
  return 0;
}

// rows: [T, d] bf16; scale: [T, k] fp32 or null; flat_slot: [T, k] int32; dst_peers: host array
// of `ep` device pointers to the ranks' [E_local, ep, capacity, d] bf16 exchange buffers.
T5X_API int t5x_moe_scatter(const void* rows, const void* scale, const void* flat_slot,
                            void* const* dst_peers, int T, int k, int capacity, int e_local,
                            int ep, int my_rank, int d, void* stream) {
  if (int rc = moe_args_ok("moe_scatter", T, k, capacity, e_local, ep, my_rank, d)) return rc;
  if (T == 0) return 0;
  MoePeers pp;
  for (int r = 0; r < ep; ++r) pp.p[r] = static_cast<__nv_bfloat16*>(dst_peers[r]);
  const long long warps = static_cast<long long>(T) * k;
  moe_scatter_kernel<<<static_cast<int>((warps + 7) / 8), 256, 0,
                       static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(rows), static_cast<const float*>(scale),
      static_cast<const int*>(flat_slot), pp, T, k, capacity, e_local, ep, my_rank, d);
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("moe_scatter: %s", cudaGetErrorString(e));
  return 0;
}

// out: [T, d] bf16 (written unless dout is given); dw: [T, k] fp32 (written when dout is
// given); w: [T, k] fp32 or null (all ones); src_peers as in t5x_moe_scatter.
T5X_API int t5x_moe_gather(void* out, void* dw, const void* dout, const void* w,
                           const void* flat_slot, void* const* src_peers, int T, int k,
                           int capacity, int e_local, int ep, int my_rank, int d, void* stream) {
  if (int rc = moe_args_ok("moe_gather", T, k, capacity, e_local, ep, my_rank, d)) return rc;
  if (T == 0) return 0;
  MoePeers pp;
  for (int r = 0; r < ep; ++r) pp.p[r] = static_cast<__nv_bfloat16*>(src_peers[r]);
  moe_gather_kernel<<<(T + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(out), static_cast<float*>(dw),
      static_cast<const __nv_bfloat16*>(dout), static_cast<const float*>(w),
      static_cast<const int*>(flat_slot), pp, T, k, capacity, e_local, ep, my_rank, d);
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("moe_gather: %s", cudaGetErrorString(e));
  return 0;
}
