// Declarations shared by the attention kernels (attention_sm100.cu: forward for short key
// ranges and the backward pass; attention_fwd_sm100.cu: the streaming forward pass).
#pragma once
#include "common.cuh"

namespace t5x {

constexpr int kAttnD = 64;
constexpr int kSoftmaxWarps = 16;
constexpr int kSoftmaxThreads = kSoftmaxWarps * 32;
constexpr int kAttnThreads = kSoftmaxThreads + 32;  // + 1 warp: TMA + MMA issue, TMEM owner
constexpr int kCtrlWarp = kSoftmaxWarps;
constexpr int kKernelIdAttnFwd = 2;
constexpr int kKernelIdAttnBwd = 3;
constexpr float kMaskValue = -1e10f;
constexpr float kLog2e = 1.4426950408889634f;

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
  asm volatile("bar.sync 1, %0;" ::"n"(kSoftmaxThreads) : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}

// Writes 8 consecutive bf16 (one 16-byte chunk) of row r, chunk c (0..7) of a [128 x 64] K-major
// 128B-swizzled tile.
__device__ __forceinline__ void store_swizzled_chunk(uint8_t* tile, int r, int c, const float* v) {
  uint4 u;
  u.x = pack_bf16x2(v[0], v[1]);
  u.y = pack_bf16x2(v[2], v[3]);
  u.z = pack_bf16x2(v[4], v[5]);
  u.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(tile + r * 128 + ((c ^ (r & 7)) << 4)) = u;
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}

// 16 fp32 values -> 16 bf16 written as two 16-byte stores.
__device__ __forceinline__ void store16_bf16(__nv_bfloat16* dst, const uint32_t (&v)[16], float scale) {
  uint4 u0, u1;
  u0.x = pack_bf16x2(__uint_as_float(v[0]) * scale, __uint_as_float(v[1]) * scale);
  u0.y = pack_bf16x2(__uint_as_float(v[2]) * scale, __uint_as_float(v[3]) * scale);
  u0.z = pack_bf16x2(__uint_as_float(v[4]) * scale, __uint_as_float(v[5]) * scale);
  u0.w = pack_bf16x2(__uint_as_float(v[6]) * scale, __uint_as_float(v[7]) * scale);
  u1.x = pack_bf16x2(__uint_as_float(v[8]) * scale, __uint_as_float(v[9]) * scale);
  u1.y = pack_bf16x2(__uint_as_float(v[10]) * scale, __uint_as_float(v[11]) * scale);
  u1.z = pack_bf16x2(__uint_as_float(v[12]) * scale, __uint_as_float(v[13]) * scale);
  u1.w = pack_bf16x2(__uint_as_float(v[14]) * scale, __uint_as_float(v[15]) * scale);
  reinterpret_cast<uint4*>(dst)[0] = u0;
  reinterpret_cast<uint4*>(dst)[1] = u1;
}


// Tensor map over a [B, L, H, D] bf16 tensor with element strides (sb, sl, sh): boxes of
// 64 channels x 128 positions of one head (one 128-byte-swizzled shared-memory panel).
inline const CUtensorMap* bhld_map(const void* ptr, int B, int L, int H, long long sb, long long sl,
                                   long long sh, int D = kAttnD) {
  uint64_t dims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(H),
                      static_cast<uint64_t>(L), static_cast<uint64_t>(B)};
  uint64_t strides[3] = {static_cast<uint64_t>(sh) * 2, static_cast<uint64_t>(sl) * 2,
                         static_cast<uint64_t>(sb) * 2};
  uint32_t box[4] = {64, 1, 128, 1};
  return get_tensor_map(ptr, 2, 4, dims, strides, box, 1);
}

}  // namespace t5x
