// Fused AdamW step (optax.adamw behind an optional global-norm clip), for the optimizers the
// GPU fine-tuning configurations use (t5x/contrib/gpu/t5/t5_1_1/adamw_opt.gin,
// t5x/optimizers.py:549-570):
//
//   g'  = g * clip_scale                          (clip_scale: device scalar, or 1)
//   mu  = b1 mu + (1 - b1) g'        nu = b2 nu + (1 - b2) g'^2
//   u   = (mu / bc1) / (sqrt(nu / bc2 + eps_root) + eps) + weight_decay * p
//   p  -= lr * u                                  and the bf16 working copy is written
//
// in one pass over the parameter. With optimizer sharding the bf16 result goes to every
// data-parallel rank's working copy (plain peer stores, or one multicast store through the
// switch), as the Adafactor kernels of comm.cu do.
#include "common.cuh"
#include "t5x_b200.h"

namespace t5x {
namespace {

constexpr int kAwThreads = 256;
constexpr int kAwMaxPeers = 16;

struct AwPeers {
  __nv_bfloat16* p[kAwMaxPeers];
};

struct AwHyper {
  float lr, b1, b2, eps, eps_root, weight_decay, bc1, bc2;
};

__device__ __forceinline__ void aw_multimem_st_b32x2(void* mc, uint32_t a, uint32_t b) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"(mc),
               "f"(__uint_as_float(a)), "f"(__uint_as_float(b))
               : "memory");
}

// n4 = n / 4 vectors of four elements; the tail (n % 4) is handled by the scalar kernel.
__global__ void __launch_bounds__(kAwThreads)
    adamw_vec_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ mu,
                     float* __restrict__ nu, AwPeers out, int world, __nv_bfloat16* out_mc,
                     long long n4, const float* __restrict__ clip_scale, AwHyper h) {
  const float cs = clip_scale != nullptr ? *clip_scale : 1.f;
  const long long stride = static_cast<long long>(gridDim.x) * kAwThreads;
  for (long long i = blockIdx.x * static_cast<long long>(kAwThreads) + threadIdx.x; i < n4;
       i += stride) {
    const float4 gv = reinterpret_cast<const float4*>(g)[i];
    const float4 pv = reinterpret_cast<const float4*>(p)[i];
    float4 mv = reinterpret_cast<const float4*>(mu)[i];
    float4 vv = reinterpret_cast<const float4*>(nu)[i];
    float gg[4] = {gv.x * cs, gv.y * cs, gv.z * cs, gv.w * cs};
    float pp[4] = {pv.x, pv.y, pv.z, pv.w};
    float mm[4] = {mv.x, mv.y, mv.z, mv.w};
    float nn[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      mm[k] = h.b1 * mm[k] + (1.f - h.b1) * gg[k];
      nn[k] = h.b2 * nn[k] + (1.f - h.b2) * gg[k] * gg[k];
      const float u = (mm[k] / h.bc1) / (sqrtf(nn[k] / h.bc2 + h.eps_root) + h.eps) +
                      h.weight_decay * pp[k];
      pp[k] -= h.lr * u;
    }
    reinterpret_cast<float4*>(mu)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(nu)[i] = make_float4(nn[0], nn[1], nn[2], nn[3]);
    reinterpret_cast<float4*>(p)[i] = make_float4(pp[0], pp[1], pp[2], pp[3]);
    __nv_bfloat162 lo = __floats2bfloat162_rn(pp[0], pp[1]);
    __nv_bfloat162 hi = __floats2bfloat162_rn(pp[2], pp[3]);
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&lo);
    packed.y = *reinterpret_cast<uint32_t*>(&hi);
    if (out_mc != nullptr)
      aw_multimem_st_b32x2(out_mc + i * 4, packed.x, packed.y);
    else
      for (int d = 0; d < world; ++d) reinterpret_cast<uint2*>(out.p[d])[i] = packed;
  }
}

__global__ void __launch_bounds__(kAwThreads)
    adamw_tail_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ mu,
                      float* __restrict__ nu, AwPeers out, int world, long long begin, long long n,
                      const float* __restrict__ clip_scale, AwHyper h) {
  const float cs = clip_scale != nullptr ? *clip_scale : 1.f;
  const long long i = begin + blockIdx.x * static_cast<long long>(kAwThreads) + threadIdx.x;
  if (i >= n) return;
  const float gg = g[i] * cs;
  const float m = h.b1 * mu[i] + (1.f - h.b1) * gg;
  const float v = h.b2 * nu[i] + (1.f - h.b2) * gg * gg;
  const float pv = p[i];
  const float u = (m / h.bc1) / (sqrtf(v / h.bc2 + h.eps_root) + h.eps) + h.weight_decay * pv;
  const float np = pv - h.lr * u;
  mu[i] = m;
  nu[i] = v;
  p[i] = np;
  for (int d = 0; d < world; ++d) out.p[d][i] = __float2bfloat16(np);
}

}  // namespace
}  // namespace t5x

// One AdamW step over a contiguous fp32 parameter of n elements. bf16_out: `world` device
// pointers to the bf16 working copies to write (world may be 0: none); bf16_mc: multicast
// address of those copies or null. clip_scale: device float that multiplies the gradient (the
// global-norm clip factor) or null. step >= 1 is the count after this update (bias correction).
T5X_API int t5x_adamw_step(void* p, const void* g, void* mu, void* nu, void* const* bf16_out,
                           int world, void* bf16_mc, long long n, float lr, float b1, float b2,
                           float eps, float eps_root, float weight_decay, int step,
                           const void* clip_scale, void* stream) {
  using namespace t5x;
  if (n <= 0) return 0;
  if (p == nullptr || g == nullptr || mu == nullptr || nu == nullptr)
    return set_error("adamw_step: null pointer");
  if (world < 0 || world > kAwMaxPeers || step < 1) return set_error("adamw_step: bad world/step");
  AwPeers out = {};
  bool aligned = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) |
                   reinterpret_cast<uintptr_t>(mu) | reinterpret_cast<uintptr_t>(nu)) & 15) == 0;
  for (int d = 0; d < world; ++d) {
    out.p[d] = static_cast<__nv_bfloat16*>(bf16_out[d]);
    aligned = aligned && (reinterpret_cast<uintptr_t>(out.p[d]) & 7) == 0;
  }
  AwHyper h;
  h.lr = lr;
  h.b1 = b1;
  h.b2 = b2;
  h.eps = eps;
  h.eps_root = eps_root;
  h.weight_decay = weight_decay;
  h.bc1 = 1.f - powf(b1, static_cast<float>(step));
  h.bc2 = 1.f - powf(b2, static_cast<float>(step));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long n4 = aligned ? n / 4 : 0;
  int launched = 0;
  if (n4 > 0) {
    long long blocks = (n4 + kAwThreads - 1) / kAwThreads;
    const long long cap = static_cast<long long>(num_sms()) * 8;
    if (blocks > cap) blocks = cap;
    adamw_vec_kernel<<<static_cast<unsigned>(blocks), kAwThreads, 0, st>>>(
        static_cast<float*>(p), static_cast<const float*>(g), static_cast<float*>(mu),
        static_cast<float*>(nu), out, world, aligned ? static_cast<__nv_bfloat16*>(bf16_mc) : nullptr,
        n4, static_cast<const float*>(clip_scale), h);
    ++launched;
  }
  const long long begin = n4 * 4;
  if (begin < n) {
    const long long rest = n - begin;
    adamw_tail_kernel<<<static_cast<unsigned>((rest + kAwThreads - 1) / kAwThreads), kAwThreads, 0,
                        st>>>(static_cast<float*>(p), static_cast<const float*>(g),
                              static_cast<float*>(mu), static_cast<float*>(nu), out, world, begin,
                              n, static_cast<const float*>(clip_scale), h);
    ++launched;
  }
  count_launches(launched);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("adamw_step: %s", cudaGetErrorString(e));
  return 0;
}
