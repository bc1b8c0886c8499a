// Tensor-parallel decode step: the all-reduce after a row-parallel projection and the gather of
// the vocabulary-sharded logits, over peer mappings of symmetric memory, for a handful of rows
// (batch x beams) where latency, not bandwidth, decides.
//
// Every all-reduce site of the captured decode step has an inbox of its own on every rank
// ([world][n] fp32) and a row of signal words of its own. The split-K GEMM leaves fp32 sums in
// a workspace; `push_partial` stores them (still fp32: a megabyte or two per site, and the sum
// then rounds once, like the single-GPU step) into slot `rank` of every rank's inbox (its own
// included), clears the workspace for the next GEMM, and, from the last CTA to finish, raises
// this rank's signal word on every rank to the current step number.
// `sum_slots` waits (bounded) until all ranks' words have reached the step number and adds the
// slots and the residual in fp32, in the same order on every rank, so all ranks hold bit-identical
// activations. The step number lives in device memory and is advanced by a kernel of the step
// itself, so a captured CUDA graph can be replayed without changing any argument.
//
// Reuse of an inbox one step later is safe without a barrier as long as a step has at least
// two all-reduce sites: before a rank writes site c again it has passed the sum of site c + 1,
// which waited for every peer's push of site c + 1, which those peers issued after their own
// sum of site c.
#include "common.cuh"
#include "t5x_b200.h"

namespace t5x {
namespace {

constexpr int kDtMaxPeers = 16;
constexpr int kDtThreads = 256;
constexpr int kDtSpinLimit = 1 << 23;  // polls >= 64 ns apart: about a second
constexpr int kKernelIdDecodeSum = 61;
constexpr int kKernelIdDecodeWait = 62;

struct DtPeers {
  void* p[kDtMaxPeers];
};

__device__ __forceinline__ void dt_signal(unsigned int* word, unsigned int value) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(word), "r"(value) : "memory");
}

__device__ __forceinline__ unsigned int dt_poll(const unsigned int* word) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(word) : "memory");
  return v;
}

// Threads 0..world-1 of the CTA wait for the peers' words; returns (to all threads) whether
// every word arrived.
__device__ __forceinline__ bool dt_wait_all(const unsigned int* sig, int world, int rank,
                                            unsigned int epoch, int* status, int kernel_id) {
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  if (threadIdx.x < world && static_cast<int>(threadIdx.x) != rank) {
    bool here = false;
    for (int it = 0; it < kDtSpinLimit; ++it) {
      if (static_cast<int>(dt_poll(sig + threadIdx.x) - epoch) >= 0) {
        here = true;
        break;
      }
      __nanosleep(64);
    }
    if (!here) {
      report_status(status, kStatusTimeoutPeerFlag, kernel_id, threadIdx.x, static_cast<int>(epoch));
      failed = 1;
    }
  }
  __syncthreads();
  return failed == 0;
}

__global__ void decode_advance_kernel(unsigned int* step) {
  if (blockIdx.x == 0 && threadIdx.x == 0) *step += 1u;
}

// One arrival per CTA: the CTA barrier orders every thread's stores before thread 0's
// system-scope fence (fences are cumulative), and the last CTA to arrive publishes the epoch.
__device__ __forceinline__ void dt_publish(DtPeers sig, int world, int rank,
                                           const unsigned int* step, unsigned int* ticket) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int done = atomicAdd(ticket, 1u);
    if (done == gridDim.x - 1) {
      *ticket = 0u;
      __threadfence_system();
      const unsigned int epoch = *step;
      for (int d = 0; d < world; ++d)
        dt_signal(static_cast<unsigned int*>(sig.p[d]) + rank, epoch);
    }
  }
}

// ws [n] fp32 -> every rank's slot; ws cleared; last CTA signals.
__global__ void __launch_bounds__(kDtThreads)
    decode_push_partial_kernel(float* __restrict__ ws, long long n4, DtPeers slot, DtPeers sig,
                               int world, int rank, const unsigned int* __restrict__ step,
                               unsigned int* ticket) {
  const long long stride = static_cast<long long>(gridDim.x) * kDtThreads;
  for (long long i = blockIdx.x * static_cast<long long>(kDtThreads) + threadIdx.x; i < n4;
       i += stride) {
    float4* src = reinterpret_cast<float4*>(ws) + i;
    const float4 a = *src;
    *src = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int d = 0; d < world; ++d) reinterpret_cast<float4*>(slot.p[d])[i] = a;
  }
  dt_publish(sig, world, rank, step, ticket);
}

__global__ void __launch_bounds__(kDtThreads)
    decode_sum_slots_kernel(const float* __restrict__ inbox, int world, int rank, long long n4,
                            const __nv_bfloat16* __restrict__ res, __nv_bfloat16* __restrict__ dst,
                            const unsigned int* __restrict__ sig,
                            const unsigned int* __restrict__ step, int* status) {
  if (!dt_wait_all(sig, world, rank, *step, status, kKernelIdDecodeSum)) return;
  const long long stride = static_cast<long long>(gridDim.x) * kDtThreads;
  for (long long i = blockIdx.x * static_cast<long long>(kDtThreads) + threadIdx.x; i < n4;
       i += stride) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (res != nullptr) {
      const uint2 u = reinterpret_cast<const uint2*>(res)[i];
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
      const float2 lo = __bfloat1622float2(p[0]), hi = __bfloat1622float2(p[1]);
      acc = make_float4(lo.x, lo.y, hi.x, hi.y);
    }
    for (int s = 0; s < world; ++s) {
      const float4 v = reinterpret_cast<const float4*>(inbox)[s * n4 + i];
      acc.x += v.x, acc.y += v.y, acc.z += v.z, acc.w += v.w;
    }
    uint2 o;
    __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&o);
    q[0] = __floats2bfloat162_rn(acc.x, acc.y);
    q[1] = __floats2bfloat162_rn(acc.z, acc.w);
    reinterpret_cast<uint2*>(dst)[i] = o;
  }
}

// The same sum, one CTA per row, followed by the RMSNorm that every residual projection of the
// decode step feeds: x = bf16(sum + residual), h = x * rsqrt(mean(x^2) + eps) * scale, with the
// statistics taken from the rounded x as the separate norm kernel would see it.
constexpr int kDtNormMaxVec = 8;  // float4 pieces per thread: d <= 256 * 4 * 8 = 8192

__global__ void __launch_bounds__(kDtThreads)
    decode_sum_slots_norm_kernel(const float* __restrict__ inbox, int world, int rank, int d,
                                 long long n, const __nv_bfloat16* __restrict__ res,
                                 const float* __restrict__ scale, float eps,
                                 __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ h,
                                 const unsigned int* __restrict__ sig,
                                 const unsigned int* __restrict__ step, int* status) {
  __shared__ float red[kDtThreads / 32];
  if (!dt_wait_all(sig, world, rank, *step, status, kKernelIdDecodeSum)) return;
  const long long row = blockIdx.x;
  const int nvec = d / 4;
  float4 vals[kDtNormMaxVec];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kDtNormMaxVec; ++i) {
    const int v = threadIdx.x + i * kDtThreads;
    if (v < nvec) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      if (res != nullptr) {
        const uint2 u = reinterpret_cast<const uint2*>(res + row * d)[v];
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
        const float2 lo = __bfloat1622float2(p[0]), hi = __bfloat1622float2(p[1]);
        acc = make_float4(lo.x, lo.y, hi.x, hi.y);
      }
      for (int s = 0; s < world; ++s) {
        const float4 t = reinterpret_cast<const float4*>(inbox + s * n + row * d)[v];
        acc.x += t.x, acc.y += t.y, acc.z += t.z, acc.w += t.w;
      }
      uint2 o;
      __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&o);
      q[0] = __floats2bfloat162_rn(acc.x, acc.y);
      q[1] = __floats2bfloat162_rn(acc.z, acc.w);
      reinterpret_cast<uint2*>(x + row * d)[v] = o;
      const float2 lo = __bfloat1622float2(q[0]), hi = __bfloat1622float2(q[1]);
      vals[i] = make_float4(lo.x, lo.y, hi.x, hi.y);
      ss += lo.x * lo.x + lo.y * lo.y + hi.x * hi.x + hi.y * hi.y;
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < kDtThreads / 32; ++w) tot += red[w];
  const float rstd = rsqrtf(tot / static_cast<float>(d) + eps);
#pragma unroll
  for (int i = 0; i < kDtNormMaxVec; ++i) {
    const int v = threadIdx.x + i * kDtThreads;
    if (v < nvec) {
      const float4 sc = reinterpret_cast<const float4*>(scale)[v];
      uint2 o;
      __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&o);
      q[0] = __floats2bfloat162_rn(vals[i].x * rstd * sc.x, vals[i].y * rstd * sc.y);
      q[1] = __floats2bfloat162_rn(vals[i].z * rstd * sc.z, vals[i].w * rstd * sc.w);
      reinterpret_cast<uint2*>(h + row * d)[v] = o;
    }
  }
}

// src [rows, cols] fp32 (this rank's vocabulary slice) -> columns [col0, col0 + cols) of every
// rank's [rows, ld] buffer; last CTA signals.
__global__ void __launch_bounds__(kDtThreads)
    decode_gather_push_kernel(const float* __restrict__ src, int rows, int cols4, int ld, int col0,
                              DtPeers full, DtPeers sig, int world, int rank,
                              const unsigned int* __restrict__ step, unsigned int* ticket) {
  const long long total = static_cast<long long>(rows) * cols4;
  const long long stride = static_cast<long long>(gridDim.x) * kDtThreads;
  for (long long i = blockIdx.x * static_cast<long long>(kDtThreads) + threadIdx.x; i < total;
       i += stride) {
    const int r = static_cast<int>(i / cols4), c = static_cast<int>(i % cols4);
    const float4 v = reinterpret_cast<const float4*>(src)[i];
    const long long off = static_cast<long long>(r) * ld + col0 + 4 * c;
    for (int d = 0; d < world; ++d)
      *reinterpret_cast<float4*>(static_cast<float*>(full.p[d]) + off) = v;
  }
  dt_publish(sig, world, rank, step, ticket);
}

__global__ void decode_wait_kernel(const unsigned int* __restrict__ sig, int world, int rank,
                                   const unsigned int* __restrict__ step, int* status) {
  dt_wait_all(sig, world, rank, *step, status, kKernelIdDecodeWait);
}

int dt_grid(long long items) {
  long long blocks = (items + kDtThreads - 1) / kDtThreads;
  // a few dozen CTAs move a megabyte or two as fast as hundreds would, with far fewer arrivals
  // to count before the signal goes out; the logits gather (tens of megabytes) takes them all
  const long long cap = items > (1ll << 19) ? static_cast<long long>(num_sms()) * 2 : 64;
  if (blocks > cap) blocks = cap;
  return static_cast<int>(blocks < 1 ? 1 : blocks);
}

bool dt_peers(DtPeers* out, void* const* ptrs, int world, int align) {
  for (int d = 0; d < world; ++d) {
    out->p[d] = ptrs[d];
    if (ptrs[d] == nullptr || (reinterpret_cast<uintptr_t>(ptrs[d]) & (align - 1))) return false;
  }
  return true;
}

}  // namespace
}  // namespace t5x

using namespace t5x;

// *step += 1 (the epoch of the decode step that follows).
T5X_API int t5x_decode_step_advance(void* step, void* stream) {
  if (step == nullptr) return set_error("decode_step_advance: null pointer");
  decode_advance_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<unsigned int*>(step));
  count_launches(1);
  return 0;
}

// ws [n] fp32 (n a multiple of 4, cleared on return) -> `slots[d]` (rank d's fp32 inbox slot for
// this rank) for every d, then signal `sigs[d][rank] = *step`.
T5X_API int t5x_decode_push_partial(void* ws, long long n, void* const* slots, void* const* sigs,
                                    int world, int rank, const void* step, void* ticket,
                                    void* stream) {
  if (n <= 0) return 0;
  if (n % 4 || world < 1 || world > kDtMaxPeers || rank < 0 || rank >= world)
    return set_error("decode_push_partial: bad arguments (n=%lld, world=%d)", n, world);
  if (ws == nullptr || step == nullptr || ticket == nullptr ||
      (reinterpret_cast<uintptr_t>(ws) & 15))
    return set_error("decode_push_partial: null or misaligned pointer");
  DtPeers slot = {}, sig = {};
  if (!dt_peers(&slot, slots, world, 16) || !dt_peers(&sig, sigs, world, 4))
    return set_error("decode_push_partial: null or misaligned peer pointer");
  decode_push_partial_kernel<<<dt_grid(n / 4), kDtThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<float*>(ws), n / 4, slot, sig, world, rank,
      static_cast<const unsigned int*>(step), static_cast<unsigned int*>(ticket));
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("decode_push_partial: %s", cudaGetErrorString(e));
  return 0;
}

// dst [n] bf16 = sum over the `world` slots of inbox ([world][n] fp32) + residual (bf16), after every
// rank's signal word in `sig` ([world] words, local) has reached *step.
T5X_API int t5x_decode_sum_slots(const void* inbox, int world, int rank, long long n,
                                 const void* residual, void* dst, const void* sig,
                                 const void* step, void* stream) {
  if (n <= 0) return 0;
  if (n % 4 || world < 1 || world > kDtMaxPeers || rank < 0 || rank >= world)
    return set_error("decode_sum_slots: bad arguments (n=%lld, world=%d)", n, world);
  if (inbox == nullptr || dst == nullptr || sig == nullptr || step == nullptr)
    return set_error("decode_sum_slots: null pointer");
  decode_sum_slots_kernel<<<dt_grid(n / 4), kDtThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(inbox), world, rank, n / 4,
      static_cast<const __nv_bfloat16*>(residual), static_cast<__nv_bfloat16*>(dst),
      static_cast<const unsigned int*>(sig), static_cast<const unsigned int*>(step),
      device_status_buffer());
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("decode_sum_slots: %s", cudaGetErrorString(e));
  return 0;
}

// x [rows, d] bf16 = sum over the `world` slots of inbox ([world][rows * d] fp32) + residual, and
// h [rows, d] = rmsnorm(x) * scale, after every rank's signal word has reached *step.
// d a multiple of 4, d <= 8192.
T5X_API int t5x_decode_sum_slots_norm(const void* inbox, int world, int rank, int rows, int d,
                                      const void* residual, const void* scale, float eps, void* x,
                                      void* h, const void* sig, const void* step, void* stream) {
  if (rows <= 0) return 0;
  if (d % 4 || d > kDtThreads * 4 * kDtNormMaxVec || world < 1 || world > kDtMaxPeers ||
      rank < 0 || rank >= world)
    return set_error("decode_sum_slots_norm: bad arguments (d=%d, world=%d)", d, world);
  if (inbox == nullptr || scale == nullptr || x == nullptr || h == nullptr || sig == nullptr ||
      step == nullptr)
    return set_error("decode_sum_slots_norm: null pointer");
  decode_sum_slots_norm_kernel<<<rows, kDtThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(inbox), world, rank, d, static_cast<long long>(rows) * d,
      static_cast<const __nv_bfloat16*>(residual), static_cast<const float*>(scale), eps,
      static_cast<__nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(h),
      static_cast<const unsigned int*>(sig), static_cast<const unsigned int*>(step),
      device_status_buffer());
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("decode_sum_slots_norm: %s", cudaGetErrorString(e));
  return 0;
}

// src [rows, cols] fp32 -> columns [col0, col0 + cols) of `fulls[d]` ([rows, ld] fp32) for every
// d, then signal. cols, col0 and ld multiples of 4.
T5X_API int t5x_decode_gather_push(const void* src, int rows, int cols, int ld, int col0,
                                   void* const* fulls, void* const* sigs, int world, int rank,
                                   const void* step, void* ticket, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if ((cols | col0 | ld) % 4 || world < 1 || world > kDtMaxPeers || rank < 0 || rank >= world)
    return set_error("decode_gather_push: bad arguments");
  if (src == nullptr || step == nullptr || ticket == nullptr ||
      (reinterpret_cast<uintptr_t>(src) & 15))
    return set_error("decode_gather_push: null or misaligned pointer");
  DtPeers full = {}, sig = {};
  if (!dt_peers(&full, fulls, world, 16) || !dt_peers(&sig, sigs, world, 4))
    return set_error("decode_gather_push: null or misaligned peer pointer");
  const long long items = static_cast<long long>(rows) * (cols / 4);
  decode_gather_push_kernel<<<dt_grid(items), kDtThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(src), rows, cols / 4, ld, col0, full, sig, world, rank,
      static_cast<const unsigned int*>(step), static_cast<unsigned int*>(ticket));
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("decode_gather_push: %s", cudaGetErrorString(e));
  return 0;
}

// Returns (in stream order) once every rank's word in `sig` has reached *step, or records a
// 'peer flag timeout' status after about a second.
T5X_API int t5x_decode_wait(const void* sig, int world, int rank, const void* step, void* stream) {
  if (sig == nullptr || step == nullptr || world < 1 || world > kDtMaxPeers)
    return set_error("decode_wait: bad arguments");
  decode_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned int*>(sig), world, rank, static_cast<const unsigned int*>(step),
      device_status_buffer());
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("decode_wait: %s", cudaGetErrorString(e));
  return 0;
}
