// Collective building blocks over NVLink peer memory, and the optimizer kernels fused with
// them. Every rank passes the same symmetric layout: `peers[d]` is rank d's mapping of one
// buffer (its own entry included), obtained from a symmetric-memory rendezvous.
//
//   barrier         : flag exchange through per-rank signal pads, bounded wait
//   peer_reduce     : dst[i] = sum_d peers[d][i]                       (pull reduce)
//   peer_push_bf16  : peers[d][i] = src[i] for all d                   (push broadcast)
//   dist_stats      : Adafactor phase 1 whose gradient is the sum over all ranks' copies,
//                     read tile by tile over NVLink while the row / column statistics of the
//                     previous tile are being accumulated (reduce-scatter fused into the
//                     optimizer's first pass; the summed gradient is kept for the later passes)
//   dist_apply      : Adafactor parameter update whose bf16 result is stored to every rank's
//                     working copy (the all-gather of updated weights fused into the update)
//
// Peer addresses are accessed with plain ld/st. When the caller also passes the NVSwitch
// multicast address of the same buffers, the gradient sum is one `multimem.ld_reduce` per 16
// bytes (the switch adds the ranks' copies and the owner receives 1/world of the bytes) and the
// weight push one `multimem.st` (the switch fans the store out). No TMA is used on peer memory.
#include "adafactor_common.cuh"
#include "common.cuh"
#include "t5x_b200.h"

namespace t5x {

constexpr int kMaxPeers = 16;
constexpr int kKernelBarrier = 40;

struct PeerF32 {
  const float* p[kMaxPeers];
};
struct PeerBf16 {
  __nv_bfloat16* p[kMaxPeers];
};
struct PeerPads {
  uint32_t* p[kMaxPeers];
};

__device__ __forceinline__ void st_release_sys(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// In-switch sum of the 16 bytes at `mc` (multicast address) over every rank's copy.
__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
// One 8-byte store that the switch delivers to every rank's copy.
__device__ __forceinline__ void multimem_st_b32x2(void* mc, uint32_t a, uint32_t b) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"(mc),
               "f"(__uint_as_float(a)), "f"(__uint_as_float(b))
               : "memory");
}

// One CTA, one thread per peer. Slot layout inside a pad: pad[channel * kMaxPeers + writer].
// `epoch` increases by one per barrier on a channel, so flags never need resetting; a waiter
// accepts any value >= epoch (signed distance, wrap-safe). A wait that exceeds `spin_limit`
// polls records kStatusTimeoutPeerFlag with the silent peer's rank and returns.
__global__ void barrier_kernel(PeerPads pads, int rank, int world, int channel, uint32_t epoch,
                               unsigned long long spin_limit, int* status) {
  const int t = threadIdx.x;
  if (t >= world) return;
  __threadfence_system();
  st_release_sys(pads.p[t] + channel * kMaxPeers + rank, epoch);
  const uint32_t* mine = pads.p[rank] + channel * kMaxPeers + t;
  unsigned long long spins = 0;
  while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
    if (++spins > spin_limit) {
      report_status(status, kStatusTimeoutPeerFlag, kKernelBarrier, t, static_cast<int>(epoch));
      return;
    }
    __nanosleep(64);
  }
}

__global__ void __launch_bounds__(256)
    peer_reduce_kernel(float* __restrict__ dst, PeerF32 src, int world, long long n4,
                       long long n) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += stride) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int d = 0; d < world; ++d) {
      const float4 v = reinterpret_cast<const float4*>(src.p[d])[i];
      acc.x += v.x;
      acc.y += v.y;
      acc.z += v.z;
      acc.w += v.w;
    }
    reinterpret_cast<float4*>(dst)[i] = acc;
  }
  // ragged tail
  for (long long i = n4 * 4 + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += stride) {
    float acc = 0.f;
    for (int d = 0; d < world; ++d) acc += src.p[d][i];
    dst[i] = acc;
  }
}

__global__ void __launch_bounds__(256)
    peer_push_bf16_kernel(PeerBf16 dst, const __nv_bfloat16* __restrict__ src, int world,
                          int skip_rank, long long n8, long long n) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += stride) {
    const uint4 v = reinterpret_cast<const uint4*>(src)[i];
    for (int d = 0; d < world; ++d)
      if (d != skip_rank) reinterpret_cast<uint4*>(dst.p[d])[i] = v;
  }
  for (long long i = n8 * 8 + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += stride) {
    const __nv_bfloat16 v = src[i];
    for (int d = 0; d < world; ++d)
      if (d != skip_rank) dst.p[d][i] = v;
  }
}


constexpr int kDsThreads = 256;
constexpr int kDsTileR = 32;
constexpr int kDsTileC = 1024;  // 256 threads x float4

// Tile walk shared by the two kernels below: CTAs stride over (batch, row tile, column tile).
// The grid is capped (t5x_comm_set_max_ctas) so that these NVLink-latency-bound kernels leave
// room on every SM for the GEMMs of the backward pass they overlap with.
struct DsTiles {
  int x;               // column tiles per row tile
  int per_batch;       // tiles per batch entry
  long long total;
};

static int g_comm_max_ctas = 0;  // 0: two per SM

static inline DsTiles ds_tiles(int batch, int R, int C) {
  DsTiles t;
  t.x = (C + kDsTileC - 1) / kDsTileC;
  t.per_batch = t.x * ((R + kDsTileR - 1) / kDsTileR);
  t.total = static_cast<long long>(t.per_batch) * batch;
  return t;
}

static inline int ds_grid(const DsTiles& t) {
  const long long cap = g_comm_max_ctas > 0 ? g_comm_max_ctas : 2LL * num_sms();
  return static_cast<int>(t.total < cap ? (t.total < 1 ? 1 : t.total) : cap);
}

// Adafactor phase 1 over the gradient summed across ranks. CTA tile: kDsTileR rows x
// kDsTileC columns; a thread owns 4 adjacent columns and walks the rows, so column sums stay
// in registers and row sums need one block reduction per row. Requires C % 4 == 0.
// W: number of ranks known at compile time, or 0 for any `world`; W = -1: grads.p[0] is the
// multicast address and the switch performs the sum.
template <int W>
__global__ void __launch_bounds__(kDsThreads)
    dist_stats_kernel(PeerF32 grads, int world, float* __restrict__ g_out,
                      const float* __restrict__ p, float* __restrict__ rowsum,
                      float* __restrict__ colsum, AdafactorScalars* __restrict__ scal, int R, int C,
                      float eps1, DsTiles tiles) {
  __shared__ float srow[kDsTileR][kDsThreads / 32];
  __shared__ float spsq[kDsThreads / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (long long tile = blockIdx.x; tile < tiles.total; tile += gridDim.x) {
  const int b = static_cast<int>(tile / tiles.per_batch);
  const int in_b = static_cast<int>(tile - static_cast<long long>(b) * tiles.per_batch);
  const long long base = static_cast<long long>(b) * R * C;
  const int r0 = (in_b / tiles.x) * kDsTileR;
  const int col = (in_b % tiles.x) * kDsTileC + threadIdx.x * 4;
  const bool active = col < C;
  float c0 = 0.f, c1 = 0.f, c2 = 0.f, c3 = 0.f, psq = 0.f;
  const int rows = min(kDsTileR, R - r0);
  // All loads of RU rows (W gradient copies and the parameter each) are issued before the
  // first use, so a thread keeps RU * (W + 1) 16-byte requests in flight over NVLink / HBM.
  constexpr int RU = W == 0 ? 1 : (W <= 2 ? 4 : 2);
  constexpr int WN = W <= 0 ? 1 : W;
  for (int rr = 0; rr < rows; rr += RU) {
    float4 v[RU][WN], pv[RU];
#pragma unroll
    for (int u = 0; u < RU; ++u) {
      const bool on = active && rr + u < rows;
      const long long off = base + static_cast<long long>(r0 + rr + u) * C + col;
      pv[u] = on ? *reinterpret_cast<const float4*>(p + off) : make_float4(0.f, 0.f, 0.f, 0.f);
      if (W == 0) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        if (on)
          for (int d = 0; d < world; ++d) {
            const float4 t = *reinterpret_cast<const float4*>(grads.p[d] + off);
            acc.x += t.x;
            acc.y += t.y;
            acc.z += t.z;
            acc.w += t.w;
          }
        v[u][0] = acc;
      } else if (W < 0) {
        v[u][0] = on ? multimem_ld_reduce_f32x4(grads.p[0] + off) : make_float4(0.f, 0.f, 0.f, 0.f);
      } else {
#pragma unroll
        for (int d = 0; d < WN; ++d)
          v[u][d] = on ? *reinterpret_cast<const float4*>(grads.p[d] + off)
                       : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
#pragma unroll
    for (int u = 0; u < RU; ++u) {
      const bool on = active && rr + u < rows;
      float4 acc = v[u][0];
#pragma unroll
      for (int d = 1; d < WN; ++d) {
        acc.x += v[u][d].x;
        acc.y += v[u][d].y;
        acc.z += v[u][d].z;
        acc.w += v[u][d].w;
      }
      float rs = 0.f;
      if (on) {
        const long long off = base + static_cast<long long>(r0 + rr + u) * C + col;
        *reinterpret_cast<float4*>(g_out + off) = acc;
        const float s0 = acc.x * acc.x + eps1, s1 = acc.y * acc.y + eps1,
                    s2 = acc.z * acc.z + eps1, s3 = acc.w * acc.w + eps1;
        c0 += s0;
        c1 += s1;
        c2 += s2;
        c3 += s3;
        rs = (s0 + s1) + (s2 + s3);
        psq += pv[u].x * pv[u].x + pv[u].y * pv[u].y + pv[u].z * pv[u].z + pv[u].w * pv[u].w;
      }
      rs = warp_sum(rs);
      if (lane == 0 && rr + u < rows) srow[rr + u][warp] = rs;
    }
  }
  psq = warp_sum(psq);
  if (lane == 0) spsq[warp] = psq;
  __syncthreads();
  if (threadIdx.x < rows) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < kDsThreads / 32; ++w) t += srow[threadIdx.x][w];
    atomicAdd(&rowsum[static_cast<long long>(b) * R + r0 + threadIdx.x], t);
  }
  if (active) {
    float* cs = colsum + static_cast<long long>(b) * C + col;
    atomicAdd(cs + 0, c0);
    atomicAdd(cs + 1, c1);
    atomicAdd(cs + 2, c2);
    atomicAdd(cs + 3, c3);
  }
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < kDsThreads / 32; ++w) t += spsq[w];
    atomicAdd(&scal[b].psq, t);
  }
  __syncthreads();  // srow / spsq are reused by the next tile
  }
}

// Factored parameter update with the bf16 result stored to every rank. Same tiling as
// dist_stats_kernel (no integer division per element). Requires C % 4 == 0.
__global__ void __launch_bounds__(kDsThreads)
    dist_apply_kernel(float* __restrict__ p, const float* __restrict__ g,
                      const float* __restrict__ rf, const float* __restrict__ cf,
                      float* __restrict__ m, PeerBf16 out, int world,
                      const AdafactorScalars* __restrict__ scal, int R, int C, float n_global,
                      AfHyper h, DsTiles tiles, __nv_bfloat16* __restrict__ out_mc) {
  for (long long tile = blockIdx.x; tile < tiles.total; tile += gridDim.x) {
  const int b = static_cast<int>(tile / tiles.per_batch);
  const int in_b = static_cast<int>(tile - static_cast<long long>(b) * tiles.per_batch);
  const long long base = static_cast<long long>(b) * R * C;
  const int r0 = (in_b / tiles.x) * kDsTileR;
  const int col = (in_b % tiles.x) * kDsTileC + threadIdx.x * 4;
  if (col >= C) continue;
  const float scale = af_update_scale(scal[b], n_global, h);
  const float4 cfv = *reinterpret_cast<const float4*>(cf + static_cast<long long>(b) * C + col);
  const float* rfb = rf + static_cast<long long>(b) * R;
  const int rows = min(kDsTileR, R - r0);
  // four rows per trip, all eight 16-byte loads issued before the first use
  constexpr int kRowUnroll = 4;
  for (int r4 = 0; r4 < rows; r4 += kRowUnroll) {
  float4 tg[kRowUnroll], to[kRowUnroll];
#pragma unroll
  for (int u = 0; u < kRowUnroll; ++u) {
    if (r4 + u < rows) {
      const long long off = base + static_cast<long long>(r0 + r4 + u) * C + col;
      tg[u] = *reinterpret_cast<const float4*>(g + off);
      to[u] = *reinterpret_cast<const float4*>(p + off);
    }
  }
#pragma unroll
  for (int u = 0; u < kRowUnroll; ++u) {
    const int rr = r4 + u;
    if (rr >= rows) break;
    const long long off = base + static_cast<long long>(r0 + rr) * C + col;
    const float rfv = rfb[r0 + rr] * scale;
    const float4 gv = tg[u];
    const float4 old = to[u];
    float sub[4] = {gv.x * rfv * cfv.x, gv.y * rfv * cfv.y, gv.z * rfv * cfv.z,
                    gv.w * rfv * cfv.w};
    const float ov[4] = {old.x, old.y, old.z, old.w};
    float nv[4];
    if (h.use_momentum) {
      float4 mv = *reinterpret_cast<const float4*>(m + off);
      float mo[4] = {mv.x, mv.y, mv.z, mv.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float nm = h.beta1 * mo[k] + (1.f - h.beta1) * sub[k];
        sub[k] = nm;
        if (h.skip_nan && isnan(nm)) nm = mo[k];
        mo[k] = nm;
      }
      *reinterpret_cast<float4*>(m + off) = make_float4(mo[0], mo[1], mo[2], mo[3]);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float np = (h.use_wd ? (1.f - h.weight_decay) * ov[k] : ov[k]) - sub[k];
      if (h.skip_nan && isnan(np)) np = ov[k];
      nv[k] = np;
    }
    *reinterpret_cast<float4*>(p + off) = make_float4(nv[0], nv[1], nv[2], nv[3]);
    __nv_bfloat162 lo = __floats2bfloat162_rn(nv[0], nv[1]);
    __nv_bfloat162 hi = __floats2bfloat162_rn(nv[2], nv[3]);
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&lo);
    packed.y = *reinterpret_cast<uint32_t*>(&hi);
    if (out_mc != nullptr)
      multimem_st_b32x2(out_mc + off, packed.x, packed.y);
    else
      for (int d = 0; d < world; ++d) *reinterpret_cast<uint2*>(out.p[d] + off) = packed;
  }
  }
  }
}

static inline int comm_grid(long long n_vec) {
  long long blocks = (n_vec + 255) / 256;
  const long long cap = static_cast<long long>(num_sms()) * 8;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

static int comm_check(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("%s: %s", what, cudaGetErrorString(e));
  return 0;
}

}  // namespace t5x

using namespace t5x;

// `pads`: host array of `world` device pointers (each rank's signal pad as mapped here).
// The pad must hold at least (channel + 1) * 16 uint32 and start at zero. `epoch` >= 1.
T5X_API int t5x_comm_barrier(const void* const* pads, int rank, int world, int channel,
                             unsigned int epoch, unsigned long long spin_limit, void* stream) {
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || channel < 0)
    return set_error("comm_barrier: bad rank/world/channel %d/%d/%d", rank, world, channel);
  PeerPads pp;
  for (int d = 0; d < world; ++d) pp.p[d] = static_cast<uint32_t*>(const_cast<void*>(pads[d]));
  barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      pp, rank, world, channel, epoch, spin_limit, device_status_buffer());
  count_launches(1);
  return comm_check("comm_barrier");
}

// dst[i] = sum over ranks of srcs[d][i], i < n (fp32). dst may alias this rank's own source.
T5X_API int t5x_peer_reduce_f32(void* dst, const void* const* srcs, int world, long long n,
                                void* stream) {
  if (n <= 0) return 0;
  if (world < 1 || world > kMaxPeers) return set_error("peer_reduce: world %d", world);
  PeerF32 ps;
  bool vec = (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
  for (int d = 0; d < world; ++d) {
    ps.p[d] = static_cast<const float*>(srcs[d]);
    vec = vec && (reinterpret_cast<uintptr_t>(srcs[d]) & 15) == 0;
  }
  const long long n4 = vec ? n / 4 : 0;
  peer_reduce_kernel<<<comm_grid(vec ? n4 : n), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<float*>(dst), ps, world, n4, n);
  count_launches(1);
  return comm_check("peer_reduce_f32");
}

// dsts[d][i] = src[i] for every rank d != skip_rank (pass -1 to write all), i < n (bf16).
T5X_API int t5x_peer_push_bf16(void* const* dsts, const void* src, int world, int skip_rank,
                               long long n, void* stream) {
  if (n <= 0) return 0;
  if (world < 1 || world > kMaxPeers) return set_error("peer_push: world %d", world);
  PeerBf16 pd;
  bool vec = (reinterpret_cast<uintptr_t>(src) & 15) == 0;
  for (int d = 0; d < world; ++d) {
    pd.p[d] = static_cast<__nv_bfloat16*>(dsts[d]);
    vec = vec && (reinterpret_cast<uintptr_t>(dsts[d]) & 15) == 0;
  }
  const long long n8 = vec ? n / 8 : 0;
  peer_push_bf16_kernel<<<comm_grid(vec ? n8 : n), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      pd, static_cast<const __nv_bfloat16*>(src), world, skip_rank, n8, n);
  count_launches(1);
  return comm_check("peer_push_bf16");
}

// Upper bound on the grid of the NVLink-fused optimizer kernels (0 restores two CTAs per SM).
T5X_API void t5x_comm_set_max_ctas(int max_ctas) { g_comm_max_ctas = max_ctas < 0 ? 0 : max_ctas; }

// Adafactor phase 1 with the gradient summed over `world` ranks' copies (grads[d], same
// layout as g_out, which receives the sum and may be this rank's own copy). Clears `scratch`
// like t5x_adafactor_stats. Requires C % 4 == 0 and 16-byte aligned pointers.
T5X_API int t5x_dist_adafactor_stats_mc(const void* p, const void* const* grads, int world,
                                        const void* grads_mc, void* g_out, void* scratch,
                                        int batch, int R, int C, float eps1, void* stream);

T5X_API int t5x_dist_adafactor_stats(const void* p, const void* const* grads, int world,
                                     void* g_out, void* scratch, int batch, int R, int C,
                                     float eps1, void* stream) {
  return t5x_dist_adafactor_stats_mc(p, grads, world, nullptr, g_out, scratch, batch, R, C, eps1,
                                     stream);
}

// The same with `grads_mc`, the multicast address of the gradient buffers (or null): the sum
// over ranks is then taken by the switch.
T5X_API int t5x_dist_adafactor_stats_mc(const void* p, const void* const* grads, int world,
                                        const void* grads_mc, void* g_out, void* scratch,
                                        int batch, int R, int C, float eps1, void* stream) {
  if (batch <= 0 || R <= 0 || C <= 0) return 0;
  if (world < 1 || world > kMaxPeers || (C & 3)) return set_error("dist_adafactor_stats: bad shape");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  PeerF32 ps;
  for (int d = 0; d < world; ++d) ps.p[d] = static_cast<const float*>(grads[d]);
  float* s = static_cast<float*>(scratch);
  cudaMemsetAsync(scratch, 0, t5x_adafactor_scratch_floats(batch, R, C) * sizeof(float), st);
  float* rowsum = s;
  float* colsum = rowsum + static_cast<long long>(batch) * R;
  AdafactorScalars* scal = reinterpret_cast<AdafactorScalars*>(
      s + 2ll * batch * (static_cast<long long>(R) + C));
  const DsTiles tiles = ds_tiles(batch, R, C);
  auto kernel = world == 2 ? dist_stats_kernel<2>
              : world == 4 ? dist_stats_kernel<4>
              : world == 8 ? dist_stats_kernel<8> : dist_stats_kernel<0>;
  if (grads_mc != nullptr) {
    if (reinterpret_cast<uintptr_t>(grads_mc) & 15)
      return set_error("dist_adafactor_stats: multicast address must be 16-byte aligned");
    kernel = dist_stats_kernel<-1>;
    ps.p[0] = static_cast<const float*>(grads_mc);
  }
  kernel<<<ds_grid(tiles), kDsThreads, 0, st>>>(
      ps, world, static_cast<float*>(g_out), static_cast<const float*>(p), rowsum, colsum, scal,
      R, C, eps1, tiles);
  count_launches(1);
  return comm_check("dist_adafactor_stats");
}

// Adafactor phase 4 storing the bf16 result into every rank's copy (bf16_out[d], contiguous
// [batch, R, C] like p). Requires C % 4 == 0.
T5X_API int t5x_dist_adafactor_apply_mc(void* p, const void* g, void* m, void* const* bf16_out,
                                        int world, void* bf16_mc, void* scratch, int batch, int R,
                                        int C, long long n_global, float lr, float eps2,
                                        float clip_threshold, float weight_decay, float beta1,
                                        float max_param_scale, int flags, void* stream);

T5X_API int t5x_dist_adafactor_apply(void* p, const void* g, void* m, void* const* bf16_out,
                                     int world, void* scratch, int batch, int R, int C,
                                     long long n_global, float lr, float eps2,
                                     float clip_threshold, float weight_decay, float beta1,
                                     float max_param_scale, int flags, void* stream) {
  return t5x_dist_adafactor_apply_mc(p, g, m, bf16_out, world, nullptr, scratch, batch, R, C,
                                     n_global, lr, eps2, clip_threshold, weight_decay, beta1,
                                     max_param_scale, flags, stream);
}

// The same with `bf16_mc`, the multicast address of the working-copy buffers (or null): one
// store per 8 bytes then reaches every rank's copy through the switch.
T5X_API int t5x_dist_adafactor_apply_mc(void* p, const void* g, void* m, void* const* bf16_out,
                                        int world, void* bf16_mc, void* scratch, int batch, int R,
                                        int C, long long n_global, float lr, float eps2,
                                        float clip_threshold, float weight_decay, float beta1,
                                        float max_param_scale, int flags, void* stream) {
  if (batch <= 0) return 0;
  if (world < 1 || world > kMaxPeers || (C & 3)) return set_error("dist_adafactor_apply: bad shape");
  PeerBf16 po;
  for (int d = 0; d < world; ++d) po.p[d] = static_cast<__nv_bfloat16*>(bf16_out[d]);
  float* s = static_cast<float*>(scratch);
  float* rf = s + static_cast<long long>(batch) * (static_cast<long long>(R) + C);
  float* cf = rf + static_cast<long long>(batch) * R;
  AdafactorScalars* scal = reinterpret_cast<AdafactorScalars*>(cf + static_cast<long long>(batch) * C);
  AfHyper h = af_hyper(lr, eps2, clip_threshold, weight_decay, beta1, max_param_scale, flags);
  const DsTiles tiles = ds_tiles(batch, R, C);
  dist_apply_kernel<<<ds_grid(tiles), kDsThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<float*>(p), static_cast<const float*>(g), rf, cf, static_cast<float*>(m), po,
      world, scal, R, C, static_cast<float>(n_global), h, tiles,
      static_cast<__nv_bfloat16*>(bf16_mc));
  count_launches(1);
  return comm_check("dist_adafactor_apply");
}
