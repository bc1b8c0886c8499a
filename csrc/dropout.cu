// Dropout with a mask shared along chosen dimensions, drawn inside the kernel.
//
// The T5 blocks use `nn.Dropout(rate, broadcast_dims=(-2,))`: for activations [batch, length, d]
// one Bernoulli mask [batch, 1, d] is shared by every position of a sequence
// (t5x/examples/t5/network.py:76-78, layers.py:476), and attention-weight dropout shares its mask
// along the query dimension (layers.py:115-126), which is the same as scaling the rows of V.
// Both are instances of one indexing rule over a 2-D view x[R, C]:
//
//     key(r, c) = ((r + row_offset) / group_rows) * key_cols + c / col_group
//
//   broadcast over length:  group_rows = length, col_group = 1      (key per (batch, feature))
//   per row (V rows):       group_rows = 1,      col_group = C      (key per row)
//   no broadcast:           group_rows = 1,      col_group = 1
//
// `row_offset` is the global index of row 0, so that a rank holding a block of rows of a
// row-sharded activation draws the same mask as a rank holding all rows. The mask is a pure
// function of (seed, stream, key): the backward pass calls the same kernel on the gradient.
#include "common.cuh"
#include "philox.cuh"

namespace t5x {
namespace {

constexpr int kDropThreads = 256;

struct DropParams {
  long long R;
  int C;
  long long ldx, ldy;
  long long row_offset;
  int group_rows, col_group, key_cols;
  unsigned long long seed;
  unsigned int stream;
  unsigned int keep_threshold;  // keep iff (bits >> 8) < keep_threshold
  float inv_keep;
};

__device__ __forceinline__ bool drop_keep(const DropParams& p, unsigned long long key,
                                          unsigned long long& cached_block, Philox4& cached) {
  const unsigned long long block = key >> 2;
  if (block != cached_block) {
    cached = philox4x32_10(p.seed, p.stream, block);
    cached_block = block;
  }
  const unsigned int lane = static_cast<unsigned int>(key & 3ull);
  const uint32_t bits = lane == 0 ? cached.x : lane == 1 ? cached.y : lane == 2 ? cached.z : cached.w;
  return (bits >> 8) < p.keep_threshold;
}

// 8 bf16 (16 bytes) per thread and iteration.
__global__ void __launch_bounds__(kDropThreads)
    dropout_vec_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                       const DropParams p) {
  const int vec_per_row = p.C / 8;
  const long long total = p.R * vec_per_row;
  unsigned long long cached_block = ~0ull;
  Philox4 cached = {0, 0, 0, 0};
  for (long long i = blockIdx.x * static_cast<long long>(kDropThreads) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * kDropThreads) {
    const long long r = i / vec_per_row;
    const int c0 = static_cast<int>(i - r * vec_per_row) * 8;
    const unsigned long long key_row =
        static_cast<unsigned long long>((r + p.row_offset) / p.group_rows) * p.key_cols;
    uint4 u = *reinterpret_cast<const uint4*>(x + r * p.ldx + c0);
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(h[j]);
      const bool k0 = drop_keep(p, key_row + (c0 + 2 * j) / p.col_group, cached_block, cached);
      const bool k1 = drop_keep(p, key_row + (c0 + 2 * j + 1) / p.col_group, cached_block, cached);
      f.x = k0 ? f.x * p.inv_keep : 0.f;
      f.y = k1 ? f.y * p.inv_keep : 0.f;
      h[j] = __floats2bfloat162_rn(f.x, f.y);
    }
    *reinterpret_cast<uint4*>(y + r * p.ldy + c0) = u;
  }
}

// The common case (mask shared along the length axis or not shared at all, col_group == 1):
// a thread owns 8 adjacent columns and walks down a tile of rows; the mask of those columns
// depends on the row only through its group, so it is drawn once per group and tile (two Philox
// blocks for 8 columns) instead of once per element, and no division is left in the loop.
constexpr int kDropTileRows = 32;

__global__ void __launch_bounds__(kDropThreads)
    dropout_coltile_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                           const DropParams p) {
  const int vec_per_row = p.C / 8;
  const int v = blockIdx.x * kDropThreads + threadIdx.x;
  if (v >= vec_per_row) return;
  const int c0 = v * 8;
  const long long r_begin = static_cast<long long>(blockIdx.y) * kDropTileRows;
  const long long r_end = min(p.R, r_begin + kDropTileRows);
  long long group = (r_begin + p.row_offset) / p.group_rows;
  long long left_in_group = p.group_rows - (r_begin + p.row_offset - group * p.group_rows);
  uint32_t keep_bits = 0;
  bool have = false;
  for (long long r = r_begin; r < r_end; ++r) {
    if (!have) {
      const unsigned long long key0 =
          static_cast<unsigned long long>(group) * p.key_cols + static_cast<unsigned long long>(c0);
      // c0 is a multiple of 8 and key_cols == C is one too: the 8 keys are two whole blocks
      const Philox4 a = philox4x32_10(p.seed, p.stream, key0 >> 2);
      const Philox4 b = philox4x32_10(p.seed, p.stream, (key0 >> 2) + 1);
      const uint32_t bits[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
      keep_bits = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) keep_bits |= ((bits[j] >> 8) < p.keep_threshold ? 1u : 0u) << j;
      have = true;
    }
    uint4 u = *reinterpret_cast<const uint4*>(x + r * p.ldx + c0);
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(h[j]);
      f.x = ((keep_bits >> (2 * j)) & 1u) ? f.x * p.inv_keep : 0.f;
      f.y = ((keep_bits >> (2 * j + 1)) & 1u) ? f.y * p.inv_keep : 0.f;
      h[j] = __floats2bfloat162_rn(f.x, f.y);
    }
    *reinterpret_cast<uint4*>(y + r * p.ldy + c0) = u;
    if (--left_in_group == 0) {
      ++group;
      left_in_group = p.group_rows;
      have = false;
    }
  }
}

__global__ void __launch_bounds__(kDropThreads)
    dropout_scalar_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                          const DropParams p) {
  const long long total = p.R * p.C;
  unsigned long long cached_block = ~0ull;
  Philox4 cached = {0, 0, 0, 0};
  for (long long i = blockIdx.x * static_cast<long long>(kDropThreads) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * kDropThreads) {
    const long long r = i / p.C;
    const int c = static_cast<int>(i - r * p.C);
    const unsigned long long key =
        static_cast<unsigned long long>((r + p.row_offset) / p.group_rows) * p.key_cols +
        c / p.col_group;
    const float v = __bfloat162float(x[r * p.ldx + c]);
    y[r * p.ldy + c] = __float2bfloat16(drop_keep(p, key, cached_block, cached) ? v * p.inv_keep : 0.f);
  }
}

}  // namespace
}  // namespace t5x

// y[R, C] = x[R, C] * mask(key(r, c)) / (1 - rate); y may be x. bf16, row strides in elements.
T5X_API int t5x_dropout_bf16(const void* x, void* y, long long R, int C, long long ldx,
                             long long ldy, long long row_offset, int group_rows, int col_group,
                             unsigned long long seed, unsigned int stream_id, float rate,
                             void* stream) {
  using namespace t5x;
  if (R <= 0 || C <= 0) return 0;
  if (x == nullptr || y == nullptr) return set_error("dropout: null pointer");
  if (!(rate >= 0.f) || !(rate < 1.f)) return set_error("dropout: rate %f is not in [0, 1)", rate);
  if (group_rows < 1 || col_group < 1) return set_error("dropout: group sizes must be >= 1");
  DropParams p;
  p.R = R;
  p.C = C;
  p.ldx = ldx;
  p.ldy = ldy;
  p.row_offset = row_offset;
  p.group_rows = group_rows;
  p.col_group = col_group;
  p.key_cols = (C + col_group - 1) / col_group;
  p.seed = seed;
  p.stream = stream_id;
  const double keep = 1.0 - static_cast<double>(rate);
  p.keep_threshold = static_cast<unsigned int>(keep * 16777216.0);
  p.inv_keep = static_cast<float>(1.0 / keep);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool vec = (C % 8 == 0) && (ldx % 8 == 0) && (ldy % 8 == 0) &&
                   ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
  const long long work = vec ? R * (C / 8) : R * static_cast<long long>(C);
  long long blocks = (work + kDropThreads - 1) / kDropThreads;
  const long long cap = static_cast<long long>(num_sms()) * 8;
  if (blocks > cap) blocks = cap;
  const long long row_tiles = (R + kDropTileRows - 1) / kDropTileRows;
  if (vec && col_group == 1 && row_tiles <= 65535) {
    const dim3 grid((C / 8 + kDropThreads - 1) / kDropThreads, static_cast<unsigned>(row_tiles));
    dropout_coltile_kernel<<<grid, kDropThreads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), p);
  } else if (vec)
    dropout_vec_kernel<<<static_cast<unsigned>(blocks), kDropThreads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), p);
  else
    dropout_scalar_kernel<<<static_cast<unsigned>(blocks), kDropThreads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), p);
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("dropout launch: %s", cudaGetErrorString(e));
  return 0;
}

// The keep decision of one key, computed on the host with the same generator: lets tests and
// CPU code reproduce the device mask exactly. Returns 1 (kept) or 0 (dropped).
T5X_API int t5x_dropout_keep_host(unsigned long long seed, unsigned int stream_id,
                                  unsigned long long key, float rate) {
  using namespace t5x;
  const double keep = 1.0 - static_cast<double>(rate);
  const unsigned int thr = static_cast<unsigned int>(keep * 16777216.0);
  const Philox4 r = philox4x32_10(seed, stream_id, key >> 2);
  const unsigned int lane = static_cast<unsigned int>(key & 3ull);
  const uint32_t bits = lane == 0 ? r.x : lane == 1 ? r.y : lane == 2 ? r.z : r.w;
  return (bits >> 8) < thr ? 1 : 0;
}
