// Beam-search and sampling steps over the vocabulary as native kernels.
//
//  t5x_beam_partial / t5x_beam_update   one beam-search step (t5x/decoding.py:1339-1506):
//      log-softmax of every live beam's logits, the best 2*beams continuations of each example
//      over beams x vocabulary, reselection of the live beams, merge into the finished set with
//      the brevity penalty, ancestry-table update and the early-termination test.
//      Two launches: per (row, vocabulary chunk) partials (max, sum of exponentials, chunk-local
//      best 2*beams), then one CTA per example that merges the partials and does all the
//      bookkeeping in shared memory. Every selection orders by value, then by lowest index, as
//      `lax.top_k` does.
//  t5x_sample_tokens                    temperature / top-k / top-p sampling
//      (t5x/decoding.py:541-621): the cutoff for top-k or top-p is found by a four-pass radix
//      select over the order-preserving bit pattern of the scaled logits (counts for top-k,
//      probability mass for top-p) instead of the reference's 32 vocabulary-wide reductions
//      (t5x/binary_search.py:167-299); the token is drawn with Gumbel noise from an in-kernel
//      counter-based generator, and its log-probability comes from the same pass.
//  t5x_topk_topp_mask                   the masking alone, for callers of topk_mask / topp_mask.
#include <float.h>

#include "common.cuh"
#include "philox.cuh"

namespace t5x {
namespace {

constexpr float kBeamNegInf = -1.0e7f;  // NEG_INF of t5x/decoding.py
constexpr int kBeamThreads = 256;
constexpr int kMaxBeams = 8;
constexpr int kMaxCand = 2 * kMaxBeams;

// (value, index) ordering of every selection here: larger value first, lower index on ties.
__device__ __forceinline__ bool cand_better(float va, int ia, float vb, int ib) {
  return va > vb || (va == vb && ia < ib);
}

__device__ __forceinline__ void warp_best(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (cand_better(ov, oi, v, i)) {
      v = ov;
      i = oi;
    }
  }
}

// Block-wide best of one (value, index) proposal per thread; every thread gets the winner.
// `red_v` / `red_i`: one slot per warp (+1 for the result).
__device__ __forceinline__ void block_best(float& v, int& i, float* red_v, int* red_i) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarps = blockDim.x >> 5;
  warp_best(v, i);
  if (lane == 0) {
    red_v[warp] = v;
    red_i[warp] = i;
  }
  __syncthreads();
  if (warp == 0) {
    float bv = lane < nwarps ? red_v[lane] : -FLT_MAX;
    int bi = lane < nwarps ? red_i[lane] : 0x7fffffff;
    warp_best(bv, bi);
    if (lane == 0) {
      red_v[nwarps] = bv;
      red_i[nwarps] = bi;
    }
  }
  __syncthreads();
  v = red_v[nwarps];
  i = red_i[nwarps];
  __syncthreads();
}

// ---------------------------------------------------------------------------------------
// Beam search, launch 1: per (row, chunk) softmax partials and chunk-local top candidates
// ---------------------------------------------------------------------------------------
template <int K2>
__global__ void __launch_bounds__(kBeamThreads)
    beam_partial_kernel(const float* __restrict__ logits, long long ld, int V, int chunk,
                        float* __restrict__ pmax, float* __restrict__ psum,
                        float* __restrict__ cand_val, int* __restrict__ cand_idx) {
  __shared__ float red_v[kBeamThreads / 32 + 1];
  __shared__ int red_i[kBeamThreads / 32 + 1];
  __shared__ float red_s[kBeamThreads / 32];
  const int row = blockIdx.y, s = blockIdx.x, S = gridDim.x;
  const float* x = logits + static_cast<long long>(row) * ld;
  const int lo = s * chunk, hi = min(V, lo + chunk);

  float tv[K2];
  int ti[K2];
#pragma unroll
  for (int j = 0; j < K2; ++j) {
    tv[j] = -FLT_MAX;
    ti[j] = 0x7fffffff;
  }
  float m = -FLT_MAX, sum = 0.f;
  for (int i = lo + threadIdx.x; i < hi; i += kBeamThreads) {
    const float v = x[i];
    if (v > m) {
      sum = sum * __expf(m - v) + 1.f;
      m = v;
    } else {
      sum += __expf(v - m);
    }
    if (v > tv[K2 - 1]) {  // indices arrive in increasing order: ties keep the earlier one
      tv[K2 - 1] = v;
      ti[K2 - 1] = i;
#pragma unroll
      for (int j = K2 - 1; j > 0; --j) {
        if (tv[j] > tv[j - 1]) {
          const float fv = tv[j];
          tv[j] = tv[j - 1];
          tv[j - 1] = fv;
          const int fi = ti[j];
          ti[j] = ti[j - 1];
          ti[j - 1] = fi;
        }
      }
    }
  }
  // softmax partials of the chunk
  float bm = m;
  {
    int who = static_cast<int>(threadIdx.x);
    block_best(bm, who, red_v, red_i);  // bm <- maximum over the block
  }
  float contrib = (m == -FLT_MAX) ? 0.f : sum * __expf(m - bm);
  contrib = warp_sum(contrib);
  if ((threadIdx.x & 31) == 0) red_s[threadIdx.x >> 5] = contrib;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < kBeamThreads / 32; ++w) t += red_s[w];
    pmax[row * S + s] = bm;
    psum[row * S + s] = t;
  }
  __syncthreads();
  // K2 rounds: the block's best remaining head wins and its owner pops it
  const long long out = (static_cast<long long>(row) * S + s) * K2;
  for (int r = 0; r < K2; ++r) {
    float v = tv[0];
    int i = ti[0];
    block_best(v, i, red_v, red_i);
    if (i == ti[0] && i != 0x7fffffff) {
#pragma unroll
      for (int j = 0; j < K2 - 1; ++j) {
        tv[j] = tv[j + 1];
        ti[j] = ti[j + 1];
      }
      tv[K2 - 1] = -FLT_MAX;
      ti[K2 - 1] = 0x7fffffff;
    }
    if (threadIdx.x == 0) {
      cand_val[out + r] = v;
      cand_idx[out + r] = i;  // 0x7fffffff marks "no candidate" (chunk shorter than K2)
    }
  }
}

// ---------------------------------------------------------------------------------------
// Beam search, launch 2: one CTA per example
// ---------------------------------------------------------------------------------------
struct BeamState {
  const float* pmax;
  const float* psum;
  const float* cand_val;
  const int* cand_idx;
  float* live_lp;            // [batch, k]
  long long* live_seqs;      // [batch, k, L]
  long long* fin_seqs;       // [batch, k, L]
  float* fin_scores;         // [batch, k]
  unsigned char* fin_flags;  // [batch, k] (bool)
  int* anc;                  // [batch, k, L]
  int* cur;                  // device scalar: position of the token the logits were computed for
  unsigned char* term_b;     // [batch] scratch
  unsigned char* terminated; // device scalar (bool)
  unsigned int* ticket;      // zero between launches
  int batch, k, L, V, S, eos;
  float alpha, min_brevity;
};

// Picks, `count` times, the best (value desc, position asc) entry of val[0..n) that has not been
// picked yet; thread 0 only (n is a few dozen). Results in order[0..count).
__device__ void serial_top(const float* val, int n, int count, int* order) {
  unsigned int taken = 0u;  // n <= 24 here
  for (int r = 0; r < count; ++r) {
    int best = -1;
    for (int j = 0; j < n; ++j) {
      if ((taken >> j) & 1u) continue;
      if (best < 0 || val[j] > val[best]) best = j;
    }
    taken |= 1u << best;
    order[r] = best;
  }
}

template <int K2>
__global__ void __launch_bounds__(kBeamThreads) beam_update_kernel(const BeamState st) {
  extern __shared__ int dyn[];
  __shared__ float red_v[kBeamThreads / 32 + 1];
  __shared__ int red_i[kBeamThreads / 32 + 1];
  __shared__ float lse[kMaxBeams];
  __shared__ float top_lp[kMaxCand];
  __shared__ int top_flat[kMaxCand];     // beam * V + token
  __shared__ int alive_src[kMaxBeams];   // candidate index feeding new live beam i
  __shared__ int fin_src[kMaxBeams];     // < k: old finished slot; >= k: candidate (j - k)
  __shared__ float new_live_lp[kMaxBeams];
  __shared__ float new_fin_score[kMaxBeams];
  __shared__ unsigned char new_fin_flag[kMaxBeams];

  const int b = blockIdx.x, k = st.k, L = st.L, S = st.S;
  const int tid = threadIdx.x;
  const int cur = *st.cur;
  int* old_live = dyn;                 // [k, L] tokens
  int* old_fin = dyn + k * L;          // [k, L]
  int* old_anc = dyn + 2 * k * L;      // [k, L]
  float* cscore = reinterpret_cast<float*>(dyn + 3 * k * L);  // [k * S * K2]
  int* cflat = reinterpret_cast<int*>(cscore + k * S * K2);

  for (int i = tid; i < k * L; i += kBeamThreads) {
    const long long g = static_cast<long long>(b) * k * L + i;
    old_live[i] = static_cast<int>(st.live_seqs[g]);
    old_fin[i] = static_cast<int>(st.fin_seqs[g]);
    old_anc[i] = st.anc[g];
  }
  if (tid < k) {
    const int row = b * k + tid;
    float m = -FLT_MAX;
    for (int s = 0; s < S; ++s) m = fmaxf(m, st.pmax[row * S + s]);
    float t = 0.f;
    for (int s = 0; s < S; ++s) t += st.psum[row * S + s] * expf(st.pmax[row * S + s] - m);
    lse[tid] = m + logf(t);
  }
  __syncthreads();
  const int ncand = k * S * K2;
  for (int c = tid; c < ncand; c += kBeamThreads) {
    const int beam = c / (S * K2);
    const long long g = static_cast<long long>(b) * k * S * K2 + c;
    const int idx = st.cand_idx[g];
    if (idx == 0x7fffffff) {
      cscore[c] = -FLT_MAX;
      cflat[c] = 0x7fffffff;
    } else {
      cscore[c] = (st.cand_val[g] - lse[beam]) + st.live_lp[b * k + beam];
      cflat[c] = beam * st.V + idx;
    }
  }
  __syncthreads();
  // best K2 over beams x vocabulary, descending
  for (int r = 0; r < K2; ++r) {
    float v = -FLT_MAX;
    int f = 0x7fffffff;
    for (int c = tid; c < ncand; c += kBeamThreads)
      if (cand_better(cscore[c], cflat[c], v, f)) {
        v = cscore[c];
        f = cflat[c];
      }
    block_best(v, f, red_v, red_i);
    for (int c = tid; c < ncand; c += kBeamThreads)
      if (cflat[c] == f) cscore[c] = -FLT_MAX, cflat[c] = 0x7fffffff;
    if (tid == 0) {
      top_lp[r] = v;
      top_flat[r] = f;
    }
    __syncthreads();
  }
  if (tid == 0) {
    // live beams: best k of the candidates that did not just end, stored ascending
    float new_lp[kMaxCand];
    int order[kMaxCand];
    for (int j = 0; j < K2; ++j) {
      const bool ended = (top_flat[j] % st.V) == st.eos;
      new_lp[j] = top_lp[j] + (ended ? kBeamNegInf : 0.f);
    }
    serial_top(new_lp, K2, k, order);
    for (int i = 0; i < k; ++i) {
      const int j = order[k - 1 - i];
      alive_src[i] = j;
      new_live_lp[i] = new_lp[j];
    }
    // finished set: old finished slots and the candidates that just ended, by penalised score
    const float length = static_cast<float>(cur + 1);
    const float penalty = powf((5.f + length) / 6.f, st.alpha);
    float all_scores[kMaxBeams + kMaxCand];
    for (int i = 0; i < k; ++i) all_scores[i] = st.fin_scores[b * k + i];
    for (int j = 0; j < K2; ++j) {
      const bool ended = (top_flat[j] % st.V) == st.eos;
      all_scores[k + j] = top_lp[j] / penalty + (ended ? 0.f : kBeamNegInf);
    }
    int forder[kMaxBeams];
    serial_top(all_scores, k + K2, k, forder);
    bool all_flags = true;
    float worst = FLT_MAX;
    for (int i = 0; i < k; ++i) {
      const int j = forder[k - 1 - i];
      fin_src[i] = j;
      new_fin_score[i] = all_scores[j];
      const bool flag = j < k ? st.fin_flags[b * k + j] != 0
                              : (top_flat[j - k] % st.V) == st.eos;
      new_fin_flag[i] = flag ? 1 : 0;
      all_flags = all_flags && flag;
      worst = fminf(worst, all_scores[j]);
    }
    // may this example stop? every finished slot is real and the worst of them beats what the
    // best live beam could still reach (t5x/decoding.py:1279-1312)
    const float best_live = new_live_lp[k - 1] / st.min_brevity;
    st.term_b[b] = (all_flags && worst > best_live) ? 1 : 0;
  }
  __syncthreads();
  // write back: sequences, ancestry, scores
  const int nxt = cur + 1;
  for (int i = tid; i < k * L; i += kBeamThreads) {
    const int beam = i / L, pos = i - beam * L;
    const long long g = static_cast<long long>(b) * k * L + i;
    {
      const int j = alive_src[beam];
      const int parent = top_flat[j] / st.V;
      int tok = old_live[parent * L + pos];
      if (pos == nxt) tok = top_flat[j] % st.V;
      st.live_seqs[g] = tok;
      st.anc[g] = (pos == cur) ? parent : old_anc[parent * L + pos];
    }
    {
      const int j = fin_src[beam];
      int tok;
      if (j < k) {
        tok = old_fin[j * L + pos];
      } else {
        const int parent = top_flat[j - k] / st.V;
        tok = old_live[parent * L + pos];
        if (pos == nxt) tok = top_flat[j - k] % st.V;
      }
      st.fin_seqs[g] = tok;
    }
  }
  if (tid < k) {
    st.live_lp[b * k + tid] = new_live_lp[tid];
    st.fin_scores[b * k + tid] = new_fin_score[tid];
    st.fin_flags[b * k + tid] = new_fin_flag[tid];
  }
  // the last CTA to get here advances the position and folds the per-example stop flags
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned int t = atomicAdd(st.ticket, 1u);
    if (t == static_cast<unsigned int>(st.batch) - 1u) {
      __threadfence();
      bool all = true;
      for (int i = 0; i < st.batch; ++i) all = all && (reinterpret_cast<volatile unsigned char*>(st.term_b)[i] != 0);
      *st.terminated = all ? 1 : 0;
      *st.cur = cur + 1;
      *st.ticket = 0u;
    }
  }
}

// ---------------------------------------------------------------------------------------
// Sampling
// ---------------------------------------------------------------------------------------
constexpr int kSampleThreads = 1024;
constexpr float kMinTemperature = 1e-4f;  // MIN_TEMPERATURE of t5x/decoding.py

__device__ __forceinline__ uint32_t float_key(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // larger float <=> larger key
}
__device__ __forceinline__ float key_float(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// Warp 0: walking the 256 bins from the top, the first bin at which the running total reaches
// `need`. Returns the bin in *digit and the total of the bins above it in *above.
template <typename T>
__device__ void bin_from_top(const T* hist, T need, int* digit, T* above) {
  const int lane = threadIdx.x;  // called by warp 0 only
  T mine = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) mine += hist[255 - (lane * 8 + j)];  // lane 0 holds the top bins
  T incl = mine;  // inclusive scan over lanes (lane 0 first)
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const T up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  const T excl = incl - mine;
  const bool here = incl >= need && excl < need;
  const unsigned int ballot = __ballot_sync(0xffffffffu, here);
  if (ballot == 0u) {  // never reached (rounding): the lowest bin
    if (lane == 31) {
      *digit = 0;
      *above = incl - hist[0];
    }
    return;
  }
  if (lane == __ffs(ballot) - 1) {
    T run = excl;
    int d = 255 - lane * 8;
    for (int j = 0; j < 8; ++j, --d) {
      if (run + hist[d] >= need || j == 7) break;
      run += hist[d];
    }
    *digit = d;
    *above = run;
  }
}

// Key of the k-th largest scaled logit of the row (k >= 1).
__device__ uint32_t select_kth_key(const float* x, int V, float inv_t, unsigned int k,
                                   unsigned int* hist, int* s_digit, unsigned int* s_above) {
  uint32_t prefix = 0u, mask = 0u;
  unsigned int need = k;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0u;
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const uint32_t key = float_key(x[i] * inv_t);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (threadIdx.x < 32) bin_from_top<unsigned int>(hist, need, s_digit, s_above);
    __syncthreads();
    prefix |= static_cast<uint32_t>(*s_digit) << shift;
    mask |= 255u << shift;
    need -= *s_above;
    __syncthreads();
  }
  return prefix;
}

// Largest key c such that the probability mass of entries with key >= c reaches `target`
// (mass = sum of exp(x - m)).
__device__ uint32_t select_mass_key(const float* x, int V, float inv_t, float m, float target,
                                    float* hist, int* s_digit, float* s_above) {
  uint32_t prefix = 0u, mask = 0u;
  float need = target;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0.f;
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = x[i] * inv_t;
      const uint32_t key = float_key(v);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], __expf(v - m));
    }
    __syncthreads();
    if (threadIdx.x < 32) bin_from_top<float>(hist, need, s_digit, s_above);
    __syncthreads();
    prefix |= static_cast<uint32_t>(*s_digit) << shift;
    mask |= 255u << shift;
    need -= *s_above;
    __syncthreads();
  }
  return prefix;
}

__device__ float block_max(float v, float* red) {
  v = warp_max(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = -FLT_MAX;
  for (int w = 0; w < (blockDim.x >> 5); ++w) r = fmaxf(r, red[w]);
  __syncthreads();
  return r;
}
__device__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = 0.f;
  for (int w = 0; w < (blockDim.x >> 5); ++w) r += red[w];
  __syncthreads();
  return r;
}

struct SampleParams {
  const float* logits;
  long long ld;
  int rows, V;
  const float* temperature;  // per row, or null
  float temperature_scalar;
  int topk;
  const float* topp;         // per row, or null
  float topp_scalar;
  int rescale_log_probs;
  unsigned long long seed;
  unsigned int stream;
  long long* tokens;         // [rows]
  float* log_probs;          // [rows]
  float* masked_out;         // mask-only mode: [rows, V] with ld_out
  long long ld_out;
  float replace_val;
};

// The cutoff key of one row: entries whose key is >= the result survive. `m_scaled` is the row
// maximum of the scaled logits.
__device__ uint32_t row_cutoff(const SampleParams& p, const float* x, float inv_t, float topp,
                               float m_scaled, float* red, unsigned int* hist_u, float* hist_f,
                               int* s_digit, unsigned int* s_above_u, float* s_above_f) {
  uint32_t cutoff = 0u;  // keep everything
  if (p.topk > 0 && p.topk < p.V)
    cutoff = select_kth_key(x, p.V, inv_t, static_cast<unsigned int>(p.topk), hist_u, s_digit,
                            s_above_u);
  if (topp > 0.f) {
    float z = 0.f;
    for (int i = threadIdx.x; i < p.V; i += blockDim.x) z += __expf(x[i] * inv_t - m_scaled);
    z = block_sum(z, red);
    const uint32_t c = select_mass_key(x, p.V, inv_t, m_scaled, topp * z, hist_f, s_digit,
                                       s_above_f);
    cutoff = max(cutoff, c);
  }
  return cutoff;
}

template <bool MASK_ONLY>
__global__ void __launch_bounds__(kSampleThreads) sample_kernel(const SampleParams p) {
  __shared__ float red[kSampleThreads / 32];
  __shared__ float red_v[kSampleThreads / 32 + 1];
  __shared__ int red_i[kSampleThreads / 32 + 1];
  __shared__ unsigned int hist_u[256];
  __shared__ float hist_f[256];
  __shared__ int s_digit;
  __shared__ unsigned int s_above_u;
  __shared__ float s_above_f;

  const int row = blockIdx.x;
  const float* x = p.logits + static_cast<long long>(row) * p.ld;
  const float temp = p.temperature ? p.temperature[row] : p.temperature_scalar;
  const float topp = p.topp ? p.topp[row] : p.topp_scalar;
  const float inv_t = MASK_ONLY ? 1.f : 1.f / fmaxf(temp, kMinTemperature);

  float m_raw = -FLT_MAX;
  for (int i = threadIdx.x; i < p.V; i += blockDim.x) m_raw = fmaxf(m_raw, x[i]);
  m_raw = block_max(m_raw, red);
  const float m_scaled = m_raw * inv_t;  // inv_t > 0

  if (MASK_ONLY) {
    const uint32_t cutoff = row_cutoff(p, x, 1.f, topp, m_raw, red, hist_u, hist_f, &s_digit,
                                       &s_above_u, &s_above_f);
    float* out = p.masked_out + static_cast<long long>(row) * p.ld_out;
    for (int i = threadIdx.x; i < p.V; i += blockDim.x)
      out[i] = float_key(x[i]) >= cutoff ? x[i] : p.replace_val;
    return;
  }

  const bool greedy = !(temp > kMinTemperature);  // the reference's switch to arg-max
  float lse_raw = 0.f;
  if (!p.rescale_log_probs) {
    float z = 0.f;
    for (int i = threadIdx.x; i < p.V; i += blockDim.x) z += __expf(x[i] - m_raw);
    lse_raw = m_raw + logf(block_sum(z, red));
  }
  if (greedy) {
    float v = -FLT_MAX;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < p.V; i += blockDim.x)
      if (cand_better(x[i], i, v, bi)) v = x[i], bi = i;
    block_best(v, bi, red_v, red_i);
    if (threadIdx.x == 0) {
      p.tokens[row] = bi;
      p.log_probs[row] = p.rescale_log_probs ? 0.f : v - lse_raw;
    }
    return;
  }
  const uint32_t cutoff = row_cutoff(p, x, inv_t, topp, m_scaled, red, hist_u, hist_f, &s_digit,
                                     &s_above_u, &s_above_f);
  // one pass over the survivors: normaliser of the masked distribution and the Gumbel argmax
  float z = 0.f, best = -FLT_MAX;
  int best_i = 0x7fffffff;
  const unsigned long long base = static_cast<unsigned long long>(row) * p.V;
  for (int i = threadIdx.x; i < p.V; i += blockDim.x) {
    const float v = x[i] * inv_t;
    if (float_key(v) < cutoff) continue;
    z += __expf(v - m_scaled);
    const unsigned long long id = base + i;
    const Philox4 r = philox4x32_10(p.seed, p.stream, id >> 2);
    const unsigned int lane = static_cast<unsigned int>(id & 3ull);
    const uint32_t bits = lane == 0 ? r.x : lane == 1 ? r.y : lane == 2 ? r.z : r.w;
    const float g = v - logf(-logf(philox_uniform(bits)));
    if (cand_better(g, i, best, best_i)) best = g, best_i = i;
  }
  z = block_sum(z, red);
  block_best(best, best_i, red_v, red_i);
  if (threadIdx.x == 0) {
    p.tokens[row] = best_i;
    const float xt = x[best_i];
    p.log_probs[row] = p.rescale_log_probs ? (xt * inv_t - (m_scaled + logf(z))) : (xt - lse_raw);
  }
}

}  // namespace
}  // namespace t5x

// ---------------------------------------------------------------------------------------
// C API
// ---------------------------------------------------------------------------------------
// Floats / ints of scratch the beam step needs for `rows` = batch * beams rows.
T5X_API int t5x_beam_chunks(int vocab) {
  // chunks of about 4096 columns: enough CTAs per row to stream the logits at full rate
  int s = (vocab + 4095) / 4096;
  return s < 1 ? 1 : (s > 32 ? 32 : s);
}

// One beam-search step. logits [batch * beams, V] fp32 (row stride ld) of the tokens at position
// *cur; state tensors as in BeamState. scratch_f: rows * S * (2 + 2 * beams) floats;
// scratch_i: rows * S * 2 * beams ints; flags: batch bytes; ticket: one zeroed uint32.
T5X_API int t5x_beam_step(const void* logits, long long ld, int batch, int beams, int L, int V,
                          int eos, float alpha, float min_brevity, void* live_lp, void* live_seqs,
                          void* fin_seqs, void* fin_scores, void* fin_flags, void* anc, void* cur,
                          void* terminated, void* scratch_f, void* scratch_i, void* flags,
                          void* ticket, void* stream) {
  using namespace t5x;
  if (batch <= 0) return 0;
  if (beams != 1 && beams != 2 && beams != 4 && beams != 8)
    return set_error("beam_step: beams must be 1, 2, 4 or 8 (got %d)", beams);
  if (static_cast<long long>(beams) * V >= 0x7fffffffLL)
    return set_error("beam_step: beams * vocab does not fit 31 bits");
  const int S = t5x_beam_chunks(V);
  const int chunk = (V + S - 1) / S;
  const int rows = batch * beams;
  const int K2 = 2 * beams;
  float* pmax = static_cast<float*>(scratch_f);
  float* psum = pmax + static_cast<long long>(rows) * S;
  float* cval = psum + static_cast<long long>(rows) * S;
  int* cidx = static_cast<int*>(scratch_i);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 g1(S, rows);
  BeamState bs;
  bs.pmax = pmax;
  bs.psum = psum;
  bs.cand_val = cval;
  bs.cand_idx = cidx;
  bs.live_lp = static_cast<float*>(live_lp);
  bs.live_seqs = static_cast<long long*>(live_seqs);
  bs.fin_seqs = static_cast<long long*>(fin_seqs);
  bs.fin_scores = static_cast<float*>(fin_scores);
  bs.fin_flags = static_cast<unsigned char*>(fin_flags);
  bs.anc = static_cast<int*>(anc);
  bs.cur = static_cast<int*>(cur);
  bs.term_b = static_cast<unsigned char*>(flags);
  bs.terminated = static_cast<unsigned char*>(terminated);
  bs.ticket = static_cast<unsigned int*>(ticket);
  bs.batch = batch;
  bs.k = beams;
  bs.L = L;
  bs.V = V;
  bs.S = S;
  bs.eos = eos;
  bs.alpha = alpha;
  bs.min_brevity = min_brevity;
  const size_t smem = static_cast<size_t>(3) * beams * L * sizeof(int) +
                      static_cast<size_t>(beams) * S * K2 * (sizeof(float) + sizeof(int));
  if (smem > 200 * 1024)
    return set_error("beam_step: beams=%d length=%d needs %zu bytes of shared memory", beams, L,
                     smem);
  const float* lg = static_cast<const float*>(logits);
  if (V < 2) return set_error("beam_step: vocabulary of %d entries", V);
  cudaError_t e = cudaSuccess;
  // the opt-in limit is raised once per (device, kernel) to the most any call can ask for
  static bool attr_set[64][4] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const int slot = K2 == 2 ? 0 : K2 == 4 ? 1 : K2 == 8 ? 2 : 3;
#define T5X_BEAM_CASE(K2V)                                                                     \
  case K2V:                                                                                    \
    if (!attr_set[dev & 63][slot]) {                                                           \
      e = cudaFuncSetAttribute(beam_update_kernel<K2V>,                                        \
                               cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);       \
      if (e != cudaSuccess) break;                                                             \
      attr_set[dev & 63][slot] = true;                                                         \
    }                                                                                          \
    beam_partial_kernel<K2V><<<g1, kBeamThreads, 0, st>>>(lg, ld, V, chunk, pmax, psum, cval, cidx); \
    beam_update_kernel<K2V><<<batch, kBeamThreads, smem, st>>>(bs);                            \
    break;
  switch (K2) {
    T5X_BEAM_CASE(2)
    T5X_BEAM_CASE(4)
    T5X_BEAM_CASE(8)
    T5X_BEAM_CASE(16)
    default:
      return set_error("beam_step: unsupported beam count");
  }
#undef T5X_BEAM_CASE
  if (e != cudaSuccess) return set_error("beam_step: %s", cudaGetErrorString(e));
  count_launches(2);
  e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("beam_step launch: %s", cudaGetErrorString(e));
  return 0;
}

// tokens[rows] (int64) and log_probs[rows] drawn from softmax(mask(logits / temperature)).
// temperature / topp: per-row device arrays, or null to use the scalars. temperature 0 takes the
// arg-max. topk 0 and topp 0 disable the respective mask.
T5X_API int t5x_sample_tokens(const void* logits, long long ld, int rows, int V,
                              const void* temperature, float temperature_scalar, int topk,
                              const void* topp, float topp_scalar, int rescale_log_probs,
                              unsigned long long seed, unsigned int stream_id, void* tokens,
                              void* log_probs, void* stream) {
  using namespace t5x;
  if (rows <= 0) return 0;
  if (V <= 0 || logits == nullptr || tokens == nullptr || log_probs == nullptr)
    return set_error("sample_tokens: bad arguments");
  SampleParams p = {};
  p.logits = static_cast<const float*>(logits);
  p.ld = ld;
  p.rows = rows;
  p.V = V;
  p.temperature = static_cast<const float*>(temperature);
  p.temperature_scalar = temperature_scalar;
  p.topk = topk;
  p.topp = static_cast<const float*>(topp);
  p.topp_scalar = topp_scalar;
  p.rescale_log_probs = rescale_log_probs;
  p.seed = seed;
  p.stream = stream_id;
  p.tokens = static_cast<long long*>(tokens);
  p.log_probs = static_cast<float*>(log_probs);
  sample_kernel<false><<<rows, kSampleThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("sample_tokens launch: %s", cudaGetErrorString(e));
  return 0;
}

// out = logits where the entry survives top-k (topk > 0) and/or top-p (topp > 0), else replace_val.
T5X_API int t5x_topk_topp_mask(const void* logits, long long ld, void* out, long long ld_out,
                               int rows, int V, int topk, const void* topp, float topp_scalar,
                               float replace_val, void* stream) {
  using namespace t5x;
  if (rows <= 0) return 0;
  if (V <= 0 || logits == nullptr || out == nullptr) return set_error("topk_topp_mask: bad arguments");
  SampleParams p = {};
  p.logits = static_cast<const float*>(logits);
  p.ld = ld;
  p.rows = rows;
  p.V = V;
  p.topk = topk;
  p.topp = static_cast<const float*>(topp);
  p.topp_scalar = topp_scalar;
  p.masked_out = static_cast<float*>(out);
  p.ld_out = ld_out;
  p.replace_val = replace_val;
  sample_kernel<true><<<rows, kSampleThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error("topk_topp_mask launch: %s", cudaGetErrorString(e));
  return 0;
}
