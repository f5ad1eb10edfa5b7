// Deterministic device-side token sampler: repetition penalty -> greedy (T <= 0) or softmax(x / T)
// -> top-k -> top-p -> renormalise -> inverse-CDF draw, one CTA per logits row, no host round trip.
//
// Policy and RNG stream follow the reference's host sampler (scirust-sciagent/src/generate.rs:202-337;
// splitmix64-seeded xorshift64, u = (s >> 11) / 2^53) and its WGSL device sampler's purpose: keep the
// token on the device. Differences by design: probabilities are turned into 32-bit fixed-point
// weights w_j = floor(exp((x_j - max) / T) * 2^32) and every sum is an integer sum, so the result does
// not depend on the order in which threads add (atomics on integers are order-free) and a seed gives
// the same tokens on every run and every grid shape. Ranking is (weight descending, id ascending),
// the host sampler's order; rank cut-offs and the draw are found with radix-select passes over the
// row instead of a sort. The host sampler adds floats sequentially, so the two can differ only when
// the uniform draw falls within rounding distance of a CDF boundary.
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include "api.h"

namespace sb {

constexpr int SAMP_THREADS = 1024;
constexpr int SAMP_MAX_WINDOW = 256;

struct SampleParams {
  const float* logits; int ld; int V;
  float temperature; int top_k; float top_p;
  float rep_penalty; int rep_window;
  const int64_t* recent; int recent_ld;   // [B, recent_ld] token history (most recent last), may be null
  const int* n_recent;                    // [B] valid entries per row
  uint64_t* rng_state;                    // [B] xorshift64 states, advanced by one draw per call
  int64_t* out_tokens;                    // [B]
  int64_t* generated; int gen_stride; int step;   // optional [B, gen_stride] log of emitted tokens
  uint32_t* work;                         // [B, V] scratch (penalised logits, then weights)
};

struct Walk {          // result of one ranked walk
  unsigned long long sum;   // inclusive weight sum where the walk stopped
  int id;                   // element at which it stopped
};

__device__ __forceinline__ float block_max(float v, float* red) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[0];
  for (int i = 1; i < SAMP_THREADS / 32; ++i) r = fmaxf(r, red[i]);
  __syncthreads();
  return r;
}

// Visits every element (index, value) of a row of 32-bit words once, thread-strided. Rows whose length is a
// multiple of 4 are read as 16-byte vectors, two loads in flight per thread: a pass over a 128 k row is then
// bound by a handful of L2 round trips instead of 125 dependent ones.
template <class F>
__device__ __forceinline__ void for_each_word(const uint32_t* w, int V, F&& f) {
  if ((V & 3) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
    const uint4* w4 = reinterpret_cast<const uint4*>(w);
    const int n4 = V >> 2;
    for (int j0 = threadIdx.x; j0 < n4; j0 += 2 * SAMP_THREADS) {
      const int j1 = j0 + SAMP_THREADS;
      const uint4 a = w4[j0];
      uint4 b = make_uint4(0u, 0u, 0u, 0u);
      if (j1 < n4) b = w4[j1];
      f(4 * j0, a.x); f(4 * j0 + 1, a.y); f(4 * j0 + 2, a.z); f(4 * j0 + 3, a.w);
      if (j1 < n4) { f(4 * j1, b.x); f(4 * j1 + 1, b.y); f(4 * j1 + 2, b.z); f(4 * j1 + 3, b.w); }
    }
  } else {
    for (int j = threadIdx.x; j < V; j += SAMP_THREADS) f(j, w[j]);
  }
}

// Ranked walk over the weights of one row (rank = weight descending, id ascending). Stops at the
// first rank r where either r + 1 == limit_count, or the inclusive sum reaches `target`
// (>= target, or > target when `strict`). Returns the inclusive sum there and, if want_id, the id.
__device__ Walk ranked_walk(const uint32_t* w, int V, unsigned long long limit_count, unsigned long long target,
                            bool strict, bool want_id, unsigned long long* h_cnt, unsigned long long* h_sum,
                            unsigned long long* s_state) {
  // s_state: [0] prefix value, [1] count before, [2] sum before, [3] chosen digit / scratch
  uint32_t prefix = 0;
  unsigned long long cnt_before = 0, sum_before = 0;
  for (int level = 0; level < 4; ++level) {
    const int shift = 24 - 8 * level;
    const uint32_t mask_hi = level == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = threadIdx.x; i < 256; i += SAMP_THREADS) { h_cnt[i] = 0; h_sum[i] = 0; }
    __syncthreads();
    {
      // most weights of a peaked distribution share one digit: a thread batches the run of equal
      // digits it sees and touches the histogram only when the digit changes
      int cur = -1;
      unsigned long long c_run = 0, s_run = 0;
      for_each_word(w, V, [&](int, uint32_t v) {
        if ((v & mask_hi) == prefix) {
          const int d = (v >> shift) & 0xff;
          if (d != cur) {
            if (c_run) { atomicAdd(&h_cnt[cur], c_run); atomicAdd(&h_sum[cur], s_run); }
            cur = d; c_run = 0; s_run = 0;
          }
          c_run += 1;
          s_run += v;
        }
      });
      if (c_run) { atomicAdd(&h_cnt[cur], c_run); atomicAdd(&h_sum[cur], s_run); }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int d = 255;
      for (; d > 0; --d) {
        const unsigned long long c = cnt_before + h_cnt[d], sm = sum_before + h_sum[d];
        const bool by_count = c >= limit_count;
        const bool by_sum = strict ? sm > target : sm >= target;
        if (h_cnt[d] != 0 && (by_count || by_sum)) break;
        cnt_before = c;
        sum_before = sm;
      }
      // d == 0 is taken when nothing above crosses (the walk then ends inside or after bin 0)
      s_state[0] = prefix | (static_cast<uint32_t>(d) << shift);
      s_state[1] = cnt_before;
      s_state[2] = sum_before;
    }
    __syncthreads();
    prefix = static_cast<uint32_t>(s_state[0]);
    cnt_before = s_state[1];
    sum_before = s_state[2];
    __syncthreads();
  }
  // all elements with weight == prefix are tied; they are taken in id order
  const unsigned long long v = prefix;
  unsigned long long n_ties = 0;
  {
    if (threadIdx.x == 0) s_state[3] = 0;
    __syncthreads();
    unsigned long long local = 0;
    for_each_word(w, V, [&](int, uint32_t x) { local += (x == prefix) ? 1 : 0; });
    if (local) atomicAdd(&s_state[3], local);
    __syncthreads();
    n_ties = s_state[3];
    __syncthreads();
  }
  unsigned long long take = n_ties;                    // ties consumed, the stopping element included
  if (limit_count - cnt_before < take) take = limit_count - cnt_before;
  if (v > 0) {
    unsigned long long need;                            // ties needed for the sum criterion
    if (strict) need = target >= sum_before ? (target - sum_before) / v + 1 : 1;
    else need = target > sum_before ? (target - sum_before + v - 1) / v : 1;
    if (need < take) take = need;
  }
  if (take < 1) take = 1;
  Walk out;
  out.sum = sum_before + take * v;
  out.id = 0;
  if (!want_id) return out;
  // id of the take-th smallest id among the ties: radix-select on the id (three 8-bit levels)
  unsigned long long k = take - 1;   // 0-based index among ties
  uint32_t id_prefix = 0;
  for (int level = 0; level < 3; ++level) {
    const int shift = 16 - 8 * level;
    const uint32_t mask_hi = level == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = threadIdx.x; i < 256; i += SAMP_THREADS) h_cnt[i] = 0;
    __syncthreads();
    for_each_word(w, V, [&](int j, uint32_t x) {
      if (x == prefix && (static_cast<uint32_t>(j) & mask_hi) == id_prefix) atomicAdd(&h_cnt[(j >> shift) & 0xff], 1ull);
    });
    __syncthreads();
    if (threadIdx.x == 0) {
      int d = 0;
      for (; d < 255; ++d) {
        if (k < h_cnt[d]) break;
        k -= h_cnt[d];
      }
      s_state[0] = id_prefix | (static_cast<uint32_t>(d) << shift);
      s_state[1] = k;
    }
    __syncthreads();
    id_prefix = static_cast<uint32_t>(s_state[0]);
    k = s_state[1];
    __syncthreads();
  }
  out.id = static_cast<int>(id_prefix);
  return out;
}

__global__ void __launch_bounds__(SAMP_THREADS)
sample_rows_kernel(const SampleParams p) {
  __shared__ unsigned long long h_cnt[256], h_sum[256], s_state[4];
  __shared__ float red[SAMP_THREADS / 32];
  __shared__ int red_i[SAMP_THREADS / 32];
  __shared__ int64_t s_tok[SAMP_MAX_WINDOW];
  __shared__ float s_val[SAMP_MAX_WINDOW];
  const int row = blockIdx.x;
  const int V = p.V;
  const float* x = p.logits + static_cast<size_t>(row) * p.ld;
  float* wf = reinterpret_cast<float*>(p.work + static_cast<size_t>(row) * V);
  uint32_t* w = p.work + static_cast<size_t>(row) * V;

  // ---- penalised copy of the row ----
  for (int j = threadIdx.x; j < V; j += SAMP_THREADS) wf[j] = x[j];
  int n_win = 0;
  if (p.rep_penalty > 1.0f && p.recent && p.n_recent) {
    const int n = p.n_recent[row];
    n_win = min(min(n, p.rep_window), SAMP_MAX_WINDOW);
    const int64_t* rec = p.recent + static_cast<size_t>(row) * p.recent_ld + (n - n_win);
    if (threadIdx.x < n_win) {
      const int64_t t = rec[threadIdx.x];
      s_tok[threadIdx.x] = t;
      s_val[threadIdx.x] = (t >= 0 && t < V) ? x[t] : 0.f;
    }
  }
  __syncthreads();
  if (n_win > 0 && threadIdx.x == 0) {
    // every occurrence in the window applies the penalty once more, oldest first
    for (int i = 0; i < n_win; ++i) {
      const int64_t t = s_tok[i];
      if (t < 0 || t >= V) continue;
      int first = i;
      for (int k = 0; k < i; ++k) if (s_tok[k] == t) { first = k; break; }
      const float l = s_val[first];
      s_val[first] = l > 0.f ? l / p.rep_penalty : l * p.rep_penalty;
    }
    for (int i = 0; i < n_win; ++i) {
      const int64_t t = s_tok[i];
      if (t < 0 || t >= V) continue;
      int first = i;
      for (int k = 0; k < i; ++k) if (s_tok[k] == t) { first = k; break; }
      if (first == i) wf[t] = s_val[i];
    }
  }
  __syncthreads();

  int token;
  if (p.temperature <= 0.f) {
    // greedy: first maximum, a NaN never wins against a number
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int j = threadIdx.x; j < V; j += SAMP_THREADS) {
      float v = wf[j];
      v = v != v ? -INFINITY : v;          // a NaN never beats a number
      if (bi == 0x7fffffff) { best = v; bi = j; }
      else if (v > best) { best = v; bi = j; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      const bool take = (ob > best) || (!(best > ob) && !(ob > best) && oi < bi);
      if (take) { best = ob; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { red[threadIdx.x >> 5] = best; red_i[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int i = 1; i < SAMP_THREADS / 32; ++i) {
        const float ob = red[i];
        const int oi = red_i[i];
        const bool take = (ob > best) || (!(best > ob) && !(ob > best) && oi < bi);
        if (take) { best = ob; bi = oi; }
      }
      // the host rule starts from element 0, so a NaN there is never displaced
      red_i[0] = (bi == 0x7fffffff || wf[0] != wf[0]) ? 0 : bi;
    }
    __syncthreads();
    token = red_i[0];
  } else {
    float mx = -INFINITY;
    for (int j = threadIdx.x; j < V; j += SAMP_THREADS) mx = fmaxf(mx, wf[j]);
    mx = block_max(mx, red);
    // fixed-point weights, total in s_state[3]
    if (threadIdx.x == 0) s_state[3] = 0;
    __syncthreads();
    unsigned long long local = 0;
    const float inv_t = 1.0f / p.temperature;
    for (int j = threadIdx.x; j < V; j += SAMP_THREADS) {
      const float e = expf((wf[j] - mx) * inv_t);              // in [0, 1]
      const float s = e * 4294967296.0f;
      const uint32_t q = s >= 4294967040.0f ? 0xffffffffu : static_cast<uint32_t>(s);
      w[j] = q;
      local += q;
    }
    atomicAdd(&s_state[3], local);
    __syncthreads();
    const unsigned long long z = s_state[3];
    __syncthreads();
    // kept set: first min(top_k, V) ranks, cut where the cumulative probability reaches top_p
    const unsigned long long limit = (p.top_k > 0 && p.top_k < V) ? static_cast<unsigned long long>(p.top_k)
                                                                   : static_cast<unsigned long long>(V);
    unsigned long long zz = z;
    if (limit < static_cast<unsigned long long>(V) || p.top_p < 1.0f) {
      unsigned long long tp = ~0ull;   // unreachable sum: only the count stops the walk
      if (p.top_p < 1.0f) {
        const double t = static_cast<double>(p.top_p) * static_cast<double>(z);
        tp = t <= 1.0 ? 1ull : static_cast<unsigned long long>(ceil(t));
      }
      zz = ranked_walk(w, V, limit, tp, false, false, h_cnt, h_sum, s_state).sum;
    }
    // one uniform draw
    if (threadIdx.x == 0) {
      uint64_t s = p.rng_state[row];
      s ^= s << 13; s ^= s >> 7; s ^= s << 17;
      p.rng_state[row] = s;
      const float u = static_cast<float>(static_cast<double>(s >> 11) / 9007199254740992.0);
      const double t = static_cast<double>(u) * static_cast<double>(zz);
      unsigned long long ti = static_cast<unsigned long long>(t);
      if (zz > 0 && ti >= zz) ti = zz - 1;
      s_state[3] = ti;
    }
    __syncthreads();
    const unsigned long long target = s_state[3];
    __syncthreads();
    token = ranked_walk(w, V, static_cast<unsigned long long>(V), target, true, true, h_cnt, h_sum, s_state).id;
  }
  if (threadIdx.x == 0) {
    p.out_tokens[row] = token;
    if (p.generated) p.generated[static_cast<size_t>(row) * p.gen_stride + p.step] = token;
  }
}

}  // namespace sb

using namespace sb;

// logits: fp32 [rows, ld]; work: rows*V 32-bit words of scratch; rng_state: one xorshift64 state per
// row (advanced by one draw when temperature > 0); recent/n_recent: optional token history for the
// repetition penalty (window <= 256). vocab < 2^24.
extern "C" int sb_sample_rows(const float* logits, int ld, int rows, int V, float temperature, int top_k, float top_p,
                              float rep_penalty, int rep_window, const int64_t* recent, int recent_ld,
                              const int* n_recent, uint64_t* rng_state, int64_t* out_tokens, int64_t* generated,
                              int gen_stride, int step, uint32_t* work, void* stream) {
  if (rows <= 0 || V <= 0 || V >= (1 << 24) || !work || !out_tokens) return SB_ERR_ARG;
  if (temperature > 0.f && !rng_state) return SB_ERR_ARG;
  SampleParams p;
  p.logits = logits; p.ld = ld; p.V = V; p.temperature = temperature; p.top_k = top_k; p.top_p = top_p;
  p.rep_penalty = rep_penalty; p.rep_window = rep_window; p.recent = recent; p.recent_ld = recent_ld;
  p.n_recent = n_recent; p.rng_state = rng_state; p.out_tokens = out_tokens; p.generated = generated;
  p.gen_stride = gen_stride; p.step = step; p.work = work;
  sample_rows_kernel<<<rows, SAMP_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}
