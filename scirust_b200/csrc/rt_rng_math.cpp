// CPU runtime, part 1: seeded random numbers and fixed-order fp32 math.
//
//  * PCG-XSH-RR 64/32 generator with the float / signed float / Box-Muller normal draws of the
//    reference initialisers (scirust-core/src/nn/rng.rs:9-53, nn/init/mod.rs:22-140). The fp32
//    operations are performed one at a time in single precision with glibc logf/cosf/sqrtf, the
//    same calls the reference's `f32::ln/cos/sqrt` resolve to on Linux, so weights initialised
//    from a seed match bit for bit.
//  * Philox4x32-10 counter-based generator (scirust-core/src/philox.rs:24-201).
//  * splitmix64 -> xorshift64 sampler stream and the `sample_row` decode policy
//    (scirust-sciagent/src/generate.rs:202-337).
//  * Fixed-order fp32 kernels for the deterministic CPU training path: GEMM with per-element
//    sequential-k accumulation (plain and fused-multiply-add variants), row soft-max
//    cross-entropy written operation by operation as the reference loss does
//    (scirust-core/src/nn/loss/cross_entropy.rs:75-134), sequential sums.
// Compiled with -ffp-contract=off so no multiply-add is fused unless asked for with fmaf.
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <numeric>
#include <vector>

extern "C" {

// ------------------------------------------------------------------ PCG32
struct SbPcg {
  uint64_t state;
  uint64_t inc;
};

uint32_t sbrt_pcg_next_u32(SbPcg* g) {
  const uint64_t old = g->state;
  g->state = old * 6364136223846793005ull + g->inc;
  const uint32_t xorshifted = static_cast<uint32_t>(((old >> 18) ^ old) >> 27);
  const uint32_t rot = static_cast<uint32_t>(old >> 59);
  return (xorshifted >> rot) | (xorshifted << ((0u - rot) & 31));
}
void sbrt_pcg_new(SbPcg* g, uint64_t seed) {
  g->state = 0;
  g->inc = (seed << 1) | 1;
  sbrt_pcg_next_u32(g);
  g->state += seed;
  sbrt_pcg_next_u32(g);
}
float sbrt_pcg_float(SbPcg* g) {
  return static_cast<float>(sbrt_pcg_next_u32(g)) / (static_cast<float>(UINT32_MAX) + 1.0f);
}
float sbrt_pcg_float_signed(SbPcg* g) { return 2.0f * sbrt_pcg_float(g) - 1.0f; }
float sbrt_pcg_normal(SbPcg* g, float mean, float stddev) {
  float u1 = sbrt_pcg_float(g);
  if (!(u1 > 1e-12f)) u1 = 1e-12f;  // f32::max(1e-12)
  const float u2 = sbrt_pcg_float(g);
  const float pi = 3.14159265358979323846f;
  const float a = -2.0f * logf(u1);
  const float z = sqrtf(a) * cosf((2.0f * pi) * u2);
  return mean + stddev * z;
}
void sbrt_pcg_fill_normal(SbPcg* g, float mean, float stddev, float* out, size_t n) {
  for (size_t i = 0; i < n; ++i) out[i] = sbrt_pcg_normal(g, mean, stddev);
}
void sbrt_pcg_fill_uniform_signed(SbPcg* g, float bound, float* out, size_t n) {
  for (size_t i = 0; i < n; ++i) out[i] = sbrt_pcg_float_signed(g) * bound;
}
void sbrt_pcg_fill_float(SbPcg* g, float* out, size_t n) {
  for (size_t i = 0; i < n; ++i) out[i] = sbrt_pcg_float(g);
}
// Fisher-Yates with the generator's u32 stream: for i in (1..n).rev(): j = u32 % (i+1).
void sbrt_pcg_shuffle(SbPcg* g, int64_t* idx, size_t n) {
  for (size_t i = n; i-- > 1;) {
    const size_t j = sbrt_pcg_next_u32(g) % (i + 1);
    std::swap(idx[i], idx[j]);
  }
}

// ------------------------------------------------------------------ Philox4x32-10
static inline void philox_round(uint32_t* c, const uint32_t* k) {
  const uint64_t p0 = static_cast<uint64_t>(0xD2511F53u) * c[0];
  const uint64_t p1 = static_cast<uint64_t>(0xCD9E8D57u) * c[2];
  const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c[1] ^ k[0];
  const uint32_t n1 = static_cast<uint32_t>(p1);
  const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c[3] ^ k[1];
  const uint32_t n3 = static_cast<uint32_t>(p0);
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}
void sbrt_philox4x32_10(const uint32_t* counter, const uint32_t* key, uint32_t* out) {
  uint32_t c[4] = {counter[0], counter[1], counter[2], counter[3]};
  uint32_t k[2] = {key[0], key[1]};
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k);
    k[0] += 0x9E3779B9u;
    k[1] += 0xBB67AE85u;
  }
  memcpy(out, c, 16);
}

// ------------------------------------------------------------------ sampler
uint64_t sbrt_seed_to_state(uint64_t seed) {
  uint64_t z = seed + 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return z == 0 ? 0x9E3779B97F4A7C15ull : z;
}
float sbrt_next_uniform(uint64_t* state) {
  uint64_t s = *state;
  s ^= s << 13;
  s ^= s >> 7;
  s ^= s << 17;
  *state = s;
  return static_cast<float>(static_cast<double>(s >> 11) / static_cast<double>(1ull << 53));
}

// Decode policy over one logits row: repetition penalty -> greedy (T <= 0) or softmax(logits/T)
// -> top-k -> top-p -> renormalise -> inverse-CDF draw. Returns the chosen token id.
int64_t sbrt_sample_row(const float* logits, int64_t vocab, float temperature, int64_t top_k, float top_p,
                        float repetition_penalty, int64_t repetition_window, const int64_t* recent,
                        int64_t n_recent, uint64_t* rng) {
  std::vector<float> row(logits, logits + vocab);
  if (repetition_penalty > 1.0f) {
    const int64_t start = n_recent > repetition_window ? n_recent - repetition_window : 0;
    for (int64_t i = start; i < n_recent; ++i) {
      const int64_t tok = recent[i];
      if (tok >= 0 && tok < vocab) {
        const float l = row[tok];
        row[tok] = l > 0.0f ? l / repetition_penalty : l * repetition_penalty;
      }
    }
  }
  if (temperature <= 0.0f) {
    int64_t best = 0;
    float best_val = row[0];
    for (int64_t j = 1; j < vocab; ++j)
      if (row[j] > best_val) { best_val = row[j]; best = j; }
    return best;
  }
  float mx = -INFINITY;
  for (int64_t j = 0; j < vocab; ++j) mx = fmaxf(mx, row[j]);
  std::vector<float> probs(vocab);
  float z = 0.0f;
  for (int64_t j = 0; j < vocab; ++j) {
    probs[j] = expf((row[j] - mx) / temperature);
    z += probs[j];  // sequential sum, as Iterator::sum
  }
  for (int64_t j = 0; j < vocab; ++j) probs[j] /= z;
  std::vector<int64_t> order(vocab);
  std::iota(order.begin(), order.end(), 0);
  // descending probability; ties keep ascending id (the reference's unstable sort leaves tie order
  // unspecified, ids ascending is the deterministic choice here)
  std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return probs[a] > probs[b]; });
  int64_t cut = vocab;
  if (top_k > 0) cut = std::min<int64_t>(cut, top_k);
  if (top_p < 1.0f) {
    float cum = 0.0f;
    for (int64_t r = 0; r < cut; ++r) {
      cum += probs[order[r]];
      if (cum >= top_p) { cut = r + 1; break; }
    }
  }
  if (cut < 1) cut = 1;
  float zz = 0.0f;
  for (int64_t r = 0; r < cut; ++r) zz += probs[order[r]];
  const float u = sbrt_next_uniform(rng) * zz;
  float acc = 0.0f;
  for (int64_t r = 0; r < cut; ++r) {
    acc += probs[order[r]];
    if (u < acc) return order[r];
  }
  return order[cut - 1];
}

// ------------------------------------------------------------------ fixed-order fp32 math
// C[m,n] = sum_k A[m,k]*B[k,n], k ascending, one accumulator per element.
// fma != 0 uses fmaf (the order a fused-multiply-add micro-kernel produces for a single
// accumulator chain); fma == 0 rounds the product and the sum separately.
void sbrt_gemm_f32(const float* A, const float* B, float* C, int64_t M, int64_t K, int64_t N, int trans_a,
                   int trans_b, int fma) {
  for (int64_t i = 0; i < M; ++i) {
    for (int64_t j = 0; j < N; ++j) {
      float acc = 0.0f;
      for (int64_t k = 0; k < K; ++k) {
        const float a = trans_a ? A[k * M + i] : A[i * K + k];
        const float b = trans_b ? B[j * K + k] : B[k * N + j];
        acc = fma ? fmaf(a, b, acc) : acc + a * b;
      }
      C[i * N + j] = acc;
    }
  }
}
float sbrt_sum_f32(const float* x, int64_t n) {
  float s = 0.0f;
  for (int64_t i = 0; i < n; ++i) s += x[i];
  return s;
}
// Soft-max cross-entropy with one-hot targets, mean over the batch, in the reference's operation
// order: row max -> sub -> exp -> row sum -> log -> log_softmax = shifted - log_sum ->
// hadamard with target -> total sum -> * (-1/B). Also returns d(loss)/d(logits).
float sbrt_softmax_ce_f32(const float* logits, const int64_t* target, float* dlogits, int64_t B, int64_t C) {
  float total = 0.0f;
  const float inv_b = 1.0f / static_cast<float>(B);
  for (int64_t i = 0; i < B; ++i) {
    const float* r = logits + i * C;
    float mx = r[0];
    for (int64_t j = 1; j < C; ++j) mx = r[j] > mx ? r[j] : mx;
    float s = 0.0f;
    for (int64_t j = 0; j < C; ++j) s += expf(r[j] - mx);
    const float ls = logf(s);
    for (int64_t j = 0; j < C; ++j) {
      const float lsm = (r[j] - mx) - ls;
      const float onehot = (j == target[i]) ? 1.0f : 0.0f;
      total += lsm * onehot;
      if (dlogits) dlogits[i * C + j] = (expf(lsm) - onehot) * inv_b;
    }
  }
  return total * (-inv_b);
}
// v = momentum*v + (g + wd*p); p -= lr*v   (scirust-core/src/autodiff/optim.rs:80-110)
void sbrt_sgd_step_f32(float* p, float* v, const float* g, int64_t n, float lr, float momentum, float wd) {
  for (int64_t i = 0; i < n; ++i) {
    float gi = g[i];
    if (wd > 0.0f) gi += wd * p[i];
    v[i] = momentum * v[i] + gi;
    p[i] -= lr * v[i];
  }
}
// Adam / AdamW with bias correction (optim.rs:176-243, 332-393). decoupled != 0 => AdamW.
void sbrt_adam_step_f32(float* p, float* m, float* v, const float* g, int64_t n, float lr, float b1, float b2,
                        float eps, float wd, float bc1, float bc2, int decoupled) {
  for (int64_t i = 0; i < n; ++i) {
    float gi = g[i];
    if (!decoupled && wd > 0.0f) gi += wd * p[i];
    m[i] = b1 * m[i] + (1.0f - b1) * gi;
    v[i] = b2 * v[i] + (1.0f - b2) * gi * gi;
    const float mhat = m[i] / bc1;
    const float vhat = v[i] / bc2;
    const float theta = p[i];
    if (decoupled) p[i] -= lr * mhat / (sqrtf(vhat) + eps) + lr * wd * theta;
    else p[i] -= lr * mhat / (sqrtf(vhat) + eps);
  }
}

}  // extern "C"

// Bit-portable GEMM: every product and sum in fp64 (an fp32 x fp32 product is exact in fp64),
// k ascending, one rounding to fp32 at the end (scirust-core/src/portable_f32.rs:1033-1075).
extern "C" void sbrt_gemm_f32_portable(const float* A, const float* B, float* C, int64_t M, int64_t K, int64_t N) {
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < N; ++j) {
      double acc = 0.0;
      for (int64_t l = 0; l < K; ++l) acc += static_cast<double>(A[i * K + l]) * static_cast<double>(B[l * N + j]);
      C[i * N + j] = static_cast<float>(acc);
    }
}
