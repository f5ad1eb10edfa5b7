// CPU runtime, part 4: transformer kernels for the host path (oracles, small deployments, tests without a GPU).
//
//  * Blockwise ("flash") attention in fp32: queries of one (batch, head) walk the key/value blocks in ascending
//    order with an online softmax (running max and normaliser), so nothing of size S x S is ever materialised.
//    GQA (query head h reads KV head h / (H / Hkv)), causal or full. Work is split over threads by (batch, head):
//    every output row is produced by one thread in a fixed order, so results do not depend on the thread count.
//  * W8A8 dynamic linear layer: activations are quantised per row to int8 (scale = max|x| / 127, round half away
//    from zero), weights are int8 with one fp32 scale per output column, the product accumulates in int32 and is
//    rescaled once: the arithmetic of scirust-core/src/quantization.rs:150-190 (`quantized_linear_forward`).
//  * An int8 decoder block (RMSNorm -> W8A8 q/k/v -> RoPE -> flash attention -> W8A8 o -> +res -> RMSNorm -> W8A8
//    gate/up -> SwiGLU -> W8A8 down -> +res) built from the pieces above (scirust-simd/src/qtransformer.rs:99-229).
//  * A KV cache with fp32 or per-row int8 storage and single-query attention over it
//    (scirust-simd/src/kv_cache.rs, attention.rs:194-389).
// The reference implements these with AVX2 / AVX-512 / NEON intrinsics behind a run-time dispatcher; this is one
// portable C++ statement of the same arithmetic (compiled with -ffp-contract=off), not a SIMD dispatch layer.
#include <math.h>
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <thread>
#include <vector>

namespace {

template <typename F>
void parallel_for(int64_t n, int threads, F f) {
  if (threads <= 1 || n <= 1) {
    for (int64_t i = 0; i < n; ++i) f(i);
    return;
  }
  const int t = static_cast<int>(std::min<int64_t>(threads, n));
  std::vector<std::thread> pool;
  for (int w = 0; w < t; ++w)
    pool.emplace_back([=]() {
      for (int64_t i = w; i < n; i += t) f(i);
    });
  for (auto& th : pool) th.join();
}

inline int8_t quant_round(float v) {
  float r = v >= 0.f ? floorf(v + 0.5f) : ceilf(v - 0.5f);
  if (r > 127.f) r = 127.f;
  if (r < -128.f) r = -128.f;
  return static_cast<int8_t>(r);
}

// one query row against keys/values [n, dh] (row pitch ld), blockwise online softmax
void attend_row(const float* q, const float* K, const float* V, int64_t ld, int64_t n, int dh, float scale, int block,
                float* out) {
  float m = -INFINITY, l = 0.f;
  for (int d = 0; d < dh; ++d) out[d] = 0.f;
  std::vector<float> s(static_cast<size_t>(block));
  for (int64_t j0 = 0; j0 < n; j0 += block) {
    const int64_t j1 = std::min<int64_t>(n, j0 + block);
    float bm = -INFINITY;
    for (int64_t j = j0; j < j1; ++j) {
      float acc = 0.f;
      const float* k = K + j * ld;
      for (int d = 0; d < dh; ++d) acc += q[d] * k[d];
      s[j - j0] = acc * scale;
      bm = std::max(bm, s[j - j0]);
    }
    const float mn = std::max(m, bm);
    const float corr = (m == -INFINITY) ? 0.f : expf(m - mn);
    l *= corr;
    for (int d = 0; d < dh; ++d) out[d] *= corr;
    for (int64_t j = j0; j < j1; ++j) {
      const float p = expf(s[j - j0] - mn);
      l += p;
      const float* v = V + j * ld;
      for (int d = 0; d < dh; ++d) out[d] += p * v[d];
    }
    m = mn;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  for (int d = 0; d < dh; ++d) out[d] *= inv;
}

}  // namespace

extern "C" {

// q [B, S, H, dh], k / v [B, S, Hkv, dh], out [B, S, H, dh] (contiguous fp32).
int sbrt_flash_attention_f32(const float* q, const float* k, const float* v, float* out, int64_t B, int64_t S, int H,
                             int Hkv, int dh, int causal, int block, int threads) {
  if (B <= 0 || S <= 0 || H <= 0 || Hkv <= 0 || dh <= 0 || H % Hkv || block <= 0) return 1;
  const float scale = 1.0f / sqrtf(static_cast<float>(dh));
  const int rep = H / Hkv;
  parallel_for(B * H, threads, [&](int64_t bh) {
    const int64_t b = bh / H;
    const int h = static_cast<int>(bh % H), hk = h / rep;
    const float* Kb = k + (b * S * Hkv + hk) * dh;
    const float* Vb = v + (b * S * Hkv + hk) * dh;
    for (int64_t i = 0; i < S; ++i) {
      const int64_t n = causal ? i + 1 : S;
      attend_row(q + ((b * S + i) * H + h) * dh, Kb, Vb, static_cast<int64_t>(Hkv) * dh, n, dh, scale, block,
                 out + ((b * S + i) * H + h) * dh);
    }
  });
  return 0;
}

// y [M, N] = dequant(quant_rows(x [M, K]) . wq [K, N]) (+ bias [N]); x_scale_out (optional) [M].
int sbrt_w8a8_linear(const float* x, const int8_t* wq, const float* w_scale, const float* bias, float* y, int64_t M,
                     int64_t K, int64_t N, float* x_scale_out, int threads) {
  if (M <= 0 || K <= 0 || N <= 0) return 1;
  parallel_for(M, threads, [&](int64_t m) {
    const float* xr = x + m * K;
    float amax = 0.f;
    for (int64_t i = 0; i < K; ++i) amax = std::max(amax, fabsf(xr[i]));
    const float sx = amax == 0.f ? 1.f : amax / 127.f;
    if (x_scale_out) x_scale_out[m] = sx;
    std::vector<int8_t> xq(static_cast<size_t>(K));
    for (int64_t i = 0; i < K; ++i) xq[i] = quant_round(xr[i] / sx);
    std::vector<int32_t> acc(static_cast<size_t>(N), 0);
    for (int64_t i = 0; i < K; ++i) {
      const int32_t xv = xq[i];
      if (xv == 0) continue;
      const int8_t* wr = wq + i * N;
      for (int64_t n = 0; n < N; ++n) acc[n] += xv * static_cast<int32_t>(wr[n]);
    }
    for (int64_t n = 0; n < N; ++n) {
      float r = static_cast<float>(acc[n]) * (sx * w_scale[n]);
      if (bias) r += bias[n];
      y[m * N + n] = r;
    }
  });
  return 0;
}

static void rmsnorm_rows(const float* x, const float* g, float* y, int64_t rows, int64_t d, float eps) {
  for (int64_t r = 0; r < rows; ++r) {
    float ss = 0.f;
    for (int64_t i = 0; i < d; ++i) ss += x[r * d + i] * x[r * d + i];
    const float inv = 1.0f / sqrtf(ss / static_cast<float>(d) + eps);
    for (int64_t i = 0; i < d; ++i) y[r * d + i] = x[r * d + i] * inv * g[i];
  }
}

static void rope_rows(float* x, int64_t S, int heads, int dh, float theta, int64_t row_pitch) {
  for (int64_t s = 0; s < S; ++s)
    for (int h = 0; h < heads; ++h)
      for (int p = 0; p < dh / 2; ++p) {
        const float freq = powf(theta, -2.0f * static_cast<float>(p) / static_cast<float>(dh));
        const float ang = static_cast<float>(s) * freq, c = cosf(ang), sn = sinf(ang);
        float* e = x + s * row_pitch + h * dh + 2 * p;
        const float x0 = e[0], x1 = e[1];
        e[0] = x0 * c - x1 * sn;
        e[1] = x0 * sn + x1 * c;
      }
}

// One decoder block on a sequence x [S, d] with int8 weights (x.W layout, per-column scales). Weight order:
// wq [d, H*dh], wk / wv [d, Hkv*dh], wo [H*dh, d], wg / wu [d, ff], wd [ff, d]; s_* their scales.
int sbrt_int8_decoder_block(const float* x, float* out, int64_t S, int d, int H, int Hkv, int ff, float theta, float eps,
                            const float* g1, const float* g2, const int8_t* wq, const float* s_q, const int8_t* wk,
                            const float* s_k, const int8_t* wv, const float* s_v, const int8_t* wo, const float* s_o,
                            const int8_t* wg, const float* s_g, const int8_t* wu, const float* s_u, const int8_t* wd,
                            const float* s_d, int threads) {
  if (S <= 0 || d <= 0 || H <= 0 || Hkv <= 0 || H % Hkv || d % H || ff <= 0) return 1;
  const int dh = d / H;
  const int64_t kvd = static_cast<int64_t>(Hkv) * dh;
  std::vector<float> h(S * d), q(S * d), k(S * kvd), v(S * kvd), ctx(S * d), x2(S * d), gt(S * ff), up(S * ff);
  rmsnorm_rows(x, g1, h.data(), S, d, eps);
  sbrt_w8a8_linear(h.data(), wq, s_q, nullptr, q.data(), S, d, d, nullptr, threads);
  sbrt_w8a8_linear(h.data(), wk, s_k, nullptr, k.data(), S, d, kvd, nullptr, threads);
  sbrt_w8a8_linear(h.data(), wv, s_v, nullptr, v.data(), S, d, kvd, nullptr, threads);
  rope_rows(q.data(), S, H, dh, theta, d);
  rope_rows(k.data(), S, Hkv, dh, theta, kvd);
  sbrt_flash_attention_f32(q.data(), k.data(), v.data(), ctx.data(), 1, S, H, Hkv, dh, 1, 64, threads);
  sbrt_w8a8_linear(ctx.data(), wo, s_o, nullptr, x2.data(), S, d, d, nullptr, threads);
  for (int64_t i = 0; i < S * d; ++i) x2[i] += x[i];
  rmsnorm_rows(x2.data(), g2, h.data(), S, d, eps);
  sbrt_w8a8_linear(h.data(), wg, s_g, nullptr, gt.data(), S, d, ff, nullptr, threads);
  sbrt_w8a8_linear(h.data(), wu, s_u, nullptr, up.data(), S, d, ff, nullptr, threads);
  for (int64_t i = 0; i < S * ff; ++i) gt[i] = gt[i] / (1.0f + expf(-gt[i])) * up[i];
  sbrt_w8a8_linear(gt.data(), wd, s_d, nullptr, out, S, ff, d, nullptr, threads);
  for (int64_t i = 0; i < S * d; ++i) out[i] += x2[i];
  return 0;
}

// ---- KV cache: rows of `dim` floats, stored fp32 or int8 (per-row scale) ------------------------------
struct SbKvCache {
  int dim, quantized;
  int64_t capacity, len;
  std::vector<float> kf, vf, ks, vs;
  std::vector<int8_t> kq, vq;
};

void* sbrt_kv_new(int dim, int64_t capacity, int quantized) {
  if (dim <= 0 || capacity <= 0) return nullptr;
  auto* c = new SbKvCache{dim, quantized, capacity, 0, {}, {}, {}, {}, {}, {}};
  if (quantized) {
    c->kq.resize(capacity * dim); c->vq.resize(capacity * dim); c->ks.resize(capacity); c->vs.resize(capacity);
  } else {
    c->kf.resize(capacity * dim); c->vf.resize(capacity * dim);
  }
  return c;
}
void sbrt_kv_free(void* h) { delete static_cast<SbKvCache*>(h); }
int64_t sbrt_kv_len(void* h) { return static_cast<SbKvCache*>(h)->len; }
int64_t sbrt_kv_bytes(void* h) {
  auto* c = static_cast<SbKvCache*>(h);
  return c->quantized ? c->len * (2 * c->dim + 8) : c->len * 2 * c->dim * 4;
}
int sbrt_kv_append(void* h, const float* k, const float* v) {
  auto* c = static_cast<SbKvCache*>(h);
  if (c->len >= c->capacity) return 5;
  const int64_t t = c->len, d = c->dim;
  if (!c->quantized) {
    memcpy(&c->kf[t * d], k, d * 4);
    memcpy(&c->vf[t * d], v, d * 4);
  } else {
    for (int which = 0; which < 2; ++which) {
      const float* src = which ? v : k;
      float amax = 0.f;
      for (int i = 0; i < d; ++i) amax = std::max(amax, fabsf(src[i]));
      const float s = amax == 0.f ? 1.f : amax / 127.f;
      (which ? c->vs : c->ks)[t] = s;
      int8_t* dst = &(which ? c->vq : c->kq)[t * d];
      for (int i = 0; i < d; ++i) dst[i] = quant_round(src[i] / s);
    }
  }
  c->len++;
  return 0;
}
// single-query attention over the cache (one head of dimension dim)
int sbrt_kv_attend(void* h, const float* q, float* out, int block) {
  auto* c = static_cast<SbKvCache*>(h);
  if (c->len == 0 || block <= 0) return 1;
  const int64_t n = c->len, d = c->dim;
  const float scale = 1.0f / sqrtf(static_cast<float>(d));
  if (!c->quantized) {
    attend_row(q, c->kf.data(), c->vf.data(), d, n, static_cast<int>(d), scale, block, out);
    return 0;
  }
  // dequantise block by block into scratch, same online softmax
  std::vector<float> kb(static_cast<size_t>(block) * d), vb(static_cast<size_t>(block) * d), s(block);
  float m = -INFINITY, l = 0.f;
  for (int i = 0; i < d; ++i) out[i] = 0.f;
  for (int64_t j0 = 0; j0 < n; j0 += block) {
    const int64_t j1 = std::min<int64_t>(n, j0 + block);
    float bm = -INFINITY;
    for (int64_t j = j0; j < j1; ++j) {
      float acc = 0.f;
      for (int i = 0; i < d; ++i) acc += q[i] * (static_cast<float>(c->kq[j * d + i]) * c->ks[j]);
      s[j - j0] = acc * scale;
      bm = std::max(bm, s[j - j0]);
    }
    const float mn = std::max(m, bm), corr = (m == -INFINITY) ? 0.f : expf(m - mn);
    l *= corr;
    for (int i = 0; i < d; ++i) out[i] *= corr;
    for (int64_t j = j0; j < j1; ++j) {
      const float p = expf(s[j - j0] - mn);
      l += p;
      for (int i = 0; i < d; ++i) out[i] += p * (static_cast<float>(c->vq[j * d + i]) * c->vs[j]);
    }
    m = mn;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  for (int i = 0; i < d; ++i) out[i] *= inv;
  return 0;
}

}  // extern "C"
