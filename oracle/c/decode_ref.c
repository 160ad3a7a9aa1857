/*
 * C restatement of the reference's Llama-2 per-token decode step on the host CPU (TEST ORACLE and
 * timed CPU baseline only; never linked into the product).  OpenMP over output rows / heads.
 *
 * Follows, op by op with an fp16 rounding wherever the reference graph holds an fp16 tensor:
 *   poptransformer/layers/rms_layer_norm.py:26-36          (RMSNorm)
 *   poptransformer/utils/param_handler/precision_strategy.py:56-60 + custom_ops/int4_to_half_codelets.cpp:18-38
 *                                                          (Int4ToHalf: half(nibble) * half scale, one rounding) then matmul
 *   poptransformer/models/llama2/attention.py:28-114        (RoPE, KVCache shift, scores, fp32 softmax without
 *                                                           max subtraction, P.V)
 *   custom_ops/kv_cache.cpp:118-132                         (newest-first shift cache)
 *   poptransformer/models/llama2/mlp.py:20-28               (SwiGLU MLP)
 * Matmul accumulation is float32 in k order (the reference's accumulation order is a PopLibs detail).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef _Float16 h16;

static inline float h2f(uint16_t b) { h16 h; memcpy(&h, &b, 2); return (float)h; }
static inline uint16_t f2h(float f) { h16 h = (h16)f; uint16_t b; memcpy(&b, &h, 2); return b; }
static inline float rh(float f) { return (float)(h16)f; } /* round through fp16 */

/* y[b][n] = fp16(sum_k float(fp16(q[n][k] * s[n][k/group])) * float(x[b][k])); w: int8 [n][k/2], high nibble = even k */
void oracle_int4_linear(const int8_t *w, const uint16_t *scale, int n, int k, int group, const uint16_t *x, int batch, uint16_t *y) {
  const int ng = k / group;
#pragma omp parallel for schedule(static)
  for (int i = 0; i < n; ++i) {
    float acc[32];
    for (int b = 0; b < batch; ++b) acc[b] = 0.f;
    const int8_t *wr = w + (size_t)i * (k / 2);
    for (int j = 0; j < k / 2; ++j) {
      const int8_t byte = wr[j];
      const float s = h2f(scale[(size_t)i * ng + (2 * j) / group]);
      const float hi = rh((float)(byte >> 4) * s);
      const float lo = rh((float)(((int8_t)(byte << 4)) >> 4) * s);
      for (int b = 0; b < batch; ++b) {
        acc[b] += hi * h2f(x[(size_t)b * k + 2 * j]);
        acc[b] += lo * h2f(x[(size_t)b * k + 2 * j + 1]);
      }
    }
    for (int b = 0; b < batch; ++b) y[(size_t)b * n + i] = f2h(acc[b]);
  }
}

/* w: fp16 [n][k] */
void oracle_f16_linear(const uint16_t *w, int n, int k, const uint16_t *x, int batch, uint16_t *y) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < n; ++i) {
    float acc[32];
    for (int b = 0; b < batch; ++b) acc[b] = 0.f;
    const uint16_t *wr = w + (size_t)i * k;
    for (int j = 0; j < k; ++j) {
      const float wv = h2f(wr[j]);
      for (int b = 0; b < batch; ++b) acc[b] += wv * h2f(x[(size_t)b * k + j]);
    }
    for (int b = 0; b < batch; ++b) y[(size_t)b * n + i] = f2h(acc[b]);
  }
}

void oracle_rms_norm(const uint16_t *x, const uint16_t *gamma, int rows, int dim, float eps, uint16_t *y) {
  for (int r = 0; r < rows; ++r) {
    float ss = 0.f;
    for (int i = 0; i < dim; ++i) { const float v = h2f(x[(size_t)r * dim + i]); ss += v * v; }
    const float rr = rh(1.0f / sqrtf(ss / (float)dim + eps));
    for (int i = 0; i < dim; ++i) y[(size_t)r * dim + i] = f2h(rh(h2f(x[(size_t)r * dim + i]) * rr) * h2f(gamma[i]));
  }
}

typedef struct {
  int d_model, n_head, ffn, max_len, group, batch; /* group == 0: fp16 weights [out][in] */
  float eps;
  const void *wq, *wk, *wv, *wo, *wgate, *wup, *wdown;        /* int8 [out][in/2] or fp16 [out][in] */
  const uint16_t *sq, *sk, *sv, *so, *sgate, *sup, *sdown;    /* fp16 [out][in/group]               */
  const uint16_t *ln1, *ln2;
  uint16_t *kcache, *vcache;                                  /* [batch][n_head][max_len][head_dim], newest first */
  const uint16_t *sin_t, *cos_t;                              /* [max_len][head_dim/2]              */
} oracle_llama_layer;

static void lin(const oracle_llama_layer *L, const void *w, const uint16_t *s, int n, int k, const uint16_t *x, uint16_t *y) {
  if (L->group) oracle_int4_linear((const int8_t *)w, s, n, k, L->group, x, L->batch, y);
  else oracle_f16_linear((const uint16_t *)w, n, k, x, L->batch, y);
}

/* One transformer block for one new token per sequence; x [batch][d_model] is updated in place.
 * scratch must hold batch * (5*d_model + 2*ffn) fp16 values. */
void oracle_llama_layer_step(const oracle_llama_layer *L, int step, uint16_t *x, uint16_t *scratch) {
  const int d = L->d_model, B = L->batch, N = L->n_head, H = d / N, ML = L->max_len, F = L->ffn;
  uint16_t *h = scratch, *q = h + (size_t)B * d, *k = q + (size_t)B * d, *v = k + (size_t)B * d, *a = v + (size_t)B * d;
  uint16_t *g = a + (size_t)B * d, *u = g + (size_t)B * F;
  oracle_rms_norm(x, L->ln1, B, d, L->eps, h);
  lin(L, L->wq, L->sq, d, d, h, q);
  lin(L, L->wk, L->sk, d, d, h, k);
  lin(L, L->wv, L->sv, d, d, h, v);
  const float scale = rh(1.0f / sqrtf((float)H));
  const uint16_t *sn = L->sin_t + (size_t)step * (H / 2), *cs = L->cos_t + (size_t)step * (H / 2);
#pragma omp parallel for collapse(2) schedule(static)
  for (int b = 0; b < B; ++b)
    for (int n = 0; n < N; ++n) {
      uint16_t *qh = q + (size_t)b * d + n * H, *kh = k + (size_t)b * d + n * H, *vh = v + (size_t)b * d + n * H;
      float qr[256], kr[256];
      for (int j = 0; j < H / 2; ++j) { /* rotate_half: rot = concat(-x2, x1) */
        const float c = h2f(cs[j]), s = h2f(sn[j]);
        const float q1 = h2f(qh[j]), q2 = h2f(qh[j + H / 2]), k1 = h2f(kh[j]), k2 = h2f(kh[j + H / 2]);
        qr[j] = rh(rh(q1 * c) + rh(-q2 * s)); qr[j + H / 2] = rh(rh(q2 * c) + rh(q1 * s));
        kr[j] = rh(rh(k1 * c) + rh(-k2 * s)); kr[j + H / 2] = rh(rh(k2 * c) + rh(k1 * s));
      }
      uint16_t *kc = L->kcache + ((size_t)b * N + n) * ML * H, *vc = L->vcache + ((size_t)b * N + n) * ML * H;
      if (step == 0) { memset(kc, 0, (size_t)ML * H * 2); memset(vc, 0, (size_t)ML * H * 2); }
      memmove(kc + H, kc, (size_t)(ML - 1) * H * 2); /* shift right by one position, newest at index 0 */
      memmove(vc + H, vc, (size_t)(ML - 1) * H * 2);
      for (int j = 0; j < H; ++j) { kc[j] = f2h(kr[j]); vc[j] = vh[j]; }
      /* scores over all max_len slots with the additive mask, float32 softmax without max subtraction */
      float *p = (float *)malloc(sizeof(float) * ML);
      float sum = 0.f;
      for (int t = 0; t < ML; ++t) {
        float s = 0.f;
        for (int j = 0; j < H; ++j) s += qr[j] * h2f(kc[(size_t)t * H + j]);
        s = rh(rh(s) * scale);
        s = rh(s + (t <= step ? 0.0f : -10000.0f));
        p[t] = expf(s);
        sum += p[t];
      }
      const float inv = 1.0f / sum;
      float o[256];
      for (int j = 0; j < H; ++j) o[j] = 0.f;
      for (int t = 0; t < ML; ++t) {
        const float pt = rh(p[t] * inv);
        if (pt == 0.f) continue;
        for (int j = 0; j < H; ++j) o[j] += pt * h2f(vc[(size_t)t * H + j]);
      }
      for (int j = 0; j < H; ++j) a[(size_t)b * d + n * H + j] = f2h(o[j]);
      free(p);
    }
  lin(L, L->wo, L->so, d, d, a, h);
  for (size_t i = 0; i < (size_t)B * d; ++i) x[i] = f2h(h2f(x[i]) + h2f(h[i]));
  oracle_rms_norm(x, L->ln2, B, d, L->eps, h);
  lin(L, L->wgate, L->sgate, F, d, h, g);
  lin(L, L->wup, L->sup, F, d, h, u);
  for (size_t i = 0; i < (size_t)B * F; ++i) {
    const float gv = h2f(g[i]);
    const float sw = rh(gv / (1.0f + expf(-gv)));
    g[i] = f2h(h2f(u[i]) * sw);
  }
  lin(L, L->wdown, L->sdown, d, F, g, h);
  for (size_t i = 0; i < (size_t)B * d; ++i) x[i] = f2h(h2f(x[i]) + h2f(h[i]));
}

/* Final norm + fp16 LM head + greedy id (lowest index wins ties). logits [batch][vocab] */
void oracle_llama_head(const uint16_t *x, const uint16_t *norm, const uint16_t *head, int batch, int d, int vocab, float eps,
                       uint16_t *h, uint16_t *logits, int32_t *next_ids) {
  oracle_rms_norm(x, norm, batch, d, eps, h);
  oracle_f16_linear(head, vocab, d, h, batch, logits);
  for (int b = 0; b < batch; ++b) {
    int best = 0;
    float bv = h2f(logits[(size_t)b * vocab]);
    for (int i = 1; i < vocab; ++i) { const float v = h2f(logits[(size_t)b * vocab + i]); if (v > bv) { bv = v; best = i; } }
    next_ids[b] = best;
  }
}
