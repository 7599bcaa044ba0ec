/*
 * CPU restatement, in C, of the reference's CPU decoder-block path — TEST INFRASTRUCTURE
 * AND CPU BASELINE ONLY; the product never links or calls this file.
 *
 * It follows the reference's CpuBackend operator by operator:
 *   forward_layer      crates/apxinf-model/src/llama/general.rs:92-146
 *   rms_norm           crates/apxinf-core/src/op_impls/cpu.rs:10-28   (x / sqrt(mean(x^2)+eps) * w)
 *   matmul             crates/apxinf-core/src/ops.rs:32-42            (naive i-j-p loop, f32)
 *   rope               crates/apxinf-core/src/op_impls/cpu.rs:60-88   (rotate-half, powf/cos/sin in f32)
 *   sdpa_prefill       crates/apxinf-core/src/op_impls/cpu.rs:140-179 (causal, f32, two-pass softmax)
 *   add / mul          crates/apxinf-core/src/op_impls/cpu.rs:36-48
 * The reference CPU backend has no GELU (crates/apxinf-core/src/backend.rs:65-70), so the
 * Gemma-style GeGLU uses the tanh formula of crates/apxinf-cuda/kernels/custom/math.cuh:8-12
 * (activation = 1); activation = 0 is the reference's own SiLU gate.
 * Single-threaded, like the reference backend. Weights are [in, out] row-major float32
 * (the reference up-casts BF16 weights to F32 before any CPU op).
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

static void sgemm_naive(int m, int k, int n, const float* a, const float* b, float* c) {
  for (int i = 0; i < m; ++i) {
    for (int j = 0; j < n; ++j) {
      float sum = 0.0f;
      for (int p = 0; p < k; ++p) sum += a[(size_t)i * k + p] * b[(size_t)p * n + j];
      c[(size_t)i * n + j] = sum;
    }
  }
}

static void rms_norm(const float* x, const float* w, float* out, int rows, int hidden, float eps) {
  for (int s = 0; s < rows; ++s) {
    const float* row = x + (size_t)s * hidden;
    float sum = 0.0f;
    for (int i = 0; i < hidden; ++i) sum += row[i] * row[i];
    const float rms = sqrtf(sum / (float)hidden + eps);
    for (int i = 0; i < hidden; ++i) out[(size_t)s * hidden + i] = (row[i] / rms) * w[i];
  }
}

static void rope(const float* in, float* out, int seq, int heads, int head_dim, float theta,
                 int pos_offset) {
  const int half = head_dim / 2;
  float* freqs = (float*)malloc(sizeof(float) * half);
  for (int i = 0; i < half; ++i) freqs[i] = 1.0f / powf(theta, 2.0f * (float)i / (float)head_dim);
  for (int s = 0; s < seq; ++s) {
    const int pos = pos_offset + s;
    for (int h = 0; h < heads; ++h) {
      const size_t base = ((size_t)s * heads + h) * head_dim;
      for (int i = 0; i < half; ++i) {
        const float angle = (float)pos * freqs[i];
        const float c = cosf(angle), sn = sinf(angle);
        const float x1 = in[base + i], x2 = in[base + half + i];
        out[base + i] = x1 * c - x2 * sn;
        out[base + half + i] = x1 * sn + x2 * c;
      }
    }
  }
  free(freqs);
}

static void sdpa_prefill(const float* q, const float* k, const float* v, float* out, int seq,
                         int heads, int kv_heads, int head_dim, int causal) {
  const float scale = 1.0f / sqrtf((float)head_dim);
  float* scores = (float*)malloc(sizeof(float) * seq);
  memset(out, 0, sizeof(float) * (size_t)seq * heads * head_dim);
  for (int s = 0; s < seq; ++s) {
    for (int h = 0; h < heads; ++h) {
      const int kvh = h * kv_heads / heads;
      const int valid = causal ? s + 1 : seq;
      const float* qrow = q + ((size_t)s * heads + h) * head_dim;
      float max_score = -INFINITY;
      for (int t = 0; t < valid; ++t) {
        const float* krow = k + ((size_t)t * kv_heads + kvh) * head_dim;
        float acc = 0.0f;
        for (int d = 0; d < head_dim; ++d) acc += qrow[d] * krow[d];
        scores[t] = acc * scale;
        if (scores[t] > max_score) max_score = scores[t];
      }
      float exp_sum = 0.0f;
      for (int t = 0; t < valid; ++t) exp_sum += expf(scores[t] - max_score);
      float* orow = out + ((size_t)s * heads + h) * head_dim;
      for (int t = 0; t < valid; ++t) {
        const float p = expf(scores[t] - max_score) / exp_sum;
        const float* vrow = v + ((size_t)t * kv_heads + kvh) * head_dim;
        for (int d = 0; d < head_dim; ++d) orow[d] += p * vrow[d];
      }
    }
  }
  free(scores);
}

static float gelu_tanh(float x) {
  const float alpha = 0.7978845608028654f;
  return 0.5f * x * (1.0f + tanhf(alpha * (x + 0.044715f * x * x * x)));
}

/* One pre-norm decoder block over `seq` tokens; returns 0, or -1 on allocation failure. */
int cpu_block_forward(const float* x, const float* attn_norm, const float* wq, const float* wk,
                      const float* wv, const float* wo, const float* ffn_norm, const float* w_gate,
                      const float* w_up, const float* w_down, int seq, int hidden, int heads,
                      int kv_heads, int head_dim, int mlp, float theta, float eps, int causal,
                      int activation, float* out) {
  const size_t qw = (size_t)heads * head_dim, kw = (size_t)kv_heads * head_dim;
  float* normed = (float*)malloc(sizeof(float) * seq * hidden);
  float* q = (float*)malloc(sizeof(float) * seq * qw);
  float* k = (float*)malloc(sizeof(float) * seq * kw);
  float* v = (float*)malloc(sizeof(float) * seq * kw);
  float* qr = (float*)malloc(sizeof(float) * seq * qw);
  float* kr = (float*)malloc(sizeof(float) * seq * kw);
  float* attn = (float*)malloc(sizeof(float) * seq * qw);
  float* proj = (float*)malloc(sizeof(float) * seq * hidden);
  float* h1 = (float*)malloc(sizeof(float) * seq * hidden);
  float* gate = (float*)malloc(sizeof(float) * (size_t)seq * mlp);
  float* up = (float*)malloc(sizeof(float) * (size_t)seq * mlp);
  if (!normed || !q || !k || !v || !qr || !kr || !attn || !proj || !h1 || !gate || !up) return -1;
  rms_norm(x, attn_norm, normed, seq, hidden, eps);
  sgemm_naive(seq, hidden, (int)qw, normed, wq, q);
  sgemm_naive(seq, hidden, (int)kw, normed, wk, k);
  sgemm_naive(seq, hidden, (int)kw, normed, wv, v);
  rope(q, qr, seq, heads, head_dim, theta, 0);
  rope(k, kr, seq, kv_heads, head_dim, theta, 0);
  sdpa_prefill(qr, kr, v, attn, seq, heads, kv_heads, head_dim, causal);
  sgemm_naive(seq, (int)qw, hidden, attn, wo, proj);
  for (size_t i = 0; i < (size_t)seq * hidden; ++i) h1[i] = x[i] + proj[i];
  rms_norm(h1, ffn_norm, normed, seq, hidden, eps);
  sgemm_naive(seq, hidden, mlp, normed, w_gate, gate);
  for (size_t i = 0; i < (size_t)seq * mlp; ++i) {
    gate[i] = activation ? gelu_tanh(gate[i]) : gate[i] / (1.0f + expf(-gate[i]));
  }
  sgemm_naive(seq, hidden, mlp, normed, w_up, up);
  for (size_t i = 0; i < (size_t)seq * mlp; ++i) gate[i] *= up[i];
  sgemm_naive(seq, mlp, hidden, gate, w_down, proj);
  for (size_t i = 0; i < (size_t)seq * hidden; ++i) out[i] = h1[i] + proj[i];
  free(normed); free(q); free(k); free(v); free(qr); free(kr); free(attn); free(proj); free(h1);
  free(gate); free(up);
  return 0;
}
