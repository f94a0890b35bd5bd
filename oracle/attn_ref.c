/*
 * Scalar C restatement of GPT-OSS attention forward + backward.
 *
 * TEST INFRASTRUCTURE ONLY: an independent checker for the CUDA library, never
 * linked into it.  Plain loops, double accumulation, no blocking and no
 * vector tricks, so that it shares no code (and no rounding pattern) with
 * either the torch restatement beside it or the kernels it checks.
 *
 * Function restated: transformers models/gpt_oss/modeling_gpt_oss.py:245-273
 * (eager_attention_forward: logits = q.k*scale + mask, a per-head sink logit
 * appended as one extra softmax column that carries no value, softmax, P.V)
 * with the visibility rule of masking_utils.py:78 (kv <= q) and :96-97
 * (kv > q - window), and its analytic gradient in the form the reference's
 * flash kernel evaluates it (attention_kernel.py:111-120 delta, :173-176
 * dSinks, :190-214 dV, dP, dS, dK, dQ).
 *
 * Layouts (all contiguous, float):  q,dq (B,Hq,S,d); k,v,dk,dv (B,Hkv,S,d);
 * o,do (B,S,Hq,d); lse (B,Hq,S); sinks,dsinks (Hq).  seqlens may be NULL.
 * Rows i >= seqlens[b] are padding: o = 0, lse = 0, no gradient contribution.
 *
 * Build: gcc -O2 -shared -fPIC -o liboracle_attn.so attn_ref.c -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static int visible(int i, int j, int window, int len) {
  if (j > i) return 0;                       /* masking_utils.py:78  */
  if (window > 0 && j <= i - window) return 0; /* masking_utils.py:96-97 */
  if (i >= len || j >= len) return 0;        /* right padding */
  return 1;
}

int oracle_attn_fwd_bwd(const float* q, const float* k, const float* v, const float* sinks,
                        const float* d_o, const int32_t* seqlens, int B, int Hq, int Hkv, int S,
                        int d, float scale, int window, float* o, float* lse, float* dq,
                        float* dk, float* dv, float* dsinks) {
  if (Hq % Hkv != 0 || d <= 0 || S <= 0) return -1;
  const int G = Hq / Hkv;
  double* p = (double*)malloc(sizeof(double) * (size_t)S);
  double* acc = (double*)malloc(sizeof(double) * (size_t)d);
  double* dkacc = (double*)calloc((size_t)B * Hkv * S * d, sizeof(double));
  double* dvacc = (double*)calloc((size_t)B * Hkv * S * d, sizeof(double));
  double* dsacc = (double*)calloc((size_t)Hq, sizeof(double));
  if (!p || !acc || !dkacc || !dvacc || !dsacc) return -2;
  memset(o, 0, sizeof(float) * (size_t)B * S * Hq * d);
  memset(lse, 0, sizeof(float) * (size_t)B * Hq * S);
  memset(dq, 0, sizeof(float) * (size_t)B * Hq * S * d);

  for (int b = 0; b < B; ++b) {
    const int len = seqlens ? seqlens[b] : S;
    for (int h = 0; h < Hq; ++h) {
      const int g = h / G;
      const float* kb = k + ((size_t)b * Hkv + g) * S * d;
      const float* vb = v + ((size_t)b * Hkv + g) * S * d;
      double* dkb = dkacc + ((size_t)b * Hkv + g) * S * d;
      double* dvb = dvacc + ((size_t)b * Hkv + g) * S * d;
      const double sink = sinks[h];
      for (int i = 0; i < len; ++i) {
        const float* qi = q + (((size_t)b * Hq + h) * S + i) * d;
        const float* doi = d_o + (((size_t)b * S + i) * Hq + h) * d;
        float* oi = o + (((size_t)b * S + i) * Hq + h) * d;
        float* dqi = dq + (((size_t)b * Hq + h) * S + i) * d;
        const int j0 = window > 0 ? (i - window + 1 > 0 ? i - window + 1 : 0) : 0;
        /* logits, running max including the sink */
        double m = sink;
        for (int j = j0; j <= i; ++j) {
          if (!visible(i, j, window, len)) { p[j] = -INFINITY; continue; }
          double s = 0;
          for (int c = 0; c < d; ++c) s += (double)qi[c] * kb[(size_t)j * d + c];
          p[j] = s * scale;
          if (p[j] > m) m = p[j];
        }
        double z = exp(sink - m);
        for (int j = j0; j <= i; ++j) { p[j] = exp(p[j] - m); z += p[j]; }
        for (int c = 0; c < d; ++c) acc[c] = 0;
        for (int j = j0; j <= i; ++j) {
          p[j] /= z;
          for (int c = 0; c < d; ++c) acc[c] += p[j] * vb[(size_t)j * d + c];
        }
        double delta = 0;
        for (int c = 0; c < d; ++c) { oi[c] = (float)acc[c]; delta += acc[c] * doi[c]; }
        const double l = m + log(z);
        lse[((size_t)b * Hq + h) * S + i] = (float)l;
        dsacc[h] += -exp(sink - l) * delta;
        for (int c = 0; c < d; ++c) acc[c] = 0; /* now dq row */
        for (int j = j0; j <= i; ++j) {
          if (p[j] == 0) continue;
          double dp = 0;
          for (int c = 0; c < d; ++c) dp += (double)doi[c] * vb[(size_t)j * d + c];
          const double ds = p[j] * (dp - delta);
          for (int c = 0; c < d; ++c) {
            dvb[(size_t)j * d + c] += p[j] * doi[c];
            dkb[(size_t)j * d + c] += ds * qi[c] * scale;
            acc[c] += ds * kb[(size_t)j * d + c] * scale;
          }
        }
        for (int c = 0; c < d; ++c) dqi[c] = (float)acc[c];
      }
    }
  }
  for (size_t t = 0; t < (size_t)B * Hkv * S * d; ++t) { dk[t] = (float)dkacc[t]; dv[t] = (float)dvacc[t]; }
  for (int h = 0; h < Hq; ++h) dsinks[h] = (float)dsacc[h];
  free(p); free(acc); free(dkacc); free(dvacc); free(dsacc);
  return 0;
}
