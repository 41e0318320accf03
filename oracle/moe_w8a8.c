/* CPU restatement (C, OpenMP) of the int8 W8A8 MoE block: router, routing, expert MLPs, combine.
 *
 * TEST / BASELINE INFRASTRUCTURE ONLY: it is the checker's fast twin of oracle/router.py and
 * oracle/moe.py (same arithmetic, same rounding points, same summation tree for the router) and
 * the CPU baseline timed by bench.py.  Nothing in the shipped package links or calls it.
 * Reference lines followed: router i8x_decode.py:99-117 and qk_route.cu:3-4,71-75,125-133;
 * W8A8 epilogue qwen36_lmhead8/w8a8.py:15-36,64-70; SwiGLU i8x_decode.py:151-156; weighted bf16
 * cache rows i8x_decode.py:420-422; combine i8x_decode.py:425-443.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline float bf2f(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint16_t f2bf(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fc0;
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
static inline float rbf(float f) { return bf2f(f2bf(f)); }

/* n > 0: use n threads from now on (a launcher may have exported OMP_NUM_THREADS=1 for its ranks) */
void oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int oracle_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* logits with the fixed tree: one fma chain from 0 per 128-deep slice (ascending k), slices added
 * in order, bias last */
void oracle_gate_logits(const uint16_t* x, const float* wr, const float* bias, int T, int H, int E, float* logits) {
  const int ns = H / 128;
#pragma omp parallel for collapse(2) schedule(static)
  for (int t = 0; t < T; ++t)
    for (int e = 0; e < E; ++e) {
      const uint16_t* xr = x + (size_t)t * H;
      const float* w = wr + (size_t)e * H;
      float tot = 0.f;
      for (int s = 0; s < ns; ++s) {
        float acc = 0.f;
        for (int k = s * 128; k < s * 128 + 128; ++k) acc = fmaf(bf2f(xr[k]), w[k], acc);
        tot = s == 0 ? acc : tot + acc;
      }
      if (bias) tot += bias[e];
      logits[(size_t)t * E + e] = tot;
    }
}

void oracle_topk(const float* logits, int T, int E, int K, int round_bf16, int32_t* ids, float* wts) {
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; ++t) {
    float* key = (float*)malloc(sizeof(float) * E);
    float* pr = (float*)malloc(sizeof(float) * E);
    float mx = -INFINITY;
    for (int e = 0; e < E; ++e) {
      float v = logits[(size_t)t * E + e];
      if (round_bf16) v = rbf(v);
      key[e] = isnan(v) ? -INFINITY : v + 0.f;
      if (key[e] > mx) mx = key[e];
    }
    float sum = 0.f;
    for (int e = 0; e < E; ++e) {
      pr[e] = isnan(logits[(size_t)t * E + e]) ? 0.f : expf(key[e] - mx);
      sum += pr[e];
    }
    float tot = 0.f;
    for (int k = 0; k < K; ++k) {
      int best = -1;
      for (int e = 0; e < E; ++e)
        if (!isnan(key[e]) && (best < 0 || key[e] > key[best])) best = e; /* first max = lowest id */
      ids[t * K + k] = best;
      wts[t * K + k] = pr[best] / sum;
      tot += wts[t * K + k];
      key[best] = NAN;
    }
    const float den = tot > 0.f ? tot : 1.f;
    for (int k = 0; k < K; ++k) wts[t * K + k] /= den;
    free(key);
    free(pr);
  }
}

static void quant_row(const float* x, int n, int8_t* q, float* scale) {
  float amax = 0.f;
  for (int i = 0; i < n; ++i) amax = fmaxf(amax, fabsf(x[i]));
  const float s = amax / 127.f, safe = amax > 0.f ? s : 1.f;
  for (int i = 0; i < n; ++i) {
    const float v = x[i] / safe;
    float r = v >= 0.f ? floorf(v + 0.5f) : -floorf(0.5f - v);
    r = fminf(fmaxf(r, -127.f), 127.f);
    q[i] = (int8_t)r;
  }
  *scale = s;
}

static inline int32_t dot_i8(const int8_t* a, const int8_t* b, int n) {
  int32_t s = 0;
  for (int i = 0; i < n; ++i) s += (int32_t)a[i] * (int32_t)b[i];
  return s;
}

/* one (row, expert) MLP: xq [H] -> cache row [H] (bf16 bits), multiplied by wt */
static void mlp_row(const int8_t* xq, float xs, const int8_t* w13, const float* s13, const int8_t* w2,
                    const float* s2, int H, int I, float wt, uint16_t* cache_row, float* hbuf, int8_t* hq) {
  for (int j = 0; j < I; ++j) {
    const float g = rbf(((float)dot_i8(xq, w13 + (size_t)j * H, H) * xs) * s13[j]);
    const float u = rbf(((float)dot_i8(xq, w13 + (size_t)(I + j) * H, H) * xs) * s13[I + j]);
    hbuf[j] = rbf(g / (1.f + expf(-g)) * u);
  }
  float hs;
  quant_row(hbuf, I, hq, &hs);
  for (int c = 0; c < H; ++c) {
    const float y = ((float)dot_i8(hq, w2 + (size_t)c * I, I) * hs) * s2[c];
    cache_row[c] = f2bf(y * wt);
  }
}

/* whole block: x bf16 bits [T,H]; ids/wts [T,K]; out bf16 bits [T,H]; cache bf16 bits [T*(K+1),H] scratch */
void oracle_moe_w8a8(const uint16_t* x, const int32_t* ids, const float* wts, int T, int H, int I, int K,
                     const int8_t* w13, const float* s13, const int8_t* w2, const float* s2, const int8_t* sh13,
                     const float* shs13, const int8_t* sh2, const float* shs2, const uint16_t* gate_w,
                     uint16_t* cache, uint16_t* out) {
  int8_t* xq = (int8_t*)malloc((size_t)T * H);
  float* xs = (float*)malloc(sizeof(float) * T);
#pragma omp parallel
  {
    float* row = (float*)malloc(sizeof(float) * H);
#pragma omp for schedule(static)
    for (int t = 0; t < T; ++t) {
      for (int k = 0; k < H; ++k) row[k] = bf2f(x[(size_t)t * H + k]);
      quant_row(row, H, xq + (size_t)t * H, &xs[t]);
    }
    free(row);
  }
  const int P = T * (K + 1);
#pragma omp parallel
  {
    float* hbuf = (float*)malloc(sizeof(float) * I);
    int8_t* hq = (int8_t*)malloc(I);
#pragma omp for schedule(dynamic, 4)
    for (int p = 0; p < P; ++p) {
      if (p < T * K) {
        const int t = p / K, e = ids[p];
        mlp_row(xq + (size_t)t * H, xs[t], w13 + (size_t)e * 2 * I * H, s13 + (size_t)e * 2 * I,
                w2 + (size_t)e * H * I, s2 + (size_t)e * H, H, I, wts[p], cache + (size_t)p * H, hbuf, hq);
      } else {
        const int t = p - T * K;
        mlp_row(xq + (size_t)t * H, xs[t], sh13, shs13, sh2, shs2, H, I, 1.f, cache + (size_t)p * H, hbuf, hq);
      }
    }
    free(hbuf);
    free(hq);
  }
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; ++t) {
    double dot = 0.0;
    for (int k = 0; k < H; ++k) dot += (double)bf2f(x[(size_t)t * H + k]) * (double)bf2f(gate_w[k]);
    const float gate = 1.f / (1.f + expf(-(float)dot));
    for (int c = 0; c < H; ++c) {
      float acc = 0.f;
      for (int j = 0; j < K; ++j) acc += bf2f(cache[((size_t)t * K + j) * H + c]);
      acc += gate * bf2f(cache[((size_t)T * K + t) * H + c]);
      out[(size_t)t * H + c] = f2bf(acc);
    }
  }
  free(xq);
  free(xs);
}
