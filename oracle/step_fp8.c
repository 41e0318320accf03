/* CPU restatement (C, OpenMP) of the fp8 block-scaled pieces of the decode step: activation quantiser, the
 * block-scaled GEMM with per-128-k promotion, the fp8 MoE block (routed + shared experts, combine).
 *
 * TEST / BASELINE INFRASTRUCTURE ONLY: the fast twin of oracle/numerics.py (quant_fp8_groups, e4m3 codec) and
 * oracle/moe.py (gemm_fp8_blocks, mlp_fp8, moe_fp8, combine), timed by bench.py as the CPU baseline of the
 * decode step.  Nothing in the shipped package links or calls it.
 * Reference lines followed: activation scale rule fp8.py:21-34; promotion order qk_lt.cu:361-364 and
 * qk_moe_prefill_i8.cu:3649-3651; SwiGLU rounding points i8x_decode.py:151-156; weighted bf16 cache rows
 * i8x_decode.py:420-422; combine i8x_decode.py:425-443; e4m3 conversion qk_attn_verify.cu:142-146.
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

static float g_e4m3[256];
static int g_e4m3_ready = 0;
static void e4m3_init(void) {
  if (g_e4m3_ready) return;
  for (int b = 0; b < 256; ++b) {
    const float s = (b & 0x80) ? -1.f : 1.f;
    const int e = (b >> 3) & 0xF, m = b & 7;
    float v;
    if (e == 0xF && m == 7)
      v = NAN;
    else if (e == 0)
      v = s * (float)m * ldexpf(1.f, -9);
    else
      v = s * (1.f + (float)m / 8.f) * ldexpf(1.f, e - 7);
    g_e4m3[b] = v;
  }
  g_e4m3_ready = 1;
}

/* fp32 -> e4m3 byte: round to nearest even, saturate to +-448, NaN -> 0x7f */
static inline uint8_t e4m3_encode(float x) {
  if (isnan(x)) return 0x7f;
  const uint8_t sign = signbit(x) ? 0x80 : 0;
  double a = fabs((double)x);
  if (a > 448.0) a = 448.0;
  if (a == 0.0) return sign;
  int e = (int)floor(log2(a));
  if (e < -6) e = -6;
  const double q = ldexp(1.0, e - 3);
  double r = rint(a / q) * q; /* default rounding mode: ties to even */
  if (r > 448.0) r = 448.0;
  if (r == 0.0) return sign;
  int e2 = (int)floor(log2(r));
  if (e2 < -6) { /* subnormal: r = m * 2^-9 */
    return sign | (uint8_t)(int)(r * 512.0);
  }
  const int m = (int)((r / ldexp(1.0, e2) - 1.0) * 8.0);
  return sign | (uint8_t)(((e2 + 7) << 3) | m);
}

void oracle_e4m3_encode(const float* x, size_t n, uint8_t* out) {
  for (size_t i = 0; i < n; ++i) out[i] = e4m3_encode(x[i]);
}

/* one row of n values -> e4m3 codes + one fp32 scale per 128 values: scale = max(amax / 448, 1e-12),
 * y = e4m3(x * (1 / scale)) */
static void quant_groups(const float* x, int n, uint8_t* q, float* scale) {
  for (int g = 0; g < n / 128; ++g) {
    float amax = 0.f;
    for (int i = 0; i < 128; ++i) amax = fmaxf(amax, fabsf(x[g * 128 + i]));
    float s = amax / 448.f;
    if (s < 1e-12f) s = 1e-12f;
    const float inv = 1.f / s;
    for (int i = 0; i < 128; ++i) q[g * 128 + i] = e4m3_encode(x[g * 128 + i] * inv);
    scale[g] = s;
  }
}

void oracle_quant_fp8_groups(const float* x, int rows, int n, uint8_t* q, float* scale) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) quant_groups(x + (size_t)r * n, n, q + (size_t)r * n, scale + (size_t)r * (n / 128));
}

/* out[m] for one weight row: acc = 0; per 128-k block g (ascending): partial = sum of the block's products
 * (exact products, summed in double, rounded once to fp32), acc = fma(partial, a_s[g] * w_s[g], acc) */
static inline float row_dot(const float* a, const float* a_s, const float* w, const float* w_s, int K) {
  float acc = 0.f;
  for (int g = 0; g < K / 128; ++g) {
    double s = 0.0;
    const float* ap = a + g * 128;
    const float* wp = w + g * 128;
    for (int k = 0; k < 128; ++k) s += (double)(ap[k] * wp[k]);
    acc = fmaf((float)s, a_s[g] * w_s[g], acc);
  }
  return acc;
}

/* out[M, N] = block-scaled GEMM of aq [M, K] (codes, scales a_s [M, K/128]) with wq [N, K] (scales w_s
 * [ceil(N/128), K/128]) */
void oracle_gemm_fp8_blocks(const uint8_t* aq, const float* a_s, int M, int K, const uint8_t* wq, const float* w_s, int N,
                            float* out) {
  e4m3_init();
  float* a = (float*)malloc(sizeof(float) * (size_t)M * K);
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m)
    for (int k = 0; k < K; ++k) a[(size_t)m * K + k] = g_e4m3[aq[(size_t)m * K + k]];
  const int KG = K / 128;
#pragma omp parallel
  {
    float* w = (float*)malloc(sizeof(float) * K);
#pragma omp for schedule(static)
    for (int n = 0; n < N; ++n) {
      for (int k = 0; k < K; ++k) w[k] = g_e4m3[wq[(size_t)n * K + k]];
      const float* ws = w_s + (size_t)(n / 128) * KG;
      for (int m = 0; m < M; ++m) out[(size_t)m * N + n] = row_dot(a + (size_t)m * K, a_s + (size_t)m * KG, w, ws, K);
    }
    free(w);
  }
  free(a);
}

/* MLP of `n` rows (n <= 16) through one expert: xdec [n][H] decoded activations, xs [n][H/128]; writes
 * cache rows (bf16 bits) at slots[], multiplied by wt[] */
static void mlp_rows(int n, const float* const* xdec, const float* const* xs, const uint8_t* w13, const float* s13,
                     const uint8_t* w2, const float* s2, int H, int I, const float* wt, uint16_t* const* cache_rows,
                     float* wrow, float* gu, float* h, uint8_t* hq, float* hdec, float* hs) {
  const int KG = H / 128, IG = I / 128;
  for (int j = 0; j < 2 * I; ++j) {
    for (int k = 0; k < H; ++k) wrow[k] = g_e4m3[w13[(size_t)j * H + k]];
    const float* ws = s13 + (size_t)(j / 128) * KG;
    for (int r = 0; r < n; ++r) gu[(size_t)r * 2 * I + j] = row_dot(xdec[r], xs[r], wrow, ws, H);
  }
  for (int r = 0; r < n; ++r) {
    for (int j = 0; j < I; ++j) {
      const float g = rbf(gu[(size_t)r * 2 * I + j]), u = rbf(gu[(size_t)r * 2 * I + I + j]);
      h[(size_t)r * I + j] = rbf(g / (1.f + expf(-g)) * u);
    }
    quant_groups(h + (size_t)r * I, I, hq + (size_t)r * I, hs + (size_t)r * IG);
    for (int j = 0; j < I; ++j) hdec[(size_t)r * I + j] = g_e4m3[hq[(size_t)r * I + j]];
  }
  for (int c = 0; c < H; ++c) {
    for (int k = 0; k < I; ++k) wrow[k] = g_e4m3[w2[(size_t)c * I + k]];
    const float* ws = s2 + (size_t)(c / 128) * IG;
    for (int r = 0; r < n; ++r) {
      const float y = row_dot(hdec + (size_t)r * I, hs + (size_t)r * IG, wrow, ws, I);
      cache_rows[r][c] = f2bf(y * wt[r]);
    }
  }
}

/* whole block: x bf16 bits [T,H]; ids/wts [T,K]; w13 e4m3 [E,2I,H], s13 [E,2I/128,H/128]; w2 [E,H,I],
 * s2 [E,H/128,I/128]; shared likewise; out bf16 bits [T,H]; cache bf16 bits [T*(K+1),H] scratch */
void oracle_moe_fp8(const uint16_t* x, const int32_t* ids, const float* wts, int T, int H, int I, int K, int E,
                    const uint8_t* w13, const float* s13, const uint8_t* w2, const float* s2, const uint8_t* sh13,
                    const float* shs13, const uint8_t* sh2, const float* shs2, const uint16_t* gate_w, uint16_t* cache,
                    uint16_t* out) {
  e4m3_init();
  const int KG = H / 128, IG = I / 128, CH = 8;
  float* xdec = (float*)malloc(sizeof(float) * (size_t)T * H);
  float* xs = (float*)malloc(sizeof(float) * (size_t)T * KG);
#pragma omp parallel
  {
    float* row = (float*)malloc(sizeof(float) * H);
    uint8_t* q = (uint8_t*)malloc(H);
#pragma omp for schedule(static)
    for (int t = 0; t < T; ++t) {
      for (int k = 0; k < H; ++k) row[k] = bf2f(x[(size_t)t * H + k]);
      quant_groups(row, H, q, xs + (size_t)t * KG);
      for (int k = 0; k < H; ++k) xdec[(size_t)t * H + k] = g_e4m3[q[k]];
    }
    free(row);
    free(q);
  }
  /* rows grouped by expert (counting sort over slots, ascending slot order inside an expert); the shared
   * expert is expert E with one row per token */
  const int P = T * K;
  int* start = (int*)calloc((size_t)E + 2, sizeof(int));
  for (int p = 0; p < P; ++p) start[ids[p] + 1]++;
  start[E + 1] = T;
  for (int e = 0; e <= E; ++e) start[e + 1] += start[e];
  int* slot_of = (int*)malloc(sizeof(int) * (size_t)(P + T));
  int* fill = (int*)malloc(sizeof(int) * (size_t)(E + 1));
  memcpy(fill, start, sizeof(int) * (size_t)(E + 1));
  for (int p = 0; p < P; ++p) slot_of[fill[ids[p]]++] = p;
  for (int t = 0; t < T; ++t) slot_of[start[E] + t] = P + t;
  /* tasks: (expert, chunk of up to CH rows) */
  int ntask = 0;
  for (int e = 0; e <= E; ++e) ntask += (start[e + 1] - start[e] + CH - 1) / CH;
  int* task_e = (int*)malloc(sizeof(int) * (size_t)(ntask > 0 ? ntask : 1));
  int* task_r0 = (int*)malloc(sizeof(int) * (size_t)(ntask > 0 ? ntask : 1));
  ntask = 0;
  for (int e = 0; e <= E; ++e)
    for (int r0 = start[e]; r0 < start[e + 1]; r0 += CH) {
      task_e[ntask] = e;
      task_r0[ntask++] = r0;
    }
#pragma omp parallel
  {
    float* wrow = (float*)malloc(sizeof(float) * (size_t)(H > I ? H : I));
    float* gu = (float*)malloc(sizeof(float) * (size_t)CH * 2 * I);
    float* h = (float*)malloc(sizeof(float) * (size_t)CH * I);
    float* hdec = (float*)malloc(sizeof(float) * (size_t)CH * I);
    float* hs = (float*)malloc(sizeof(float) * (size_t)CH * IG);
    uint8_t* hq = (uint8_t*)malloc((size_t)CH * I);
#pragma omp for schedule(dynamic, 1)
    for (int ti = 0; ti < ntask; ++ti) {
      const int e = task_e[ti], r0 = task_r0[ti];
      const int n = start[e + 1] - r0 < CH ? start[e + 1] - r0 : CH;
      const float* xd[8];
      const float* xsc[8];
      float wt[8];
      uint16_t* rows[8];
      for (int r = 0; r < n; ++r) {
        const int slot = slot_of[r0 + r];
        const int t = slot < P ? slot / K : slot - P;
        xd[r] = xdec + (size_t)t * H;
        xsc[r] = xs + (size_t)t * KG;
        wt[r] = slot < P ? wts[slot] : 1.f;
        rows[r] = cache + (size_t)slot * H;
      }
      if (e < E)
        mlp_rows(n, xd, xsc, w13 + (size_t)e * 2 * I * H, s13 + (size_t)e * (2 * I / 128) * KG, w2 + (size_t)e * H * I,
                 s2 + (size_t)e * KG * IG, H, I, wt, rows, wrow, gu, h, hq, hdec, hs);
      else
        mlp_rows(n, xd, xsc, sh13, shs13, sh2, shs2, H, I, wt, rows, wrow, gu, h, hq, hdec, hs);
    }
    free(wrow);
    free(gu);
    free(h);
    free(hdec);
    free(hs);
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
      acc += gate * bf2f(cache[((size_t)P + t) * H + c]);
      out[(size_t)t * H + c] = f2bf(acc);
    }
  }
  free(xdec);
  free(xs);
  free(start);
  free(slot_of);
  free(fill);
  free(task_e);
  free(task_r0);
}
