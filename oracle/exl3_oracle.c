/* CPU restatement in C of the EXL3 hot path (decode + GEMV in the device arithmetic order). TEST INFRASTRUCTURE ONLY:
 * tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / --impl reference legs may load it, nothing else.
 *
 * It restates, for speed, what oracle/exl3_codec.py and oracle/opref_port.py state in numpy (tests check the two
 * against each other), following the reference's device readers (kernels/ne_common.h:105-161,
 * kernels/trunk6/trunk6.metal:87-127) and its kernel-arithmetic recipe (tests/trunk6/check_kernels.py:47-60,93-99;
 * kernels/fn_moe.metal:304-343,370-445). PARITY UNPINNED for the bit layout, as stated in oracle/exl3_codec.py.
 *
 * Threads: a small pthread parallel-for (this image has no libgomp); ORACLE_THREADS overrides the core count.
 * Build: gcc -O3 -pthread -mf16c -mavx2 -mfma -shared -fPIC (oracle/Makefile).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>
#include <unistd.h>

/* ---- parallel for over [0, n): body(i, ctx), contiguous chunks per thread */
typedef void (*body_fn)(int i, void *ctx);
typedef struct { body_fn body; void *ctx; int lo, hi; } pf_job;
static void *pf_run(void *a) {
  pf_job *j = (pf_job *)a;
  for (int i = j->lo; i < j->hi; i++) j->body(i, j->ctx);
  return NULL;
}
int oracle_threads(void) {
  const char *e = getenv("ORACLE_THREADS");
  long n = e ? atol(e) : sysconf(_SC_NPROCESSORS_ONLN);
  return n < 1 ? 1 : (n > 256 ? 256 : (int)n);
}
static void parallel_for(int n, body_fn body, void *ctx) {
  int T = oracle_threads();
  if (T > n) T = n;
  if (T <= 1) { for (int i = 0; i < n; i++) body(i, ctx); return; }
  pthread_t th[256];
  pf_job jobs[256];
  for (int t = 0; t < T; t++) {
    jobs[t].body = body; jobs[t].ctx = ctx;
    jobs[t].lo = (int)((long)n * t / T); jobs[t].hi = (int)((long)n * (t + 1) / T);
    pthread_create(&th[t], NULL, pf_run, &jobs[t]);
  }
  for (int t = 0; t < T; t++) pthread_join(th[t], NULL);
}

static float g_lut[1 << 15];      /* the weight as the format defines it: fp16(lo + hi) */
static float g_lut_sum[1 << 15];  /* lo + hi unrounded: what a product accumulates that takes lo and hi as separate terms */
static int g_lut_ready = 0;
/* which of the two the *_emul functions multiply with: 0 = the rounded value (the reference's kernels and every CUDA
 * kernel by default), 1 = the summands (the CUDA decode kernels' opt-in product mode) */
static int g_summands = 0;
void exl3_emul_summands(int on) { g_summands = on ? 1 : 0; }

static float half_bits_to_float(uint16_t h) {
  _Float16 f;
  memcpy(&f, &h, 2);
  return (float)f;
}
static float round_to_half(float v) { return (float)(_Float16)v; }

/* value of a 15-bit codeword: r = ((cw * 0xCBAC1FED) & 0x8FFF8FFF) ^ 0x3B603B60; fp16(lo) + fp16(hi), half RN */
static void lut_init(void) {
  if (g_lut_ready) return;
  for (uint32_t cw = 0; cw < (1u << 15); cw++) {
    const uint32_t r = ((cw * 0xCBAC1FEDu) & 0x8FFF8FFFu) ^ 0x3B603B60u;
    /* the exact sum of the two halfs fits a float; one rounding to half = the half-precision add */
    g_lut_sum[cw] = half_bits_to_float((uint16_t)(r & 0xFFFF)) + half_bits_to_float((uint16_t)(r >> 16));
    g_lut[cw] = round_to_half(g_lut_sum[cw]);
  }
  g_lut_ready = 1;
}

/* 256 values of one tile in slot order; words = 8K little-endian u32, ring read MSB-first, slot t ends at bit (t+1)K */
static void decode_tile(const uint32_t *words, int K, float *v, const float *lut) {
  const int TOT = 256 * K, NW = 8 * K;
  for (int t = 0; t < 256; t++) {
    int end = (t + 1) * K;               /* exclusive */
    int start = end - 15;                /* 15 codeword bits */
    if (start < 0) start += TOT;
    uint32_t cw = 0;
    int wi = start >> 5, bo = start & 31; /* bit offset from the MSB of word wi */
    int need = 15;
    while (need > 0) {
      const int avail = 32 - bo, take = need < avail ? need : avail;
      const uint32_t chunk = (words[wi] << bo) >> (32 - take);
      cw = (cw << take) | chunk;
      need -= take;
      bo = 0;
      wi = wi + 1 == NW ? 0 : wi + 1;
    }
    v[t] = lut[cw & 0x7FFF];
  }
}

static inline int slot_row(int t) {
  const int lane = t >> 3, j = t & 7, q = lane & 3;
  const int r4[4] = {2 * q, 2 * q + 1, 2 * q + 8, 2 * q + 9};
  return r4[j & 3];
}
static inline int slot_col(int t) { return (t >> 5) + 8 * ((t & 7) >> 2); }

static int had_size(int d) { return d % 128 == 0 ? 128 : d % 64 == 0 ? 64 : d % 32 == 0 ? 32 : 16; }

/* in-place float32 FWHT over blocks of n (butterflies over index bits 0,1,2,...), then * 1/sqrt(n) */
static void fwht_f32(float *x, int len, int n) {
  const float s = (float)(1.0 / sqrt((double)n));
  for (int b0 = 0; b0 < len; b0 += n) {
    float *v = x + b0;
    for (int b = 1; b < n; b <<= 1)
      for (int i = 0; i < n; i += 2 * b)
        for (int j = i; j < i + b; j++) {
          const float lo = v[j], hi = v[j + b];
          v[j] = lo + hi;
          v[j + b] = lo - hi;
        }
    for (int i = 0; i < n; i++) v[i] *= s;
  }
}
static void fwht_f64(double *x, int len, int n) {
  const double s = 1.0 / sqrt((double)n);
  for (int b0 = 0; b0 < len; b0 += n) {
    double *v = x + b0;
    for (int b = 1; b < n; b <<= 1)
      for (int i = 0; i < n; i += 2 * b)
        for (int j = i; j < i + b; j++) {
          const double lo = v[j], hi = v[j + b];
          v[j] = lo + hi;
          v[j + b] = lo - hi;
        }
    for (int i = 0; i < n; i++) v[i] *= s;
  }
}

/* W' [in][out] float32 (exact fp16 values) */
typedef struct { const uint16_t *trellis; int IT, OT, K; float *out; } dec_ctx;
static void dec_body(int tile, void *p) {
  dec_ctx *c = (dec_ctx *)p;
  float v[256];
  decode_tile((const uint32_t *)(c->trellis + (size_t)tile * 16 * c->K), c->K, v, g_lut);
  const int tk = tile / c->OT, tn = tile % c->OT, n_out = c->OT * 16;
  for (int t = 0; t < 256; t++) c->out[(size_t)(tk * 16 + slot_row(t)) * n_out + tn * 16 + slot_col(t)] = v[t];
}
void exl3_decode_inner(const uint16_t *trellis, int IT, int OT, int K, float *out) {
  lut_init();
  dec_ctx c = {trellis, IT, OT, K, out};
  parallel_for(IT * OT, dec_body, &c);
}

/* xh[rows][in] = float(fp16(H(x * suh))) with the product and butterflies in float32 */
void exl3_prep_emul(const float *x, const uint16_t *suh, int rows, int in, float *xh) {
  const int n = had_size(in);
  for (int r = 0; r < rows; r++) {
    float *o = xh + (size_t)r * in;
    for (int i = 0; i < in; i++) o[i] = x[(size_t)r * in + i] * half_bits_to_float(suh[i]);
    fwht_f32(o, in, n);
    for (int i = 0; i < in; i++) o[i] = round_to_half(o[i]);
  }
}

/* raw[rows][out] (double) = xh[rows][in] @ W', W' decoded tile by tile, never materialised */
typedef struct { const uint16_t *trellis; int in, out, K; const float *xh; int rows; double *raw; } gemm_ctx;
static void gemm_body(int tn, void *p) {
  gemm_ctx *g = (gemm_ctx *)p;
  const uint16_t *trellis = g->trellis;
  const int in = g->in, out = g->out, K = g->K, rows = g->rows, IT = in / 16, OT = out / 16;
  const float *xh = g->xh;
  double *raw = g->raw;
  {
    double acc[64][16];
    float v[256];
    for (int r = 0; r < rows; r++)
      for (int c = 0; c < 16; c++) acc[r][c] = 0.0;
    for (int tk = 0; tk < IT; tk++) {
      decode_tile((const uint32_t *)(trellis + ((size_t)tk * OT + tn) * 16 * K), K, v, g_summands ? g_lut_sum : g_lut);
      float w[16][16];
      for (int t = 0; t < 256; t++) w[slot_row(t)][slot_col(t)] = v[t];
      for (int r = 0; r < rows; r++) {
        const float *xr = xh + (size_t)r * in + tk * 16;
        for (int k = 0; k < 16; k++) {
          const double xv = xr[k];
          for (int c = 0; c < 16; c++) acc[r][c] += xv * (double)w[k][c];
        }
      }
    }
    for (int r = 0; r < rows; r++)
      for (int c = 0; c < 16; c++) raw[(size_t)r * out + tn * 16 + c] = acc[r][c];
  }
}
void exl3_raw_gemm(const uint16_t *trellis, int in, int out, int K, const float *xh, int rows, double *raw) {
  lut_init();
  gemm_ctx g = {trellis, in, out, K, xh, rows, raw};
  parallel_for(out / 16, gemm_body, &g);
}

/* y[rows][out] = (H_out raw) * svh, double in, float out */
void exl3_finish(const double *raw, const uint16_t *svh, int rows, int out, float *y) {
  const int n = had_size(out);
  double *tmp = (double *)malloc(sizeof(double) * (size_t)out);
  for (int r = 0; r < rows; r++) {
    memcpy(tmp, raw + (size_t)r * out, sizeof(double) * (size_t)out);
    fwht_f64(tmp, out, n);
    for (int c = 0; c < out; c++) y[(size_t)r * out + c] = (float)(tmp[c] * (double)half_bits_to_float(svh[c]));
  }
  free(tmp);
}

/* the whole Linear in the device arithmetic (y_emul of the reference's kernel check); rows <= 64 */
void exl3_linear_emul(const uint16_t *trellis, const uint16_t *suh, const uint16_t *svh, int in, int out, int K,
                      const float *x, int rows, float *y) {
  float *xh = (float *)malloc(sizeof(float) * (size_t)rows * in);
  double *raw = (double *)malloc(sizeof(double) * (size_t)rows * out);
  exl3_prep_emul(x, suh, rows, in, xh);
  exl3_raw_gemm(trellis, in, out, K, xh, rows, raw);
  exl3_finish(raw, svh, rows, out, y);
  free(xh);
  free(raw);
}

/* logits[rows][E] = x @ W^T with W bf16 [E][H], double accumulation rounded to float */
typedef struct { const uint16_t *w_bf16; int E, H; const float *x; int rows; float *logits; } rt_ctx;
static void rt_body(int e, void *p) {
  rt_ctx *c = (rt_ctx *)p;
  const uint16_t *w_bf16 = c->w_bf16;
  const int E = c->E, H = c->H, rows = c->rows;
  const float *x = c->x;
  float *logits = c->logits;
    for (int r = 0; r < rows; r++) {
      double a = 0.0;
      for (int i = 0; i < H; i++) {
        const uint32_t u = (uint32_t)w_bf16[(size_t)e * H + i] << 16;
        float f;
        memcpy(&f, &u, 4);
        a += (double)x[(size_t)r * H + i] * (double)f;
      }
      logits[(size_t)r * E + e] = (float)a;
    }
}
void router_logits(const uint16_t *w_bf16, int E, int H, const float *x, int rows, float *logits) {
  rt_ctx c = {w_bf16, E, H, x, rows, logits};
  parallel_for(E, rt_body, &c);
}

/* One routed expert applied to one row in the device arithmetic: out[H] (double) += w * down(silu(gate x) * up x).
 * Also returns the raw gate / up inner products (gu[2][I]) when gu != NULL. */
void moe_expert_emul(const uint16_t *gt, const uint16_t *gsu, const uint16_t *gsv, const uint16_t *ut,
                     const uint16_t *usu, const uint16_t *usv, const uint16_t *dt, const uint16_t *dsu,
                     const uint16_t *dsv, int H, int I, int K, const float *x, double weight, double *out, float *gu) {
  float *xh = (float *)malloc(sizeof(float) * (size_t)(H > I ? H : I));
  double *rg = (double *)malloc(sizeof(double) * (size_t)I), *ru = (double *)malloc(sizeof(double) * (size_t)I);
  double *rd = (double *)malloc(sizeof(double) * (size_t)H);
  float *mid = (float *)malloc(sizeof(float) * (size_t)I);
  exl3_prep_emul(x, gsu, 1, H, xh);
  exl3_raw_gemm(gt, H, I, K, xh, 1, rg);
  exl3_prep_emul(x, usu, 1, H, xh);
  exl3_raw_gemm(ut, H, I, K, xh, 1, ru);
  if (gu)
    for (int i = 0; i < I; i++) { gu[i] = (float)rg[i]; gu[I + i] = (float)ru[i]; }
  fwht_f64(rg, I, 128);
  fwht_f64(ru, I, 128);
  for (int i = 0; i < I; i++) {
    const float g = (float)(rg[i] * (double)half_bits_to_float(gsv[i]));
    const float u = (float)(ru[i] * (double)half_bits_to_float(usv[i]));
    mid[i] = g / (1.0f + expf(-g)) * u;
  }
  exl3_prep_emul(mid, dsu, 1, I, xh);
  exl3_raw_gemm(dt, I, H, K, xh, 1, rd);
  fwht_f64(rd, H, 128);
  for (int c = 0; c < H; c++) out[c] += weight * rd[c] * (double)half_bits_to_float(dsv[c]);
  free(xh); free(rg); free(ru); free(rd); free(mid);
}
