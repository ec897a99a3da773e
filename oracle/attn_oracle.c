/*
 * CPU oracle for the gated GQA full-attention mixer.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker, never the product: only the test-suite, the smoke
 * entry and the benchmark's cpu-baseline leg may load it.  The product path is
 * the CUDA library and has no CPU fallback.
 *
 * It restates, in plain C with double accumulation, the arithmetic of the
 * reference engine's full-attention layer (paths are relative to the reference
 * project root):
 *   - partial RoPE, half-split pairs (i, i+rot/2), angle = pos * theta^(-2i/rot),
 *     optional 3-component mrope positions ........ src/elem.cu:112-137
 *   - KV-cache append at slot pos+b ................ src/mixers.cu:416-425
 *   - decode / verify attention, row b sees keys [0, pos+b], GQA map
 *     kv = h / (q_heads/kv_heads), max-subtracted softmax  src/mixers.cu:436-525
 *   - prefill attention, same maths with a per-query causal limit
 *     t <= pos+q0+i ................................ src/mixers.cu:546-649
 *   - sigmoid output gate .......................... src/mixers.cu:653-657
 *   - operation order rope(q), rope(k), append, attend, gate
 *     ............................ src/model.cu:228-240, src/prefill.cu:142-156
 *   - the steps that feed the path from the fused q/k/v projection row (oracle_fused_rows):
 *     scatter of [q|gate x heads, k, v] .............. src/elem.cu:226-237
 *     per-head de-interleave of query and gate ....... src/mixers.cu:382-390
 *     per-head RMSNorm with (1 + weight) on q and k .. src/mixers.cu:393-413
 *     in the order of ................................ src/model.cu:219-226
 *
 * Differences from the reference, all deliberate:
 *   - libm pow/sincos/exp in double instead of the __powf/__sincosf/__expf fast
 *     intrinsics, so the oracle is the exact value the reference approximates;
 *   - the per-row log-sum-exp (m + ln sum exp) is also returned;
 *   - the cache element type is selectable: fp32 (what the reference stores) or
 *     bf16 with round-to-nearest-even on store (what the B200 path stores), so
 *     both sides of a parity test read identical cached values;
 *   - many independent sequences per call (the reference serves one).
 *
 * Pinning: the reference ships no golden vector and no unit test for this path.
 * The oracle is pinned (a) against fixtures produced by running the reference's
 * own CUDA kernels, rebuilt for sm_100a, on seeded inputs, and (b) against the
 * Hugging Face Qwen3.5 attention functions the reference cites as its source.
 * Both fixture sets and their generator scripts live in tests/golden/.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>
#include <unistd.h>

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* Round-to-nearest-even fp32 -> bf16 (NaN kept quiet). */
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

/* Which of the three mrope positions (t, h, w) frequency slot `slot` uses.
 * Sections [11, 11, 10] interleaved T,H,W,T,H,W,...  (src/elem.cu:112-117) */
static inline int mrope_component(int slot) {
  const int m = slot % 3;
  if (m == 1 && slot <= 31) return 1;
  if (m == 2 && slot <= 29) return 2;
  return 0;
}

/* Rotate one head vector in place (fp32 values, double arithmetic).
 * pos3 holds the (t, h, w) positions; text rows pass the same value three times. */
static void rope_head(float *x, int rot, double theta, const int *pos3) {
  const int half = rot / 2;
  for (int i = 0; i < half; ++i) {
    const int comp = mrope_component(i);
    const double freq = pow(theta, -2.0 * (double)i / (double)rot);
    const double a = (double)pos3[comp] * freq;
    const double c = cos(a), s = sin(a);
    const double u = x[i], v = x[i + half];
    x[i] = (float)(u * c - v * s);
    x[i + half] = (float)(u * s + v * c);
  }
}

/* ---- a small pthread parallel-for (dynamic, one index at a time) ---------------- */
static int g_threads = 0; /* 0: one per online core */

void oracle_set_threads(int n) { g_threads = n; }

int oracle_num_threads(void) {
  if (g_threads > 0) return g_threads;
  const char *e = getenv("ORACLE_THREADS");
  if (e && atoi(e) > 0) return atoi(e);
  long n = sysconf(_SC_NPROCESSORS_ONLN);
  return n > 0 ? (int)n : 1;
}

typedef struct {
  void (*fn)(int64_t, void *);
  void *ctx;
  int64_t n;
  int64_t next; /* claimed with an atomic add */
} pf_job;

static void *pf_worker(void *p) {
  pf_job *j = (pf_job *)p;
  for (;;) {
    const int64_t i = __atomic_fetch_add(&j->next, 1, __ATOMIC_RELAXED);
    if (i >= j->n) break;
    j->fn(i, j->ctx);
  }
  return NULL;
}

static void parallel_for(int64_t n, void (*fn)(int64_t, void *), void *ctx) {
  pf_job job = {fn, ctx, n, 0};
  int nt = oracle_num_threads();
  if (nt > n) nt = (int)n;
  if (nt <= 1) { pf_worker(&job); return; }
  pthread_t *th = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)nt);
  int started = 0;
  for (int t = 0; t < nt - 1; ++t)
    if (pthread_create(&th[started], NULL, pf_worker, &job) == 0) ++started;
  pf_worker(&job);
  for (int t = 0; t < started; ++t) pthread_join(th[t], NULL);
  free(th);
}

/* In-place partial RoPE on v[B][heads][dim] (fp32), the rope() launcher of
 * src/elem.cu:255-259.  pos0 is the scalar position of row 0 (*dpos); mpos is
 * NULL or [B][3]. */
void oracle_rope_f32(float *v, int B, int heads, int dim, int rot, int pos0,
                     double theta, const int *mpos) {
  for (int b = 0; b < B; ++b) {
    int p3[3] = {pos0 + b, pos0 + b, pos0 + b};
    if (mpos) { p3[0] = mpos[3 * b]; p3[1] = mpos[3 * b + 1]; p3[2] = mpos[3 * b + 2]; }
    for (int h = 0; h < heads; ++h) rope_head(v + ((size_t)b * heads + h) * dim, rot, theta, p3);
  }
}

typedef struct {
  int n_seq;          /* sequences in the batch                                  */
  int n_new;          /* new rows (tokens) per sequence                          */
  int q_heads, kv_heads, head_dim, rotary_dim;
  double theta;       /* RoPE base                                               */
  double scale;       /* softmax scale                                           */
  int cache_is_bf16;  /* 1: cache holds bf16 (uint16_t), 0: cache holds fp32     */
  int do_rope, do_append, do_gate;
} oracle_geom;

typedef struct {
  const oracle_geom *g;
  const float *q, *k_new, *v_new, *gate;
  void *kc, *vc;
  const int *pos;
  const int64_t *cache_row;
  const int *mpos;
  const int64_t *rows;
  float *out, *lse;
  int fail;
} mixer_ctx;

/* Steps 1-3 for flat row r = s*n_new+b: rope(k), then append K and V at slot pos+b. */
static void append_row(int64_t r, void *p) {
  mixer_ctx *c = (mixer_ctx *)p;
  const oracle_geom *g = c->g;
  const int D = g->head_dim, Hkv = g->kv_heads;
  const size_t kvdim = (size_t)Hkv * D;
  const int s = (int)(r / g->n_new), b = (int)(r % g->n_new);
  const int pz = c->pos[s] + b;
  int p3[3] = {pz, pz, pz};
  if (c->mpos) { p3[0] = c->mpos[3 * r]; p3[1] = c->mpos[3 * r + 1]; p3[2] = c->mpos[3 * r + 2]; }
  const size_t slot = ((size_t)c->cache_row[s] + (size_t)pz) * kvdim;
  float *kr = (float *)malloc(sizeof(float) * (size_t)D);
  if (!kr) { c->fail = 1; return; }
  for (int h = 0; h < Hkv; ++h) {
    const float *ks = c->k_new + ((size_t)r * Hkv + h) * D;
    const float *vs = c->v_new + ((size_t)r * Hkv + h) * D;
    memcpy(kr, ks, sizeof(float) * (size_t)D);
    if (g->do_rope) rope_head(kr, g->rotary_dim, g->theta, p3);
    for (int d = 0; d < D; ++d) {
      if (g->cache_is_bf16) {
        ((uint16_t *)c->kc)[slot + (size_t)h * D + d] = f32_to_bf16(kr[d]);
        ((uint16_t *)c->vc)[slot + (size_t)h * D + d] = f32_to_bf16(vs[d]);
      } else {
        ((float *)c->kc)[slot + (size_t)h * D + d] = kr[d];
        ((float *)c->vc)[slot + (size_t)h * D + d] = vs[d];
      }
    }
  }
  free(kr);
}

/* Steps 4-6 for work item w = e*q_heads + h: one output row of one query head. */
static void attend_row_head(int64_t w, void *p) {
  mixer_ctx *c = (mixer_ctx *)p;
  const oracle_geom *g = c->g;
  const int D = g->head_dim, Hq = g->q_heads, Hkv = g->kv_heads, G = Hq / Hkv;
  const size_t kvdim = (size_t)Hkv * D;
  const int64_t e = w / Hq;
  const int h = (int)(w % Hq);
  const int64_t r = c->rows ? c->rows[e] : e;
  const int s = (int)(r / g->n_new), b = (int)(r % g->n_new);
  const int pz = c->pos[s] + b;
  const int T = pz + 1; /* keys visible to this row, itself included */
  const int kvh = h / G;
  int p3[3] = {pz, pz, pz};
  if (c->mpos) { p3[0] = c->mpos[3 * r]; p3[1] = c->mpos[3 * r + 1]; p3[2] = c->mpos[3 * r + 2]; }

  float *qr = (float *)malloc(sizeof(float) * (size_t)D);
  double *sc = (double *)malloc(sizeof(double) * (size_t)T);
  double *acc = (double *)calloc((size_t)D, sizeof(double));
  if (!qr || !sc || !acc) { c->fail = 1; free(qr); free(sc); free(acc); return; }
  memcpy(qr, c->q + ((size_t)r * Hq + h) * D, sizeof(float) * (size_t)D);
  if (g->do_rope) rope_head(qr, g->rotary_dim, g->theta, p3);

  const size_t base = (size_t)c->cache_row[s] * kvdim + (size_t)kvh * D;
  const uint16_t *kc16 = (const uint16_t *)c->kc, *vc16 = (const uint16_t *)c->vc;
  const float *kc32 = (const float *)c->kc, *vc32 = (const float *)c->vc;
  double m = -INFINITY;
  for (int t = 0; t < T; ++t) {
    double dot = 0.0;
    if (g->cache_is_bf16) {
      const uint16_t *kt = kc16 + base + (size_t)t * kvdim;
      for (int d = 0; d < D; ++d) dot += (double)qr[d] * (double)bf16_to_f32(kt[d]);
    } else {
      const float *kt = kc32 + base + (size_t)t * kvdim;
      for (int d = 0; d < D; ++d) dot += (double)qr[d] * (double)kt[d];
    }
    sc[t] = dot * g->scale;
    if (sc[t] > m) m = sc[t];
  }
  double l = 0.0;
  for (int t = 0; t < T; ++t) {
    const double e_ = exp(sc[t] - m);
    l += e_;
    if (g->cache_is_bf16) {
      const uint16_t *vt = vc16 + base + (size_t)t * kvdim;
      for (int d = 0; d < D; ++d) acc[d] += e_ * (double)bf16_to_f32(vt[d]);
    } else {
      const float *vt = vc32 + base + (size_t)t * kvdim;
      for (int d = 0; d < D; ++d) acc[d] += e_ * (double)vt[d];
    }
  }
  float *o = c->out + ((size_t)e * Hq + h) * D;
  const float *gt = c->gate ? c->gate + ((size_t)r * Hq + h) * D : NULL;
  for (int d = 0; d < D; ++d) {
    double v = acc[d] / l;
    if (g->do_gate && gt) v *= 1.0 / (1.0 + exp(-(double)gt[d]));
    o[d] = (float)v;
  }
  if (c->lse) c->lse[(size_t)e * Hq + h] = (float)(m + log(l));
  free(qr); free(sc); free(acc);
}

/*
 * The whole mixer for a batch of sequences.
 *   q      [n_seq][n_new][q_heads][dim]   fp32 (already QK-normed, un-rotated if do_rope)
 *   k_new  [n_seq][n_new][kv_heads][dim]  fp32
 *   v_new  same shape
 *   gate   same shape as q (ignored unless do_gate)
 *   kc, vc cache pools; sequence s owns rows cache_row[s] .. ; row = kv_heads*dim elements
 *   pos    [n_seq] tokens already cached for each sequence (*dpos of the reference)
 *   mpos   NULL or [n_seq][n_new][3]
 *   rows   NULL (all rows) or n_rows flat indices s*n_new+b of the rows to evaluate;
 *          the append always covers every row so the cache is complete either way
 *   out    [n_eval][q_heads][dim] fp32 (post-gate), lse [n_eval][q_heads] (may be NULL)
 * Returns 0, -1 on a bad argument, -2 when memory ran out.
 */
int oracle_mixer(const oracle_geom *g, const float *q, const float *k_new,
                 const float *v_new, const float *gate, void *kc, void *vc,
                 const int *pos, const int64_t *cache_row, const int *mpos,
                 const int64_t *rows, int64_t n_rows, float *out, float *lse) {
  if (!g || g->n_seq < 0 || g->n_new < 0 || g->head_dim <= 0 || g->kv_heads <= 0 ||
      g->q_heads % g->kv_heads || g->rotary_dim > g->head_dim || (g->rotary_dim & 1))
    return -1;
  mixer_ctx c = {g, q, k_new, v_new, gate, kc, vc, pos, cache_row, mpos, rows, out, lse, 0};
  if (g->do_append) parallel_for((int64_t)g->n_seq * g->n_new, append_row, &c);
  const int64_t n_eval = rows ? n_rows : (int64_t)g->n_seq * g->n_new;
  parallel_for(n_eval * g->q_heads, attend_row_head, &c);
  return c.fail ? -2 : 0;
}

/* out *= sigmoid(gate), n elements (src/mixers.cu:653-657). */
void oracle_gate_sigmoid_f32(float *x, const float *gate, int64_t n) {
  for (int64_t i = 0; i < n; ++i)
    x[i] = (float)((double)x[i] * (1.0 / (1.0 + exp(-(double)gate[i]))));
}

/* Merge two split-KV partials of one row the way a cross-GPU combine does:
 * (o, m, l) with o = sum exp(s-m) v un-normalised.  Used to check the combine kernel. */
void oracle_combine2(const float *o1, float m1, float l1, const float *o2, float m2,
                     float l2, int dim, float *o, float *m, float *l) {
  const double mm = m1 > m2 ? m1 : m2;
  const double a1 = l1 > 0 ? exp((double)m1 - mm) : 0.0, a2 = l2 > 0 ? exp((double)m2 - mm) : 0.0;
  for (int d = 0; d < dim; ++d) o[d] = (float)(a1 * o1[d] + a2 * o2[d]);
  *m = (float)mm;
  *l = (float)(a1 * l1 + a2 * l2);
}

/* From the fused projection rows to the mixer's inputs.
 * fused[r] = [ (q[256] | gate[256]) x q_heads | k[kv_heads*256] | v[kv_heads*256] ]  (src/model.cu:219-222).
 * k_unpack3 (src/elem.cu:226-237) scatters the three parts, k_split_qgate (src/mixers.cu:382-390)
 * separates query and gate per head, k_rmsnorm_head (src/mixers.cu:393-413) scales every q and k
 * head by rsqrt(mean(x^2) + eps) * (1 + w[d]) with bf16 weights shared by all heads.  Sums in double.
 * round_bf16 != 0 rounds q and gate to bf16 on the way out: that is where the B200 path stores them (its
 * activations are bf16; k and v are rounded once, when the mixer writes them into a bf16 cache);
 * 0 keeps the reference's fp32 values. */
void oracle_fused_rows(const float *fused, int64_t n_rows, int q_heads, int kv_heads, int dim,
                       const uint16_t *q_norm_w, const uint16_t *k_norm_w, double eps, int round_bf16,
                       float *q, float *gate, float *k, float *v) {
  const int64_t width = (int64_t)q_heads * 2 * dim + 2 * (int64_t)kv_heads * dim;
  for (int64_t r = 0; r < n_rows; ++r) {
    const float *row = fused + r * width;
    const float *krow = row + (int64_t)q_heads * 2 * dim;
    const float *vrow = krow + (int64_t)kv_heads * dim;
    for (int h = 0; h < q_heads + kv_heads; ++h) {
      const int is_q = h < q_heads;
      const float *x = is_q ? row + (int64_t)h * 2 * dim : krow + (int64_t)(h - q_heads) * dim;
      const uint16_t *w = is_q ? q_norm_w : k_norm_w;
      float *dst = is_q ? q + (r * q_heads + h) * dim : k + (r * kv_heads + (h - q_heads)) * dim;
      double ss = 0.0;
      for (int d = 0; d < dim; ++d) ss += (double)x[d] * (double)x[d];
      const double sc = 1.0 / sqrt(ss / dim + eps);
      for (int d = 0; d < dim; ++d) {
        const float y = (float)((double)x[d] * sc * (1.0 + (double)bf16_to_f32(w[d])));
        dst[d] = (round_bf16 && is_q) ? bf16_to_f32(f32_to_bf16(y)) : y;
      }
      if (is_q) {
        float *gd = gate + (r * q_heads + h) * dim;
        for (int d = 0; d < dim; ++d) gd[d] = round_bf16 ? bf16_to_f32(f32_to_bf16(x[dim + d])) : x[dim + d];
      }
    }
    for (int64_t i = 0; i < (int64_t)kv_heads * dim; ++i)
      v[r * kv_heads * dim + i] = vrow[i];
  }
}

/* Exposed so tests can check the rounding rule itself. */
uint16_t oracle_f32_to_bf16(float f) { return f32_to_bf16(f); }
float oracle_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }
