/*
 * CPU golden walker -- TEST INFRASTRUCTURE ONLY.
 *
 * Nothing in the product library links, loads or calls this file.  It is an
 * independent plain-C restatement of the walk semantics, used by the tests,
 * by the smoke check and by the bench's CPU-baseline leg as the checker for
 * the CUDA engine.
 *
 * Parity status: UNPINNED BY THE REFERENCE.  The reference ships no tests,
 * no golden vectors and no CPU path, and its walks are not reproducible
 * (XORWOW streams are tied to physical threads racing for an atomic counter,
 * include/myrand.cuh:271-292, include/walker.cuh:1323-1350).  What this
 * oracle pins instead:
 *   - Philox4x32-10 against the published Random123 known-answer vectors;
 *   - the walk semantics of the reference, restated from
 *       include/app.cuh:58-152      (four biases and stop rules),
 *       include/gpu_task.cuh:36-77  (state update order),
 *       include/walker.cuh:1372-1385, 1422-1432 (write result, then stop test),
 *       include/sampler.cuh:46-85   (weighted pick, -1 iff no positive bias),
 *       include/gpu_graph.cuh:97-118 (membership by binary search, sorted rows),
 *       src/main.cu:93-111          (what counts as a step / a scanned edge);
 *   - the sampling law P(i) = bias_i / sum(bias), checked by chi-square in tests.
 *
 * Sampler (replaces the reference's prefix-sum reservoir with an exponential
 * race, which has the same law and is independent of the visiting order):
 * every candidate group gets key = E / W, E ~ Exp (in log2 units) drawn from a
 * counter-based Philox stream keyed by (seed; query id, step, group index),
 * W = total bias of the group; the smallest (key, group index) wins.  Group
 * mode 1: one neighbour per group.  Group mode 64: a "strip" of up to 64
 * neighbours (sixteen 16-byte quads 512 bytes apart); the neighbour inside the
 * winning strip is then drawn by inverse CDF with the fourth word of the
 * strip's Philox block (words 0..2 are the keys of three strips).
 *
 * Floating point: only +, *, /, fmaf (correctly rounded on host and device);
 * build with -ffp-contract=off.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define FWO_APP_DEEPWALK 0
#define FWO_APP_PPR 1
#define FWO_APP_NODE2VEC 2
#define FWO_APP_METAPATH 3

#define FWO_PURPOSE_SCAN 0u
#define FWO_PURPOSE_STOP 1u

/* ---- Philox4x32-10 (Salmon et al., SC'11), restated ---- */
void fwo_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2],
                       uint32_t out[4]) {
  uint32_t c0 = ctr[0], c1 = ctr[1], c2 = ctr[2], c3 = ctr[3];
  uint32_t k0 = key[0], k1 = key[1];
  for (int r = 0; r < 10; ++r) {
    uint64_t p0 = (uint64_t)0xD2511F53u * c0;
    uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
    uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
    uint32_t n1 = (uint32_t)p1;
    uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
    uint32_t n3 = (uint32_t)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

static inline int clz32(uint32_t x) { return x ? __builtin_clz(x) : 32; }

/* 32 random bits -> exponential variate in log2 units, E = g + f(m):
 * g = number of leading zero bits (geometric), m = the bits after the
 * leading one as a fraction in (0,1], f(m) = -log2(1 - m/2) by a fixed
 * degree-5 polynomial m*P(m).  Small E keeps full relative precision. */
float fwo_exp_key(uint32_t x) {
  int g = clz32(x);
  uint32_t t = x << (g & 31);
  uint32_t mb = t << 1;
  float m = fmaf((float)mb, 0x1p-32f, 0x1p-33f);
  float p = 0x1.3897a4p-6f;
  p = fmaf(p, m, -0x1.cb946cp-7f);
  p = fmaf(p, m, 0x1.29f26p-5f);
  p = fmaf(p, m, 0x1.cf6494p-5f);
  p = fmaf(p, m, 0x1.71fdcap-3f);
  p = fmaf(p, m, 0x1.7153dap-1f);
  return fmaf(p, m, (float)g);
}

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

uint32_t fwo_tp_threshold(double tp) {
  double t = tp * 4294967296.0;
  if (!(t > 0.0)) return 0u;
  if (t >= 4294967295.0) return 0xFFFFFFFFu;
  return (uint32_t)t;
}

typedef struct {
  int64_t V;
  const void* xadj;
  int xadj_bits;
  const int32_t* adj;
  const float* weight;
  const int32_t* label;
  int app, d;
  uint32_t tp_thresh;
  float inv_p, inv_q;
  const int32_t* schema;
  int schema_len;
  uint32_t key[2];
  int group_mode;
} fwo_ctx;

static inline int64_t row_at(const fwo_ctx* c, int64_t v) {
  return c->xadj_bits == 64 ? ((const int64_t*)c->xadj)[v]
                            : (int64_t)((const uint32_t*)c->xadj)[v];
}

/* include/gpu_graph.cuh:97-118: is `target` in the sorted row of `src`? */
static int connected(const fwo_ctx* c, int32_t src, int32_t target) {
  int64_t lo = row_at(c, src), hi = row_at(c, src + 1) - 1;
  while (lo <= hi) {
    int64_t mid = lo + (hi - lo) / 2;
    int32_t a = c->adj[mid];
    if (a == target) return 1;
    if (a < target) lo = mid + 1; else hi = mid - 1;
  }
  return 0;
}

/* Bias of edge i for step k (0-based) of a walk that came from `prev`;
 * non-positive and NaN biases are returned as 0 (never selected). */
static float bias_of(const fwo_ctx* c, int64_t i, int k, int32_t prev) {
  float b;
  switch (c->app) {
    case FWO_APP_METAPATH:  /* include/app.cuh:142-147 */
      b = (c->label[i] == c->schema[k % c->schema_len]) ? 1.0f : 0.0f;
      break;
    case FWO_APP_NODE2VEC: {  /* include/app.cuh:109-122 */
      b = c->weight[i];
      if (prev >= 0) {
        int32_t x = c->adj[i];
        if (x == prev) b = b * c->inv_p;
        else if (!connected(c, prev, x)) b = b * c->inv_q;
      }
      break;
    }
    default:  /* include/app.cuh:64-66, 84-86 */
      b = c->weight[i];
  }
  return (b > 0.0f) ? b : 0.0f;
}

/* Biases (w64, canonical order: quad j, edge cc) and edge indices of strip (s,l) of the row
 * [b,e): its 16 quads are s*512 + j*32 + l.  Returns the strip's total bias, summed in the
 * fixed order ((S0+S1)+(S2+S3)) per group of four quads, then (A0+A1)+(A2+A3). */
static float strip_fill(const fwo_ctx* c, int64_t b, int64_t e, int64_t q0, int64_t nq, int64_t s, int l,
                        int k, int32_t prev, float* w64, int64_t* i64) {
  float A[4];
  for (int g4 = 0; g4 < 4; ++g4) {
    float S[4];
    for (int jj = 0; jj < 4; ++jj) {
      int j = 4 * g4 + jj;
      int64_t q = s * 512 + j * 32 + l;
      for (int cc = 0; cc < 4; ++cc) {
        int64_t i = 4 * (q0 + q) + cc;
        i64[4 * j + cc] = i;
        w64[4 * j + cc] = (q < nq && i >= b && i < e) ? bias_of(c, i, k, prev) : 0.f;
      }
      S[jj] = (w64[4 * j] + w64[4 * j + 1]) + (w64[4 * j + 2] + w64[4 * j + 3]);
    }
    A[g4] = (S[0] + S[1]) + (S[2] + S[3]);
  }
  return (A[0] + A[1]) + (A[2] + A[3]);
}

/* One weighted pick in row [b,e).  Returns the absolute edge index or -1. */
static int64_t sample_row(const fwo_ctx* c, int64_t b, int64_t e, int k,
                          int32_t prev, uint64_t qid) {
  if (e <= b) return -1;
  const int64_t q0 = b >> 2;
  const int64_t nq = ((e + 3) >> 2) - q0;
  uint32_t ctr[4], r[4];
  ctr[1] = (uint32_t)k | (FWO_PURPOSE_SCAN << 28);
  ctr[2] = (uint32_t)qid;
  ctr[3] = (uint32_t)(qid >> 32);
  uint64_t best = ~(uint64_t)0;
  if (c->group_mode == 1) {
    for (int64_t q = 0; q < nq; ++q) {
      ctr[0] = (uint32_t)q;
      fwo_philox4x32_10(ctr, c->key, r);
      for (int cc = 0; cc < 4; ++cc) {
        int64_t i = 4 * (q0 + q) + cc;
        if (i < b || i >= e) continue;
        float w = bias_of(c, i, k, prev);
        if (!(w > 0.0f)) continue;
        float key = fwo_exp_key(r[cc]) / w;
        uint64_t packed = ((uint64_t)f2u(key) << 32) | (uint32_t)(i - 4 * q0);
        if (packed < best) best = packed;
      }
    }
    if (best == ~(uint64_t)0) return -1;
    return 4 * q0 + (int64_t)(uint32_t)best;
  }
  /* strips: group B = (s,l) holds quads s*512 + j*32 + l, j = 0..15 */
  const int64_t nsuper = (nq + 511) >> 9;
  float w64[64];
  int64_t i64[64];
  for (int64_t s = 0; s < nsuper; ++s) {
    for (int l = 0; l < 32; ++l) {
      if (s * 512 + l >= nq) continue;  /* the strip has no quad inside the row */
      float W = strip_fill(c, b, e, q0, nq, s, l, k, prev, w64, i64);
      if (!(W > 0.0f)) continue;
      uint32_t B = (uint32_t)(s * 32 + l);
      ctr[0] = (uint32_t)((s / 3) * 32 + l);  /* one block serves supergroups 3g..3g+2 of lane l */
      fwo_philox4x32_10(ctr, c->key, r);
      float key = fwo_exp_key(r[s % 3]) / W;
      uint64_t packed = ((uint64_t)f2u(key) << 32) | B;
      if (packed < best) best = packed;
    }
  }
  if (best == ~(uint64_t)0) return -1;
  /* inverse-CDF pick inside the winning strip: word 3 of the strip's scan block;
   * the first edge (canonical order) whose running sum exceeds u * W */
  uint32_t B = (uint32_t)best;
  int64_t s = B >> 5;
  int l = (int)(B & 31u);
  ctr[0] = (uint32_t)((s / 3) * 32 + l);
  fwo_philox4x32_10(ctr, c->key, r);
  float W = strip_fill(c, b, e, q0, nq, s, l, k, prev, w64, i64);
  float u = (float)(r[3] >> 8) * 0x1p-24f;
  float t = u * W;
  float acc = 0.f;
  int64_t last = -1;
  for (int z = 0; z < 64; ++z) {
    if (w64[z] > 0.f) {
      last = i64[z];
      acc = acc + w64[z];
      if (acc > t) return last;
    }
  }
  return last;
}

/* One query: fills row[0..d] (-1 padded); returns steps, adds scanned edges. */
static int walk_one(const fwo_ctx* c, int32_t start, uint64_t qid, int32_t* row,
                    uint64_t* scanned) {
  const int d = c->d;
  for (int z = 0; z <= d; ++z) row[z] = -1;
  row[0] = start;
  int32_t cur = start, prev = -1;
  int k = 0;
  while (k < d) {
    if (cur < 0 || (int64_t)cur >= c->V) break;
    int64_t b = row_at(c, cur), e = row_at(c, (int64_t)cur + 1);
    int64_t sel = sample_row(c, b, e, k, prev, qid);
    if (sel < 0) break;                 /* walker.cuh:1373-1374 */
    int32_t nxt = c->adj[sel];
    row[k + 1] = nxt;                   /* walker.cuh:1380-1381 */
    *scanned += (uint64_t)(e - b);      /* main.cu:104-105 */
    prev = cur;                         /* gpu_task.cuh:70-77 */
    cur = nxt;
    ++k;
    if (c->app == FWO_APP_PPR) {        /* app.cuh:88-94, after the step */
      uint32_t ctr[4] = {0u, (uint32_t)(k - 1) | (FWO_PURPOSE_STOP << 28),
                         (uint32_t)qid, (uint32_t)(qid >> 32)};
      uint32_t r[4];
      fwo_philox4x32_10(ctr, c->key, r);
      if (r[0] < c->tp_thresh) break;
    }
  }
  return k;
}

/*
 * Walk n queries.  result is int32 [n x (d+1)], row-major, -1 padded
 * (layout of src/walk.cu:586, src/main.cu:151-181).  stats (may be NULL):
 * [0] steps, [1] scanned edges, [2..2+d] histogram of walk lengths.
 * Returns 0, or a negative code on bad arguments.
 */
int fwo_walk(int64_t V, const void* xadj, int xadj_bits, const int32_t* adj,
             const float* weight, const int32_t* label, int app, int d,
             double tp, double p, double q, const int32_t* schema,
             int schema_len, uint64_t seed, uint64_t query_id_base,
             uint64_t query_id_stride, int group_mode, const int32_t* starts, int64_t n, int32_t* result,
             uint64_t* stats, int threads) {
  if (V < 0 || n < 0 || d < 0 || d >= (1 << 28)) return -1;
  if (xadj_bits != 32 && xadj_bits != 64) return -2;
  if (group_mode != 1 && group_mode != 64) return -3;
  if (app < 0 || app > 3) return -4;
  if (app == FWO_APP_METAPATH && (!label || !schema || schema_len <= 0)) return -5;
  if (app != FWO_APP_METAPATH && !weight) return -6;
  fwo_ctx c;
  c.V = V; c.xadj = xadj; c.xadj_bits = xadj_bits; c.adj = adj;
  c.weight = weight; c.label = label; c.app = app; c.d = d;
  c.tp_thresh = fwo_tp_threshold(tp);
  c.inv_p = (float)(1.0 / p);
  c.inv_q = (float)(1.0 / q);
  c.schema = schema; c.schema_len = schema_len;
  c.key[0] = (uint32_t)seed; c.key[1] = (uint32_t)(seed >> 32);
  c.group_mode = group_mode;
  uint64_t steps = 0, scanned = 0;
  uint64_t* hist = stats ? stats + 2 : NULL;
  if (stats) memset(stats, 0, sizeof(uint64_t) * (size_t)(d + 3));
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#endif
  (void)threads;
#pragma omp parallel
  {
    uint64_t my_steps = 0, my_scanned = 0;
    uint64_t* my_hist = hist ? (uint64_t*)calloc((size_t)d + 1, 8) : NULL;
#pragma omp for schedule(dynamic, 64)
    for (int64_t i = 0; i < n; ++i) {
      int len = walk_one(&c, starts[i], query_id_base + (uint64_t)i * (query_id_stride ? query_id_stride : 1),
                         result + i * (int64_t)(d + 1), &my_scanned);
      my_steps += (uint64_t)len;
      if (my_hist) my_hist[len]++;
    }
#pragma omp critical
    {
      steps += my_steps;
      scanned += my_scanned;
      if (my_hist) for (int z = 0; z <= d; ++z) hist[z] += my_hist[z];
    }
    free(my_hist);
  }
  if (stats) { stats[0] = steps; stats[1] = scanned; }
  return 0;
}

int fwo_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
