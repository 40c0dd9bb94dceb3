/*
 * CPU oracle for the HNSW hot path (search + per-level graph construction).
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, loads or
 * calls this file; it exists so that the CUDA path can be checked against an
 * independent plain-C restatement of the algorithm, and so that a host-CPU
 * baseline can be timed beside the GPU numbers.
 *
 * Pinning status: PINNED against the reference's own code.  The reference ships
 * no golden vectors, so fixtures were produced by running it: level draws by
 * executing the body of its set_random_levels (cuhnsw/pyhnsw.py:65-71), search
 * results and index files by its unmodified CUDA sources compiled for sm_100
 * and run on a B200 (generators and fixtures sit under tests/golden/).  On
 * continuous data this oracle returns exactly the reference's ids; on data with
 * exact distance ties only tie-independent facts can agree, because the
 * reference orders ties by heap position.  Parity with hnswlib proper (the CPU
 * library the reference names, examples/requirements.txt:3) stays unpinned: it
 * is not part of the reference's tree and not installable offline.
 *
 * What each function follows in the reference (paths inside that project):
 *   canonical distance       cpp/include/cuda_dist_kernels.cuh:31-124
 *                            (dot / squaresum / GetDistanceByVec: -dot, squared l2)
 *   greedy upper descent     cpp/include/cuda_search_kernels.cuh:22-66
 *   layer-0 bounded search   cpp/include/cuda_search_kernels.cuh:99-162
 *                            cpp/include/cuda_utils_kernels.cuh:104-151,212-227
 *   level membership, enter  cpp/src/cuhnsw_base.cu:130-156
 *   per-level construction   cpp/src/cuhnsw_build.cu:104-208
 *                            cpp/include/cuda_build_kernels.cuh:164-338
 *   neighbour selection      cpp/include/cuda_build_kernels.cuh:68-162
 *
 * Two deliberate, documented choices that the CUDA path shares bit for bit:
 *  (1) One total order everywhere: (distance, node id), packed into a 64-bit
 *      key.  The reference breaks distance ties by heap position, which is
 *      incidental; a total order makes every result unique.
 *  (2) One fp32 summation order ("canonical distance"): W = 32 accumulators
 *      for d <= 128, else 128; element i is fused-multiply-added into
 *      accumulator i mod W in increasing i; accumulators are folded as
 *      lane t = (a[4t]+a[4t+1]) + (a[4t+2]+a[4t+3]) and lanes by an xor
 *      butterfly (offsets T/2 .. 1, T = W/4).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define DIST_DOT 0
#define DIST_L2 1

/* ------------------------------------------------------------------ */
/* canonical distance                                                  */
/* ------------------------------------------------------------------ */

static inline float fold_lanes(const float *acc, int lanes) {
  float s[32], t[32];
  for (int i = 0; i < lanes; ++i)
    s[i] = (acc[4 * i] + acc[4 * i + 1]) + (acc[4 * i + 2] + acc[4 * i + 3]);
  for (int off = lanes / 2; off > 0; off >>= 1) {
    for (int i = 0; i < lanes; ++i) t[i] = s[i] + s[i ^ off];
    for (int i = 0; i < lanes; ++i) s[i] = t[i];
  }
  return s[0];
}

static inline float dist_dot_w(const float *a, const float *b, int d, int w) {
  float acc[128];
  for (int e = 0; e < w; ++e) acc[e] = 0.0f;
  int full = d / w;
  for (int c = 0; c < full; ++c) {
    const float *pa = a + (size_t)c * w, *pb = b + (size_t)c * w;
    for (int e = 0; e < w; ++e) acc[e] = fmaf(pa[e], pb[e], acc[e]);
  }
  int rem = d - full * w;
  const float *pa = a + (size_t)full * w, *pb = b + (size_t)full * w;
  for (int e = 0; e < rem; ++e) acc[e] = fmaf(pa[e], pb[e], acc[e]);
  return -fold_lanes(acc, w / 4);
}

static inline float dist_l2_w(const float *a, const float *b, int d, int w) {
  float acc[128];
  for (int e = 0; e < w; ++e) acc[e] = 0.0f;
  int full = d / w;
  for (int c = 0; c < full; ++c) {
    const float *pa = a + (size_t)c * w, *pb = b + (size_t)c * w;
    for (int e = 0; e < w; ++e) {
      float df = pa[e] - pb[e];
      acc[e] = fmaf(df, df, acc[e]);
    }
  }
  int rem = d - full * w;
  const float *pa = a + (size_t)full * w, *pb = b + (size_t)full * w;
  for (int e = 0; e < rem; ++e) {
    float df = pa[e] - pb[e];
    acc[e] = fmaf(df, df, acc[e]);
  }
  return fold_lanes(acc, w / 4);
}

float oracle_distance(const float *a, const float *b, int d, int dist_type) {
  int w = d <= 128 ? 32 : 128;
  if (dist_type == DIST_DOT) return w == 32 ? dist_dot_w(a, b, d, 32) : dist_dot_w(a, b, d, 128);
  return w == 32 ? dist_l2_w(a, b, d, 32) : dist_l2_w(a, b, d, 128);
}

/* ------------------------------------------------------------------ */
/* (distance, id) keys                                                 */
/* ------------------------------------------------------------------ */

static inline uint32_t f2ord(float x) {
  x = x + 0.0f; /* -0 -> +0 so that equal floats map to equal keys */
  uint32_t u;
  memcpy(&u, &x, 4);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
static inline float ord2f(uint32_t o) {
  uint32_t u = (o & 0x80000000u) ? (o & 0x7fffffffu) : ~o;
  float x;
  memcpy(&x, &u, 4);
  return x;
}
static inline uint64_t mkkey(float dist, int id) {
  return ((uint64_t)f2ord(dist) << 32) | (uint32_t)id;
}
static inline int key_id(uint64_t k) { return (int)(uint32_t)k; }
static inline float key_dist(uint64_t k) { return ord2f((uint32_t)(k >> 32)); }

/* binary heaps over 64-bit keys */
static inline void minheap_push(uint64_t *h, int *n, uint64_t k) {
  int i = (*n)++;
  while (i > 0) {
    int p = (i - 1) >> 1;
    if (h[p] <= k) break;
    h[i] = h[p];
    i = p;
  }
  h[i] = k;
}
static inline uint64_t minheap_pop(uint64_t *h, int *n) {
  uint64_t top = h[0];
  uint64_t last = h[--(*n)];
  int i = 0, sz = *n;
  for (;;) {
    int c = 2 * i + 1;
    if (c >= sz) break;
    if (c + 1 < sz && h[c + 1] < h[c]) c++;
    if (h[c] >= last) break;
    h[i] = h[c];
    i = c;
  }
  if (sz > 0) h[i] = last;
  return top;
}
static inline void maxheap_push(uint64_t *h, int *n, uint64_t k) {
  int i = (*n)++;
  while (i > 0) {
    int p = (i - 1) >> 1;
    if (h[p] >= k) break;
    h[i] = h[p];
    i = p;
  }
  h[i] = k;
}
static inline uint64_t maxheap_pop(uint64_t *h, int *n) {
  uint64_t top = h[0];
  uint64_t last = h[--(*n)];
  int i = 0, sz = *n;
  for (;;) {
    int c = 2 * i + 1;
    if (c >= sz) break;
    if (c + 1 < sz && h[c + 1] > h[c]) c++;
    if (h[c] <= last) break;
    h[i] = h[c];
    i = c;
  }
  if (sz > 0) h[i] = last;
  return top;
}

/* ------------------------------------------------------------------ */
/* graph view                                                          */
/* ------------------------------------------------------------------ */

typedef struct {
  int64_t n;
  int d, dist_type, max_m, max_m0;
  const float *vec;     /* n x d, row-major, unpadded                     */
  int *rows0;           /* n x max_m0 node ids                             */
  int *deg0;            /* n                                               */
  float *dist0;         /* n x max_m0 stored edge distances (build only)   */
  const int *upper_base; /* n: index of the node's level-1 row in rowsU    */
  int *rowsU;           /* total_upper x max_m                             */
  int *degU;            /* total_upper                                     */
  float *distU;         /* total_upper x max_m (build only)                */
  int max_level, enter_point;
  int reverse_cand;     /* expand the farthest unexpanded key first (cuda_utils_kernels.cuh:113-124) */
} graph_t;

static inline int level_stride(const graph_t *g, int l) { return l ? g->max_m : g->max_m0; }
static inline int *row_ids(const graph_t *g, int i, int l) {
  return l ? g->rowsU + ((size_t)g->upper_base[i] + l - 1) * g->max_m : g->rows0 + (size_t)i * g->max_m0;
}
static inline float *row_dist(const graph_t *g, int i, int l) {
  return l ? g->distU + ((size_t)g->upper_base[i] + l - 1) * g->max_m : g->dist0 + (size_t)i * g->max_m0;
}
static inline int *row_deg(const graph_t *g, int i, int l) {
  return l ? g->degU + ((size_t)g->upper_base[i] + l - 1) : g->deg0 + i;
}
static inline float gdist(const graph_t *g, const float *q, int id) {
  return oracle_distance(q, g->vec + (size_t)id * g->d, g->d, g->dist_type);
}

typedef struct {
  int *stamp; /* n, epoch-stamped visited set */
  int epoch;
  uint64_t *cand; /* min-heap */
  uint64_t *res;  /* max-heap, capacity ef */
  int cap;
} scratch_t;

static void scratch_init(scratch_t *s, int64_t n, int cap) {
  s->stamp = (int *)calloc((size_t)(n > 0 ? n : 1), sizeof(int));
  s->epoch = 0;
  s->cap = cap;
  s->cand = (uint64_t *)malloc(sizeof(uint64_t) * ((size_t)n + 64));
  s->res = (uint64_t *)malloc(sizeof(uint64_t) * ((size_t)cap + 64));
}
static void scratch_free(scratch_t *s) {
  free(s->stamp);
  free(s->cand);
  free(s->res);
}
static inline void scratch_next(scratch_t *s, int64_t n) {
  if (++s->epoch == 0x7fffffff) {
    memset(s->stamp, 0, sizeof(int) * (size_t)n);
    s->epoch = 1;
  }
}

/* Greedy 1-NN walk in one upper layer: sweep the neighbour list of the current
 * node (the list is fixed when the sweep starts), move on strictly smaller
 * distance, repeat while a sweep moved.  Returns the new current node.
 * (cuda_search_kernels.cuh:38-66) */
static int greedy_level(const graph_t *g, const float *q, int cur, float *dcur, int l, scratch_t *sc,
                        int64_t *evals, int64_t *sweeps) {
  int changed = 1;
  while (changed) {
    changed = 0;
    const int *row = row_ids(g, cur, l);
    int deg = *row_deg(g, cur, l);
    if (sweeps) (*sweeps)++;
    for (int j = 0; j < deg; ++j) {
      int nb = row[j];
      if (evals && sc->stamp[nb] != sc->epoch) {
        sc->stamp[nb] = sc->epoch;
        (*evals)++;
      }
      float dd = gdist(g, q, nb);
      if (dd < *dcur) {
        *dcur = dd;
        cur = nb;
        changed = 1;
      }
    }
  }
  return cur;
}

/* copies a max-heap into an ascending array without keeping the heap; returns count */
static int drain_sorted_keep(uint64_t *heap, int n, uint64_t *out) {
  int total = n;
  while (n > 0) {
    int pos = n - 1;
    out[pos] = maxheap_pop(heap, &n);
  }
  return total;
}

/* ef-bounded best-first search in one layer.  `res` holds the result set as a
 * max-heap of at most ef keys; a node enters iff the set is not full or its
 * key is smaller than the largest key; expansion always takes the smallest
 * unexpanded key and stops when that key is larger than the largest key of a
 * full result set (cuda_search_kernels.cuh:114-139,
 * cuda_utils_kernels.cuh:220-225).  Seeds must already be in cand/res/visited.
 * `self` (>= 0) is never inserted (build: cuda_utils_kernels.cuh:157). */
#define ORACLE_FLAG 0x80000000ull
/* reverse_cand variant: the result set is a sorted array with an "expanded" flag per key (bit 31 of the
 * id word, masked in comparisons); every step expands the LARGEST unexpanded key and the walk ends when
 * every key of the set is expanded.  Uses sc->cand as the array; leaves sc->res a valid max-heap. */
static void beam_layer_reverse(const graph_t *g, const float *q, int l, int ef, scratch_t *sc, int *nres, int self,
                               int64_t *evals, int64_t *expansions) {
  uint64_t *w = sc->cand;
  int n = drain_sorted_keep(sc->res, *nres, w);
  for (;;) {
    int at = n - 1;
    while (at >= 0 && (w[at] & ORACLE_FLAG)) --at;
    if (at < 0) break;
    int c = (int)((uint32_t)w[at] & 0x7fffffffu);
    w[at] |= ORACLE_FLAG;
    const int *row = row_ids(g, c, l);
    int deg = *row_deg(g, c, l);
    if (expansions) (*expansions)++;
    for (int j = 0; j < deg; ++j) {
      int nb = row[j];
      if (nb == self || sc->stamp[nb] == sc->epoch) continue;
      sc->stamp[nb] = sc->epoch;
      uint64_t k = mkkey(gdist(g, q, nb), nb);
      if (evals) (*evals)++;
      if (n >= ef) {
        if (!(k < (w[n - 1] & ~ORACLE_FLAG))) continue;
        --n; /* evict the largest key */
      }
      int pos = n;
      while (pos > 0 && (w[pos - 1] & ~ORACLE_FLAG) > k) { w[pos] = w[pos - 1]; --pos; }
      w[pos] = k;
      ++n;
    }
  }
  *nres = 0;
  for (int i = 0; i < n; ++i) maxheap_push(sc->res, nres, w[i] & ~ORACLE_FLAG);
}

static void beam_layer(const graph_t *g, const float *q, int l, int ef, scratch_t *sc, int *ncand, int *nres,
                       int self, int64_t *evals, int64_t *expansions) {
  if (g->reverse_cand) {
    beam_layer_reverse(g, q, l, ef, sc, nres, self, evals, expansions);
    *ncand = 0;
    return;
  }
  while (*ncand > 0) {
    uint64_t ck = sc->cand[0];
    if (*nres >= ef && ck > sc->res[0]) break;
    minheap_pop(sc->cand, ncand);
    int c = key_id(ck);
    const int *row = row_ids(g, c, l);
    int deg = *row_deg(g, c, l);
    if (expansions) (*expansions)++;
    for (int j = 0; j < deg; ++j) {
      int nb = row[j];
      if (nb == self) continue;
      if (sc->stamp[nb] == sc->epoch) continue;
      sc->stamp[nb] = sc->epoch;
      float dd = gdist(g, q, nb);
      if (evals) (*evals)++;
      uint64_t k = mkkey(dd, nb);
      if (*nres < ef) {
        maxheap_push(sc->res, nres, k);
        minheap_push(sc->cand, ncand, k);
      } else if (k < sc->res[0]) {
        maxheap_pop(sc->res, nres);
        maxheap_push(sc->res, nres, k);
        minheap_push(sc->cand, ncand, k);
      }
    }
  }
}

/* drain a max-heap into an ascending array; returns count */
static int drain_sorted(uint64_t *heap, int n, uint64_t *out) {
  int total = n;
  while (n > 0) {
    int pos = n - 1;
    out[pos] = maxheap_pop(heap, &n);
  }
  return total;
}

/* ------------------------------------------------------------------ */
/* search                                                              */
/* ------------------------------------------------------------------ */

/* counters (optional, 3 per query): distinct distance evaluations,
 * layer-0 expansions, upper-layer sweeps. */
int oracle_search(int64_t n, int d, int dist_type, const float *vec, int max_m, int max_m0, const int *rows0,
                  const int *deg0, const int *upper_base, const int *rowsU, const int *degU, int max_level,
                  int enter_point, const float *queries, int64_t nq, int topk, int ef, int *out_ids,
                  float *out_dist, int *out_found, int64_t *counters, int nthreads, int reverse_cand) {
  if (ef < topk) ef = topk;
  graph_t g;
  memset(&g, 0, sizeof(g));
  g.n = n; g.d = d; g.dist_type = dist_type; g.max_m = max_m; g.max_m0 = max_m0;
  g.vec = vec; g.rows0 = (int *)rows0; g.deg0 = (int *)deg0; g.upper_base = upper_base;
  g.rowsU = (int *)rowsU; g.degU = (int *)degU; g.max_level = max_level; g.enter_point = enter_point;
  g.reverse_cand = reverse_cand;
  if (n <= 0) {
    for (int64_t i = 0; i < nq; ++i) out_found[i] = 0;
    return 0;
  }
#ifdef _OPENMP
  if (nthreads <= 0) nthreads = omp_get_max_threads();
#else
  nthreads = 1;
#endif
#pragma omp parallel num_threads(nthreads)
  {
    scratch_t sc;
    scratch_init(&sc, n, ef);
    uint64_t *sorted = (uint64_t *)malloc(sizeof(uint64_t) * ((size_t)ef + 8));
#pragma omp for schedule(dynamic, 16)
    for (int64_t qi = 0; qi < nq; ++qi) {
      const float *q = queries + (size_t)qi * d;
      int64_t ev = 0, ex = 0, sw = 0;
      int64_t *pev = counters ? &ev : NULL;
      scratch_next(&sc, n);
      int cur = enter_point;
      float dcur = gdist(&g, q, cur);
      if (pev) { sc.stamp[cur] = sc.epoch; ev++; }
      for (int l = max_level; l >= 1; --l) cur = greedy_level(&g, q, cur, &dcur, l, &sc, pev, counters ? &sw : NULL);
      /* layer 0 uses a fresh visited set: {entry} (cuda_search_kernels.cuh:108-112) */
      int64_t ev_upper = ev;
      scratch_next(&sc, n);
      int ncand = 0, nres = 0;
      uint64_t k0 = mkkey(dcur, cur);
      sc.stamp[cur] = sc.epoch;
      maxheap_push(sc.res, &nres, k0);
      minheap_push(sc.cand, &ncand, k0);
      ev = 0;
      beam_layer(&g, q, 0, ef, &sc, &ncand, &nres, -1, counters ? &ev : NULL, counters ? &ex : NULL);
      int total = drain_sorted(sc.res, nres, sorted);
      int found = total < topk ? total : topk;
      out_found[qi] = found;
      for (int j = 0; j < found; ++j) {
        out_ids[(size_t)qi * topk + j] = key_id(sorted[j]);
        out_dist[(size_t)qi * topk + j] = key_dist(sorted[j]);
      }
      if (counters) {
        /* the entry's distance is evaluated once (upper count); layer-0 first visits add to it */
        counters[3 * qi + 0] = ev_upper + ev;
        counters[3 * qi + 1] = ex;
        counters[3 * qi + 2] = sw;
      }
    }
    free(sorted);
    scratch_free(&sc);
  }
  return 0;
}

/* ------------------------------------------------------------------ */
/* neighbour selection (SearchHeuristic)                               */
/* ------------------------------------------------------------------ */

/* cands: ascending keys (distance to src, id).  Writes at most m ids/dists
 * and returns the new degree.  new_comer < 0: full test of every candidate
 * against the already accepted ones; new_comer >= 0: candidates before the
 * newcomer pass untested, the newcomer gets the full test, later candidates
 * are tested against the newcomer only (cuda_build_kernels.cuh:99-160). */
static int select_neighbors(const graph_t *g, const uint64_t *cands, int ncands, int m, double heuristic_coef,
                            int save_remains, int new_comer, int *out_ids, float *out_dist, int64_t *evals) {
  int head = 0;
  int tail = m - 1;
  if (tail > ncands - 1) tail = ncands - 1;
  const int max_head = tail + 1;
  const int nn_num = (int)(m * heuristic_coef);
  int new_comer_inserted = 0;
  for (int j = 0; j < ncands; ++j) {
    if (head >= m) break;
    int cid = key_id(cands[j]);
    float cd = key_dist(cands[j]);
    int freepass = head < nn_num || (new_comer >= 0 && !new_comer_inserted && cid != new_comer);
    if (freepass) {
      out_ids[head] = cid;
      out_dist[head] = cd;
      head++;
      continue;
    }
    int skip = 0;
    const float *cv = g->vec + (size_t)cid * g->d;
    if (new_comer >= 0 && new_comer_inserted) {
      float dd = gdist(g, cv, new_comer);
      *evals += 1;
      skip = cd > dd;
    } else {
      for (int k = 0; k < head; ++k) {
        float dd = gdist(g, cv, out_ids[k]);
        *evals += 1;
        if (cd > dd) { skip = 1; break; }
      }
    }
    if (cid == new_comer && !skip) new_comer_inserted = 1;
    if (skip && tail >= head) {
      out_ids[tail] = cid;
      out_dist[tail] = cd;
      tail--;
    } else if (!skip) {
      out_ids[head] = cid;
      out_dist[head] = cd;
      head++;
    }
  }
  return save_remains ? max_head : head;
}

/* ------------------------------------------------------------------ */
/* build                                                               */
/* ------------------------------------------------------------------ */

typedef struct { uint64_t key; float dist; } proposal_t; /* key = dst<<32 | batch position */
static int cmp_proposal(const void *a, const void *b) {
  uint64_t x = ((const proposal_t *)a)->key, y = ((const proposal_t *)b)->key;
  return x < y ? -1 : (x > y ? 1 : 0);
}

/* Number of nodes taken by the next insertion batch of a level: a fixed
 * function of how many nodes are already linked (`reachable` = nodes copied
 * down from the level above + nodes processed so far).  bmax = 1 gives the
 * strictly sequential schedule (the reference kernel run with one block). */
static int64_t next_batch(int64_t reachable, int64_t left, int64_t bmax, int64_t ramp_div) {
  int64_t b = reachable / ramp_div;
  if (b < 1) b = 1;
  if (b > bmax) b = bmax;
  if (b > left) b = left;
  return b;
}

/* Fills rows0/deg0/dist0, rowsU/degU/distU (caller-allocated from levels[]),
 * max_level and enter_point.  upper_base must be the exclusive prefix sum of
 * levels[].  Deterministic for any thread count. */
int oracle_build(int64_t n, int d, int dist_type, const float *vec, const int *levels, int max_m, int max_m0,
                 int ef_construction, double heuristic_coef, int save_remains, int64_t bmax, int64_t ramp_div,
                 int *rows0, int *deg0, float *dist0, const int *upper_base, int *rowsU, int *degU,
                 float *distU, int *out_max_level, int *out_enter_point, int64_t *build_counters, int nthreads,
                 int reverse_cand) {
  graph_t g;
  memset(&g, 0, sizeof(g));
  g.n = n; g.d = d; g.dist_type = dist_type; g.max_m = max_m; g.max_m0 = max_m0;
  g.vec = vec; g.rows0 = rows0; g.deg0 = deg0; g.dist0 = dist0; g.upper_base = upper_base;
  g.rowsU = rowsU; g.degU = degU; g.distU = distU;
  g.reverse_cand = reverse_cand;
  /* first node that reaches the maximum level (cuhnsw_base.cu:134-141) */
  int max_level = 0, enter = 0;
  for (int64_t i = 0; i < n; ++i)
    if (levels[i] > max_level) { max_level = levels[i]; enter = (int)i; }
  g.max_level = max_level; g.enter_point = enter;
  *out_max_level = max_level; *out_enter_point = enter;
  if (n == 0) return 0;
  if (bmax < 1) bmax = 1;
  if (ramp_div < 1) ramp_div = 1;
#ifdef _OPENMP
  if (nthreads <= 0) nthreads = omp_get_max_threads();
#else
  nthreads = 1;
#endif
  const int efc = ef_construction;
  scratch_t *scs = (scratch_t *)malloc(sizeof(scratch_t) * nthreads);
  uint64_t **sorted = (uint64_t **)malloc(sizeof(uint64_t *) * nthreads);
  for (int t = 0; t < nthreads; ++t) {
    scratch_init(&scs[t], n, efc);
    sorted[t] = (uint64_t *)malloc(sizeof(uint64_t) * ((size_t)efc + 8));
  }
  int *nodes = (int *)malloc(sizeof(int) * (size_t)n);
  unsigned char *went = (unsigned char *)malloc((size_t)n);
  int64_t cap = bmax < n ? bmax : n;
  const int mmax = max_m0 > max_m ? max_m0 : max_m;
  int *st_ids = (int *)malloc(sizeof(int) * (size_t)cap * mmax);
  float *st_dist = (float *)malloc(sizeof(float) * (size_t)cap * mmax);
  int *st_deg = (int *)malloc(sizeof(int) * (size_t)cap);
  proposal_t *props = (proposal_t *)malloc(sizeof(proposal_t) * (size_t)cap * mmax);
  int64_t *seg = (int64_t *)malloc(sizeof(int64_t) * ((size_t)cap * mmax + 1));
  /* work counters: rows gathered for a distance (descent, beam search, neighbour selection with its early
   * exit), adjacency rows read or written, and the bytes of those rows (ids + stored distances + degree:
   * 8 * (1 + link budget of the level) each) */
  int64_t c_evals = 0, c_rows = 0, c_row_bytes = 0;

  for (int l = max_level; l >= 0; --l) {
    const int m = level_stride(&g, l);
    const int64_t rows_before = c_rows;
    int64_t nl = 0, upper_cnt = 0;
    for (int64_t i = 0; i < n; ++i)
      if (levels[i] >= l) {
        nodes[nl++] = (int)i;
        if (levels[i] > l) upper_cnt++;
      }
    /* initial rows (cuhnsw_build.cu:113-142): nodes of the level above keep
     * their finished row from there (with its distances); every other node
     * gets one edge to the node a greedy descent from the enter point
     * reaches on the level above. */
#pragma omp parallel for schedule(dynamic, 64) num_threads(nthreads) reduction(+ : c_evals, c_rows)
    for (int64_t t = 0; t < nl; ++t) {
      int i = nodes[t];
      int *ids = row_ids(&g, i, l);
      float *ds = row_dist(&g, i, l);
      went[i] = 0;
      c_rows += 1 + (levels[i] > l);  /* the initial row is written; a copied-down row is also read */
      if (levels[i] > l) {
        const int *uids = row_ids(&g, i, l + 1);
        const float *uds = row_dist(&g, i, l + 1);
        int udeg = *row_deg(&g, i, l + 1);
        for (int j = 0; j < udeg; ++j) { ids[j] = uids[j]; ds[j] = uds[j]; }
        *row_deg(&g, i, l) = udeg;
      } else if (l == max_level) {
        if (i == enter) {
          *row_deg(&g, i, l) = 0;
        } else {
          ids[0] = enter;
          ds[0] = gdist(&g, vec + (size_t)i * d, enter);
          *row_deg(&g, i, l) = 1;
        }
      } else {
#ifdef _OPENMP
        scratch_t *sc = &scs[omp_get_thread_num()];
#else
        scratch_t *sc = &scs[0];
#endif
        const float *q = vec + (size_t)i * d;
        int cur = enter;
        float dcur = gdist(&g, q, cur);
        int64_t ev = 1;
        scratch_next(sc, n);
        for (int ll = max_level; ll > l; --ll) cur = greedy_level(&g, q, cur, &dcur, ll, sc, &ev, NULL);
        c_evals += ev;
        ids[0] = cur;
        ds[0] = dcur;
        *row_deg(&g, i, l) = 1;
      }
    }

    int64_t p = 0;
    while (p < nl) {
      int64_t b = next_batch(upper_cnt + p, nl - p, bmax, ramp_div);
      /* phase A: search + own-row selection against the frozen graph */
#pragma omp parallel for schedule(dynamic, 4) num_threads(nthreads) reduction(+ : c_evals, c_rows)
      for (int64_t t = 0; t < b; ++t) {
#ifdef _OPENMP
        int tid = omp_get_thread_num();
#else
        int tid = 0;
#endif
        scratch_t *sc = &scs[tid];
        int s = nodes[p + t];
        const float *q = vec + (size_t)s * d;
        scratch_next(sc, n);
        sc->stamp[s] = sc->epoch;
        int ncand = 0, nres = 0;
        const int *row = row_ids(&g, s, l);
        int deg = *row_deg(&g, s, l);
        int64_t ev = 0, ex = 0;
        for (int j = 0; j < deg; ++j) {
          int nb = row[j];
          if (nb == s || sc->stamp[nb] == sc->epoch) continue;
          sc->stamp[nb] = sc->epoch;
          uint64_t k = mkkey(gdist(&g, q, nb), nb);
          ev++;
          if (nres < efc) {
            maxheap_push(sc->res, &nres, k);
            minheap_push(sc->cand, &ncand, k);
          } else if (k < sc->res[0]) {
            maxheap_pop(sc->res, &nres);
            maxheap_push(sc->res, &nres, k);
            minheap_push(sc->cand, &ncand, k);
          }
        }
        beam_layer(&g, q, l, efc, sc, &ncand, &nres, s, &ev, &ex);
        int total = drain_sorted(sc->res, nres, sorted[tid]);
        st_deg[t] = select_neighbors(&g, sorted[tid], total, m, heuristic_coef, save_remains, -1,
                                     st_ids + (size_t)t * m, st_dist + (size_t)t * m, &ev);
        c_evals += ev;
        c_rows += ex + 1;
      }
      /* apply own rows, emit reverse-link proposals */
      int64_t np = 0;
      for (int64_t t = 0; t < b; ++t) {
        int s = nodes[p + t];
        int *ids = row_ids(&g, s, l);
        float *ds = row_dist(&g, s, l);
        for (int j = 0; j < st_deg[t]; ++j) {
          ids[j] = st_ids[(size_t)t * m + j];
          ds[j] = st_dist[(size_t)t * m + j];
          props[np].key = ((uint64_t)(uint32_t)ids[j] << 32) | (uint64_t)t;
          props[np].dist = ds[j];
          np++;
        }
        *row_deg(&g, s, l) = st_deg[t];
        went[s] = 1;
      }
      qsort(props, (size_t)np, sizeof(proposal_t), cmp_proposal);
      int64_t nseg = 0;
      for (int64_t i = 0; i < np; ++i)
        if (i == 0 || (props[i].key >> 32) != (props[i - 1].key >> 32)) seg[nseg++] = i;
      seg[nseg] = np;
      /* phase C: per target node, newcomers in ascending source order
       * (cuda_build_kernels.cuh:295-332) */
#pragma omp parallel for schedule(dynamic, 16) num_threads(nthreads) reduction(+ : c_rows, c_evals)
      for (int64_t si = 0; si < nseg; ++si) {
        int dst = (int)(props[seg[si]].key >> 32);
        int *ids = row_ids(&g, dst, l);
        float *ds = row_dist(&g, dst, l);
        int *pdeg = row_deg(&g, dst, l);
        uint64_t ck[72];
        int tmp_ids[64];
        float tmp_ds[64];
        for (int64_t pi = seg[si]; pi < seg[si + 1]; ++pi) {
          int s = nodes[p + (int64_t)(props[pi].key & 0xffffffffu)];
          int deg = *pdeg;
          int present = 0;
          for (int j = 0; j < deg; ++j)
            if (ids[j] == s) { present = 1; break; }
          if (present) continue;
          int nc = 0;
          ck[nc++] = mkkey(props[pi].dist, s);
          for (int j = 0; j < deg; ++j)
            if (ids[j] != dst) ck[nc++] = mkkey(ds[j], ids[j]);
          /* insertion sort ascending (nc <= m + 1) */
          for (int a = 1; a < nc; ++a) {
            uint64_t v = ck[a];
            int bpos = a - 1;
            while (bpos >= 0 && ck[bpos] > v) { ck[bpos + 1] = ck[bpos]; bpos--; }
            ck[bpos + 1] = v;
          }
          if (nc > efc) nc = efc;
          int new_comer = (!save_remains && went[dst]) ? s : -1;
          int64_t sev = 0;
          int ndeg = select_neighbors(&g, ck, nc, m, heuristic_coef, save_remains, new_comer, tmp_ids, tmp_ds, &sev);
          c_evals += sev;
          for (int j = 0; j < ndeg; ++j) { ids[j] = tmp_ids[j]; ds[j] = tmp_ds[j]; }
          *pdeg = ndeg;
          went[dst] = 1;
          c_rows += 2;
        }
      }
      p += b;
    }
    c_row_bytes += (c_rows - rows_before) * 8 * (1 + (int64_t)m);
  }
  if (build_counters) { build_counters[0] = c_evals; build_counters[1] = c_rows; build_counters[2] = c_row_bytes; }
  for (int t = 0; t < nthreads; ++t) { scratch_free(&scs[t]); free(sorted[t]); }
  free(scs); free(sorted); free(nodes); free(went); free(st_ids); free(st_dist); free(st_deg);
  free(props); free(seg);
  return 0;
}

/* Exact top-k by brute force under the same (distance, id) order. */
int oracle_bruteforce(int64_t n, int d, int dist_type, const float *vec, const float *queries, int64_t nq,
                      int topk, int *out_ids, float *out_dist, int nthreads) {
#ifdef _OPENMP
  if (nthreads <= 0) nthreads = omp_get_max_threads();
#else
  nthreads = 1;
#endif
#pragma omp parallel num_threads(nthreads)
  {
    uint64_t *heap = (uint64_t *)malloc(sizeof(uint64_t) * ((size_t)topk + 8));
    uint64_t *srt = (uint64_t *)malloc(sizeof(uint64_t) * ((size_t)topk + 8));
#pragma omp for schedule(dynamic, 4)
    for (int64_t qi = 0; qi < nq; ++qi) {
      const float *q = queries + (size_t)qi * d;
      int nh = 0;
      for (int64_t i = 0; i < n; ++i) {
        uint64_t k = mkkey(oracle_distance(q, vec + (size_t)i * d, d, dist_type), (int)i);
        if (nh < topk) maxheap_push(heap, &nh, k);
        else if (k < heap[0]) { maxheap_pop(heap, &nh); maxheap_push(heap, &nh, k); }
      }
      int total = drain_sorted(heap, nh, srt);
      for (int j = 0; j < topk; ++j) {
        out_ids[(size_t)qi * topk + j] = j < total ? key_id(srt[j]) : -1;
        out_dist[(size_t)qi * topk + j] = j < total ? key_dist(srt[j]) : INFINITY;
      }
    }
    free(heap);
    free(srt);
  }
  return 0;
}

int oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
