/*
 * nd_oracle.c -- CPU oracle for the NextDoor sampling path.  TEST INFRASTRUCTURE ONLY:
 * see nd_oracle.h for what may load it and for the parity status of each app.
 *
 * Build: gcc -O2 -std=c11 -ffp-contract=off -fopenmp -shared -fPIC nd_oracle.c -o libnd_oracle.so
 * (-ffp-contract=off: every float expression below must round like a lone fp32 operation,
 *  the way the device code spells it with __fmul_rn.)
 */
#include "nd_oracle.h"

#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------ RNG */

/* Philox4x32-10 (Salmon et al., SC'11).  Round constants are the published ones; the CUDA
 * toolkit lists the same four in curand_philox4x32_x.h. */
void ndo_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]) {
  uint32_t c0 = ctr[0], c1 = ctr[1], c2 = ctr[2], c3 = ctr[3];
  uint32_t k0 = key[0], k1 = key[1];
  for (int r = 0; r < 10; r++) {
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

/* Draw contract: key = run seed; counter = (sample, step, slot, draw/4); lane = draw%4.
 * `draw` counts the uniform draws inside one next() invocation, from 0.  The reference ties
 * draws to a per-thread XORWOW stream (src/nextdoor.cu:1838-1843), which is not
 * reproducible across schedules; this keyed contract replaces it. */
uint32_t ndo_draw_u32(uint64_t seed, uint32_t sample, uint32_t step, uint32_t slot, uint32_t draw) {
  uint32_t ctr[4] = {sample, step, slot, draw >> 2};
  uint32_t key[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
  uint32_t o[4];
  ndo_philox4x32_10(ctr, key, o);
  return o[draw & 3];
}

/* (0,1] mapping of cuRAND's curand_uniform: x*2^-32 + 2^-33 in fp32 (curand_uniform.h:69-72). */
float ndo_u32_to_uniform(uint32_t x) {
  float f = (float)x;
  f = f * 2.3283064365386963e-10f;
  return f + 1.1641532182693481e-10f;
}

float ndo_uniform(uint64_t seed, uint32_t sample, uint32_t step, uint32_t slot, uint32_t draw) {
  return ndo_u32_to_uniform(ndo_draw_u32(seed, sample, step, slot, draw));
}

/* RandNumGen::rand_int, src/rand_num_gen.cuh:117-122 */
int32_t ndo_rand_int(float u, int32_t n) {
  float ff = u * (float)n;
  int32_t id = (int32_t)ff;
  return id < n - 1 ? id : n - 1;
}

typedef struct {
  uint64_t seed;
  uint32_t sample, step, slot, draw;
} rng_t;

static inline float rng_uniform(rng_t *r) {
  float u = ndo_uniform(r->seed, r->sample, r->step, r->slot, r->draw);
  r->draw++;
  return u;
}
static inline int32_t rng_int(rng_t *r, int32_t n) { return ndo_rand_int(rng_uniform(r), n); }

/* ------------------------------------------------------------------ synthetic graph */

/* R-MAT (a,b,c,d) = (.57,.19,.19,.05).  Undirected edge e, attempt t: counter (e_lo, e_hi, t, blk),
 * key = seed ^ "RMAT".  Level l uses draw l; quadrant thresholds are integers so host and
 * device agree bit for bit.  An attempt is rejected when an endpoint >= V or src == dst.
 * The weight uses draw `scale` of the accepted attempt: 1 + 4 * (x>>8) * 2^-24, in [1,5). */
static const uint32_t RMAT_T1 = 2448131358u; /* floor(0.57 * 2^32) */
static const uint32_t RMAT_T2 = 3264175144u; /* floor(0.76 * 2^32) */
static const uint32_t RMAT_T3 = 4080218931u; /* floor(0.95 * 2^32) */

static void rmat_edge(int32_t V, int scale, uint64_t e, uint64_t seed, int32_t *ps, int32_t *pd, float *pw) {
  uint32_t key[2] = {(uint32_t)seed ^ 0x524D4154u, (uint32_t)(seed >> 32)};
  for (uint32_t attempt = 0;; attempt++) {
    uint32_t o[4];
    int32_t s = 0, d = 0;
    for (int l = 0; l <= scale; l++) {
      if ((l & 3) == 0) {
        uint32_t ctr[4] = {(uint32_t)e, (uint32_t)(e >> 32), attempt, (uint32_t)(l >> 2)};
        ndo_philox4x32_10(ctr, key, o);
      }
      uint32_t x = o[l & 3];
      if (l == scale) {
        if (s < V && d < V && s != d) {
          *ps = s; *pd = d;
          *pw = 1.0f + 4.0f * ((float)(x >> 8) * 5.9604644775390625e-08f);
          return;
        }
        break;
      }
      int sb = 0, db = 0;
      if (x < RMAT_T1) { sb = 0; db = 0; }
      else if (x < RMAT_T2) { sb = 0; db = 1; }
      else if (x < RMAT_T3) { sb = 1; db = 0; }
      else { sb = 1; db = 1; }
      s = (s << 1) | sb;
      d = (d << 1) | db;
    }
  }
}

void ndo_rmat_records(int32_t V, int64_t M, uint64_t seed, int32_t *src, int32_t *dst, float *w) {
  int scale = 0;
  while (((int64_t)1 << scale) < V) scale++;
#pragma omp parallel for schedule(static)
  for (int64_t e = 0; e < M; e++) {
    int32_t s, d; float ww;
    rmat_edge(V, scale, (uint64_t)e, seed, &s, &d, &ww);
    src[2 * e] = s; dst[2 * e] = d; w[2 * e] = ww;
    src[2 * e + 1] = d; dst[2 * e + 1] = s; w[2 * e + 1] = ww;
  }
}

typedef struct { int32_t d; float w; } adj_t;
static int adj_cmp(const void *a, const void *b) {
  const adj_t *x = (const adj_t *)a, *y = (const adj_t *)b;
  if (x->d != y->d) return x->d < y->d ? -1 : 1;
  if (x->w != y->w) return x->w < y->w ? -1 : 1;
  return 0;
}

/* Graph::load_from_edge_list_binary (src/graph.hpp:106-159): vertex count = max id + 1,
 * duplicates kept, each adjacency list sorted by (dst, weight) (graph.hpp:38);
 * csr_from_graph (src/csr.hpp:399-424) lays the lists out back to back;
 * Vertex::max_weight (graph.hpp:71-80) starts from 0. */
int32_t ndo_csr_from_records(int64_t n, const int32_t *src, const int32_t *dst, const float *w,
                             int32_t V, int32_t *row_ptr, int32_t *col, float *wout, float *max_w) {
  if (V <= 0) {
    int32_t m = -1;
    for (int64_t i = 0; i < n; i++) {
      if (src[i] > m) m = src[i];
      if (dst[i] > m) m = dst[i];
    }
    V = m + 1;
  }
  if (!row_ptr) return V;
  /* records are grouped by source with a counting pass, then every list is sorted on its own
   * (lists in parallel): the same order as one sort by (src, dst, weight) */
  adj_t *r = (adj_t *)malloc(sizeof(adj_t) * (size_t)(n > 0 ? n : 1));
  int64_t *pos = (int64_t *)malloc(sizeof(int64_t) * ((size_t)V + 1));
  for (int32_t v = 0; v <= V; v++) row_ptr[v] = 0;
  for (int64_t i = 0; i < n; i++) row_ptr[src[i] + 1]++;
  for (int32_t v = 0; v < V; v++) row_ptr[v + 1] += row_ptr[v];
  for (int32_t v = 0; v < V; v++) pos[v] = row_ptr[v];
  for (int64_t i = 0; i < n; i++) {
    adj_t *q = &r[pos[src[i]]++];
    q->d = dst[i]; q->w = w[i];
  }
#pragma omp parallel for schedule(dynamic, 1024)
  for (int32_t v = 0; v < V; v++) {
    const int64_t a = row_ptr[v], b = row_ptr[v + 1];
    if (b - a > 1) qsort(r + a, (size_t)(b - a), sizeof(adj_t), adj_cmp);
    float m = 0.0f;
    for (int64_t i = a; i < b; i++) {
      col[i] = r[i].d; wout[i] = r[i].w;
      if (r[i].w > m) m = r[i].w;
    }
    max_w[v] = m;
  }
  free(pos);
  free(r);
  return V;
}

/* Range partitioner after create_csr_partitions (src/graph_partitioner.cuh:1-173, dead code in
 * the reference): contiguous vertex ranges, a vertex record costs 16 B and an edge 4 B, a
 * partition is closed before the first vertex whose list would make it reach the budget, or
 * after it when it lands exactly on the budget.  Extension: a vertex whose own list does not
 * fit an empty partition is cut across partitions (same vertex id closes one and opens the next). */
void ndo_partition(int32_t V, const int32_t *row_ptr, int64_t budget, int32_t max_parts,
                   int32_t *first_v, int32_t *last_v, int64_t *first_e, int64_t *last_e,
                   int32_t *n_parts) {
  int32_t np = 0;
  int32_t u = 0;
  int64_t e_start = 0;
  while (u < V && np < max_parts) {
    int64_t n_edges = 0;
    int32_t v = u;
    int64_t e_end = -1;
    int32_t u_end = V - 1;
    int closed = 0;
    for (; v < V; v++) {
      int64_t s = row_ptr[v], e = row_ptr[v + 1];
      if (v == u && e_start > s) s = e_start;
      int64_t edges = e - s;
      int64_t nv = v - u + 1;
      if ((n_edges + edges) * 4 + nv * 16 >= budget) {
        int64_t room = (budget - nv * 16) / 4 - n_edges;
        if (room < 0) room = 0;
        if (room >= edges) { /* exactly fits */
          u_end = v; e_end = s + edges - 1;
        } else if (v > u) { /* close before v */
          u_end = v - 1; e_end = s - 1;
        } else { /* a single list larger than the budget: cut it */
          if (room == 0) room = 1;
          u_end = v; e_end = s + room - 1;
        }
        closed = 1;
        break;
      }
      n_edges += edges;
    }
    if (!closed) { u_end = V - 1; e_end = (int64_t)row_ptr[V] - 1; }
    first_v[np] = u; last_v[np] = u_end; first_e[np] = e_start; last_e[np] = e_end;
    np++;
    if (!closed) break;
    e_start = e_end + 1;
    if (e_start >= row_ptr[u_end + 1]) u = u_end + 1; else u = u_end; /* continue a cut list */
  }
  *n_parts = np;
}

/* ------------------------------------------------------------------ app bodies */

static int is_walk(int app) { return app <= NDO_APP_NODE2VEC; }
static int is_khop(int app) { return app == NDO_APP_KHOP || app == NDO_APP_KHOP_DISTINCT; }
static int is_collective(int app) { return app >= NDO_APP_FASTGCN_REF; }

int32_t ndo_initial_sample_size(const ndo_params *p) { return is_collective(p->app) ? p->batch : 1; }

/* getFinalSampleSize, src/nextdoor.cu:1913-1929 */
int32_t ndo_final_sample_size(const ndo_params *p) {
  if (is_walk(p->app)) return p->steps;
  if (is_khop(p->app)) {
    int64_t n = 1, tot = 0;
    for (int k = 0; k < p->steps; k++) { n *= p->fanout[k]; tot += n; }
    return (int32_t)tot;
  }
  return p->steps * p->fanout[0];
}

/* utils::binarySearch, src/utils.hpp:30-48; counts probes */
static int bsearch_i32(const int32_t *a, int32_t x, int32_t size, int64_t *probes) {
  int32_t l = 0, r = size - 1;
  while (l <= r) {
    int32_t m = l + (r - l) / 2;
    (*probes)++;
    int32_t am = a[m];
    if (am == x) return 1;
    if (am < x) l = m + 1; else r = m - 1;
  }
  return 0;
}

/* one next() of a walk app; returns -1 for "no vertex" */
static int32_t walk_next(const ndo_graph *g, const ndo_params *p, int step, int32_t transit,
                         int32_t *state_t, rng_t *rng, ndo_counters *c) {
  const int32_t rs = g->row_ptr[transit];
  const int32_t n = g->row_ptr[transit + 1] - rs;
  const int32_t *edges = g->col + rs;
  const float *weights = g->w + rs;
  const float max_w = g->max_w[transit];
  switch (p->app) {
    case NDO_APP_UNIFORM_WALK: { /* example/uniformRandWalk.cu:35-36 */
      return edges[rng_int(rng, n)];
    }
    case NDO_APP_DEEPWALK:
    case NDO_APP_PPR: { /* randomWalks.cu:74-90, 102-124 */
      if (n == 0) return -1;
      if (p->app == NDO_APP_PPR) {
        float pr = rng_uniform(rng);
        if (pr < p->stop_prob) return -1;
      }
      if (n == 1) return edges[0];
      int32_t x = rng_int(rng, n);
      float y = rng_uniform(rng) * max_w;
      c->weight_tries++;
      while (y > weights[x]) {
        x = rng_int(rng, n);
        y = rng_uniform(rng) * max_w;
        c->weight_tries++;
      }
      return edges[x];
    }
    case NDO_APP_NODE2VEC: { /* randomWalks.cu:141-172 */
      if (n == 0) return -1;
      if (n == 1 || step == 0) { *state_t = transit; return edges[0]; }
      const float pp = p->p, qq = p->q;
      float bound = pp > 1.0f / qq ? pp : 1.0f / qq;
      if (bound < 1.0f) bound = 1.0f;
      for (;;) {
        int32_t x = rng_int(rng, n);
        int32_t v = edges[x];
        float y = rng_uniform(rng) * bound;
        const int32_t t = *state_t;
        const int32_t ts = g->row_ptr[t];
        const int32_t tn = g->row_ptr[t + 1] - ts;
        float h;
        c->n2v_tries++;
        int is_ret = p->n2v_ref_compat ? (x == t) : (v == t); /* randomWalks.cu:159 compares the index */
        if (is_ret) h = pp;
        else if (bsearch_i32(g->col + ts, v, tn, &c->n2v_probes)) h = 1.0f / qq;
        else h = 1.0f;
        if (y < h) { *state_t = transit; return v; }
      }
    }
  }
  return -1;
}

/* CSRPartition::has_edge_logn, src/csr.hpp:343-359 */
static int has_edge_logn(const ndo_graph *g, int32_t src, int32_t dst) {
  int32_t l = g->row_ptr[src], r = g->row_ptr[src + 1] - 1;
  while (l <= r) {
    int32_t m = l + (r - l) / 2;
    if (g->col[m] == dst) return 1;
    if (g->col[m] < dst) l = m + 1; else r = m - 1;
  }
  return 0;
}

static int i32_cmp(const void *a, const void *b) {
  int32_t x = *(const int32_t *)a, y = *(const int32_t *)b;
  return x < y ? -1 : (x > y ? 1 : 0);
}

/* semantics of remove_duplicates_in_hop_per_block (src/distinct.cuh:45-111): ascending,
 * equal neighbours dropped, compacted to the front, count returned; tail padded with invalid */
int32_t ndo_distinct(int32_t *seg, int32_t n, int32_t invalid) {
  int32_t m = 0;
  for (int32_t i = 0; i < n; i++) if (seg[i] != invalid && seg[i] != -1) seg[m++] = seg[i];
  qsort(seg, (size_t)m, sizeof(int32_t), i32_cmp);
  int32_t u = 0;
  for (int32_t i = 0; i < m; i++) if (i == 0 || seg[i] != seg[i - 1]) seg[u++] = seg[i];
  for (int32_t i = u; i < n; i++) seg[i] = invalid;
  return u;
}

static void sample_walk(const ndo_graph *g, const ndo_params *p, int64_t gs, int32_t init,
                        int32_t *out, ndo_counters *c) {
  const int32_t INV = g->V;
  int32_t cur = init;
  int32_t state_t = 0;
  for (int step = 0; step < p->steps; step++) {
    int32_t nbr = -1;
    if (cur != INV && cur != -1) {
      c->live_pairs++;
      /* the kernels call next() only when the transit has edges (src/nextdoor.cu:255,412,1143) */
      if (g->row_ptr[cur + 1] - g->row_ptr[cur] != 0) {
        rng_t rng = {p->seed, (uint32_t)gs, (uint32_t)step, 0u, 0u};
        c->next_calls++;
        nbr = walk_next(g, p, step, cur, &state_t, &rng, c);
      }
    }
    if (nbr != -1) { out[step] = nbr; c->sampled_edges++; cur = nbr; }
    else { out[step] = INV; cur = INV; }
  }
}

/* k-hop: hop k expands every slot of hop k-1; child j of parent slot i is written at
 * prefix_k + i*fanout_k + j (the reference assigns racy positions inside [prefix_k, prefix_k+n_k),
 * src/nextdoor.cu:295-305; this layout is one of its legal outcomes).  Draw key slot =
 * i*fanout_k + j. */
static void sample_khop(const ndo_graph *g, const ndo_params *p, int64_t gs, int32_t init,
                        int32_t *out, int32_t *hop_counts, ndo_counters *c) {
  const int32_t INV = g->V;
  int32_t prefix_prev = 0, n_prev = 1, prefix = 0;
  for (int step = 0; step < p->steps; step++) {
    const int32_t k = p->fanout[step];
    for (int32_t i = 0; i < n_prev; i++) {
      const int32_t transit = step == 0 ? init : out[prefix_prev + i];
      int32_t *dst = out + prefix + (int64_t)i * k;
      if (transit == INV || transit == -1) { for (int j = 0; j < k; j++) dst[j] = INV; continue; }
      c->live_pairs++;
      const int32_t rs = g->row_ptr[transit];
      const int32_t n = g->row_ptr[transit + 1] - rs;
      if (n == 0) { for (int j = 0; j < k; j++) dst[j] = INV; continue; }
      if (p->app == NDO_APP_KHOP) { /* khop.cu:18-22: independent draws, with replacement */
        for (int j = 0; j < k; j++) {
          rng_t rng = {p->seed, (uint32_t)gs, (uint32_t)step, (uint32_t)(i * k + j), 0u};
          dst[j] = g->col[rs + rng_int(&rng, n)];
          c->next_calls++; c->sampled_edges++;
        }
      } else { /* without replacement */
        if (n <= k) {
          for (int j = 0; j < k; j++) {
            if (j < n) { dst[j] = g->col[rs + j]; c->sampled_edges++; } else dst[j] = INV;
          }
          c->next_calls += k;
        } else { /* Floyd's algorithm, one keyed draw per slot */
          int32_t picks[64];
          for (int j = 0; j < k; j++) {
            rng_t rng = {p->seed, (uint32_t)gs, (uint32_t)step, (uint32_t)(i * k + j), 0u};
            const int32_t m = n - k + j;
            int32_t t = rng_int(&rng, m + 1);
            for (int q = 0; q < j; q++) if (picks[q] == t) { t = m; break; }
            picks[j] = t;
            dst[j] = g->col[rs + t];
            c->next_calls++; c->sampled_edges++;
          }
        }
      }
    }
    prefix_prev = prefix;
    prefix += n_prev * k;
    n_prev *= k;
  }
  if (p->app == NDO_APP_KHOP_DISTINCT) {
    int32_t off = 0, n = 1;
    for (int step = 0; step < p->steps; step++) {
      n *= p->fanout[step];
      int32_t cnt = ndo_distinct(out + off, n, INV);
      if (hop_counts) hop_counts[step] = cnt;
      off += n;
    }
  }
}

/* collective apps: layer k draws fanout[0] vertices for the whole transit set of the sample.
 * transits of layer 0 = the batch, of layer k = layer k-1's output (src/nextdoor.cu:1402-1411).
 * adjacency entry (i,j) of layer k lives at [k*stride + i*L + j], stride = max(batch,L)*L
 * (fastgcnSampling.cu:32-44 with i over the transits and j the slot). */
static void sample_collective(const ndo_graph *g, const ndo_params *p, int64_t gs,
                              const int32_t *init, int32_t *out, int32_t *adj_row,
                              int32_t *adj_col, float *prob, ndo_counters *c) {
  const int32_t INV = g->V;
  const int32_t L = p->fanout[0];
  const int32_t B = p->batch;
  const int32_t stride = (B > L ? B : L) * L;
  for (int step = 0; step < p->steps; step++) {
    const int32_t *transits = step == 0 ? init : out + (int64_t)(step - 1) * L;
    const int32_t ntr = step == 0 ? B : L;
    int32_t *arow = adj_row ? adj_row + (int64_t)step * stride : NULL;
    int32_t *acol = adj_col ? adj_col + (int64_t)step * stride : NULL;
    int32_t *dst = out + (int64_t)step * L;
    float *pdst = prob ? prob + (int64_t)step * L : NULL;
    if (arow) for (int32_t e = 0; e < stride; e++) { arow[e] = -1; acol[e] = -1; }
    c->live_pairs += ntr;
    if (p->app == NDO_APP_FASTGCN_REF || p->app == NDO_APP_LADIES_REF) {
      for (int32_t j = 0; j < L; j++) {
        rng_t rng = {p->seed, (uint32_t)gs, (uint32_t)step, (uint32_t)j, 0u};
        int32_t id = rng_int(&rng, g->V);
        c->next_calls++; c->sampled_edges++;
        dst[j] = id;
        if (pdst) pdst[j] = 0.0f;
        if (arow) for (int32_t i = 0; i < ntr; i++) {
          int32_t t = transits[i];
          if (t != INV && t != -1 && has_edge_logn(g, t, id)) { arow[i * L + j] = i; acol[i * L + j] = j; }
        }
      }
      continue;
    }
    /* importance sampling over the sorted unique union of the transits' neighbours */
    int64_t tot_deg = 0;
    for (int32_t i = 0; i < ntr; i++) {
      int32_t t = transits[i];
      if (t == INV || t == -1) continue;
      tot_deg += g->row_ptr[t + 1] - g->row_ptr[t];
    }
    c->union_ids += tot_deg;
    int32_t *cand = (int32_t *)malloc(sizeof(int32_t) * (size_t)(tot_deg > 0 ? tot_deg : 1));
    int64_t m = 0;
    for (int32_t i = 0; i < ntr; i++) {
      int32_t t = transits[i];
      if (t == INV || t == -1) continue;
      for (int32_t e = g->row_ptr[t]; e < g->row_ptr[t + 1]; e++) cand[m++] = g->col[e];
    }
    qsort(cand, (size_t)m, sizeof(int32_t), i32_cmp);
    int64_t U = 0;
    for (int64_t i = 0; i < m; i++) if (i == 0 || cand[i] != cand[i - 1]) cand[U++] = cand[i];
    c->union_unique += U;
    float *wt = (float *)calloc((size_t)(U > 0 ? U : 1), sizeof(float));
    double *cdf = (double *)malloc(sizeof(double) * (size_t)(U > 0 ? U : 1));
    if (p->app == NDO_APP_FASTGCN_IS) {
      for (int64_t u = 0; u < U; u++) {
        float d = (float)(g->row_ptr[cand[u] + 1] - g->row_ptr[cand[u]]);
        wt[u] = d * d;
      }
    } else {
      for (int32_t i = 0; i < ntr; i++) {
        int32_t t = transits[i];
        if (t == INV || t == -1) continue;
        double rowsum_d = 0.0; /* summed in fp64 so that the order of the adds does not matter */
        for (int32_t e = g->row_ptr[t]; e < g->row_ptr[t + 1]; e++) rowsum_d += (double)g->w[e];
        const float rowsum = (float)rowsum_d;
        for (int32_t e = g->row_ptr[t]; e < g->row_ptr[t + 1]; e++) {
          int32_t v = g->col[e];
          int64_t lo = 0, hi = U - 1, pos = -1;
          while (lo <= hi) { int64_t mid = lo + (hi - lo) / 2; if (cand[mid] == v) { pos = mid; break; } if (cand[mid] < v) lo = mid + 1; else hi = mid - 1; }
          float r = g->w[e] / rowsum;
          wt[pos] = wt[pos] + r * r;
        }
      }
    }
    /* the CDF is accumulated in fp64: sums of fp32 weights then agree between any two orders
     * of addition to ~1e-16, far inside the 1e-5 the probabilities are held to */
    double run = 0.0;
    for (int64_t u = 0; u < U; u++) { run += (double)wt[u]; cdf[u] = run; }
    const double total = U > 0 ? cdf[U - 1] : 0.0;
    for (int32_t j = 0; j < L; j++) {
      if (U == 0 || !(total > 0.0)) { dst[j] = INV; if (pdst) pdst[j] = 0.0f; continue; }
      rng_t rng = {p->seed, (uint32_t)gs, (uint32_t)step, (uint32_t)j, 0u};
      double target = (double)rng_uniform(&rng) * total;
      int64_t lo = 0, hi = U - 1; /* first index with cdf >= target */
      while (lo < hi) { int64_t mid = lo + (hi - lo) / 2; if (cdf[mid] >= target) hi = mid; else lo = mid + 1; }
      dst[j] = cand[lo];
      if (pdst) pdst[j] = (float)((double)wt[lo] / total);
      c->next_calls++; c->sampled_edges++;
      if (arow) for (int32_t i = 0; i < ntr; i++) {
        int32_t t = transits[i];
        if (t != INV && t != -1 && has_edge_logn(g, t, cand[lo])) { arow[i * L + j] = i; acol[i * L + j] = j; }
      }
    }
    free(cand); free(wt); free(cdf);
  }
}

static void ctr_add(ndo_counters *a, const ndo_counters *b) {
  a->sampled_edges += b->sampled_edges; a->next_calls += b->next_calls;
  a->weight_tries += b->weight_tries; a->n2v_tries += b->n2v_tries;
  a->n2v_probes += b->n2v_probes; a->live_pairs += b->live_pairs;
  a->union_ids += b->union_ids; a->union_unique += b->union_unique;
}

int ndo_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

int ndo_sample(const ndo_graph *g, const ndo_params *p, int64_t S, int64_t first_sample,
               const int32_t *initial, int32_t *out, int32_t *adj_row, int32_t *adj_col,
               float *prob, int32_t *hop_counts, ndo_counters *ctr, int threads) {
  const int32_t fs = ndo_final_sample_size(p);
  const int32_t is = ndo_initial_sample_size(p);
  ndo_counters total;
  memset(&total, 0, sizeof(total));
  if (is_khop(p->app)) for (int k = 0; k < p->steps; k++) if (p->fanout[k] > 64 || p->fanout[k] < 1) return -1;
  const int32_t L = p->fanout[0], B = p->batch;
  const int64_t astride = is_collective(p->app) ? (int64_t)p->steps * (B > L ? B : L) * L : 0;
#ifdef _OPENMP
  if (threads <= 0) threads = omp_get_max_threads();
#else
  threads = 1;
#endif
#pragma omp parallel num_threads(threads)
  {
    ndo_counters c;
    memset(&c, 0, sizeof(c));
#pragma omp for schedule(dynamic, 256)
    for (int64_t s = 0; s < S; s++) {
      const int64_t gs = first_sample + s;
      int32_t *o = out + s * fs;
      if (is_walk(p->app)) sample_walk(g, p, gs, initial[s], o, &c);
      else if (is_khop(p->app)) sample_khop(g, p, gs, initial[s], o, hop_counts ? hop_counts + s * p->steps : NULL, &c);
      else sample_collective(g, p, gs, initial + s * is, o, adj_row ? adj_row + s * astride : NULL,
                             adj_col ? adj_col + s * astride : NULL, prob ? prob + s * fs : NULL, &c);
    }
#pragma omp critical
    ctr_add(&total, &c);
  }
  if (ctr) *ctr = total;
  return 0;
}

/* ------------------------------------------------------------------ map inversion */

/* what cub::DeviceRadixSort::SortPairs does at src/nextdoor.cu:2930-2933 (stable, by transit),
 * with the dead pairs (key == invalid, which the reference sorts last and skips via
 * invalidVertexStartPos, :1804-1836) dropped. */
int64_t ndo_invert_map(int64_t n, const int32_t *keys, const int32_t *vals, int32_t invalid,
                       int32_t *keys_out, int32_t *vals_out) {
  int64_t *cnt = (int64_t *)calloc((size_t)invalid + 1, sizeof(int64_t));
  for (int64_t i = 0; i < n; i++) if (keys[i] != invalid && keys[i] >= 0) cnt[keys[i] + 1]++;
  for (int32_t v = 0; v < invalid; v++) cnt[v + 1] += cnt[v];
  int64_t live = cnt[invalid];
  for (int64_t i = 0; i < n; i++) {
    if (keys[i] == invalid || keys[i] < 0) continue;
    int64_t pos = cnt[keys[i]]++;
    keys_out[pos] = keys[i]; vals_out[pos] = vals[i];
  }
  free(cnt);
  return live;
}

/* ------------------------------------------------------------------ validators */

/* checkSampledVerticesResult (src/check_results.cu:162-299): every vertex of step k is adjacent
 * to some vertex of step k-1 of the same sample, and a step is not empty when the previous
 * step had neighbours to offer.  All steps are checked (the reference stops after 4). */
int64_t ndo_check_sampled_vertices(const ndo_graph *g, const ndo_params *p, int64_t S,
                                   const int32_t *initial, const int32_t *out) {
  const int32_t INV = g->V;
  const int32_t fs = ndo_final_sample_size(p);
  int64_t bad = 0;
  if (is_collective(p->app)) return -1;
#pragma omp parallel for reduction(+ : bad) schedule(dynamic, 256)
  for (int64_t s = 0; s < S; s++) {
    const int32_t *o = out + s * fs;
    int32_t prev_off = 0, prev_n = 1, off = 0;
    for (int step = 0; step < p->steps; step++) {
      const int32_t k = is_walk(p->app) ? 1 : p->fanout[step];
      const int32_t n = prev_n * k;
      int64_t offered = 0, got = 0;
      for (int32_t i = 0; i < prev_n; i++) {
        int32_t t = step == 0 ? initial[s] : o[prev_off + i];
        if (t != INV) offered += g->row_ptr[t + 1] - g->row_ptr[t];
      }
      for (int32_t j = 0; j < n; j++) {
        int32_t v = o[off + j];
        if (v == INV) continue;
        got++;
        if (v < 0 || v > INV) { bad++; continue; }
        int found = 0;
        for (int32_t i = 0; i < prev_n && !found; i++) {
          int32_t t = step == 0 ? initial[s] : o[prev_off + i];
          if (t != INV && has_edge_logn(g, t, v)) found = 1;
        }
        if (!found) bad++;
      }
      /* PPR may stop a walk by choice and distinct may shrink a hop: emptiness is only an
       * error for the apps that must sample when they can */
      if (got == 0 && offered > 0 && p->app != NDO_APP_PPR) bad++;
      prev_off = off; prev_n = n; off += n;
    }
  }
  return bad;
}

/* checkAdjacencyMatrixResult (src/check_results.cu:46-160): (1) every recorded (row,col) is an
 * edge of the graph; (2) every graph edge between a transit and a sampled vertex is recorded. */
int64_t ndo_check_adjacency(const ndo_graph *g, const ndo_params *p, int64_t S,
                            const int32_t *initial, const int32_t *out, const int32_t *adj_row,
                            const int32_t *adj_col) {
  const int32_t INV = g->V;
  const int32_t fs = ndo_final_sample_size(p);
  const int32_t L = p->fanout[0], B = p->batch;
  const int32_t stride = (B > L ? B : L) * L;
  int64_t bad = 0;
  for (int64_t s = 0; s < S; s++) {
    for (int step = 0; step < p->steps; step++) {
      const int32_t *tr = step == 0 ? initial + s * B : out + s * fs + (int64_t)(step - 1) * L;
      const int32_t ntr = step == 0 ? B : L;
      const int32_t *lay = out + s * fs + (int64_t)step * L;
      const int32_t *ar = adj_row + (s * p->steps + step) * (int64_t)stride;
      const int32_t *ac = adj_col + (s * p->steps + step) * (int64_t)stride;
      for (int32_t i = 0; i < ntr; i++) for (int32_t j = 0; j < L; j++) {
        int rec = ar[i * L + j] != -1 || ac[i * L + j] != -1;
        int edge = tr[i] != INV && lay[j] != INV && has_edge_logn(g, tr[i], lay[j]);
        if (rec && (ar[i * L + j] != i || ac[i * L + j] != j)) bad++;
        if (rec != edge) bad++;
      }
    }
  }
  return bad;
}
