/*
 * nd_oracle.h -- CPU oracle for the NextDoor sampling path.  TEST INFRASTRUCTURE ONLY.
 *
 * This is a plain-C restatement of the sampling semantics of the reference
 * (plasma-umass/NextDoor).  Each function cites the reference file:line it follows.
 * It exists to check the CUDA library; nothing that ships may link it, call it or fall
 * back to it.  Only tests, the smoke check and the CPU-baseline leg of the benchmark
 * load this library.
 *
 * Parity status: the reference holds no golden vectors or seeds for this path (its tests
 * are property checks on external graph files), so exact values are pinned in two ways:
 *   (1) Philox4x32-10 against the published known-answer vectors of the algorithm;
 *   (2) every app body against the reference's own next() source, compiled for the host
 *       through a shim (oracle/ref_shim, output oracle/_ref), fed the same keyed draws.
 * The apps the reference does not implement (k-hop without replacement + distinct,
 * FastGCN/LADIES importance sampling, PPR with a configurable stop probability) are defined
 * here and nowhere else: parity unpinned for those three.
 */
#ifndef ND_ORACLE_H
#define ND_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* App ids (shared numbering with the CUDA library's nd_app enum). */
enum {
  NDO_APP_UNIFORM_WALK = 0, /* example/uniformRandWalk.cu:27-37 */
  NDO_APP_DEEPWALK = 1,     /* src/apps/randomwalks/randomWalks.cu:65-91 */
  NDO_APP_PPR = 2,          /* src/apps/randomwalks/randomWalks.cu:93-125 */
  NDO_APP_NODE2VEC = 3,     /* src/apps/randomwalks/randomWalks.cu:132-173 */
  NDO_APP_KHOP = 4,         /* src/apps/khop/khop.cu:10-23 (with replacement) */
  NDO_APP_KHOP_DISTINCT = 5,/* extension: without replacement, then per-hop distinct */
  NDO_APP_FASTGCN_REF = 6,  /* src/apps/fastgcn/fastgcnSampling.cu:23-47 */
  NDO_APP_LADIES_REF = 7,   /* src/apps/ladies/ladiessampling.cu:23-47 (same code) */
  NDO_APP_FASTGCN_IS = 8,   /* extension: importance ~ degree^2 over the neighbour union */
  NDO_APP_LADIES_IS = 9     /* extension: importance ~ sum of squared row-normalised weights */
};

#define NDO_MAX_STEPS_FANOUT 8

typedef struct ndo_params {
  int32_t app;
  int32_t steps;               /* walks: walk length; k-hop: hops; collective: layers */
  int32_t fanout[NDO_MAX_STEPS_FANOUT]; /* k-hop stepSize per hop; collective: layer size in [0] */
  int32_t batch;               /* collective: transits per sample (initialSampleSize) */
  int32_t n2v_ref_compat;      /* node2vec: 1 = compare edge index with t (reference quirk) */
  float p, q;                  /* node2vec */
  float stop_prob;             /* PPR */
  uint64_t seed;               /* Philox key */
} ndo_params;

typedef struct ndo_graph {
  int32_t V;
  int64_t E;
  const int32_t *row_ptr; /* V+1, exclusive end */
  const int32_t *col;
  const float *w;
  const float *max_w; /* per vertex: max(0, max weight), src/graph.hpp:71-80 */
} ndo_graph;

/* event counters from which the algorithmic-bytes model is evaluated */
typedef struct ndo_counters {
  int64_t sampled_edges; /* valid vertices written */
  int64_t next_calls;    /* (pair,slot) evaluations with a live transit */
  int64_t weight_tries;  /* rejection tries that read a weight */
  int64_t n2v_tries;     /* node2vec tries */
  int64_t n2v_probes;    /* binary-search probes */
  int64_t live_pairs;    /* sum over steps of live (transit,sample) pairs */
  int64_t union_ids;     /* collective: sum of degrees copied */
  int64_t union_unique;  /* collective: candidate-set sizes */
} ndo_counters;

/* --- RNG --- */
void ndo_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]);
uint32_t ndo_draw_u32(uint64_t seed, uint32_t sample, uint32_t step, uint32_t slot, uint32_t draw);
float ndo_u32_to_uniform(uint32_t x);
float ndo_uniform(uint64_t seed, uint32_t sample, uint32_t step, uint32_t slot, uint32_t draw);
int32_t ndo_rand_int(float u, int32_t n);

/* --- synthetic graph + CSR build --- */
/* writes 2*M directed records (both directions of every undirected edge) */
void ndo_rmat_records(int32_t V, int64_t M, uint64_t seed, int32_t *src, int32_t *dst, float *w);
/* sorts by (src,dst,w) and builds exclusive row_ptr; n_vertices = max id + 1 if V<=0 */
int32_t ndo_csr_from_records(int64_t n, const int32_t *src, const int32_t *dst, const float *w,
                             int32_t V, int32_t *row_ptr, int32_t *col, float *wout, float *max_w);
void ndo_partition(int32_t V, const int32_t *row_ptr, int64_t budget_bytes, int32_t max_parts,
                   int32_t *first_v, int32_t *last_v, int64_t *first_e, int64_t *last_e,
                   int32_t *n_parts);

/* --- sampling --- */
int32_t ndo_final_sample_size(const ndo_params *p);
int32_t ndo_initial_sample_size(const ndo_params *p);
/*
 * Samples [first_sample, first_sample+S).  initial: S*initialSampleSize transits.
 * out: S*finalSampleSize.  Collective apps: adj_row/adj_col are S*steps*batch*layer ints,
 * prob (importance apps) S*finalSampleSize floats; pass NULL when not applicable.
 * hop_counts (KHOP_DISTINCT): S*steps ints.
 */
int ndo_sample(const ndo_graph *g, const ndo_params *p, int64_t S, int64_t first_sample,
               const int32_t *initial, int32_t *out, int32_t *adj_row, int32_t *adj_col,
               float *prob, int32_t *hop_counts, ndo_counters *ctr, int threads);

/* map inversion: stable sort of (key,val) by key; keys == invalid are dropped. returns live count */
int64_t ndo_invert_map(int64_t n, const int32_t *keys, const int32_t *vals, int32_t invalid,
                       int32_t *keys_out, int32_t *vals_out);
/* per-segment ascending unique; returns count, pads with invalid */
int32_t ndo_distinct(int32_t *seg, int32_t n, int32_t invalid);

/* validators, restated from src/check_results.cu:162-299: returns number of violations */
int64_t ndo_check_sampled_vertices(const ndo_graph *g, const ndo_params *p, int64_t S,
                                   const int32_t *initial, const int32_t *out);
int64_t ndo_check_adjacency(const ndo_graph *g, const ndo_params *p, int64_t S,
                            const int32_t *initial, const int32_t *out, const int32_t *adj_row,
                            const int32_t *adj_col);
int ndo_max_threads(void);

#ifdef __cplusplus
}
#endif
#endif
