// Shared declarations of the sm_100a sampling library: error plumbing, the device-resident
// graph and sampler records, and the launch geometry every kernel file uses.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <string>
#include <vector>

#include "../../include/nextdoor_b200.h"

// ---------------------------------------------------------------- errors

void nd_set_error(const char *fmt, ...);
void nd_count_launches(int n);  // bookkeeping behind nd_launch_count()

#define ND_CUDA(call)                                                                      \
  do {                                                                                     \
    cudaError_t e__ = (call);                                                              \
    if (e__ != cudaSuccess) {                                                              \
      nd_set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__), __FILE__, __LINE__); \
      return ND_ERR_CUDA;                                                                  \
    }                                                                                      \
  } while (0)

#define ND_TRY(call)             \
  do {                           \
    int s__ = (call);            \
    if (s__ != ND_OK) return s__; \
  } while (0)

#define ND_REQUIRE(cond, code, ...) \
  do {                              \
    if (!(cond)) {                  \
      nd_set_error(__VA_ARGS__);    \
      return (code);                \
    }                               \
  } while (0)

// bits of the device status word (a kernel ORs a bit in and carries on with bounded work)
enum : int {
  ND_DEV_BAD_TRANSIT = 1,   // a transit id outside [0, V)
  ND_DEV_WAIT_TIMEOUT = 2,  // a bounded mbarrier / flag wait gave up
  ND_DEV_OVERFLOW = 4,      // a work list or candidate buffer would overflow
  ND_DEV_RETRY_LIMIT = 8    // a rejection loop hit its iteration cap
};

// ---------------------------------------------------------------- device info

struct NdDeviceInfo {
  int device = -1;
  int sms = 0;
  int smem_optin = 0;
};
int nd_device_info(int device, NdDeviceInfo *info);

// ---------------------------------------------------------------- graph replica (SoA in HBM)
//
// row_ptr[V+1] int32 exclusive ends (the reference's 16-byte AoS vertex record, src/csr.hpp:49-79,
// becomes 8 bytes of row offsets + 4 bytes of max weight), col[E] int32 sorted per row by
// (neighbour, weight), w[E] fp32.

struct nd_graph {
  int device = 0;
  int32_t V = 0;
  int64_t E = 0;
  int32_t max_degree = 0;
  int32_t *row_ptr = nullptr;
  int32_t *col = nullptr;
  float *w = nullptr;
  float *max_w = nullptr;
  // Derived layouts, built on the first sampler that needs them and shared by all samplers of the graph:
  mutable int2 *colw = nullptr;        // [E] (neighbour id, weight bits) records: one 8-byte gather per weighted try
  mutable int2 *vrec = nullptr;        // [V+1] (row start, max weight bits) per vertex: what a thread-per-walk kernel needs of a vertex in one sector
  mutable int32_t *adjset = nullptr;   // node2vec membership: per-vertex hash sets of the neighbour ids, 8-slot buckets
};

struct NdGraphView {
  int32_t V;
  const int32_t *__restrict__ row_ptr;
  const int32_t *__restrict__ col;
  const float *__restrict__ w;
  const float *__restrict__ max_w;
};

static inline NdGraphView nd_view(const nd_graph *g) {
  return NdGraphView{g->V, g->row_ptr, g->col, g->w, g->max_w};
}

// ---------------------------------------------------------------- radix sort (map inversion, CSR build)

struct NdRadixPlan {
  int key_bits = 0;     // significant bits of the key
  int passes = 0;
  int bits[8] = {0};    // digit width per pass (LSD first)
  int shift[8] = {0};
  int max_bins = 0;
  int tile = 0;         // pairs per tile
  int64_t max_n = 0;
  int64_t max_tiles = 0;
};

struct NdRadixScratch {
  NdRadixPlan plan;
  uint32_t *tile_hist = nullptr;  // [max_bins][max_tiles]
  uint32_t *ghist = nullptr;      // [8][cap_bins]
  int cap_bins = 0;
  size_t bytes = 0;
};

NdRadixPlan nd_radix_plan(int key_bits, int64_t max_n);
int nd_radix_scratch_alloc(NdRadixScratch *s, int key_bits, int64_t max_n);
void nd_radix_scratch_free(NdRadixScratch *s);

// Sorts NW parallel 32-bit arrays by word `key_word` (stable, LSD, bits [0,key_bits)).  n is read
// from *d_n on the device.  Pairs whose key equals `drop_key` are dropped in the first pass when
// drop_enable; *d_n_out receives the surviving count.  If first_hist_done, the tile histogram of
// pass 0 over buf_a was already produced (fused into the producer kernel).  The sorted result
// lands in result (== a or b, reported through *result_in_b).
struct NdSortArrays {
  uint32_t *a[3];
  uint32_t *b[3];
  int nwords;
};
int nd_radix_sort(const NdDeviceInfo &dev, cudaStream_t st, NdRadixScratch *scr, const NdRadixPlan &pl,
                  NdSortArrays arr, int key_word, const int32_t *d_n, int32_t *d_n_out, bool drop_enable,
                  uint32_t drop_key, bool first_hist_done, bool *result_in_b);

// geometry shared with producers that fuse the first tile histogram
static constexpr int ND_RADIX_THREADS = 256;

// ---------------------------------------------------------------- sampler

struct NdPhaseTimer {
  bool on = false;
  std::vector<cudaEvent_t> ev;        // pairs
  std::vector<int> phase_of_pair;
  float ms[ND_PHASE_COUNT] = {0};
  int launches[ND_PHASE_COUNT] = {0};
};

struct NdHostRows;   // state of the sparse result update of a caller's host array (nd_hostrows.cu)

struct nd_sampler {
  const nd_graph *g = nullptr;
  NdDeviceInfo dev;
  nd_app_params p;
  int64_t S = 0;       // samples of this shard
  int64_t first = 0;   // global index of sample 0 of the shard
  int32_t fs = 0;      // final sample size
  int32_t isz = 0;     // initial sample size
  cudaStream_t stream = nullptr;
  bool sampled = false;

  int32_t *d_initial = nullptr;   // [S*isz]
  int32_t *d_out = nullptr;       // [S*fs] final samples, sample-major (src/nextdoor.cu:2041)
  // walks
  int32_t *d_tmp = nullptr;       // [steps][S] step-major staging of the walk output
  int32_t *d_len = nullptr;       // [S] number of valid steps of each walk
  int32_t *d_plen = nullptr;      // [S] walks: leading slots of the sample's row in d_out that may hold a vertex (the rest is invalid)
  int32_t *d_state = nullptr;     // [S] per-sample app state (node2vec: previous vertex)
  // transit maps (ping-pong); key = transit, val = pair id
  int32_t *d_map_key[2] = {nullptr, nullptr};
  int32_t *d_map_val[2] = {nullptr, nullptr};
  int32_t *d_init_key = nullptr;  // initial map, sorted by transit once
  int32_t *d_init_val = nullptr;
  int64_t map_cap = 0;
  int32_t *d_nlive = nullptr;     // [steps+2] live pairs entering each step
  unsigned long long *d_stats = nullptr;  // [8]
  int *d_status = nullptr;
  NdRadixScratch radix;
  // counting inversion of the walk maps: per-vertex counters, their exclusive scan, chunk sums, ranks
  uint32_t *d_cnt = nullptr, *d_offs = nullptr, *d_bsum = nullptr;
  int32_t *d_rank = nullptr;
  // load-balanced walk loop: the transit-sorted map as records (8 bytes, node2vec 32 bytes), ping-pong,
  // the initial map in the same form, and (node2vec) what next() hands to the scatter per pair
  void *d_srec[2] = {nullptr, nullptr};
  void *d_init_rec = nullptr;
  int4 *d_uext = nullptr;
  // the step loop of a walk job captured once per mode and replayed (needs a non-default stream)
  cudaGraphExec_t graph_exec[3] = {nullptr, nullptr, nullptr};
  int graph_launches[3] = {0, 0, 0};
  bool graph_off = false;
  // PPR, load-balanced mode: the tail launch runs on this stream beside the result update of the walks that ended
  cudaStream_t side = nullptr;
  cudaEvent_t side_fork = nullptr, side_join = nullptr;
  // ... and the number of walks whose start vertex has neighbours, counted when the seeds are set (pinned word + event):
  // the hand-over to the tail launch is placed by the pairs the maps will really hold
  int32_t *h_active = nullptr;
  cudaEvent_t active_done = nullptr;
  int64_t active_starts = -1;   // -1: not read yet
  cudaEvent_t copy_event = nullptr;  // orders a result copy on another stream after the sampling
  cudaEvent_t copy_done = nullptr;   // ... and the next sampling (which overwrites the result) after that copy
  bool copy_pending = false;
  // k-hop LB bins
  int32_t *d_runs = nullptr;      // work lists
  int64_t runs_cap = 0;
  int32_t *d_bin_counts = nullptr;
  int32_t *d_hop_counts = nullptr;
  // collective
  int32_t *d_adj_row = nullptr, *d_adj_col = nullptr;
  float *d_prob = nullptr;
  int32_t *d_cand = nullptr;
  float *d_cand_w = nullptr;
  int64_t cand_cap = 0;
  bool coll_bitmap = false;       // importance sampling through the shared-memory bitmap kernel
  int coll_grid = 0;
  double *d_acc = nullptr;        // LADIES: per-CTA accumulators of the candidates' weights
  unsigned char *d_bm = nullptr;  // per-CTA bitmap slices when a bit per vertex does not fit shared memory

  NdHostRows *hostrows = nullptr;

  NdPhaseTimer timer;
  int64_t host_stats[8] = {0};
};
void nd_hostrows_free(nd_sampler *s);

// phase timing helpers (no-ops unless profiling is on)
void nd_phase_begin(nd_sampler *s, int phase);
void nd_phase_end(nd_sampler *s);

// ---------------------------------------------------------------- per-family entry points
int nd_graph_ensure_colw(const nd_graph *g, int sms);
int nd_walk_step_packed_launch(const nd_graph *g, const nd_app_params *p, int step, int64_t n, const uint64_t *d_in,
                               uint64_t *d_out, cudaStream_t st);
int nd_walk_step_launch(const nd_graph *g, const nd_app_params *p, int step, int64_t n, const int32_t *d_transits,
                        const int64_t *d_samples, int32_t *d_next, cudaStream_t st);

int nd_walk_step_status_read(cudaStream_t st, int *status);

int nd_walk_alloc(nd_sampler *s);
int nd_walk_sample(nd_sampler *s, int mode);
int nd_khop_alloc(nd_sampler *s);
int nd_khop_sample(nd_sampler *s, int mode);
int nd_collective_alloc(nd_sampler *s);
int nd_collective_sample(nd_sampler *s, int mode);
const char *nd_collective_kernel_name(const nd_sampler *s);  // union path of the importance samplers
int nd_sampler_build_initial_map(nd_sampler *s);

int nd_graph_finish(nd_graph *g, cudaStream_t st);  // max_w (if null) + max_degree
int nd_distinct_launch(cudaStream_t st, int32_t *data, int64_t n_segments, int32_t seg_len,
                       int32_t seg_stride, int32_t invalid, int32_t *counts, int32_t counts_stride);

static inline bool nd_is_walk(int app) { return app >= ND_APP_UNIFORM_WALK && app <= ND_APP_NODE2VEC; }
static inline bool nd_is_khop(int app) { return app == ND_APP_KHOP || app == ND_APP_KHOP_DISTINCT; }
static inline bool nd_is_collective(int app) { return app >= ND_APP_FASTGCN_REF && app <= ND_APP_LADIES_IS; }

static inline int nd_bit_length(uint32_t x) {
  int b = 0;
  while (x) { b++; x >>= 1; }
  return b;
}
