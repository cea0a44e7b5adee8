/*
 * nextdoor_b200.h -- C ABI of the B200-native NextDoor sampling engine (libnextdoor_b200.so).
 *
 * Plain pointers and sizes only.  Every function returns an nd_status (0 = ND_OK); the text of
 * the last failure on the calling thread is available through nd_last_error().  The library
 * never aborts and has no CPU fallback: without a CUDA device every compute call fails with
 * ND_ERR_CUDA.
 *
 * Each entry point names the piece of the reference (plasma-umass/NextDoor, paths relative to
 * its tree) that it replaces.
 */
#ifndef NEXTDOOR_B200_H
#define NEXTDOOR_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum nd_status {
  ND_OK = 0,
  ND_ERR_ARG = 1,     /* bad argument (null pointer, size out of range, unknown app) */
  ND_ERR_CUDA = 2,    /* a CUDA runtime call failed */
  ND_ERR_IO = 3,      /* file not found / short read */
  ND_ERR_RANGE = 4,   /* vertex or edge count does not fit int32 (src/csr.hpp:6-8) */
  ND_ERR_DEVICE = 5,  /* a kernel reported a problem through the device status word */
  ND_ERR_STATE = 6    /* call order violated (e.g. final samples before sample) */
} nd_status;

/* Built-in applications: the App structs of the reference, same sampling rule each. */
typedef enum nd_app {
  ND_APP_UNIFORM_WALK = 0,  /* UniformRandomWalkApp, example/uniformRandWalk.cu:15-93 */
  ND_APP_DEEPWALK = 1,      /* DeepWalkApp, src/apps/randomwalks/randomWalks.cu:65-91 */
  ND_APP_PPR = 2,           /* PPRApp, src/apps/randomwalks/randomWalks.cu:93-125 */
  ND_APP_NODE2VEC = 3,      /* Node2VecApp, src/apps/randomwalks/randomWalks.cu:132-173 */
  ND_APP_KHOP = 4,          /* KHopApp, src/apps/khop/khop.cu:1-77 (with replacement) */
  ND_APP_KHOP_DISTINCT = 5, /* no counterpart: without replacement, then distinct per hop
                               (semantics of src/distinct.cuh:45-111) */
  ND_APP_FASTGCN_REF = 6,   /* FastGCNSamplingApp, src/apps/fastgcn/fastgcnSampling.cu:15-100 */
  ND_APP_LADIES_REF = 7,    /* ImportanceSampleApp, src/apps/ladies/ladiessampling.cu:15-100 */
  ND_APP_FASTGCN_IS = 8,    /* no counterpart: importance ~ degree^2 over the neighbour union */
  ND_APP_LADIES_IS = 9      /* no counterpart: importance ~ sum of squared row-normalised weights */
} nd_app;

/* kernelType + load-balancing flag of nextdoor<>() (src/nextdoor.cu:3239-3243, src/main.cu:21-29) */
typedef enum nd_mode {
  ND_MODE_TRANSIT_PARALLEL = 0,    /* "TransitParallel", -l off: no bins */
  ND_MODE_TRANSIT_PARALLEL_LB = 1, /* "TransitParallel", -l on: sub-warp / block / grid bins */
  ND_MODE_SAMPLE_PARALLEL = 2      /* "SampleParallel" (what the Python sample() runs) */
} nd_mode;

#define ND_MAX_STEPS_FANOUT 8

/* The compile-time constants of the reference's App structs, as run-time parameters. */
typedef struct nd_app_params {
  int32_t app;     /* nd_app */
  int32_t steps;   /* App::steps(): walk length / hops / layers */
  int32_t fanout[ND_MAX_STEPS_FANOUT]; /* App::stepSize(k) for k-hop; layer size in [0] for collective apps */
  int32_t batch;   /* App::initialSampleSize() of the collective apps (VERTICES_PER_SAMPLE) */
  int32_t n2v_ref_compat; /* 1: keep the index-vs-vertex comparison of randomWalks.cu:159; 0: compare vertices */
  float p, q;      /* node2vec (randomWalks.cu:149-150) */
  float stop_prob; /* PPR walkEndProb (randomWalks.cu:105) */
  uint64_t seed;   /* Philox key; draws are keyed by (seed, global sample index, step, slot, draw) */
} nd_app_params;

typedef struct nd_graph nd_graph;     /* CSR replica resident on one device */
typedef struct nd_sampler nd_sampler; /* NextDoorData<SampleType,App> of one device (src/libNextDoor.hpp:13-37) */

const char *nd_last_error(void);
int nd_version(void);
/* number of CUDA devices visible, 0 when there is none (never fails) */
int nd_device_count(void);
/* kernels launched by the library in this process so far (all devices, all handles) */
int64_t nd_launch_count(void);

/* ------------------------------------------------------------------ graph */

/* transferCSRToGPUs / copyPartitionToGPU (src/nextdoor.cu:1893-1911, src/utils.hpp:378-395):
 * upload a host CSR.  row_ptr has V+1 entries with exclusive ends; max_w may be NULL (computed
 * on the device as Vertex::max_weight does, src/graph.hpp:71-80). */
int nd_graph_from_csr(int device, int32_t V, int64_t E, const int32_t *row_ptr, const int32_t *col,
                      const float *w, const float *max_w, nd_graph **out);
/* Graph::load_from_edge_list_binary + csr_from_graph (src/graph.hpp:106-159, src/csr.hpp:399-424),
 * done on the device: n 12-byte records {int32 src, int32 dst, float32 w} in host memory are
 * sorted by (src, dst, w) with the library's radix sort; vertex count = max id + 1; duplicates kept. */
int nd_graph_from_edge_records(int device, int64_t n, const void *records, nd_graph **out);
/* loadGraph(file, "edge-list", "binary") (src/nextdoor.cu:1845-1891) */
int nd_graph_load_edge_list_binary(int device, const char *path, nd_graph **out);
/* loadGraph(file, type, format) with all three formats of the reference (src/nextdoor.cu:1845-1891):
 * ("edge-list","binary"), ("edge-list","text") (src/graph.hpp:162-254: topology only, weights are
 * stored as 0 as the reference does) and ("adj-list","text") (src/graph.hpp:256-326: vertices
 * renumbered by line).  Parsing is on the host, the CSR is built on the device. */
int nd_graph_load(int device, const char *path, const char *graph_type, const char *graph_format, nd_graph **out);
/* Synthetic R-MAT graph (a,b,c,d)=(.57,.19,.19,.05) generated and built on the device: M
 * undirected edges, both directions stored, weights uniform [1,5).  Stands in for the graph
 * files the reference's tests read (src/tests/testBase.h:6-12). */
int nd_graph_rmat(int device, int32_t V, int64_t M, uint64_t seed, nd_graph **out);
int nd_graph_info(const nd_graph *g, int32_t *V, int64_t *E, int32_t *max_degree, int *device);
/* copies to host buffers; any pointer may be NULL */
int nd_graph_to_host(const nd_graph *g, int32_t *row_ptr, int32_t *col, float *w, float *max_w);
/* device addresses of the replica (GPUCSRPartition, src/csr.hpp:387-393) */
int nd_graph_device_ptrs(const nd_graph *g, const int32_t **row_ptr, const int32_t **col,
                         const float **w, const float **max_w);
int nd_graph_destroy(nd_graph *g);
/* create_csr_partitions (src/graph_partitioner.cuh:1-173): contiguous vertex ranges under a byte
 * budget (16 B per vertex record, 4 B per edge); boundaries are found on the device. */
int nd_graph_partition(const nd_graph *g, int64_t budget_bytes, int32_t max_parts, int32_t *first_v,
                       int32_t *last_v, int64_t *first_e, int64_t *last_e, int32_t *n_parts);

/* ------------------------------------------------------------------ sampler */

/* App::steps/stepSize folded as getFinalSampleSize (src/nextdoor.cu:1913-1929) */
int nd_final_sample_size(const nd_app_params *p);
int nd_initial_sample_size(const nd_app_params *p);
/* PartStartPointer / PartDivisionSize (src/utils.hpp:26-27): samples of part `idx` of `parts` */
int nd_shard_range(int64_t total, int idx, int parts, int64_t *first, int64_t *count);

/* allocNextDoorDataOnGPU (src/nextdoor.cu:1931-2086) for this device's shard: samples
 * [first_sample, first_sample + num_samples) of the job.  `initial` (host, num_samples *
 * initialSampleSize transits) may be NULL: then App::initialSample of the reference app is used
 * (sample i starts at vertex i % V; collective batches take consecutive ids). */
int nd_sampler_create(const nd_graph *g, const nd_app_params *p, int64_t num_samples,
                      int64_t first_sample, const int32_t *initial, nd_sampler **out);
/* replaces the initial transits (host pointer) without reallocating: one H2D copy + map set-up */
int nd_sampler_set_initial(nd_sampler *s, const int32_t *initial);
/* run on the caller's stream (a cudaStream_t); NULL = the legacy default stream */
int nd_sampler_set_stream(nd_sampler *s, void *stream);
/* doTransitParallelSampling / doSampleParallelSampling (src/nextdoor.cu:2191-3006, 3009-3209).
 * Asynchronous on the sampler's stream. */
int nd_sampler_sample(nd_sampler *s, int mode);
/* waits for the stream, checks the device status word */
int nd_sampler_sync(nd_sampler *s);
/* getFinalSamples (src/nextdoor.cu:3211-3237): D2H into `out` (num_samples * finalSampleSize) */
int nd_sampler_final_samples(nd_sampler *s, int32_t *out);
/* same copy, enqueued without waiting: on `copy_stream` (a cudaStream_t) after the sampling issued
 * so far on the sampler's stream, or on the sampler's stream itself when copy_stream is NULL.  With
 * pinned `out` the copy overlaps the sampling of the next chunk.  Wait for the copy stream
 * (nd_stream_sync) before reading `out` and before the next sample() of this sampler. */
int nd_sampler_final_samples_async(nd_sampler *s, int32_t *out, void *copy_stream);
/* Walk apps: bring a caller's dense host array `out` [num_samples, finalSampleSize] up to date with the
 * sampler's result while moving only the rows' valid prefixes over PCIe (no counterpart in the reference, whose
 * getFinalSamples copies the dense array, src/nextdoor.cu:3211-3237; the array the caller ends up with is the
 * same).  `row_len` [num_samples] belongs to `out`: the number of leading slots of each row that may hold a
 * vertex, every other slot of `out` holding the invalid id (= V).  Start with `out` filled with the invalid id
 * and `row_len` zero (nd_host_fill_int32), hand the same pair to every later update and leave both alone in
 * between: an update rewrites only the slots a walk fills now or filled at the array's previous update.
 *   begin:  packs the prefixes on the device (sampler's stream) and enqueues the copy of the row lengths on
 *           `copy_stream` (NULL: the sampler's stream); returns at once.
 *   fetch:  waits for the lengths, then enqueues the copy of the packed vertices (or of the dense array when
 *           more than half of its slots are in use); optional -- finish calls it when the caller did not.
 *   finish: waits for that copy and writes the rows with host threads (ND_HOST_THREADS, default: the hardware
 *           threads, at most 32); `values_copied` (may be NULL) receives the number of vertex slots that crossed.
 * One update at a time per sampler; the sampler's next sample() waits on the device for the copies. */
int nd_sampler_host_update_begin(nd_sampler *s, int32_t *out, int32_t *row_len, void *copy_stream);
int nd_sampler_host_update_fetch(nd_sampler *s);
int nd_sampler_host_update_finish(nd_sampler *s, int64_t *values_copied);
/* dst[0..n) = value with the same host threads (first fill of a result array) */
int nd_host_fill_int32(int32_t *dst, int64_t n, int32_t value);
/* The same packing between GPUs (no counterpart in the reference, which concatenates dense per-device arrays on the
 * host, src/nextdoor.cu:3211-3237).  nd_sampler_pack_rows enqueues the packing on the sampler's stream and returns
 * the device addresses of the row lengths [num_samples] and of the packed vertices (valid until the sampler's next
 * sample()); nd_sampler_pack_rows_total waits for it and returns the number of packed vertices, i.e. how much of
 * `d_vals` to send.  On the receiving GPU nd_rows_unpack writes `n_rows` rows into the dense array `d_out`
 * [n_rows, steps] whose per-row state `d_row_len` it keeps (all zero over an array filled with `invalid` to start
 * with): vertices from d_vals, the invalid id into slots a row held before and does not hold now.  `d_scratch`:
 * nd_rows_scratch_words(n_rows) 32-bit words.  Everything is stream-ordered; nothing allocates. */
int nd_sampler_pack_rows(nd_sampler *s, const int32_t **d_row_len, const int32_t **d_vals);
int nd_sampler_pack_rows_total(nd_sampler *s, int64_t *total);
int64_t nd_rows_scratch_words(int64_t n_rows);
int nd_rows_unpack(int device, void *stream, int64_t n_rows, int steps, int32_t invalid, const int32_t *d_len,
                   const int32_t *d_vals, int32_t *d_out, int32_t *d_row_len, uint32_t *d_scratch);
int nd_stream_sync(int device, void *stream);
/* zero-copy variant: device address of the same array.  READ-ONLY for the caller: for the walk
 * applications the library keeps the array between sample() calls and rewrites only the slots a
 * walk uses now or used in the previous call (the rest holds the invalid id already). */
int nd_sampler_final_samples_device(nd_sampler *s, const int32_t **out);
/* collective apps: adjacency rows/cols (num_samples*steps*max(batch,L)*L each) and, for the
 * importance apps, the probability of every sampled vertex; k-hop distinct: per-hop counts */
int nd_sampler_aux(nd_sampler *s, int32_t *adj_row, int32_t *adj_col, float *prob, int32_t *hop_counts);
/* counters of the last sample(): [0] sampled edges (valid vertices written), [1] live
 * (transit,sample) pairs summed over steps, [2] weight reads of the rejection loops, [3] node2vec
 * tries, [4] node2vec binary-search probes, [5] neighbour ids gathered for collective unions,
 * [6] unique candidates, [7] PPR in the load-balanced mode: pairs counted in [1] that never entered a
 * map because their walk was known to stop at that step (its stop draw does not depend on the vertex);
 * n <= 8 */
int nd_sampler_stats(nd_sampler *s, int64_t *stats, int n);
/* walks in a transit-parallel mode: live[k] = (transit, sample) pairs that entered step k of the last
 * sample(), i.e. the size of the step's map (the reference prints the same as "totalThreads" per
 * step, src/nextdoor.cu:2400-2410); entries of steps the run did not take step by step are those of
 * an earlier run or zero.  n <= steps. */
int nd_sampler_live_pairs(nd_sampler *s, int32_t *live, int n);
/* per-phase device time of the last sample() when profiling is on: see nd_phase */
typedef enum nd_phase {
  ND_PHASE_NEXT = 0, ND_PHASE_INVERT = 1, ND_PHASE_BIN = 2, ND_PHASE_FINALIZE = 3,
  ND_PHASE_DEDUP = 4, ND_PHASE_COLLECT = 5,
  ND_PHASE_TAIL = 6,   /* the one launch that finishes the surviving walks of a PPR job (also next() work) */
  ND_PHASE_COUNT = 7
} nd_phase;
int nd_sampler_set_profiling(nd_sampler *s, int on);
int nd_sampler_phase_ms(nd_sampler *s, float *ms, int32_t *launches, int n);
/* Name of the next() kernel (for walks: with the app) that nd_sampler_sample(s, mode) launches: the
 * reference picks its kernels by kernelType and the load-balancing flag (src/nextdoor.cu:2400-2928),
 * this library also by app, graph size and its environment switches, so a measurement can label
 * itself with what ran.  `name` receives at most n bytes including the terminator. */
int nd_sampler_next_kernel(const nd_sampler *s, int mode, char *name, int n);
/* freeDeviceData (src/nextdoor.cu:2088-2115) */
int nd_sampler_destroy(nd_sampler *s);

/* ------------------------------------------------------------------ single operators (device pointers) */

/* The map inversion of the step loop: cub::DeviceRadixSort::SortPairs + invalidVertexStartPos
 * (src/nextdoor.cu:2930-2933, 1804-1836).  Stable sort of n (key,val) pairs by key; pairs whose
 * key equals `invalid` are dropped.  All pointers are device pointers on `device`; keys_in/vals_in
 * are clobbered.  *n_live_out (host) receives the surviving count. */
int nd_invert_map(int device, int64_t n, int32_t *keys_in, int32_t *vals_in, int32_t invalid,
                  int32_t *keys_out, int32_t *vals_out, int64_t *n_live_out);
/* The same inversion as a stream-ordered operation for a step loop: the scratch is allocated once
 * (the reference sizes its cub temp storage once before its loop, src/nextdoor.cu:2335, and sorts in
 * every step, :2930-2933).  nd_inverter_run enqueues the sort of n pairs on `stream` and returns
 * without waiting and without touching the allocator; the surviving count stays on the device:
 * *d_n_live (may be NULL) receives the address of an int32 that holds it once the stream reaches
 * that point (valid until the next run on this inverter).  The sorted pairs occupy the first
 * *d_n_live slots of keys_out / vals_out; keys_in / vals_in are clobbered.  max_pairs bounds n;
 * `invalid` (= the vertex count) is the dead key and bounds the key range. */
typedef struct nd_inverter nd_inverter;
int nd_inverter_create(int device, int64_t max_pairs, int32_t invalid, nd_inverter **out);
int nd_inverter_run(nd_inverter *inv, void *stream, int64_t n, int32_t *keys_in, int32_t *vals_in, int32_t *keys_out,
                    int32_t *vals_out, const int32_t **d_n_live);
int nd_inverter_destroy(nd_inverter *inv);
/* No counterpart in the reference.  nd_invert_map for callers that must not allocate device
 * memory: a sampler sharing a process with a training job, where cudaMalloc/cudaFree would
 * synchronise the device and stall the training streams, or where the framework's allocator has
 * already taken nearly all of HBM so a raw cudaMalloc may fail.  Same arguments and result as
 * nd_invert_map, but the scratch is a fixed array inside the library image (about 2 MB, resident
 * on every GPU that loads the library until the process exits) and no cudaMalloc/cudaFree is
 * made.  n must not exceed nd_static_max_pairs() (2^20), else ND_ERR_RANGE.  All calls on a device
 * share the array: calls that overlap on the GPU race, so issue them one after the other.  The
 * first call on each device looks the array's device address up and should happen before any
 * stream capture begins. */
int nd_invert_map_static(int device, int64_t n, int32_t *keys_in, int32_t *vals_in, int32_t invalid,
                         int32_t *keys_out, int32_t *vals_out, int64_t *n_live_out);
/* The same on a stream of the caller's (a cudaStream_t): every copy and kernel is enqueued on
 * `stream` and only that stream is waited for before the call returns, so work on the device's
 * other streams is not held up.  nd_invert_map_static is this with stream = NULL, the legacy
 * default stream, which synchronises with every blocking stream of the device.  No counterpart in
 * the reference either. */
int nd_invert_map_static_on(int device, void *stream, int64_t n, int32_t *keys_in, int32_t *vals_in, int32_t invalid,
                            int32_t *keys_out, int32_t *vals_out, int64_t *n_live_out);
int64_t nd_static_max_pairs(void);
/* remove_duplicates_in_hop_per_block (src/distinct.cuh:1-111): every segment of seg_len ints is
 * sorted ascending, made unique, compacted to the front and padded with `invalid`;
 * counts (device, may be NULL) receives the unique count per segment. */
int nd_distinct_segments(int device, int32_t *data, int64_t n_segments, int32_t seg_len,
                         int32_t invalid, int32_t *counts);
/* the keyed draw the kernels use, evaluated on the device for n (sample, step, slot, draw) tuples */
int nd_philox_uniform(int device, uint64_t seed, int64_t n, const uint32_t *tuples4, float *out);
/* One next() of a walk application (uniform walk, DeepWalk, PPR) for n explicit (transit, sample)
 * pairs: the transit-parallel next() kernel (samplingKernel, src/nextdoor.cu:212-336) as an
 * operator.  d_transits[n] int32, d_samples[n] int64 (GLOBAL sample ids: the draws are keyed by
 * them) and d_next[n] int32 are DEVICE pointers; d_next[i] = the sampled neighbour, or -1 (no
 * edges, walk ended, transit outside [0, V)).  Enqueued on `stream`, no synchronisation.  With a
 * graph that holds only the rows of one vertex range (other rows empty) this is the per-step
 * building block of sampling over a graph partitioned across GPUs -- the use the reference's
 * CSR partitioner was written for (src/graph_partitioner.cuh:1-173; the multi-GPU partitioned
 * path itself is a stub there, ENABLE_GRAPH_PARTITION_FOR_GLOBAL_MEM, src/csr.hpp:371-374). */
int nd_walk_step(const nd_graph *g, const nd_app_params *p, int step, int64_t n, const int32_t *d_transits,
                 const int64_t *d_samples, int32_t *d_next, void *stream);
/* nd_walk_step for walkers packed into one 64-bit word each, (global sample id << 32) | vertex;
 * a walk that ended comes back as all ones.  Device pointers, enqueued on `stream`. */
int nd_walk_step_packed(const nd_graph *g, const nd_app_params *p, int step, int64_t n, const uint64_t *d_walkers_in,
                        uint64_t *d_walkers_out, void *stream);
/* Device status of nd_walk_step / nd_walk_step_packed on `device` (the reference aborts inside
 * CHK_CU instead, src/utils.hpp:16): waits for `stream`, then *status receives the bits the step
 * kernels have set since the last call (8 = a rejection loop hit its iteration cap and took
 * edges[0]) and the word is cleared. */
int nd_walk_step_status(int device, void *stream, int *status);
/* Routing of packed walkers between the ranks of a partitioned job (no counterpart in the
 * reference, whose multi-GPU path replicates the graph, src/nextdoor.cu:1893-1911).  `d_bounds`
 * (device, parts + 1 int64) are the contiguous key ranges of the parts; the key of a walker is its
 * vertex, or its sample id when by_sample != 0 (records going to the samples' home ranks).
 * nd_route_count: d_counts[parts] = live walkers per destination (ended walkers are skipped).
 * nd_route_scatter: d_out = the live walkers grouped by destination, segment p starting at
 * sum(d_counts[0..p)); d_cursor[parts] is scratch.  Device pointers, enqueued on `stream`. */
int nd_route_count(int device, int64_t n, const uint64_t *d_walkers, int by_sample, const int64_t *d_bounds, int parts,
                   uint64_t *d_counts, void *stream);
int nd_route_scatter(int device, int64_t n, const uint64_t *d_walkers, int by_sample, const int64_t *d_bounds, int parts,
                     const uint64_t *d_counts, uint64_t *d_cursor, uint64_t *d_out, void *stream);
/* d_records[n] = (sample << 32 | vertex) words of ONE step that arrived at their home rank:
 * d_out[(sample - first_sample) * steps + step] = vertex for the samples in [first_sample,
 * first_sample + count); d_out is the rank's [count, steps] result array. */
int nd_records_store(int device, int64_t n, const uint64_t *d_records, int step, int64_t first_sample, int64_t count,
                     int steps, int32_t *d_out, void *stream);
#ifdef __cplusplus
}
#endif
#endif
