// Random-walk applications (stepSize == 1): uniform walk, DeepWalk, PPR, node2vec.
//
// Transit-parallel path (doTransitParallelSampling, src/nextdoor.cu:2191-3006): every step runs
// one next() kernel over the transit-sorted (transit, sample) map -- the role of samplingKernel /
// identityKernel (src/nextdoor.cu:212-336, 338-504) -- and then inverts the freshly written
// sample->transit pairs with the in-house radix sort.  The next() kernel already counts the first
// radix digit of the keys it writes, so the inversion starts at its scan.
// Sample-parallel path (sampleParallelKernel, src/nextdoor.cu:1348-1518): one thread owns a walk
// for all its steps and keeps the walk state in registers.
//
// Both paths write the walk step-major (tmp[step][sample], 4-byte stores that the L2 merges into
// full sectors) and a last kernel transposes that into the reference's sample-major layout
// finalSamples[sample*steps + step] (src/nextdoor.cu:2041, 293-334) with coalesced row stores.
// Why no adjacency staging here: a walk draws one neighbour per visit, and at stationarity a
// transit of degree d is visited by about d * S / E walks per step (1/32 of d on the 2^20-vertex
// graph), so the visits touch fewer sectors than the list holds; staging pays for k-hop, not for walks.
#include <mutex>

#include "nd_cache.cuh"
#include "nd_common.cuh"
#include "nd_philox.cuh"

namespace {

using ndrng::Rng;

struct WalkParams {
  uint64_t seed;
  float p, q, stop_prob;
  int n2v_compat;
  int steps;
  const int32_t *adjset;  // node2vec: per-vertex hash sets of the neighbour ids
  const int2 *colw;       // DeepWalk / PPR: (neighbour id, weight bits) records
  const int2 *vrec = nullptr;  // DeepWalk / PPR: (row start, max weight bits) per vertex, V + 1 entries
  int keep_all_step = -1; // PPR, load-balanced loop: the step whose map goes to the tail launch keeps every pair (see walk_next_count_kernel)
};

// node2vec asks "is v a neighbour of the previous vertex t?" for its candidates, and t is usually a
// hub (a 17-probe bisection of dependent loads).  Every vertex with at least SET_MIN_DEG
// neighbours gets an open-addressing hash set of its neighbour ids instead: buckets of 8 ids (one
// 32-byte sector), the buckets [row_ptr[t]/4, (row_ptr[t]+deg)/4) of one array (regions of
// consecutive vertices cannot overlap; at least deg slots each, load factor about 1/2).  An id
// lives in the first free slot at or after its home bucket, so a lookup reads the home bucket and
// is done unless that bucket is full and does not hold the id (about 5 % of the lookups).  The
// answer is exact, i.e. the answer of utils::binarySearch (src/utils.hpp:30-48).
constexpr int SET_MIN_DEG = 8;
constexpr int32_t SET_EMPTY = -1;

__device__ __forceinline__ uint32_t set_mix(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return x;
}
__device__ __forceinline__ uint32_t set_bucket(int32_t v, uint32_t n_buckets) {
  return (uint32_t)(((unsigned long long)set_mix((uint32_t)v) * n_buckets) >> 32);
}

constexpr int RETRY_CAP = 1 << 16;

// events the algorithmic-bytes model is evaluated from (stats[2..4]); kept per thread and
// flushed once per warp when the kernel ends
struct Events {
  uint32_t weight_tries = 0, n2v_tries = 0, n2v_probes = 0;
  uint32_t not_entered = 0;  // PPR: pairs left out of the next map because the walk is known to stop there (stats[7])
  __device__ __forceinline__ void flush(unsigned long long *stats) {
    uint32_t a = weight_tries, b = n2v_tries, c = n2v_probes, d = not_entered;
    for (int o = 16; o > 0; o >>= 1) {
      a += __shfl_xor_sync(0xffffffffu, a, o);
      b += __shfl_xor_sync(0xffffffffu, b, o);
      c += __shfl_xor_sync(0xffffffffu, c, o);
      d += __shfl_xor_sync(0xffffffffu, d, o);
    }
    if ((threadIdx.x & 31) == 0) {
      if (a) atomicAdd(&stats[2], (unsigned long long)a);
      if (b) atomicAdd(&stats[3], (unsigned long long)b);
      if (c) atomicAdd(&stats[4], (unsigned long long)c);
      if (d) atomicAdd(&stats[7], (unsigned long long)d);
    }
  }
  // The same for a kernel whose CTAs are short-lived (a tile each): the warps' sums meet in shared
  // memory and the CTA adds them once -- with one atomic per warp the half a million warps of a large
  // step queue up on the four counters (measured: 0.4 ms per pass and counter on the 2^24-vertex job).
  // Every thread of the CTA must call it.
  __device__ __forceinline__ void flush_cta(unsigned long long *stats) {
    __shared__ uint32_t sums[4];
    uint32_t a = weight_tries, b = n2v_tries, c = n2v_probes, d = not_entered;
    for (int o = 16; o > 0; o >>= 1) {
      a += __shfl_xor_sync(0xffffffffu, a, o);
      b += __shfl_xor_sync(0xffffffffu, b, o);
      c += __shfl_xor_sync(0xffffffffu, c, o);
      d += __shfl_xor_sync(0xffffffffu, d, o);
    }
    __syncthreads();
    if (threadIdx.x < 4) sums[threadIdx.x] = 0u;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) {
      if (a) atomicAdd(&sums[0], a);
      if (b) atomicAdd(&sums[1], b);
      if (c) atomicAdd(&sums[2], c);
      if (d) atomicAdd(&sums[3], d);
    }
    __syncthreads();
    if (threadIdx.x < 4 && sums[threadIdx.x]) atomicAdd(&stats[threadIdx.x < 3 ? 2 + threadIdx.x : 7], (unsigned long long)sums[threadIdx.x]);
  }
};

// Gathers from the big graph arrays (neighbour ids, weight records, set buckets) are used once per
// launch in the transit-parallel kernels: there they are loaded with the streaming policy
// (evict-first) so that they do not push the small per-sample and per-vertex arrays (maps,
// counters, staged output row, row offsets) out of L2.  A sample-parallel walk revisits hub lists
// from the same thread step after step and is faster with the default policy.
template <bool STREAM, typename T>
__device__ __forceinline__ T ld_graph(const T *p) { return STREAM ? __ldcs(p) : __ldg(p); }

// Exact membership of v in the neighbour list [ts, ts+tn) of t.  `probes` counts the 4-byte words read.
template <bool STREAM>
__device__ __forceinline__ bool n2v_member_slow(const NdGraphView &g, const int32_t *adjset, int32_t ts, int32_t tn,
                                                int32_t v, uint32_t bucket, uint32_t n_buckets, uint32_t &probes) {
  if (tn < SET_MIN_DEG) {  // short list: read it
    bool found = false;
#pragma unroll
    for (int k = 0; k < SET_MIN_DEG - 1; k++) {
      const int32_t e = k < tn ? ld_graph<STREAM>(g.col + ts + k) : -1;
      found |= e == v;
    }
    probes += tn;
    return found;
  }
  const int4 *region = reinterpret_cast<const int4 *>(adjset) + 2 * (size_t)((uint32_t)ts >> 2);
  for (uint32_t it = 0; it < n_buckets; it++) {  // the home bucket was full: walk on
    bucket = bucket + 1 < n_buckets ? bucket + 1 : 0;
    const int4 a = ld_graph<STREAM>(region + 2 * (size_t)bucket), b = ld_graph<STREAM>(region + 2 * (size_t)bucket + 1);
    probes += 8;
    if (a.x == v || a.y == v || a.z == v || a.w == v || b.x == v || b.y == v || b.z == v || b.w == v) return true;
    if (b.w == SET_EMPTY) return false;  // slots fill front to back inside a bucket
  }
  return false;
}

// node2vec tries whose gathers are issued together (template argument of app_next): measured
// best are 3 in the ticket kernel and 2 in the sample-parallel kernel at four CTAs of 256 per SM,
// and 4 at three CTAs per SM in the kernel that also keeps the radix histogram
constexpr int N2V_BATCH_COUNT = 3, N2V_BATCH_SP = 2, N2V_BATCH_TP = 4;
// Weighted tries per round.  Every try of a round is gathered, so a larger batch buys latency with
// gathers that a 60 % acceptance rate wastes: two per round, except PPR in the sample-parallel
// kernel (walks die young there, the kernel is short of loads in flight; four measured faster).
template <int APP, bool STREAM>
__host__ __device__ constexpr int weight_batch() { return APP == ND_APP_PPR && !STREAM ? 4 : 2; }

constexpr int32_t ROUND_AGAIN = -2;   // a round of tries ended without an accepted vertex

// The rejection loops of DeepWalk / PPR / node2vec draw their tries from the keyed stream in
// order, so try k of an invocation is a pure function of (sample, step, k).  A ROUND evaluates a
// batch of tries: the gathers of the whole round are issued together (one memory latency instead
// of one per try) and the first try that accepts, in draw order, wins -- the same vertex the
// one-try-at-a-time loop returns.  Only the tries up to the winner are counted.  `rng` carries the
// draw position from round to round.

// weighted rejection (randomWalks.cu:81-89): {x = rand_int(n); y = u * max_w} until !(y > w[x])
template <bool STREAM, int BATCH>
__device__ __forceinline__ int32_t weighted_round(const WalkParams &wp, int32_t rs, int32_t n, float max_w, Rng &rng,
                                                  Events &ev) {
  const int2 *__restrict__ recs = wp.colw + rs;
  float y[BATCH];
  int2 rec[BATCH];
#pragma unroll
  for (int k = 0; k < BATCH; k++) {
    const int32_t x = rng.rand_int(n);
    y[k] = __fmul_rn(rng.uniform(), max_w);
    rec[k] = ld_graph<STREAM>(recs + x);
  }
#pragma unroll
  for (int k = 0; k < BATCH; k++) {
    ev.weight_tries++;
    if (!(y[k] > __int_as_float(rec[k].y))) return rec[k].x;
  }
  return ROUND_AGAIN;
}

// node2vec (randomWalks.cu:151-171).  A candidate that is not the previous vertex t is accepted
// when y < 1/q (neighbour of t) or y < 1 (not a neighbour): below `lo` the membership does not
// matter, at or above `hi` neither; below `sure` nothing about the candidate matters.
struct N2vConsts {
  float inv_q, bound, lo, hi, sure;
  __device__ __forceinline__ explicit N2vConsts(const WalkParams &wp) {
    inv_q = __fdiv_rn(1.0f, wp.q);
    bound = wp.p > inv_q ? wp.p : inv_q;
    if (bound < 1.0f) bound = 1.0f;
    lo = inv_q < 1.0f ? inv_q : 1.0f;
    hi = inv_q < 1.0f ? 1.0f : inv_q;
    sure = lo < wp.p ? lo : wp.p;
  }
};

// t = previous vertex, [ts, ts + tn) its row
template <bool STREAM, int BATCH>
__device__ __forceinline__ int32_t n2v_round(const NdGraphView &g, const WalkParams &wp, const N2vConsts &c, int32_t rs,
                                             int32_t n, int32_t t, int32_t ts, int32_t tn, Rng &rng, Events &ev) {
  const int32_t *__restrict__ edges = g.col + rs;
  const uint32_t n_buckets = ((uint32_t)(ts + tn) >> 2) - ((uint32_t)ts >> 2);
  const int4 *__restrict__ region = reinterpret_cast<const int4 *>(wp.adjset) + 2 * (size_t)((uint32_t)ts >> 2);
  const bool use_set = tn >= SET_MIN_DEG;
  int32_t x[BATCH], v[BATCH];
  float y[BATCH];
  int n_try = BATCH;  // the round ends at the first try that is sure to accept
#pragma unroll
  for (int k = 0; k < BATCH; k++) {
    if (k < n_try) {
      x[k] = rng.rand_int(n);
      y[k] = __fmul_rn(rng.uniform(), c.bound);
      if (y[k] < c.sure) n_try = k + 1;
    }
  }
#pragma unroll
  for (int k = 0; k < BATCH; k++) v[k] = k < n_try ? ld_graph<STREAM>(edges + x[k]) : -1;
  // membership gathers of the tries that need one, issued together
  bool is_ret[BATCH], need[BATCH];
  uint32_t bucket[BATCH];
  int4 ba[BATCH], bb[BATCH];
#pragma unroll
  for (int k = 0; k < BATCH; k++) {
    is_ret[k] = wp.n2v_compat ? (x[k] == t) : (v[k] == t);  // randomWalks.cu:159 compares the index
    need[k] = k < n_try && !is_ret[k] && y[k] >= c.lo && y[k] < c.hi;
    bucket[k] = set_bucket(v[k], n_buckets);
    if (need[k] && use_set) {
      ba[k] = ld_graph<STREAM>(region + 2 * (size_t)bucket[k]);
      bb[k] = ld_graph<STREAM>(region + 2 * (size_t)bucket[k] + 1);
    } else {
      ba[k] = make_int4(SET_EMPTY, SET_EMPTY, SET_EMPTY, SET_EMPTY);
      bb[k] = ba[k];
    }
  }
#pragma unroll
  for (int k = 0; k < BATCH; k++) {
    if (k < n_try) {
      ev.n2v_tries++;
      bool accept;
      if (is_ret[k]) {
        accept = y[k] < wp.p;
      } else if (!need[k]) {
        accept = y[k] < c.lo;
      } else {
        bool found = ba[k].x == v[k] || ba[k].y == v[k] || ba[k].z == v[k] || ba[k].w == v[k] ||
                     bb[k].x == v[k] || bb[k].y == v[k] || bb[k].z == v[k] || bb[k].w == v[k];
        if (use_set) ev.n2v_probes += 8;
        if (!found && (!use_set || bb[k].w != SET_EMPTY))
          found = n2v_member_slow<STREAM>(g, wp.adjset, ts, tn, v[k], bucket[k], n_buckets, ev.n2v_probes);
        accept = y[k] < (found ? c.inv_q : 1.0f);
      }
      if (accept) return v[k];
    }
  }
  return ROUND_AGAIN;
}

// node2vec next() on a transit with n > 1 neighbours at a step > 0 when the row [ts, ts + tn) of the
// previous vertex t is known already
template <bool STREAM, int N2V_BATCH>
__device__ __forceinline__ int32_t n2v_next_known(const NdGraphView &g, const WalkParams &wp, int32_t rs, int32_t n,
                                                  int32_t t, int32_t ts, int32_t tn, Rng &rng, int *status, Events &ev) {
  const N2vConsts c(wp);
  for (int it = 0; it <= RETRY_CAP; it += N2V_BATCH) {
    const int32_t r = n2v_round<STREAM, N2V_BATCH>(g, wp, c, rs, n, t, ts, tn, rng, ev);
    if (r != ROUND_AGAIN) return r;
  }
  atomicOr(status, ND_DEV_RETRY_LIMIT);
  return ld_graph<STREAM>(g.col + rs);
}

// One next() of the app on a transit with n > 0 neighbours; -1 = no vertex.
template <int APP, bool STREAM = true, int N2V_BATCH = N2V_BATCH_COUNT>
__device__ __forceinline__ int32_t app_next(const NdGraphView &g, const WalkParams &wp, int step,
                                            int32_t transit, int32_t rs, int32_t n, int32_t &state_t,
                                            Rng &rng, int *status, Events &ev, bool have_max_w = false,
                                            float max_w_in = 0.f) {  // weighted apps: the transit's maximum weight, if the caller fetched it beside the row offsets
  const int32_t *__restrict__ edges = g.col + rs;
  if (APP == ND_APP_UNIFORM_WALK) {  // example/uniformRandWalk.cu:35-36
    return ld_graph<STREAM>(edges + rng.rand_int(n));
  }
  if (APP == ND_APP_DEEPWALK || APP == ND_APP_PPR) {  // randomWalks.cu:74-90, 102-124
    if (APP == ND_APP_PPR) {
      const float pr = rng.uniform();
      if (pr < wp.stop_prob) return -1;
    }
    if (n == 1) return ld_graph<STREAM>(edges);
    const float max_w = have_max_w ? max_w_in : __ldg(g.max_w + transit);
    constexpr int WEIGHT_BATCH = weight_batch<APP, STREAM>();
    for (int it = 0; it <= RETRY_CAP; it += WEIGHT_BATCH) {
      const int32_t r = weighted_round<STREAM, WEIGHT_BATCH>(wp, rs, n, max_w, rng, ev);
      if (r != ROUND_AGAIN) return r;
    }
    atomicOr(status, ND_DEV_RETRY_LIMIT);
    return ld_graph<STREAM>(edges);
  }
  if (APP == ND_APP_NODE2VEC) {  // randomWalks.cu:141-172
    if (n == 1 || step == 0) { state_t = transit; return ld_graph<STREAM>(edges); }
    const int32_t t = state_t;
    const int32_t ts = __ldg(g.row_ptr + t);
    const int32_t tn = __ldg(g.row_ptr + t + 1) - ts;
    state_t = transit;
    return n2v_next_known<STREAM, N2V_BATCH>(g, wp, rs, n, t, ts, tn, rng, status, ev);
  }
  return -1;
}

// ---------------------------------------------------------------- set-up kernels

// thread per CSR entry: find the entry's source vertex by bisection of the row offsets and insert
// the neighbour id into the source's set (first free slot at or after the home bucket)
__global__ void adjset_build_kernel(NdGraphView g, int64_t E, int32_t *__restrict__ adjset, int *__restrict__ status) {
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < E; e += (int64_t)gridDim.x * blockDim.x) {
    int32_t lo = 0, hi = g.V;  // last vertex with row_ptr[v] <= e
    while (hi - lo > 1) {
      const int32_t mid = lo + ((hi - lo) >> 1);
      if ((int64_t)g.row_ptr[mid] <= e) lo = mid; else hi = mid;
    }
    const int32_t rs = g.row_ptr[lo], deg = g.row_ptr[lo + 1] - rs;
    if (deg < SET_MIN_DEG) continue;
    const uint32_t n_buckets = ((uint32_t)(rs + deg) >> 2) - ((uint32_t)rs >> 2);
    int32_t *region = adjset + 8 * (size_t)((uint32_t)rs >> 2);
    const int32_t v = g.col[e];
    uint32_t b = set_bucket(v, n_buckets);
    bool done = false;
    for (uint32_t it = 0; it < n_buckets && !done; it++) {
      for (int i = 0; i < 8 && !done; i++) {
        int32_t *slot = region + 8 * (size_t)b + i;
        int32_t cur = *(volatile int32_t *)slot;
        if (cur == SET_EMPTY) cur = atomicCAS(slot, SET_EMPTY, v);
        done = cur == SET_EMPTY || cur == v;  // placed, or the id is in the set already (repeated edge)
      }
      b = b + 1 < n_buckets ? b + 1 : 0;
    }
    if (!done) atomicOr(status, ND_DEV_RETRY_LIMIT);  // cannot happen: a region has at least deg slots
  }
}

__global__ void colw_build_kernel(const int32_t *__restrict__ col, const float *__restrict__ w, int64_t E,
                                  int2 *__restrict__ colw) {
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < E; e += (int64_t)gridDim.x * blockDim.x)
    colw[e] = make_int2(col[e], __float_as_int(w[e]));
}

__global__ void vrec_build_kernel(const int32_t *__restrict__ row_ptr, const float *__restrict__ max_w, int32_t V,
                                  int2 *__restrict__ vrec) {
  for (int64_t v = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; v <= V; v += (int64_t)gridDim.x * blockDim.x)
    vrec[v] = make_int2(row_ptr[v], v < V ? __float_as_int(max_w[v]) : 0);
}

__global__ void walk_reset_kernel(const int32_t *__restrict__ initial, int32_t V, int64_t S, int steps,
                                  int32_t *__restrict__ len, int32_t *__restrict__ state,
                                  unsigned long long *__restrict__ stats, int32_t *__restrict__ tail_ctr) {
  const int64_t s = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (s < 8 && stats) stats[s] = 0ull;
  if (s == 0 && tail_ctr) *tail_ctr = 0;
  if (s >= S) return;
  const int32_t t = initial[s];
  len[s] = (t >= 0 && t < V) ? steps : -1;
  if (state) state[s] = 0;
}

// walks whose start vertex is valid and has neighbours
__global__ void count_active_kernel(const int32_t *__restrict__ initial, int64_t n, int32_t V,
                                    const int32_t *__restrict__ row_ptr, int32_t *__restrict__ out) {
  int c = 0;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int32_t t = initial[i];
    if (t >= 0 && t < V && row_ptr[t + 1] > row_ptr[t]) c++;
  }
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0 && c) atomicAdd(out, c);
}

__global__ void init_map_kernel(const int32_t *__restrict__ initial, int32_t V, int64_t n,
                                int32_t *__restrict__ keys, int32_t *__restrict__ vals) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int32_t t = initial[i];
  keys[i] = (t >= 0 && t < V) ? t : V;
  vals[i] = (int32_t)i;
}

// ---------------------------------------------------------------- transit-parallel next()

// node2vec keeps a round of candidates and set buckets in registers: four CTAs of 256 per SM (64
// registers) with rounds of 2-3 tries measured faster than three CTAs with rounds of 4
// (the weighted apps: five CTAs per SM in the ticket kernel, six in the sample-parallel one,
// measured against 4-8 on the 2^20- and 2^24-vertex graphs)
template <int APP>
constexpr int walk_min_ctas() { return APP == ND_APP_NODE2VEC ? 4 : (APP == ND_APP_UNIFORM_WALK ? 1 : 5); }
template <int APP>
constexpr int walk_min_ctas_sp() { return APP == ND_APP_NODE2VEC ? 4 : (APP == ND_APP_UNIFORM_WALK ? 1 : 6); }

constexpr int NEXT_THREADS = 256;

// One CTA per radix tile of the transit->sample map.  HIST: also count the first radix digit of the
// new keys (layout and digit as the radix scatter of pass 0 expects them).
template <int APP, bool HIST>
__global__ void __launch_bounds__(NEXT_THREADS, APP == ND_APP_NODE2VEC ? 3 : 1)
walk_next_tp_kernel(NdGraphView g, WalkParams wp, int step, int64_t first_sample, int tile_size,
                    const int32_t *__restrict__ in_key, const int32_t *__restrict__ in_val,
                    const int32_t *__restrict__ d_n, int32_t *__restrict__ out_key,
                    int32_t *__restrict__ out_val, int32_t *__restrict__ tmp_step,
                    int32_t *__restrict__ len, int32_t *__restrict__ state, int shift, int bins,
                    uint32_t *__restrict__ tile_hist, int64_t max_tiles, uint32_t *__restrict__ ghist,
                    int *__restrict__ status, unsigned long long *__restrict__ stats) {
  extern __shared__ uint32_t sh_hist[];
  Events ev;
  const int n = *d_n;
  const int tiles = (n + tile_size - 1) / tile_size;
  const uint32_t mask = bins - 1;
  if (HIST) for (int b = threadIdx.x; b < bins; b += NEXT_THREADS) sh_hist[bins + b] = 0;
  for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    if (HIST) {
      for (int b = threadIdx.x; b < bins; b += NEXT_THREADS) sh_hist[b] = 0;
      __syncthreads();
    }
    const int base = tile * tile_size;
    for (int i = base + threadIdx.x; i < base + tile_size && i < n; i += NEXT_THREADS) {
      const int32_t t = in_key[i];
      const int32_t s = in_val[i];
      int32_t nbr = -1;
      if (t < 0 || t >= g.V) {
        atomicOr(status, ND_DEV_BAD_TRANSIT);
      } else {
        const int32_t rs = __ldg(g.row_ptr + t);
        const int32_t deg = __ldg(g.row_ptr + t + 1) - rs;
        if (deg > 0) {  // next() runs only on transits with edges (src/nextdoor.cu:255,412)
          Rng rng(wp.seed, (uint32_t)(first_sample + s), (uint32_t)step, 0u);
          int32_t st = 0;
          if (APP == ND_APP_NODE2VEC && step > 0) st = state[s];
          nbr = app_next<APP, true, N2V_BATCH_TP>(g, wp, step, t, rs, deg, st, rng, status, ev);
          if (APP == ND_APP_NODE2VEC && nbr >= 0) state[s] = st;
        }
      }
      if (nbr >= 0) tmp_step[s] = nbr; else len[s] = step;
      if (HIST) {
        out_key[i] = nbr >= 0 ? nbr : g.V;
        out_val[i] = s;
        if (nbr >= 0) atomicAdd(&sh_hist[((uint32_t)nbr >> shift) & mask], 1u);
      }
    }
    if (HIST) {
      __syncthreads();
      for (int b = threadIdx.x; b < bins; b += NEXT_THREADS) {  // a bin is always handled by the same thread
        const uint32_t c = sh_hist[b];
        tile_hist[(int64_t)b * max_tiles + tile] = c;
        sh_hist[bins + b] += c;
      }
      __syncthreads();
    }
  }
  if (HIST)  // one global atomic per bin and CTA
    for (int b = threadIdx.x; b < bins; b += NEXT_THREADS)
      if (sh_hist[bins + b]) atomicAdd(&ghist[b], sh_hist[bins + b]);
  if (APP != ND_APP_UNIFORM_WALK) ev.flush(stats);
}

// ---------------------------------------------------------------- next() + counting inversion (load-balanced mode)
//
// The transit ids are a dense key space (< V) and the map holds at most one pair per walk, so
// the inversion does not need a multi-pass sort: next() takes a ticket on its new transit
// (atomicAdd on cnt[transit], the ticket is the pair's rank inside the transit's run) and counts
// the pair in a coarse histogram (one bin per CNT_SUPER vertices, kept in shared memory and
// flushed once per CTA); one kernel turns the counters into run offsets (a CTA per bin: the bins
// before it give its base, then an exclusive scan of its own counters, which also clears them and
// publishes the live count); one kernel moves every pair to offs[transit] + rank.  Three launches
// and 16 B read + 8 B written per pair beside the counter traffic, against 2-3 radix passes of
// three launches each.  The order of the pairs inside one transit's run depends on the order the
// tickets were drawn; results do not, because every draw is keyed by the sample.
// node2vec: the previous vertex of a walk travels with the sorted map (the scatter copies the
// transit the pair was read under), so next() reads it with a coalesced load instead of a gather
// by sample id.

constexpr int CNT_SUPER = 4096;                             // counters per scan CTA = vertices per coarse bin
constexpr int CNT_SUPER_SHIFT = 12;
constexpr int SCAN_THREADS = 512;
constexpr int SCAN_PER_THREAD = CNT_SUPER / SCAN_THREADS;   // 32 consecutive counters per thread
constexpr int MAX_SMEM_BINS = 8192;                         // coarse bins kept in shared memory (V <= 2^25)

// ---- opt-in: the reference's grid bin for walks (staged adjacency list shared by all samples on a hub)
//
// A tile of HUB_TILE consecutive pairs of the sorted map whose pairs all stand on ONE transit is a
// hub tile; the consecutive hub tiles of a transit form its run.  The CTA that finds the first
// tile of a run streams the transit's adjacency list through shared memory once per pass of
// HUB_PASS tiles and serves all their draws from it (uniform walk: the index is drawn first, the
// pair picks its neighbour when the chunk that holds the index is staged).  The pairs outside
// whole hub tiles stay with the thread-per-pair kernel.  Measured slower than plain gathers (a
// transit of degree d holds d * S / E walkers, so 128 bytes of list are streamed per gather of one
// sector that is saved), hence off unless ND_WALK_STAGING=1; the weighted apps and node2vec probe
// several random positions per try and cannot be served from a streamed chunk at all.
constexpr int HUB_TILE = 256;
constexpr int HUB_PASS = 8;        // tiles whose pairs a CTA serves per sweep of the list
constexpr int HUB_CHUNK = 8192;    // neighbour ids staged at once (32 KB)

// transit of hub tile `tau` of the 8-byte-record map, or -1 if the tile is not one
__device__ __forceinline__ int32_t hub_tile(const void *in_rec, int n, int tau) {
  const int base = tau * HUB_TILE;
  if (tau < 0 || base + HUB_TILE > n) return -1;
  const int2 *rec = reinterpret_cast<const int2 *>(in_rec);
  const int32_t a = rec[base].x, b = rec[base + HUB_TILE - 1].x;
  return a == b ? a : -1;
}

// The kernel.  CTAs take tiles of 256 * PPT pairs of the sorted map (PPT = pairs a thread works on
// at once, phase by phase; 1 measured best for every app, larger values are kept as a tuning macro).
//  * uniform walk, DeepWalk, PPR: next() in place, up to 16 CTAs per SM, a tile each.
//  * node2vec: the first round of tries of a pair is straight-line code (no divergence: the
//    round's candidate gathers are issued together, then its set buckets); a pair the first round
//    does not settle (every try rejected, or a membership test that has to walk past a full
//    bucket: about one pair in eight) goes on a per-warp queue in shared memory, and whenever a
//    queue holds 32 pairs the warp runs them through the general loop with all lanes busy --
//    continuing behind the rejected tries in the pair's draw sequence, so nothing is gathered
//    twice.  The draws of a pair depend only on (sample, step), so the queue changes no sample.
//    The CTAs are persistent here (as many as are resident), so that the queues fill over tiles.
//  * the coarse histogram (pairs per 4096 vertices, for the scan) is kept in shared memory and flushed once per CTA.
// What bounds it: a pair costs a few random 32-byte sector reads that miss the L2 (one neighbour id;
// node2vec about 2.6 candidates and 1.3 set buckets in a first round of four tries), and the memory system serves those at a
// rate far below its streaming bandwidth; occupancy, pairs per thread, cache hints and the L2
// fetch granularity were all measured and do not move the kernel's time by more than a few per cent.
constexpr int COUNT_THREADS = 256;
constexpr int COUNT_WARPS = COUNT_THREADS / 32;

#ifndef ND_TUNE_PPT_UNIFORM
#define ND_TUNE_PPT_UNIFORM 1
#endif
#ifndef ND_TUNE_PPT_WEIGHTED
#define ND_TUNE_PPT_WEIGHTED 1
#endif
#ifndef ND_TUNE_PPT_N2V
#define ND_TUNE_PPT_N2V 1
#endif
#ifndef ND_TUNE_N2V_FIRST
#define ND_TUNE_N2V_FIRST 4
#endif
#ifndef ND_TUNE_CTAS_UNIFORM
#define ND_TUNE_CTAS_UNIFORM 4
#endif
#ifndef ND_TUNE_CTAS_WEIGHTED
#define ND_TUNE_CTAS_WEIGHTED 5
#endif
#ifndef ND_TUNE_CTAS_N2V
#define ND_TUNE_CTAS_N2V 3
#endif
template <int APP>
__host__ __device__ constexpr int count_ppt() {
  return APP == ND_APP_NODE2VEC ? ND_TUNE_PPT_N2V : (APP == ND_APP_UNIFORM_WALK ? ND_TUNE_PPT_UNIFORM : ND_TUNE_PPT_WEIGHTED);
}
template <int APP>
__host__ __device__ constexpr int count_ctas() {
  return APP == ND_APP_NODE2VEC ? ND_TUNE_CTAS_N2V : (APP == ND_APP_UNIFORM_WALK ? ND_TUNE_CTAS_UNIFORM : ND_TUNE_CTAS_WEIGHTED);
}
constexpr int N2V_FIRST = ND_TUNE_N2V_FIRST;   // tries of the straight-line first round

// A record of the transit-sorted map in the load-balanced mode.  One record = one aligned piece
// of one 32-byte sector, so the scatter kernel places a pair with ONE random sector write:
// {transit, sample} (8 bytes), or for node2vec 32 bytes {transit, sample, previous vertex, row
// start of the previous vertex, its degree, 0, 0, 0} -- the previous vertex's row travels with
// the pair, so next() never gathers row offsets by a random vertex id.
template <bool N2V>
struct MapRec {
  int32_t t, s, pv;
  int2 prow;
};
template <bool N2V>
__host__ __device__ constexpr size_t map_rec_bytes() { return N2V ? 32 : 8; }

template <bool N2V>
__device__ __forceinline__ MapRec<N2V> map_rec_load(const ndmem::Keep &keep, const void *base, int i) {
  MapRec<N2V> r;
  if (N2V) {
    const int4 *p = reinterpret_cast<const int4 *>(base) + 2 * (size_t)i;
    const int4 a = keep.ld(p);
    r.t = a.x; r.s = a.y; r.pv = a.z;
    r.prow = make_int2(a.w, keep.ld(reinterpret_cast<const int32_t *>(p + 1)));
  } else {
    const int2 a = keep.ld(reinterpret_cast<const int2 *>(base) + i);
    r.t = a.x; r.s = a.y; r.pv = 0;
    r.prow = make_int2(0, 0);
  }
  return r;
}

// what the kernel writes for one settled pair
template <bool COUNT>
__device__ __forceinline__ void count_emit(const ndmem::Keep &keep, int i, int32_t s, int32_t nbr, int32_t V, int step,
                                           bool smem_bins, uint32_t *sh_bins, int32_t *__restrict__ out_key,
                                           int32_t *__restrict__ out_val, int32_t *__restrict__ out_rank,
                                           uint32_t *__restrict__ cnt, uint32_t *__restrict__ bsum,
                                           int32_t *__restrict__ tmp_step, int32_t *__restrict__ len,
                                           int4 *__restrict__ out_ext, int32_t t, int32_t rs, int32_t deg,
                                           bool ends_next = false) {  // the walk takes this vertex and is known to stop at the next step
  if (nbr >= 0) keep.st(tmp_step + s, nbr); else len[s] = step;
  if (ends_next) len[s] = step + 1;
  if (COUNT) {
    const bool in_map = nbr >= 0 && !ends_next;
    keep.st(out_key + i, in_map ? nbr : V);
    if (in_map) {
      keep.st(out_val + i, s);
      keep.st(out_rank + i, (int32_t)keep.atom_add(cnt + nbr, 1u));
      if (out_ext) keep.st(out_ext + i, make_int4(t, rs, deg, 0));  // node2vec: this transit is the pair's previous vertex next step
      if (smem_bins) atomicAdd(&sh_bins[nbr >> CNT_SUPER_SHIFT], 1u);
      else atomicAdd(&bsum[nbr >> CNT_SUPER_SHIFT], 1u);
    }
  }
}

template <int APP, bool COUNT>
__global__ void __launch_bounds__(COUNT_THREADS, count_ctas<APP>())
walk_next_count_kernel(NdGraphView g, WalkParams wp, int step, int64_t first_sample,
                       const void *__restrict__ in_rec, const int32_t *__restrict__ d_n,
                       int32_t *__restrict__ out_key, int32_t *__restrict__ out_val, int32_t *__restrict__ out_rank,
                       int4 *__restrict__ out_ext, uint32_t *__restrict__ cnt, uint32_t *__restrict__ bsum, int bins, int32_t *__restrict__ tmp_step,
                       int32_t *__restrict__ len, int *__restrict__ status, unsigned long long *__restrict__ stats,
                       int skip_hub_tiles) {
  constexpr int PPT = count_ppt<APP>();
  constexpr int QCAP = 32 * PPT + 32;
  constexpr bool N2V = APP == ND_APP_NODE2VEC;
  constexpr bool WEIGHTED = APP == ND_APP_DEEPWALK || APP == ND_APP_PPR;
  extern __shared__ uint32_t sh_dyn[];
  Events ev;
  const int n = *d_n;
  constexpr int TILE = COUNT_THREADS * PPT;
  if ((int64_t)blockIdx.x * TILE >= n) return;  // no pair for this CTA
  const bool smem_bins = COUNT && bins <= MAX_SMEM_BINS;
  uint32_t *sh_bins = sh_dyn;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int32_t *queue = reinterpret_cast<int32_t *>(sh_dyn + (smem_bins ? bins : 0)) + warp * QCAP;
  int q_count = 0;  // warp-uniform
  if (smem_bins) {
#pragma unroll 1
    for (int b = threadIdx.x; b < bins; b += COUNT_THREADS) sh_bins[b] = 0u;
    __syncthreads();
  }
  const N2vConsts c(wp);
  const ndmem::Keep keep;

  // runs 32 queued pairs (or the rest, when `all`) through the general loop.  A queue entry is the
  // pair's position in the map; bit 31 set = the first round rejected all its tries, so the loop
  // continues behind them in the pair's draw sequence; clear = the pair starts over (node2vec, a
  // membership test that the home bucket did not answer).
  constexpr uint32_t Q_CONTINUE = 0x80000000u;
  auto drain = [&](bool all) {
    while (q_count >= 32 || (all && q_count > 0)) {
      const int take = q_count < 32 ? q_count : 32;
      q_count -= take;
      __syncwarp();
      if (lane < take) {
        const uint32_t q = (uint32_t)queue[q_count + lane];
        const int i = (int)(q & ~Q_CONTINUE);
        const bool cont = (q & Q_CONTINUE) != 0u;
        const MapRec<N2V> r = map_rec_load<N2V>(keep, in_rec, i);
        const int32_t rs = keep.ld_const(g.row_ptr + r.t);
        const int32_t deg = keep.ld_const(g.row_ptr + r.t + 1) - rs;
        Rng rng(wp.seed, (uint32_t)(first_sample + r.s), (uint32_t)step, 0u);
        int32_t nbr = ROUND_AGAIN;
        if (N2V) {
          if (cont) { rng.seek(2u * N2V_FIRST); ev.n2v_tries += N2V_FIRST; }
          nbr = n2v_next_known<true, N2V_BATCH_COUNT>(g, wp, rs, deg, r.pv, r.prow.x, r.prow.y, rng, status, ev);
        }
        count_emit<COUNT>(keep, i, r.s, nbr, g.V, step, smem_bins, sh_bins, out_key, out_val, out_rank, cnt, bsum, tmp_step, len,
                          out_ext, r.t, rs, deg);
      }
      __syncwarp();
    }
  };

  for (int base = blockIdx.x * TILE; base < n; base += gridDim.x * TILE) {
    // opt-in staging of hub lists (uniform walk): a tile whose 256 pairs all stand on one transit
    // belongs to walk_next_hub_kernel
    if (APP == ND_APP_UNIFORM_WALK && PPT == 1 && skip_hub_tiles && hub_tile(in_rec, n, base / HUB_TILE) >= 0) continue;
    int idx[PPT];
    int32_t t[PPT], s[PPT], rs[PPT], deg[PPT], nbr[PPT];
    bool live[PPT], settled[PPT], cont[PPT];
    // ---- map entries
    int32_t pv[PPT];
    int2 prow[PPT];
#pragma unroll
    for (int k = 0; k < PPT; k++) {
      idx[k] = base + k * COUNT_THREADS + threadIdx.x;
      live[k] = idx[k] < n;
      MapRec<N2V> r;
      r.t = 0; r.s = 0; r.pv = 0; r.prow = make_int2(0, 0);
      if (live[k]) r = map_rec_load<N2V>(keep, in_rec, idx[k]);
      t[k] = r.t; s[k] = r.s; pv[k] = r.pv; prow[k] = r.prow;
    }
    // ---- row offsets
    float mw[PPT];
#pragma unroll
    for (int k = 0; k < PPT; k++) {
      mw[k] = 0.f;
      const bool ok = live[k] && t[k] >= 0 && t[k] < g.V;
      if (live[k] && !ok) atomicOr(status, ND_DEV_BAD_TRANSIT);
      rs[k] = ok ? keep.ld_const(g.row_ptr + t[k]) : 0;
      deg[k] = ok ? keep.ld_const(g.row_ptr + t[k] + 1) - rs[k] : 0;
      if (WEIGHTED) mw[k] = ok ? __ldg(g.max_w + t[k]) : 0.f;   // independent of the row offsets: one latency, not two
      nbr[k] = -1;
      cont[k] = false;
      settled[k] = deg[k] <= 0;  // next() runs only on transits with edges (src/nextdoor.cu:255,412)
    }
    // ---- first round
    if (APP == ND_APP_UNIFORM_WALK) {  // example/uniformRandWalk.cu:35-36
#pragma unroll
      for (int k = 0; k < PPT; k++) {
        Rng rng(wp.seed, (uint32_t)(first_sample + s[k]), (uint32_t)step, 0u);
        const int32_t x = rng.rand_int(deg[k] > 0 ? deg[k] : 1);
        if (deg[k] > 0) nbr[k] = __ldcs(g.col + rs[k] + x);
        settled[k] = true;
      }
    }
    if (WEIGHTED) {  // randomWalks.cu:74-90, 102-124: the rejection loop in place (rounds of two tries)
#pragma unroll
      for (int k = 0; k < PPT; k++) {
        if (deg[k] > 0) {
          Rng rng(wp.seed, (uint32_t)(first_sample + s[k]), (uint32_t)step, 0u);
          int32_t st = 0;
          nbr[k] = app_next<APP>(g, wp, step, t[k], rs[k], deg[k], st, rng, status, ev, true, mw[k]);
          settled[k] = true;
        }
      }
    }
    if (N2V) {  // randomWalks.cu:141-172
      int32_t x[PPT][N2V_FIRST], v[PPT][N2V_FIRST];
      float y[PPT][N2V_FIRST];
      int n_try[PPT];
      bool simple[PPT];
#pragma unroll
      for (int k = 0; k < PPT; k++) {
        simple[k] = deg[k] == 1 || step == 0;
        Rng rng(wp.seed, (uint32_t)(first_sample + s[k]), (uint32_t)step, 0u);
        n_try[k] = N2V_FIRST;
#pragma unroll
        for (int j = 0; j < N2V_FIRST; j++) {
          x[k][j] = 0; y[k][j] = 0.f;
          if (j < n_try[k]) {
            x[k][j] = rng.rand_int(deg[k] > 0 ? deg[k] : 1);
            y[k][j] = __fmul_rn(rng.uniform(), c.bound);
            if (y[k][j] < c.sure) n_try[k] = j + 1;
          }
        }
        if (simple[k]) { n_try[k] = 1; x[k][0] = 0; }
        if (deg[k] <= 0) n_try[k] = 0;
      }
#pragma unroll
      for (int k = 0; k < PPT; k++)
#pragma unroll
        for (int j = 0; j < N2V_FIRST; j++) v[k][j] = j < n_try[k] ? __ldcs(g.col + rs[k] + x[k][j]) : -1;
      bool is_ret[PPT][N2V_FIRST], need[PPT][N2V_FIRST];
      int4 ba[PPT][N2V_FIRST], bb[PPT][N2V_FIRST];
#pragma unroll
      for (int k = 0; k < PPT; k++) {
        const int32_t ts = prow[k].x, tn = prow[k].y;
        const uint32_t n_buckets = ((uint32_t)(ts + tn) >> 2) - ((uint32_t)ts >> 2);
        const int4 *__restrict__ region = reinterpret_cast<const int4 *>(wp.adjset) + 2 * (size_t)((uint32_t)ts >> 2);
#pragma unroll
        for (int j = 0; j < N2V_FIRST; j++) {
          is_ret[k][j] = wp.n2v_compat ? (x[k][j] == pv[k]) : (v[k][j] == pv[k]);  // randomWalks.cu:159 compares the index
          need[k][j] = !simple[k] && j < n_try[k] && !is_ret[k][j] && y[k][j] >= c.lo && y[k][j] < c.hi;
          const uint32_t bucket = set_bucket(v[k][j], n_buckets);
          const bool fetch = need[k][j] && tn >= SET_MIN_DEG;
          ba[k][j] = fetch ? __ldcs(region + 2 * (size_t)bucket) : make_int4(SET_EMPTY, SET_EMPTY, SET_EMPTY, SET_EMPTY);
          bb[k][j] = fetch ? __ldcs(region + 2 * (size_t)bucket + 1) : make_int4(SET_EMPTY, SET_EMPTY, SET_EMPTY, SET_EMPTY);
        }
      }
#pragma unroll
      for (int k = 0; k < PPT; k++) {
        if (deg[k] > 0) {
          if (simple[k]) {
            nbr[k] = v[k][0];
            settled[k] = true;
          } else {
            const bool use_set = prow[k].y >= SET_MIN_DEG;
            int32_t res = ROUND_AGAIN;
            uint32_t tries = (uint32_t)n_try[k], probes = 0;
            bool slow = false;  // a membership test the home bucket does not answer, before any accepted try
#pragma unroll
            for (int j = N2V_FIRST - 1; j >= 0; j--) {
              if (j < n_try[k]) {
                bool accept, unsure = false;
                uint32_t pj = 0;
                if (is_ret[k][j]) {
                  accept = y[k][j] < wp.p;
                } else if (!need[k][j]) {
                  accept = y[k][j] < c.lo;
                } else {
                  const int32_t vv = v[k][j];
                  const bool found = ba[k][j].x == vv || ba[k][j].y == vv || ba[k][j].z == vv || ba[k][j].w == vv ||
                                     bb[k][j].x == vv || bb[k][j].y == vv || bb[k][j].z == vv || bb[k][j].w == vv;
                  if (use_set) pj = 8;
                  unsure = !found && (!use_set || bb[k][j].w != SET_EMPTY);
                  accept = y[k][j] < (found ? c.inv_q : 1.0f);
                }
                // walking from the last try to the first: an earlier try overrides what later ones said
                if (unsure) { slow = true; res = ROUND_AGAIN; probes = 0; }
                else if (accept) { slow = false; res = v[k][j]; tries = j + 1; probes = pj; }
                else { probes += pj; }
              }
            }
            if (!slow && res != ROUND_AGAIN) {
              nbr[k] = res; settled[k] = true;
              ev.n2v_tries += tries; ev.n2v_probes += probes;
            } else if (!slow) {  // every try rejected: the queue continues behind them
              cont[k] = true;
              ev.n2v_probes += probes;
            }
          }
        }
      }
    }
    // ---- settled pairs are written, the others queued
#pragma unroll
    for (int k = 0; k < PPT; k++)
      if (live[k] && settled[k]) {
        // PPR: whether a walk stops at a step is the first draw of that step's keyed sequence and does
        // not depend on where the walk stands, so the next step's verdict is known now: a pair that
        // would only enter the next map to be dropped from it takes no ticket and is not scattered.
        // (Not in the step that feeds the tail launch: the result update that runs beside the tail
        // tells the tail's walks from the others by their length, and a walk ended here would have
        // the length of one that the tail is about to continue.)
        bool ends_next = false;
        if (APP == ND_APP_PPR && COUNT && nbr[k] >= 0 && step != wp.keep_all_step) {
          Rng ahead(wp.seed, (uint32_t)(first_sample + s[k]), (uint32_t)(step + 1), 0u);
          ends_next = ahead.uniform() < wp.stop_prob;
          ev.not_entered += ends_next ? 1u : 0u;
        }
        count_emit<COUNT>(keep, idx[k], s[k], nbr[k], g.V, step, smem_bins, sh_bins, out_key, out_val, out_rank, cnt, bsum, tmp_step, len,
                          out_ext, t[k], rs[k], deg[k], ends_next);
      }
    if (APP != ND_APP_UNIFORM_WALK) {
#pragma unroll
      for (int k = 0; k < PPT; k++) {
        const bool push = live[k] && !settled[k];
        const uint32_t m = __ballot_sync(0xffffffffu, push);
        if (push) queue[q_count + __popc(m & ((1u << lane) - 1u))] = (int32_t)((uint32_t)idx[k] | (cont[k] ? Q_CONTINUE : 0u));
        q_count += __popc(m);
      }
      drain(false);
    }
  }
  if (APP != ND_APP_UNIFORM_WALK) drain(true);
  if (smem_bins) {
    __syncthreads();
#pragma unroll 1
    for (int b = threadIdx.x; b < bins; b += COUNT_THREADS) {
      const uint32_t cb = sh_bins[b];
      if (cb) atomicAdd(&bsum[b], cb);
    }
  }
  if (APP != ND_APP_UNIFORM_WALK) ev.flush_cta(stats);
}

template <bool COUNT>
__global__ void __launch_bounds__(HUB_TILE)
walk_next_hub_kernel(NdGraphView g, WalkParams wp, int step, int64_t first_sample, const void *__restrict__ in_rec,
                     const int32_t *__restrict__ d_n, int32_t *__restrict__ out_key, int32_t *__restrict__ out_val,
                     int32_t *__restrict__ out_rank, uint32_t *__restrict__ cnt, uint32_t *__restrict__ bsum,
                     int32_t *__restrict__ tmp_step, int32_t *__restrict__ len) {
  __shared__ int32_t sh_list[HUB_CHUNK];
  const ndmem::Keep keep;
  const int n = *d_n;
  const int tiles = n / HUB_TILE;
  const int2 *rec = reinterpret_cast<const int2 *>(in_rec);
  for (int tau = blockIdx.x; tau < tiles; tau += gridDim.x) {
    const int32_t t = hub_tile(in_rec, n, tau);
    if (t < 0 || hub_tile(in_rec, n, tau - 1) == t) continue;       // not the first tile of a run
    int nt = 1;
    while (hub_tile(in_rec, n, tau + nt) == t) nt++;
    const bool ok = t < g.V;
    const int32_t rs = ok ? __ldg(g.row_ptr + t) : 0;
    const int32_t deg = ok ? __ldg(g.row_ptr + t + 1) - rs : 0;
    for (int j0 = 0; j0 < nt; j0 += HUB_PASS) {
      const int m = nt - j0 < HUB_PASS ? nt - j0 : HUB_PASS;
      int32_t smp[HUB_PASS], x[HUB_PASS], nbr[HUB_PASS];
#pragma unroll
      for (int j = 0; j < HUB_PASS; j++) {
        smp[j] = 0; x[j] = -1; nbr[j] = -1;
        if (j < m) {
          smp[j] = rec[(tau + j0 + j) * HUB_TILE + threadIdx.x].y;
          Rng rng(wp.seed, (uint32_t)(first_sample + smp[j]), (uint32_t)step, 0u);
          if (deg > 0) x[j] = rng.rand_int(deg);
        }
      }
      for (int c0 = 0; c0 < deg; c0 += HUB_CHUNK) {
        const int cn = deg - c0 < HUB_CHUNK ? deg - c0 : HUB_CHUNK;
        for (int i = threadIdx.x; i < cn; i += HUB_TILE) sh_list[i] = __ldg(g.col + rs + c0 + i);
        __syncthreads();
#pragma unroll
        for (int j = 0; j < HUB_PASS; j++)
          if (x[j] >= c0 && x[j] < c0 + cn) nbr[j] = sh_list[x[j] - c0];
        __syncthreads();
      }
#pragma unroll
      for (int j = 0; j < HUB_PASS; j++)
        if (j < m)
          count_emit<COUNT>(keep, (int)((tau + j0 + j) * HUB_TILE + threadIdx.x), smp[j], nbr[j], g.V, step, false, nullptr, out_key,
                            out_val, out_rank, cnt, bsum, tmp_step, len, nullptr, 0, 0, 0);
    }
  }
}

// CTA b owns the counters of coarse bin b: its base is the sum of the bins before it; exclusive
// scan of its counters into offs; counters cleared for the next step; the last CTA publishes the
// number of live pairs.  A bin nobody drew a ticket in holds no transit of the next step: its
// offsets are never read and its counters are zero already.
__global__ void __launch_bounds__(SCAN_THREADS)
cnt_scan_kernel(uint32_t *__restrict__ cnt, const uint32_t *__restrict__ bsum, uint32_t *__restrict__ offs,
                int32_t *__restrict__ d_n_out) {
  __shared__ uint32_t wsum[SCAN_THREADS / 32];
  __shared__ uint32_t base_sh;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool is_last = blockIdx.x == gridDim.x - 1;
  const uint32_t own = bsum[blockIdx.x];
  if (own == 0u && !is_last) return;
  uint32_t part = 0;
  for (int i = threadIdx.x; i < (int)blockIdx.x; i += SCAN_THREADS) part += bsum[i];
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  if (lane == 0) wsum[warp] = part;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t t = 0;
    for (int w = 0; w < SCAN_THREADS / 32; w++) t += wsum[w];
    base_sh = t;
  }
  __syncthreads();
  if (own == 0u) {  // last CTA, empty bin
    if (threadIdx.x == 0) *d_n_out = (int32_t)base_sh;
    return;
  }
  // each thread owns SCAN_PER_THREAD consecutive counters (the arrays are padded to whole bins)
  const size_t first = (size_t)blockIdx.x * CNT_SUPER + (size_t)threadIdx.x * SCAN_PER_THREAD;
  uint32_t c[SCAN_PER_THREAD];
  uint32_t tsum = 0;
#pragma unroll
  for (int r = 0; r < SCAN_PER_THREAD / 4; r++) {
    const uint4 a = *reinterpret_cast<const uint4 *>(cnt + first + 4 * r);
    c[4 * r] = a.x; c[4 * r + 1] = a.y; c[4 * r + 2] = a.z; c[4 * r + 3] = a.w;
    tsum += a.x + a.y + a.z + a.w;
  }
  uint32_t inc = tsum;
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  __syncthreads();  // wsum reuse
  if (lane == 31) wsum[warp] = inc;
  __syncthreads();
  uint32_t run = base_sh + inc - tsum;
  for (int w = 0; w < warp; w++) run += wsum[w];
  if (tsum != 0u) {  // a thread without tickets has nothing to publish or clear
#pragma unroll
    for (int r = 0; r < SCAN_PER_THREAD / 4; r++) {
      uint4 o;
      o.x = run; run += c[4 * r];
      o.y = run; run += c[4 * r + 1];
      o.z = run; run += c[4 * r + 2];
      o.w = run; run += c[4 * r + 3];
      *reinterpret_cast<uint4 *>(offs + first + 4 * r) = o;
      *reinterpret_cast<uint4 *>(cnt + first + 4 * r) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  if (is_last && threadIdx.x == SCAN_THREADS - 1) *d_n_out = (int32_t)run;
}

// Moves every live pair to its place in the sorted map of the next step -- one record, one random
// sector write (see MapRec) -- and clears the coarse bins (the scan before it was their last reader).
constexpr int SCATTER_PPT = 2;
template <bool N2V>
__global__ void __launch_bounds__(256)
walk_scatter_kernel(const int32_t *__restrict__ d_n, int32_t V, const int32_t *__restrict__ ukey,
                    const int32_t *__restrict__ uval, const int32_t *__restrict__ urank,
                    const int4 *__restrict__ uext, const uint32_t *__restrict__ offs, void *__restrict__ out_rec,
                    uint32_t *__restrict__ bsum, int bins) {
  const int n = *d_n;
  const ndmem::Keep keep;
  for (int b = blockIdx.x * blockDim.x + threadIdx.x; b < bins; b += gridDim.x * blockDim.x) bsum[b] = 0u;
  constexpr int TILE = 256 * SCATTER_PPT;
  for (int base = blockIdx.x * TILE; base < n; base += gridDim.x * TILE) {
    int32_t k[SCATTER_PPT], v[SCATTER_PPT], r[SCATTER_PPT];
    int4 ext[SCATTER_PPT];
    uint32_t pos[SCATTER_PPT];
#pragma unroll
    for (int j = 0; j < SCATTER_PPT; j++) {
      const int i = base + j * 256 + threadIdx.x;
      k[j] = i < n ? keep.ld(ukey + i) : V;
      const bool ok = k[j] != V;
      v[j] = ok ? keep.ld(uval + i) : 0;
      r[j] = ok ? keep.ld(urank + i) : 0;
      if (N2V) ext[j] = ok ? keep.ld(uext + i) : make_int4(0, 0, 0, 0);
    }
#pragma unroll
    for (int j = 0; j < SCATTER_PPT; j++) pos[j] = k[j] != V ? keep.ld(offs + k[j]) + (uint32_t)r[j] : 0u;
#pragma unroll
    for (int j = 0; j < SCATTER_PPT; j++) {
      if (k[j] != V) {
        if (N2V) {
          int4 *dst = reinterpret_cast<int4 *>(out_rec) + 2 * (size_t)pos[j];
          keep.st(dst, make_int4(k[j], v[j], ext[j].x, ext[j].y));
          keep.st(dst + 1, make_int4(ext[j].z, 0, 0, 0));
        } else {
          keep.st(reinterpret_cast<int2 *>(out_rec) + pos[j], make_int2(k[j], v[j]));
        }
      }
    }
  }
}

// the transit-sorted initial map (key, value arrays) as records
template <bool N2V>
__global__ void __launch_bounds__(256)
pack_map_kernel(const int32_t *__restrict__ d_n, const int32_t *__restrict__ key, const int32_t *__restrict__ val,
                void *__restrict__ rec) {
  const int n = *d_n;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    if (N2V) {
      int4 *dst = reinterpret_cast<int4 *>(rec) + 2 * (size_t)i;
      dst[0] = make_int4(key[i], val[i], 0, 0);
      dst[1] = make_int4(0, 0, 0, 0);
    } else {
      reinterpret_cast<int2 *>(rec)[i] = make_int2(key[i], val[i]);
    }
  }
}

// Row start, degree and maximum weight of a vertex for a kernel that reaches it by a random id: the
// two neighbouring 8-byte records share a 32-byte sector three times out of four, where the row
// offsets and the maximum weights are two arrays and two sectors.
__device__ __forceinline__ void vertex_of(const WalkParams &wp, int32_t v, int32_t &rs, int32_t &deg, float &max_w) {
  const int2 a = __ldg(wp.vrec + v), b = __ldg(wp.vrec + v + 1);
  rs = a.x;
  deg = b.x - rs;
  max_w = __int_as_float(a.y);
}

// The tail of a job whose walks end early (PPR): once few walks are still alive, a step of the
// transit-parallel loop is three launches whose fixed cost outweighs the per-pair work.  From
// there on one launch finishes the job, a lane per walk: a lane takes a pair of the sorted map
// (a batch of indices per warp from a device counter, so that the lanes end together) and walks its sample to
// the end; a warp makes one round of tries per trip as walk_sp_rounds_kernel does, and a lane
// whose walk ended takes the next pair.  The draws are keyed by (sample, step), so the samples are
// the ones the step-by-step loop would have produced.
// DIRECT: the launch lasts at least as long as the longest surviving walk's chain of dependent
// loads and leaves most of the memory system idle, so it runs on a second stream beside the result
// update of the walks that ended in the step loop (walk_finalize_sparse_kernel with tail_from =
// first_step).  The two kernels split the result rows between them: a survivor's slots from
// first_step on, its entry of plen and its share of the counters belong to this kernel, everything
// else to the other.
template <int APP, bool DIRECT>
__global__ void __launch_bounds__(256, walk_min_ctas_sp<APP>())
walk_tail_kernel(NdGraphView g, WalkParams wp, int first_step, int64_t first_sample, const void *__restrict__ in_rec,
                 const int32_t *__restrict__ d_n, int32_t *__restrict__ next_pair, int64_t S, int32_t *__restrict__ tmp,
                 int32_t *__restrict__ len, int32_t *__restrict__ plen, int32_t *__restrict__ out, int *__restrict__ status,
                 unsigned long long *__restrict__ stats) {
  static_assert(APP == ND_APP_DEEPWALK || APP == ND_APP_PPR, "weighted walks only");
  Events ev;
  const ndmem::Keep keep;
  const int n = *d_n;
  const int lane = threadIdx.x & 31;
  constexpr int TAIL_BATCH = 64;   // at least the 32 indices one trip can ask for
  bool have = false, fresh = true, done = false;
  int32_t s = 0, cur = 0, rs = 0, deg = 0, had = 0;
  int step = 0, rounds = 0;
  int w_cur = 0, w_end = 0;
  float max_w = 0.f;
  int32_t *row = nullptr;
  unsigned int edges = 0, live = 0;
  Rng rng(wp.seed, 0u, 0u, 0u);
  while (true) {
    // The lanes without a walk take the next pair indices of the warp's batch; the warp draws a
    // batch of TAIL_BATCH indices from the device counter when the batch runs out.  (Some lane's
    // walk ends in almost every trip, and an atomic with its round trip to the L2 in every trip
    // doubled the trip: the 1 M-pair tail of the 2^24-vertex job took 0.75 ms with one atomic per
    // trip.)  w_cur / w_end are the same in all lanes.
    const unsigned want = __ballot_sync(0xffffffffu, !done && !have);
    if (want) {
      const int need = __popc(want), avail = w_end - w_cur;
      const int my = __popc(want & ((1u << lane) - 1u));
      int i = w_cur + my;
      if (need <= avail) {
        w_cur += need;
      } else {
        int nb = 0;
        if (lane == 0) nb = atomicAdd(next_pair, TAIL_BATCH);
        nb = __shfl_sync(0xffffffffu, nb, 0);
        if (my >= avail) i = nb + (my - avail);
        w_cur = nb + (need - avail);
        w_end = nb + TAIL_BATCH;
      }
      if (!done && !have) {
        if (i >= n) {
          done = true;
        } else {
          const MapRec<false> r = map_rec_load<false>(keep, in_rec, i);
          s = r.s;
          cur = r.t;
          step = first_step;
          have = true;
          fresh = true;
          if (cur >= 0 && cur < g.V) {
            vertex_of(wp, cur, rs, deg, max_w);
          } else {
            deg = 0;
          }
          if (DIRECT) {
            row = out + (int64_t)s * wp.steps;
            had = plen[s];
          }
        }
      }
    }
    if (!__any_sync(0xffffffffu, have)) break;   // no lane holds a walk, so every lane found the map exhausted
    if (have) {
      int32_t nbr = ROUND_AGAIN;
      if (deg == 0) {
        nbr = -1;
      } else if (fresh) {  // first trip of a step: the draws of the step start, the cases without a rejection loop
        rng = Rng(wp.seed, (uint32_t)(first_sample + s), (uint32_t)step, 0u);
        rounds = 0;
        fresh = false;
        if (APP == ND_APP_PPR) {
          const float pr = rng.uniform();
          if (pr < wp.stop_prob) nbr = -1;
        }
        if (nbr == ROUND_AGAIN && deg == 1) nbr = __ldg(g.col + rs);
      }
      if (nbr == ROUND_AGAIN) {
        nbr = weighted_round<false, 2>(wp, rs, deg, max_w, rng, ev);
        if (nbr == ROUND_AGAIN && ++rounds > RETRY_CAP) {
          atomicOr(status, ND_DEV_RETRY_LIMIT);
          nbr = __ldg(g.col + rs);
        }
      }
      if (nbr >= 0) {
        if (DIRECT) row[step] = nbr;
        else tmp[(int64_t)step * S + s] = nbr;
        cur = nbr;
        if (++step < wp.steps) {
          vertex_of(wp, cur, rs, deg, max_w);
          fresh = true;
        }
      }
      if (nbr == -1 || step == wp.steps) {  // the walk ends here, after `step` vertices
        if (step < wp.steps) len[s] = step;
        if (DIRECT) {
          for (int k = step; k < had; k++) row[k] = g.V;   // slots the previous pass filled beyond this walk's end
          if (had != step) plen[s] = step;
          edges += step - first_step;
          live += (step < wp.steps ? step + 1 : wp.steps) - first_step;
        }
        have = false;
      }  // ROUND_AGAIN: the lane stays on its step
    }
  }
  if (DIRECT) {
    for (int o = 16; o > 0; o >>= 1) {
      edges += __shfl_xor_sync(0xffffffffu, edges, o);
      live += __shfl_xor_sync(0xffffffffu, live, o);
    }
    if (lane == 0) {
      if (edges) atomicAdd(&stats[0], (unsigned long long)edges);
      if (live) atomicAdd(&stats[1], (unsigned long long)live);
    }
  }
  ev.flush(stats);
}

// ---------------------------------------------------------------- sample-parallel: a thread owns a walk

template <int APP>
__global__ void __launch_bounds__(256, walk_min_ctas_sp<APP>())
walk_sp_kernel(NdGraphView g, WalkParams wp, int64_t first_sample, int64_t S,
               const int32_t *__restrict__ initial, int32_t *__restrict__ tmp,
               int32_t *__restrict__ len, int *__restrict__ status, unsigned long long *__restrict__ stats) {
  Events ev;
  for (int64_t s = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; s < S;
       s += (int64_t)gridDim.x * blockDim.x) {
    int32_t cur = initial[s];
    if (cur < 0 || cur >= g.V) continue;  // len already -1
    int32_t st = 0;
    int step = 0;
    for (; step < wp.steps; step++) {
      const int32_t rs = __ldg(g.row_ptr + cur);
      const int32_t deg = __ldg(g.row_ptr + cur + 1) - rs;
      int32_t nbr = -1;
      if (deg > 0) {
        Rng rng(wp.seed, (uint32_t)(first_sample + s), (uint32_t)step, 0u);
        nbr = app_next<APP, false, N2V_BATCH_SP>(g, wp, step, cur, rs, deg, st, rng, status, ev);
      }
      if (nbr < 0) break;
      tmp[(int64_t)step * S + s] = nbr;
      cur = nbr;
    }
    if (step < wp.steps) len[s] = step;
  }
  if (APP != ND_APP_UNIFORM_WALK) ev.flush(stats);
}

// Sample-parallel walks of the apps with a rejection loop, as a per-lane state machine.  In
// walk_sp_kernel a warp spends, at every step, as many rounds as its unluckiest lane (about 2.2
// rounds per step for node2vec although a walk needs 1.13 on average).  Here a loop trip is ONE
// round for every lane, wherever its walk stands: a lane whose try was accepted moves on to its
// next step (the row offsets of the new vertex are fetched at the end of the trip, so that the
// next trip starts with them in registers), a lane that was rejected stays on its step, a lane
// whose walk ended takes the next walk.  Over 100 steps the lanes' round counts even out, so a
// warp makes about as many trips as the average walk needs rounds.  Draws are keyed by (sample,
// step) and counted per step, so the walks are the same as in every other kernel.
template <int APP>
__global__ void __launch_bounds__(256, walk_min_ctas_sp<APP>())
walk_sp_rounds_kernel(NdGraphView g, WalkParams wp, int64_t first_sample, int64_t S,
                      const int32_t *__restrict__ initial, int32_t *__restrict__ tmp,
                      int32_t *__restrict__ len, int *__restrict__ status, unsigned long long *__restrict__ stats) {
  constexpr bool N2V = APP == ND_APP_NODE2VEC;
  Events ev;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t s = blockIdx.x * (int64_t)blockDim.x + threadIdx.x - stride;
  bool have = false, fresh = true;
  int32_t cur = 0, rs = 0, deg = 0, prev = 0, ts = 0, tn = 0;
  int step = 0, rounds = 0;
  float max_w = 0.f;
  Rng rng(wp.seed, 0u, 0u, 0u);
  const N2vConsts c(wp);
  bool done = false;  // this lane has no walk left
  // every lane of the warp stays in the loop until the last one is done: the vote at the loop
  // head is where the lanes meet again after a trip, so that a trip runs as one instruction stream
  while (__any_sync(0xffffffffu, !done)) {
    if (!done && !have) {  // take the next walk of this lane
      s += stride;
      if (s >= S) {
        done = true;
      } else {
        cur = initial[s];
        if (cur >= 0 && cur < g.V) {  // otherwise len is -1 already and the lane tries the next walk in the next trip
          if (N2V) {
            rs = __ldg(g.row_ptr + cur);
            deg = __ldg(g.row_ptr + cur + 1) - rs;
          } else {
            vertex_of(wp, cur, rs, deg, max_w);
          }
          step = 0;
          have = true;
          fresh = true;
        }
      }
    }
    if (have) {
      int32_t nbr = ROUND_AGAIN;
      if (deg == 0) {
        nbr = -1;
      } else if (fresh) {  // first trip of a step: the draws of the step start, the cases without a rejection loop
        rng = Rng(wp.seed, (uint32_t)(first_sample + s), (uint32_t)step, 0u);
        rounds = 0;
        fresh = false;
        if (APP == ND_APP_PPR) {
          const float pr = rng.uniform();
          if (pr < wp.stop_prob) nbr = -1;
        }
        if (nbr == ROUND_AGAIN && (deg == 1 || (N2V && step == 0))) nbr = __ldg(g.col + rs);
      }
      if (nbr == ROUND_AGAIN) {
        if (N2V) nbr = n2v_round<false, N2V_BATCH_SP>(g, wp, c, rs, deg, prev, ts, tn, rng, ev);
        else nbr = weighted_round<false, 2>(wp, rs, deg, max_w, rng, ev);
        if (nbr == ROUND_AGAIN && ++rounds > RETRY_CAP) {
          atomicOr(status, ND_DEV_RETRY_LIMIT);
          nbr = __ldg(g.col + rs);
        }
      }
      if (nbr == -1) {  // the walk ends here
        len[s] = step;
        have = false;
      } else if (nbr >= 0) {
        tmp[(int64_t)step * S + s] = nbr;
        prev = cur; ts = rs; tn = deg;
        cur = nbr;
        if (++step == wp.steps) {
          have = false;
        } else {
          if (N2V) {
            rs = __ldg(g.row_ptr + cur);
            deg = __ldg(g.row_ptr + cur + 1) - rs;
          } else {
            vertex_of(wp, cur, rs, deg, max_w);
          }
          fresh = true;
        }
      }  // ROUND_AGAIN: the lane stays on its step
    }
  }
  ev.flush(stats);
}

// ---------------------------------------------------------------- finalize: step-major -> sample-major

constexpr int FIN_SAMPLES = 32;   // samples per CTA
constexpr int FIN_THREADS = 256;

// Step-major staging -> the reference's sample-major rows, every row written whole: a CTA takes 32
// samples, transposes through shared memory and stores 16 bytes per thread.  The kernel of the
// apps whose walks run their full length (uniform walk, DeepWalk, node2vec).
constexpr int FIN_MAX_STEPS = 128;  // steps per smem chunk
__global__ void __launch_bounds__(FIN_THREADS)
walk_finalize_kernel(const int32_t *__restrict__ tmp, const int32_t *__restrict__ len, int32_t *__restrict__ plen, int64_t S,
                     int steps, int32_t invalid, int32_t *__restrict__ out,
                     unsigned long long *__restrict__ stats) {
  __shared__ int32_t tile[FIN_MAX_STEPS][FIN_SAMPLES + 1];
  __shared__ int32_t sh_len[FIN_SAMPLES];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t groups = (S + FIN_SAMPLES - 1) / FIN_SAMPLES;
  unsigned long long edges = 0, live = 0;
  for (int64_t grp = blockIdx.x; grp < groups; grp += gridDim.x) {
    const int64_t s0 = grp * FIN_SAMPLES;
    const int ns = (int)(S - s0 < FIN_SAMPLES ? S - s0 : FIN_SAMPLES);
    if (threadIdx.x < FIN_SAMPLES) {
      const int32_t l = threadIdx.x < ns ? len[s0 + threadIdx.x] : -1;
      sh_len[threadIdx.x] = l;
      if (threadIdx.x < ns) {
        plen[s0 + threadIdx.x] = l > 0 ? l : 0;   // every row is written whole: its slots beyond the walk hold the invalid id
        edges += l > 0 ? l : 0;
        live += l < 0 ? 0 : (l < steps ? l + 1 : steps);
      }
    }
    __syncthreads();
    for (int k0 = 0; k0 < steps; k0 += FIN_MAX_STEPS) {
      const int kc = steps - k0 < FIN_MAX_STEPS ? steps - k0 : FIN_MAX_STEPS;
      const int32_t mylen = sh_len[lane];
      for (int k = warp; k < kc; k += FIN_THREADS / 32) {
        int32_t v = invalid;
        if (lane < ns && k0 + k < mylen) v = tmp[(int64_t)(k0 + k) * S + s0 + lane];
        tile[k][lane] = v;
      }
      __syncthreads();
      // rows of `steps` ints, ns of them back to back
      if (kc == steps) {  // the group's rows are one contiguous, 128-byte aligned piece: 16-byte stores
        int32_t *dst = out + s0 * steps;
        const int total = ns * steps, quads = total >> 2;
        for (int q = threadIdx.x; q < quads; q += FIN_THREADS) {
          int i = (4 * q) / steps, k = 4 * q - i * steps;
          int32_t e[4];
#pragma unroll
          for (int c = 0; c < 4; c++) {
            e[c] = tile[k][i];
            if (++k == steps) { k = 0; i++; }
          }
          __stcs(reinterpret_cast<int4 *>(dst) + q, make_int4(e[0], e[1], e[2], e[3]));
        }
        for (int j = (quads << 2) + threadIdx.x; j < total; j += FIN_THREADS) dst[j] = tile[j % steps][j / steps];
      } else {
        for (int j = threadIdx.x; j < ns * kc; j += FIN_THREADS) {
          const int i = j / kc, k = j % kc;
          out[(s0 + i) * steps + k0 + k] = tile[k][i];
        }
      }
      __syncthreads();
    }
  }
  // CTA-level reduction of the counters, one atomic each
  for (int o = 16; o > 0; o >>= 1) {
    edges += __shfl_xor_sync(0xffffffffu, edges, o);
    live += __shfl_xor_sync(0xffffffffu, live, o);
  }
  if (threadIdx.x == 0 && stats) {  // only warp 0 accumulated
    if (edges) atomicAdd(&stats[0], edges);
    if (live) atomicAdd(&stats[1], live);
  }
}


// The result array keeps its contents from pass to pass, and the kernel keeps the invariant that
// out[s][k] holds the invalid id for every k >= plen[s]: a pass therefore only has to write the
// slots a walk fills now or filled last time.  For walks that end early (PPR: 3 valid steps on
// average in rows of 100) that is a few per cent of the array, where writing every row in full is
// 6.7 GB per pass on the 2^24-vertex job and as long as a quarter of the sampling itself.  Groups
// of 32 samples whose rows need more than FIN_SPARSE slots on average (a scattered 4-byte store
// costs the memory system a sector, so beyond that writing the rows whole is cheaper) go through
// the shared-memory transpose and are written whole, with 16-byte stores.
constexpr int FIN_SPARSE = 8;
constexpr int FIN_BATCH = 8;    // staged rows a lane reads at once
constexpr float FIN_SPARSE_STOP = 0.04f;  // PPR stop probability from which the result update takes this kernel

__global__ void __launch_bounds__(FIN_THREADS)
walk_finalize_sparse_kernel(const int32_t *__restrict__ tmp, const int32_t *__restrict__ len, int32_t *__restrict__ plen, int64_t S,
                     int steps, int32_t invalid, int32_t *__restrict__ out,
                     unsigned long long *__restrict__ stats, int tail_from) {
  // a warp owns a group of 32 samples (lane = sample) from start to end: no block barrier anywhere
  __shared__ int32_t tiles[FIN_THREADS / 32][32][FIN_SAMPLES + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int32_t (*tile)[FIN_SAMPLES + 1] = tiles[warp];
  const int64_t groups = (S + FIN_SAMPLES - 1) / FIN_SAMPLES;
  const int64_t warps = (int64_t)gridDim.x * (FIN_THREADS / 32);
  unsigned long long edges = 0, live = 0;
  for (int64_t grp = (int64_t)blockIdx.x * (FIN_THREADS / 32) + warp; grp < groups; grp += warps) {
    const int64_t s0 = grp * FIN_SAMPLES;
    const int ns = (int)(S - s0 < FIN_SAMPLES ? S - s0 : FIN_SAMPLES);
    const int32_t l = lane < ns ? len[s0 + lane] : -1;
    // A walk that was alive after step tail_from - 1 is being finished by the tail kernel while this
    // kernel runs (tail_from > steps: no such kernel).  Its length entry reads as `steps` or as its
    // final length, at least tail_from either way; this kernel writes its slots below tail_from and
    // leaves the rest of the row, the row's plen entry and the rest of its counts to the tail kernel.
    const bool surv = l >= tail_from;
    const int32_t had = lane < ns && !surv ? plen[s0 + lane] : 0;
    const int32_t now = surv ? tail_from : (l > 0 ? l : 0);
    const int32_t need = now > had ? now : had;
    if (lane < ns) {
      edges += now;
      live += surv ? tail_from : (l < 0 ? 0 : (l < steps ? l + 1 : steps));
      if (!surv && now != had) plen[s0 + lane] = now;
    }
    const int width = __reduce_max_sync(0xffffffffu, need);   // slots the widest row of the group has to (re)write
    const int total = __reduce_add_sync(0xffffffffu, need);   // ... and all its rows together
    // (a group with a survivor never takes the whole-row path: that one would write the tail kernel's slots)
    if (total <= FIN_SPARSE * FIN_SAMPLES || (steps & 3) != 0 || __any_sync(0xffffffffu, surv)) {
      // the staged row k is read coalesced, each sample's row gets only its few slots
      int32_t *row = out + (s0 + lane) * steps;
      for (int k0 = 0; k0 < width; k0 += FIN_BATCH) {   // the loads of a batch are in flight together
        int32_t v[FIN_BATCH];
#pragma unroll
        for (int j = 0; j < FIN_BATCH; j++) v[j] = k0 + j < now ? tmp[(int64_t)(k0 + j) * S + s0 + lane] : invalid;
#pragma unroll
        for (int j = 0; j < FIN_BATCH; j++)
          if (k0 + j < need) row[k0 + j] = v[j];
      }
      continue;
    }
    // rows written whole, 32 steps at a time through the warp's tile, 16-byte stores
    for (int k0 = 0; k0 < steps; k0 += 32) {
      const int kc = steps - k0 < 32 ? steps - k0 : 32;   // a multiple of 4
      for (int kb = 0; kb < kc; kb += FIN_BATCH) {
        int32_t v[FIN_BATCH];
#pragma unroll
        for (int j = 0; j < FIN_BATCH; j++) {
          const int k = k0 + kb + j;
          v[j] = (lane < ns && kb + j < kc && k < now) ? tmp[(int64_t)k * S + s0 + lane] : invalid;
        }
#pragma unroll
        for (int j = 0; j < FIN_BATCH; j++)
          if (kb + j < kc) tile[kb + j][lane] = v[j];
      }
      __syncwarp();
      const int qn = kc >> 2;                              // 16-byte pieces per sample in this chunk
      for (int q = lane; q < ns * qn; q += 32) {
        const int i = q / qn, c = q - i * qn;
        const int4 v = make_int4(tile[4 * c][i], tile[4 * c + 1][i], tile[4 * c + 2][i], tile[4 * c + 3][i]);
        __stcs(reinterpret_cast<int4 *>(out + (s0 + i) * steps + k0) + c, v);
      }
      __syncwarp();
    }
  }
  // CTA-level reduction of the counters, one atomic per warp
  for (int o = 16; o > 0; o >>= 1) {
    edges += __shfl_xor_sync(0xffffffffu, edges, o);
    live += __shfl_xor_sync(0xffffffffu, live, o);
  }
  if (lane == 0 && stats) {
    if (edges) atomicAdd(&stats[0], edges);
    if (live) atomicAdd(&stats[1], live);
  }
}

// fills the result array with the invalid id once, when the sampler is made (see walk_finalize_kernel)
__global__ void walk_fill_kernel(int32_t *__restrict__ out, int64_t n4, int64_t n, int32_t v) {
  const int4 q = make_int4(v, v, v, v);
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x)
    reinterpret_cast<int4 *>(out)[i] = q;
  for (int64_t i = 4 * n4 + blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) out[i] = v;
}

template <int APP>
int launch_next_tp(nd_sampler *s, const WalkParams &wp, int step, bool hist, int grid, const int32_t *in_key,
                   const int32_t *in_val, const int32_t *d_n, int32_t *out_key, int32_t *out_val) {
  const NdRadixPlan &pl = s->radix.plan;
  const int bins = 1 << pl.bits[0];
  NdGraphView gv = nd_view(s->g);
  int32_t *tmp_step = s->d_tmp + (int64_t)step * s->S;
  if (hist) {
    walk_next_tp_kernel<APP, true><<<grid, NEXT_THREADS, 2 * bins * sizeof(uint32_t), s->stream>>>(
        gv, wp, step, s->first, pl.tile, in_key, in_val, d_n, out_key, out_val, tmp_step, s->d_len,
        s->d_state, pl.shift[0], bins, s->radix.tile_hist, pl.max_tiles, s->radix.ghist, s->d_status, s->d_stats);
  } else {
    walk_next_tp_kernel<APP, false><<<grid, NEXT_THREADS, 0, s->stream>>>(
        gv, wp, step, s->first, pl.tile, in_key, in_val, d_n, out_key, out_val, tmp_step, s->d_len,
        s->d_state, 0, 1, nullptr, 0, nullptr, s->d_status, s->d_stats);
  }
  return ND_OK;
}

// next() of one step in the load-balanced mode: as many CTAs as are resident, at most one per tile
template <int APP>
int launch_count(nd_sampler *s, const WalkParams &wp, int step, bool last, int bins, const void *in_rec, const int32_t *d_n,
                 int32_t *ukey, int32_t *uval, int32_t *tmp_step) {
  constexpr int PPT = count_ppt<APP>();
  const size_t smem = sizeof(uint32_t) * ((bins <= MAX_SMEM_BINS && !last ? (size_t)bins : 0) + (size_t)COUNT_WARPS * (32 * PPT + 32));
  static int resident[2] = {0, 0};  // CTAs per SM (with and without the histogram), asked once
  int &res = resident[last ? 1 : 0];
  if (res == 0) {
    int r = 0;
    cudaError_t e = last ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&r, walk_next_count_kernel<APP, false>, COUNT_THREADS, smem)
                         : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&r, walk_next_count_kernel<APP, true>, COUNT_THREADS, smem);
    if (e != cudaSuccess || r < 1) { cudaGetLastError(); r = count_ctas<APP>(); }
    res = r;
  }
  const int64_t tiles = (s->S + COUNT_THREADS * PPT - 1) / (COUNT_THREADS * PPT);
  // node2vec: as many CTAs as are resident, each working through several tiles (its per-warp queues
  // fill up over the tiles); the others measured best with up to 16 CTAs per SM, a tile each
  const int64_t cap = (int64_t)s->dev.sms * (APP == ND_APP_NODE2VEC ? res : 16);
  const int grid = (int)(tiles < cap ? (tiles > 0 ? tiles : 1) : cap);
  NdGraphView gv = nd_view(s->g);
  int4 *uext = APP == ND_APP_NODE2VEC && !last ? s->d_uext : nullptr;
  const char *staging_env = getenv("ND_WALK_STAGING");   // opt-in: hub tiles of the uniform walk through walk_next_hub_kernel
  const int staging = APP == ND_APP_UNIFORM_WALK && count_ppt<APP>() == 1 && staging_env && staging_env[0] == '1' ? 1 : 0;
  if (last)
    walk_next_count_kernel<APP, false><<<grid, COUNT_THREADS, smem, s->stream>>>(
        gv, wp, step, s->first, in_rec, d_n, ukey, uval, s->d_rank, uext, s->d_cnt, s->d_bsum, bins,
        tmp_step, s->d_len, s->d_status, s->d_stats, staging);
  else
    walk_next_count_kernel<APP, true><<<grid, COUNT_THREADS, smem, s->stream>>>(
        gv, wp, step, s->first, in_rec, d_n, ukey, uval, s->d_rank, uext, s->d_cnt, s->d_bsum, bins,
        tmp_step, s->d_len, s->d_status, s->d_stats, staging);
  if (staging) {  // the hub tiles the kernel above left out
    const int hgrid = (int)(tiles < (int64_t)s->dev.sms * 8 ? (tiles > 0 ? tiles : 1) : (int64_t)s->dev.sms * 8);
    if (last)
      walk_next_hub_kernel<false><<<hgrid, HUB_TILE, 0, s->stream>>>(gv, wp, step, s->first, in_rec, d_n, ukey, uval, s->d_rank,
                                                                     s->d_cnt, s->d_bsum, tmp_step, s->d_len);
    else
      walk_next_hub_kernel<true><<<hgrid, HUB_TILE, 0, s->stream>>>(gv, wp, step, s->first, in_rec, d_n, ukey, uval, s->d_rank,
                                                                    s->d_cnt, s->d_bsum, tmp_step, s->d_len);
    nd_count_launches(1);
  }
  return ND_OK;
}

template <int APP>
int launch_sp(nd_sampler *s, const WalkParams &wp) {
  const int64_t blocks = (s->S + 255) / 256;
  const int grid = (int)(blocks < (int64_t)s->dev.sms * 32 ? blocks : (int64_t)s->dev.sms * 32);
  static const bool plain = getenv("ND_SP_PLAIN") != nullptr;
  if (APP == ND_APP_UNIFORM_WALK || plain)   // no rejection loop: one round per step for every lane anyway
    walk_sp_kernel<APP><<<grid, 256, 0, s->stream>>>(nd_view(s->g), wp, s->first, s->S, s->d_initial,
                                                      s->d_tmp, s->d_len, s->d_status, s->d_stats);
  else
    walk_sp_rounds_kernel<APP><<<grid, 256, 0, s->stream>>>(nd_view(s->g), wp, s->first, s->S, s->d_initial,
                                                             s->d_tmp, s->d_len, s->d_status, s->d_stats);
  return ND_OK;
}

}  // namespace

// The derived layouts of a graph are built by the first sampler that needs them; samplers of one
// graph may be created from several host threads, so the builds are serialised.
static std::mutex g_derived_mutex;

// interleaved (neighbour id, weight) records of a graph, built on first use
int nd_graph_ensure_colw(const nd_graph *g, int sms) {
  std::lock_guard<std::mutex> lock(g_derived_mutex);
  if (g->colw || g->E == 0) return ND_OK;
  int2 *cw = nullptr, *vr = nullptr;
  ND_CUDA(cudaMalloc(&cw, sizeof(int2) * (size_t)g->E));
  if (cudaMalloc(&vr, sizeof(int2) * ((size_t)g->V + 1)) != cudaSuccess) {
    cudaFree(cw);
    nd_set_error("per-vertex records: out of device memory");
    cudaGetLastError();
    return ND_ERR_CUDA;
  }
  colw_build_kernel<<<sms * 16, 256>>>(g->col, g->w, g->E, cw);
  vrec_build_kernel<<<sms * 16, 256>>>(g->row_ptr, g->max_w, g->V, vr);
  ND_CUDA(cudaDeviceSynchronize());
  g->vrec = vr;
  g->colw = cw;
  return ND_OK;
}

namespace {
__device__ int g_step_status;                       // device status word of nd_walk_step
__device__ unsigned long long g_step_stats[8];      // its event counters (not reported)

// One next() per explicit (transit, sample) pair; the sample id is the global one the draws are keyed by.
template <int APP>
__global__ void __launch_bounds__(256)
walk_step_kernel(NdGraphView g, WalkParams wp, int step, int64_t n, const int32_t *__restrict__ transit,
                 const int64_t *__restrict__ sample, int32_t *__restrict__ next) {
  Events ev;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int32_t t = transit[i];
    int32_t nbr = -1;
    if (t >= 0 && t < g.V) {
      const int32_t rs = __ldg(g.row_ptr + t);
      const int32_t deg = __ldg(g.row_ptr + t + 1) - rs;
      if (deg > 0) {
        Rng rng(wp.seed, (uint32_t)sample[i], (uint32_t)step, 0u);
        int32_t st = 0;
        nbr = app_next<APP, false>(g, wp, step, t, rs, deg, st, rng, &g_step_status, ev);
      }
    }
    next[i] = nbr;
  }
}
// The same for walkers packed as (global sample id << 32) | vertex; an ended walk becomes all ones.
template <int APP>
__global__ void __launch_bounds__(256)
walk_step_packed_kernel(NdGraphView g, WalkParams wp, int step, int64_t n, const unsigned long long *__restrict__ in,
                        unsigned long long *__restrict__ out) {
  Events ev;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const unsigned long long x = in[i];
    const int32_t t = (int32_t)(uint32_t)x;
    const uint32_t sample = (uint32_t)(x >> 32);
    int32_t nbr = -1;
    if (x != ~0ull && t >= 0 && t < g.V) {
      const int32_t rs = __ldg(g.row_ptr + t);
      const int32_t deg = __ldg(g.row_ptr + t + 1) - rs;
      if (deg > 0) {
        Rng rng(wp.seed, sample, (uint32_t)step, 0u);
        int32_t st = 0;
        nbr = app_next<APP, false>(g, wp, step, t, rs, deg, st, rng, &g_step_status, ev);
      }
    }
    out[i] = nbr >= 0 ? (((unsigned long long)sample << 32) | (uint32_t)nbr) : ~0ull;
  }
}
}  // namespace

// reads and clears the status word of the two step operators on the current device, after `st` drained
int nd_walk_step_status_read(cudaStream_t st, int *status) {
  ND_CUDA(cudaStreamSynchronize(st));
  int h = 0;
  ND_CUDA(cudaMemcpyFromSymbol(&h, g_step_status, sizeof(int)));
  if (h != 0) {
    const int zero = 0;
    ND_CUDA(cudaMemcpyToSymbol(g_step_status, &zero, sizeof(int)));
  }
  *status = h;
  return ND_OK;
}

int nd_walk_step_packed_launch(const nd_graph *g, const nd_app_params *p, int step, int64_t n, const uint64_t *d_in,
                               uint64_t *d_out, cudaStream_t st) {
  NdDeviceInfo dev;
  ND_TRY(nd_device_info(g->device, &dev));
  if (p->app == ND_APP_DEEPWALK || p->app == ND_APP_PPR) ND_TRY(nd_graph_ensure_colw(g, dev.sms));
  WalkParams wp{p->seed, p->p, p->q, p->stop_prob, p->n2v_ref_compat, p->steps, nullptr, g->colw};
  const int64_t blocks = (n + 255) / 256;
  const int grid = (int)(blocks < (int64_t)dev.sms * 16 ? blocks : (int64_t)dev.sms * 16);
  NdGraphView gv = nd_view(g);
  const unsigned long long *in = (const unsigned long long *)d_in;
  unsigned long long *out = (unsigned long long *)d_out;
  switch (p->app) {
    case ND_APP_UNIFORM_WALK: walk_step_packed_kernel<ND_APP_UNIFORM_WALK><<<grid, 256, 0, st>>>(gv, wp, step, n, in, out); break;
    case ND_APP_DEEPWALK: walk_step_packed_kernel<ND_APP_DEEPWALK><<<grid, 256, 0, st>>>(gv, wp, step, n, in, out); break;
    default: walk_step_packed_kernel<ND_APP_PPR><<<grid, 256, 0, st>>>(gv, wp, step, n, in, out); break;
  }
  nd_count_launches(1);
  ND_CUDA(cudaGetLastError());
  return ND_OK;
}

int nd_walk_step_launch(const nd_graph *g, const nd_app_params *p, int step, int64_t n, const int32_t *d_transits,
                        const int64_t *d_samples, int32_t *d_next, cudaStream_t st) {
  NdDeviceInfo dev;
  ND_TRY(nd_device_info(g->device, &dev));
  if (p->app == ND_APP_DEEPWALK || p->app == ND_APP_PPR) ND_TRY(nd_graph_ensure_colw(g, dev.sms));
  WalkParams wp{p->seed, p->p, p->q, p->stop_prob, p->n2v_ref_compat, p->steps, nullptr, g->colw};
  const int64_t blocks = (n + 255) / 256;
  const int grid = (int)(blocks < (int64_t)dev.sms * 16 ? blocks : (int64_t)dev.sms * 16);
  NdGraphView gv = nd_view(g);
  switch (p->app) {
    case ND_APP_UNIFORM_WALK: walk_step_kernel<ND_APP_UNIFORM_WALK><<<grid, 256, 0, st>>>(gv, wp, step, n, d_transits, d_samples, d_next); break;
    case ND_APP_DEEPWALK: walk_step_kernel<ND_APP_DEEPWALK><<<grid, 256, 0, st>>>(gv, wp, step, n, d_transits, d_samples, d_next); break;
    default: walk_step_kernel<ND_APP_PPR><<<grid, 256, 0, st>>>(gv, wp, step, n, d_transits, d_samples, d_next); break;
  }
  nd_count_launches(1);
  ND_CUDA(cudaGetLastError());
  return ND_OK;
}

int nd_walk_alloc(nd_sampler *s) {
  const int64_t S = s->S;
  const int steps = s->p.steps;
  ND_REQUIRE(steps >= 1 && steps <= 4096, ND_ERR_ARG, "walk length %d out of range [1,4096]", steps);
  ND_CUDA(cudaMalloc(&s->d_tmp, sizeof(int32_t) * (size_t)S * steps));
  ND_CUDA(cudaMalloc(&s->d_len, sizeof(int32_t) * (size_t)S));
  // the result array starts out all-invalid with no slot in use (walk_finalize_kernel keeps it that way)
  ND_CUDA(cudaMalloc(&s->d_plen, sizeof(int32_t) * (size_t)(S > 0 ? S : 1)));
  ND_CUDA(cudaMemset(s->d_plen, 0, sizeof(int32_t) * (size_t)(S > 0 ? S : 1)));
  if (S > 0) walk_fill_kernel<<<s->dev.sms * 8, 256>>>(s->d_out, S * steps / 4, S * steps, s->g->V);
  if (s->p.app == ND_APP_NODE2VEC) {
    ND_CUDA(cudaMalloc(&s->d_state, sizeof(int32_t) * (size_t)S));
    std::lock_guard<std::mutex> lock(g_derived_mutex);
    if (!s->g->adjset) {  // 8 bytes per CSR entry, built once per graph
      const size_t slots = 8 * ((size_t)(s->g->E / 4) + 2);
      int32_t *set = nullptr;
      ND_CUDA(cudaMalloc(&set, sizeof(int32_t) * slots));
      ND_CUDA(cudaMemset(set, 0xff, sizeof(int32_t) * slots));
      ND_CUDA(cudaMemset(s->d_status, 0, sizeof(int)));
      adjset_build_kernel<<<s->dev.sms * 16, 256>>>(nd_view(s->g), s->g->E, set, s->d_status);
      int st = 0;
      ND_CUDA(cudaMemcpy(&st, s->d_status, sizeof(int), cudaMemcpyDeviceToHost));
      if (st) { cudaFree(set); ND_REQUIRE(false, ND_ERR_DEVICE, "neighbour-set construction failed (status %d)", st); }
      s->g->adjset = set;
    }
  }
  if (s->p.app == ND_APP_DEEPWALK || s->p.app == ND_APP_PPR) ND_TRY(nd_graph_ensure_colw(s->g, s->dev.sms));
  s->map_cap = S;
  for (int i = 0; i < 2; i++) {
    ND_CUDA(cudaMalloc(&s->d_map_key[i], sizeof(int32_t) * (size_t)S));
    ND_CUDA(cudaMalloc(&s->d_map_val[i], sizeof(int32_t) * (size_t)S));
  }
  ND_CUDA(cudaMalloc(&s->d_init_key, sizeof(int32_t) * (size_t)S));
  ND_CUDA(cudaMalloc(&s->d_init_val, sizeof(int32_t) * (size_t)S));
  ND_CUDA(cudaMalloc(&s->d_nlive, sizeof(int32_t) * (size_t)(steps + 4)));  // live pairs per step, a spare slot, the tail launch's work counter, walks that can start
  const int key_bits = nd_bit_length((uint32_t)(s->g->V > 1 ? s->g->V - 1 : 1));
  ND_TRY(nd_radix_scratch_alloc(&s->radix, key_bits, S));
  // counting inversion (load-balanced mode)
  const size_t V = (size_t)s->g->V;
  const size_t bins = (V + CNT_SUPER - 1) / CNT_SUPER;
  ND_CUDA(cudaMalloc(&s->d_cnt, sizeof(uint32_t) * bins * CNT_SUPER));   // padded to whole bins
  ND_CUDA(cudaMalloc(&s->d_offs, sizeof(uint32_t) * bins * CNT_SUPER));
  ND_CUDA(cudaMalloc(&s->d_bsum, sizeof(uint32_t) * bins));
  ND_CUDA(cudaMalloc(&s->d_rank, sizeof(int32_t) * (size_t)(S > 0 ? S : 1)));
  ND_CUDA(cudaMemset(s->d_cnt, 0, sizeof(uint32_t) * bins * CNT_SUPER));
  ND_CUDA(cudaMemset(s->d_bsum, 0, sizeof(uint32_t) * bins));
  const size_t rec = s->p.app == ND_APP_NODE2VEC ? map_rec_bytes<true>() : map_rec_bytes<false>();
  const size_t S1 = (size_t)(S > 0 ? S : 1);
  for (int i = 0; i < 2; i++) ND_CUDA(cudaMalloc(&s->d_srec[i], rec * S1));
  ND_CUDA(cudaMalloc(&s->d_init_rec, rec * S1));
  if (s->p.app == ND_APP_NODE2VEC) ND_CUDA(cudaMalloc(&s->d_uext, sizeof(int4) * S1));
  if (s->p.app == ND_APP_PPR && s->p.stop_prob > 0.f) {  // the tail launch runs beside the result update
    ND_CUDA(cudaStreamCreateWithFlags(&s->side, cudaStreamNonBlocking));
    ND_CUDA(cudaEventCreateWithFlags(&s->side_fork, cudaEventDisableTiming));
    ND_CUDA(cudaEventCreateWithFlags(&s->side_join, cudaEventDisableTiming));
    ND_CUDA(cudaMallocHost(&s->h_active, sizeof(int32_t)));
    *s->h_active = -1;
    ND_CUDA(cudaEventCreateWithFlags(&s->active_done, cudaEventDisableTiming));
  }
  return ND_OK;
}

// Sort the initial transit->sample map once (the reference uploads it unsorted in the prologue of
// doTransitParallelSampling, src/nextdoor.cu:2207-2231, and never balances step 0, :2400).
int nd_sampler_build_initial_map(nd_sampler *s) {
  const int64_t n = s->S * s->isz;
  ND_REQUIRE(n < ((int64_t)1 << 31), ND_ERR_RANGE, "initial map of %lld pairs does not fit int32", (long long)n);
  const int32_t n32 = (int32_t)n;
  int32_t *d_n_in = s->d_nlive + s->p.steps + 1;  // spare slot
  ND_CUDA(cudaMemcpyAsync(d_n_in, &n32, sizeof(int32_t), cudaMemcpyHostToDevice, s->stream));
  const int blocks = (int)((n + 255) / 256);
  init_map_kernel<<<blocks > 0 ? blocks : 1, 256, 0, s->stream>>>(s->d_initial, s->g->V, n, s->d_map_key[0], s->d_map_val[0]);
  NdSortArrays arr;
  arr.nwords = 2;
  arr.a[0] = (uint32_t *)s->d_map_key[0]; arr.a[1] = (uint32_t *)s->d_map_val[0]; arr.a[2] = nullptr;
  arr.b[0] = (uint32_t *)s->d_map_key[1]; arr.b[1] = (uint32_t *)s->d_map_val[1]; arr.b[2] = nullptr;
  bool in_b = false;
  ND_TRY(nd_radix_sort(s->dev, s->stream, &s->radix, s->radix.plan, arr, 0, d_n_in, s->d_nlive, true, (uint32_t)s->g->V, false, &in_b));
  const int src = in_b ? 1 : 0;
  ND_CUDA(cudaMemcpyAsync(s->d_init_key, s->d_map_key[src], sizeof(int32_t) * n, cudaMemcpyDeviceToDevice, s->stream));
  ND_CUDA(cudaMemcpyAsync(s->d_init_val, s->d_map_val[src], sizeof(int32_t) * n, cudaMemcpyDeviceToDevice, s->stream));
  if (s->d_init_rec) {  // walks: the records the load-balanced mode starts from
    const int pg = (int)(blocks < s->dev.sms * 16 ? (blocks > 0 ? blocks : 1) : s->dev.sms * 16);
    if (s->p.app == ND_APP_NODE2VEC) pack_map_kernel<true><<<pg, 256, 0, s->stream>>>(s->d_nlive, s->d_map_key[src], s->d_map_val[src], s->d_init_rec);
    else pack_map_kernel<false><<<pg, 256, 0, s->stream>>>(s->d_nlive, s->d_map_key[src], s->d_map_val[src], s->d_init_rec);
  }
  if (s->h_active) {  // PPR: how many walks can start (read when the step loop is laid out, not waited for here)
    s->active_starts = -1;
    *s->h_active = -1;
    int32_t *d_active = s->d_nlive + s->p.steps + 3;
    ND_CUDA(cudaMemsetAsync(d_active, 0, sizeof(int32_t), s->stream));
    count_active_kernel<<<s->dev.sms * 4, 256, 0, s->stream>>>(s->d_initial, n, s->g->V, s->g->row_ptr, d_active);
    ND_CUDA(cudaMemcpyAsync(s->h_active, d_active, sizeof(int32_t), cudaMemcpyDeviceToHost, s->stream));
    ND_CUDA(cudaEventRecord(s->active_done, s->stream));
  }
  return ND_OK;  // stream-ordered: no host synchronisation, so chunks on different streams overlap
}

// Enqueues one whole job on the sampler's stream: no host synchronisation, no allocation, every
// size that changes from step to step is read from device memory -- so the sequence can be
// captured into a CUDA graph once and replayed.
static int walk_enqueue(nd_sampler *s, int mode) {
  const int64_t S = s->S;
  const int steps = s->p.steps;
  const int app = s->p.app;
  cudaStream_t st = s->stream;
  WalkParams wp{s->p.seed, s->p.p, s->p.q, s->p.stop_prob, s->p.n2v_ref_compat, steps, s->g->adjset, s->g->colw, s->g->vrec};
  bool tail_direct = false, join = false;   // PPR tail launch: writes the result rows itself / runs on the side stream
  int tail_from = 0x7fffffff;               // first step of that launch
  const int rblocks = (int)((S + 255) / 256);
  walk_reset_kernel<<<rblocks > 1 ? rblocks : 1, 256, 0, st>>>(s->d_initial, s->g->V, S, steps, s->d_len, s->d_state, s->d_stats,
                                                                s->d_nlive + steps + 2);
  nd_count_launches(1);
  if (mode == ND_MODE_SAMPLE_PARALLEL) {
    nd_phase_begin(s, ND_PHASE_NEXT);
    switch (app) {
      case ND_APP_UNIFORM_WALK: launch_sp<ND_APP_UNIFORM_WALK>(s, wp); break;
      case ND_APP_DEEPWALK: launch_sp<ND_APP_DEEPWALK>(s, wp); break;
      case ND_APP_PPR: launch_sp<ND_APP_PPR>(s, wp); break;
      default: launch_sp<ND_APP_NODE2VEC>(s, wp); break;
    }
    nd_phase_end(s);
    nd_count_launches(1);
  } else if (mode == ND_MODE_TRANSIT_PARALLEL) {
    // plain transit-parallel: sort-based inversion, first digit histogram fused into next()
    const NdRadixPlan &pl = s->radix.plan;
    const int64_t tiles = pl.max_tiles;
    const int grid = (int)(tiles < (int64_t)s->dev.sms * 8 ? tiles : (int64_t)s->dev.sms * 8);
    const int32_t *in_key = s->d_init_key, *in_val = s->d_init_val;
    int cur = 0;  // buffer the next kernel writes into
    for (int step = 0; step < steps; step++) {
      const bool last = step == steps - 1;
      int32_t *ok = s->d_map_key[cur], *ov = s->d_map_val[cur];
      const int32_t *d_n = s->d_nlive + step;
      nd_phase_begin(s, ND_PHASE_NEXT);
      switch (app) {
        case ND_APP_UNIFORM_WALK: launch_next_tp<ND_APP_UNIFORM_WALK>(s, wp, step, !last, grid, in_key, in_val, d_n, ok, ov); break;
        case ND_APP_DEEPWALK: launch_next_tp<ND_APP_DEEPWALK>(s, wp, step, !last, grid, in_key, in_val, d_n, ok, ov); break;
        case ND_APP_PPR: launch_next_tp<ND_APP_PPR>(s, wp, step, !last, grid, in_key, in_val, d_n, ok, ov); break;
        default: launch_next_tp<ND_APP_NODE2VEC>(s, wp, step, !last, grid, in_key, in_val, d_n, ok, ov); break;
      }
      nd_phase_end(s);
      nd_count_launches(1);
      if (last) break;
      nd_phase_begin(s, ND_PHASE_INVERT);
      NdSortArrays arr;
      arr.nwords = 2;
      arr.a[0] = (uint32_t *)s->d_map_key[cur]; arr.a[1] = (uint32_t *)s->d_map_val[cur]; arr.a[2] = nullptr;
      arr.b[0] = (uint32_t *)s->d_map_key[cur ^ 1]; arr.b[1] = (uint32_t *)s->d_map_val[cur ^ 1]; arr.b[2] = nullptr;
      bool in_b = false;
      ND_TRY(nd_radix_sort(s->dev, st, &s->radix, s->radix.plan, arr, 0, d_n, s->d_nlive + step + 1, true,
                           (uint32_t)s->g->V, true, &in_b));
      nd_phase_end(s);
      const int res = in_b ? (cur ^ 1) : cur;
      in_key = s->d_map_key[res];
      in_val = s->d_map_val[res];
      cur = res ^ 1;
    }
  } else {
    // load-balanced transit-parallel: next() draws tickets, counting inversion
    const int V = s->g->V;
    const int bins = (V + CNT_SUPER - 1) / CNT_SUPER;
    const bool n2v = app == ND_APP_NODE2VEC;
    // unsorted pairs written by next(): key/val in d_map_*[0], rank, (node2vec) d_uext; the sorted
    // maps are records that ping-pong between d_srec[0] and d_srec[1]
    int32_t *ukey = s->d_map_key[0], *uval = s->d_map_val[0];
    const void *in_rec = s->d_init_rec;
    const int64_t sblocks = (S + 256 * SCATTER_PPT - 1) / (256 * SCATTER_PPT);
    const int sgrid = (int)(sblocks < (int64_t)s->dev.sms * 16 ? (sblocks > 0 ? sblocks : 1) : (int64_t)s->dev.sms * 16);
    // PPR: a step of the loop costs about 40 us of launches and of the scan over the per-vertex
    // counters whatever the number of pairs, which is what a million pairs cost on top of it.  The
    // map of step k >= 1 holds the walks that can start and pass the stop draws of steps 1..k
    // (pairs known to stop are not entered): active * (1 - stop probability)^(k+1).  The loop runs
    // while that is above a million, one tail launch finishes the rest (ND_WALK_TAIL_PAIRS moves the
    // hand-over, for tests and A/B runs).  `active` was counted when the seeds were set; the layout
    // is fixed when the loop is first captured and kept for later seeds.
    int tp_steps = steps;
    if (app == ND_APP_PPR && s->p.stop_prob > 0.f && !getenv("ND_WALK_NO_TAIL")) {
      const char *e = getenv("ND_WALK_TAIL_PAIRS");
      const double floor_pairs = e ? atof(e) : 1048576.0;
      const double active = s->active_starts >= 0 ? (double)s->active_starts : (double)S;
      const double keep = 1.0 - (double)s->p.stop_prob;
      double in_map = active * keep * keep;   // step 1
      int k = 1;
      while (k < steps && in_map > floor_pairs) { in_map *= keep; k++; }
      tp_steps = k;
    }
    wp.keep_all_step = tp_steps < steps ? tp_steps - 1 : -1;
    int cur = 0;  // sorted map the scatter of this step writes
    for (int step = 0; step < tp_steps; step++) {
      const bool last = step == steps - 1;
      const int32_t *d_n = s->d_nlive + step;
      int32_t *tmp_step = s->d_tmp + (int64_t)step * S;
      nd_phase_begin(s, ND_PHASE_NEXT);
      switch (app) {
        case ND_APP_UNIFORM_WALK: ND_TRY(launch_count<ND_APP_UNIFORM_WALK>(s, wp, step, last, bins, in_rec, d_n, ukey, uval, tmp_step)); break;
        case ND_APP_DEEPWALK: ND_TRY(launch_count<ND_APP_DEEPWALK>(s, wp, step, last, bins, in_rec, d_n, ukey, uval, tmp_step)); break;
        case ND_APP_PPR: ND_TRY(launch_count<ND_APP_PPR>(s, wp, step, last, bins, in_rec, d_n, ukey, uval, tmp_step)); break;
        default: ND_TRY(launch_count<ND_APP_NODE2VEC>(s, wp, step, last, bins, in_rec, d_n, ukey, uval, tmp_step)); break;
      }
      nd_phase_end(s);
      nd_count_launches(1);
      if (last) break;
      nd_phase_begin(s, ND_PHASE_INVERT);
      cnt_scan_kernel<<<bins, SCAN_THREADS, 0, st>>>(s->d_cnt, s->d_bsum, s->d_offs, s->d_nlive + step + 1);
      if (n2v) walk_scatter_kernel<true><<<sgrid, 256, 0, st>>>(d_n, V, ukey, uval, s->d_rank, s->d_uext, s->d_offs, s->d_srec[cur], s->d_bsum, bins);
      else walk_scatter_kernel<false><<<sgrid, 256, 0, st>>>(d_n, V, ukey, uval, s->d_rank, nullptr, s->d_offs, s->d_srec[cur], s->d_bsum, bins);
      nd_phase_end(s);
      nd_count_launches(2);
      in_rec = s->d_srec[cur];
      cur ^= 1;
    }
    if (tp_steps < steps) {
      // with the sparse result update the tail writes its walks' slots itself and runs beside that
      // update on the side stream (one after the other on the main stream when the phases are timed)
      tail_direct = s->p.stop_prob >= FIN_SPARSE_STOP && s->side != nullptr;
      const char *ti = getenv("ND_WALK_TAIL_INLINE");   // A/B switch: anything but empty or 0 keeps the tail on the main stream
      const bool forked = tail_direct && !s->timer.on && !(ti && ti[0] && ti[0] != '0');
      cudaStream_t ts = st;
      if (forked) {
        ND_CUDA(cudaEventRecord(s->side_fork, st));
        ND_CUDA(cudaStreamWaitEvent(s->side, s->side_fork, 0));
        ts = s->side;
      }
      nd_phase_begin(s, ND_PHASE_TAIL);
      const int tgrid = s->dev.sms * walk_min_ctas_sp<ND_APP_PPR>();   // resident CTAs; the lanes draw their pairs from a counter
      int32_t *next_pair = s->d_nlive + steps + 2;
      if (tail_direct)
        walk_tail_kernel<ND_APP_PPR, true><<<tgrid, 256, 0, ts>>>(nd_view(s->g), wp, tp_steps, s->first, in_rec, s->d_nlive + tp_steps, next_pair,
                                                                 S, s->d_tmp, s->d_len, s->d_plen, s->d_out, s->d_status, s->d_stats);
      else
        walk_tail_kernel<ND_APP_PPR, false><<<tgrid, 256, 0, ts>>>(nd_view(s->g), wp, tp_steps, s->first, in_rec, s->d_nlive + tp_steps, next_pair,
                                                                  S, s->d_tmp, s->d_len, s->d_plen, s->d_out, s->d_status, s->d_stats);
      nd_phase_end(s);
      nd_count_launches(1);
      if (forked) {
        ND_CUDA(cudaEventRecord(s->side_join, s->side));
        join = true;
      }
      tail_from = tail_direct ? tp_steps : tail_from;
    }
  }
  nd_phase_begin(s, ND_PHASE_FINALIZE);
  const int64_t groups = (S + FIN_SAMPLES - 1) / FIN_SAMPLES, fblocks = (groups + FIN_THREADS / 32 - 1) / (FIN_THREADS / 32);
  const int fgrid = (int)(fblocks < (int64_t)s->dev.sms * 16 ? fblocks : (int64_t)s->dev.sms * 16);
  const int dgrid = (int)(groups < (int64_t)s->dev.sms * 16 ? groups : (int64_t)s->dev.sms * 16);
  // walks that end early leave most of a row invalid: the sparse kernel; full-length walks: whole rows
  if (app == ND_APP_PPR && s->p.stop_prob >= FIN_SPARSE_STOP)
    walk_finalize_sparse_kernel<<<fgrid > 0 ? fgrid : 1, FIN_THREADS, 0, st>>>(s->d_tmp, s->d_len, s->d_plen, S, steps, s->g->V, s->d_out, s->d_stats, tail_from);
  else
    walk_finalize_kernel<<<dgrid > 0 ? dgrid : 1, FIN_THREADS, 0, st>>>(s->d_tmp, s->d_len, s->d_plen, S, steps, s->g->V, s->d_out, s->d_stats);
  nd_phase_end(s);
  nd_count_launches(1);
  if (join) ND_CUDA(cudaStreamWaitEvent(st, s->side_join, 0));
  ND_CUDA(cudaGetLastError());
  return ND_OK;
}

int nd_walk_sample(nd_sampler *s, int mode) {
  // the count of walks that can start is waited for here, outside any stream capture, the first
  // time a step loop is laid out after the seeds were set
  if (s->h_active && s->active_starts < 0 && s->active_done) {
    const bool lays_out = s->stream != nullptr && s->stream != cudaStreamLegacy && s->stream != cudaStreamPerThread &&
                          !s->timer.on && !s->graph_off && !s->graph_exec[mode];   // about to capture this mode's loop
    const cudaError_t ready = lays_out ? cudaEventSynchronize(s->active_done) : cudaEventQuery(s->active_done);
    if (ready == cudaSuccess) s->active_starts = *s->h_active;
    else cudaGetLastError();   // not there yet: this (uncaptured) run is laid out by the number of samples
  }
  // Graph replay needs a capturable stream (not the legacy default stream) and no phase timers.
  const bool capturable = s->stream != nullptr && s->stream != cudaStreamLegacy && s->stream != cudaStreamPerThread;
  if (!capturable || s->timer.on || s->graph_off) return walk_enqueue(s, mode);
  if (!s->graph_exec[mode]) {
    const long long before = nd_launch_count();
    cudaGraph_t graph = nullptr;
    if (cudaStreamBeginCapture(s->stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
      cudaGetLastError();
      s->graph_off = true;
      return walk_enqueue(s, mode);
    }
    const int rc = walk_enqueue(s, mode);
    const cudaError_t ec = cudaStreamEndCapture(s->stream, &graph);
    s->graph_launches[mode] = (int)(nd_launch_count() - before);
    nd_count_launches(-s->graph_launches[mode]);  // nothing ran yet
    if (rc != ND_OK || ec != cudaSuccess || !graph ||
        cudaGraphInstantiate(&s->graph_exec[mode], graph, 0) != cudaSuccess) {
      cudaGetLastError();
      if (graph) cudaGraphDestroy(graph);
      s->graph_exec[mode] = nullptr;
      s->graph_off = true;
      return walk_enqueue(s, mode);
    }
    cudaGraphDestroy(graph);
  }
  ND_CUDA(cudaGraphLaunch(s->graph_exec[mode], s->stream));
  nd_count_launches(s->graph_launches[mode]);
  return ND_OK;
}
