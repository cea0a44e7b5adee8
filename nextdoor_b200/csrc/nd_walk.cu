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
#include "nd_common.cuh"
#include "nd_philox.cuh"

namespace {

using ndrng::Rng;

struct WalkParams {
  uint64_t seed;
  float p, q, stop_prob;
  int n2v_compat;
  int steps;
  const unsigned long long *filter;  // node2vec: adjacency pre-filter of the high-degree vertices (may be null)
};

// node2vec asks "is v a neighbour of the previous vertex t?" once per try, and t is usually a hub
// (a 17-probe bisection).  Most answers are "no", so every vertex with at least FILTER_MIN_DEG
// neighbours gets a blocked Bloom filter over its list: 16 bits per neighbour, stored in the 64-bit
// words [row_ptr[t]/4, row_ptr[t]/4 + deg/4) of one array (regions of consecutive vertices cannot
// overlap), two bits per neighbour inside one word, so a test is a single 8-byte load.  A filter
// has no false negatives: when it says "no" the bisection is skipped, otherwise it runs as usual,
// and the accepted vertex is the same either way.
constexpr int FILTER_MIN_DEG = 32;

__device__ __forceinline__ uint32_t filter_mix(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return x;
}
__device__ __forceinline__ void filter_slot(int32_t v, uint32_t n_words, uint32_t &word, unsigned long long &mask) {
  const uint32_t h = filter_mix((uint32_t)v);
  word = (uint32_t)(((unsigned long long)h * n_words) >> 32);
  const uint32_t g = filter_mix(h ^ 0x9e3779b9u);
  mask = (1ull << (g & 63u)) | (1ull << ((g >> 6) & 63u));
}

constexpr int RETRY_CAP = 1 << 16;

// events the algorithmic-bytes model is evaluated from (stats[2..4]); kept per thread and
// flushed once per warp when the kernel ends
struct Events {
  uint32_t weight_tries = 0, n2v_tries = 0, n2v_probes = 0;
  __device__ __forceinline__ void flush(unsigned long long *stats) {
    uint32_t a = weight_tries, b = n2v_tries, c = n2v_probes;
    for (int o = 16; o > 0; o >>= 1) {
      a += __shfl_xor_sync(0xffffffffu, a, o);
      b += __shfl_xor_sync(0xffffffffu, b, o);
      c += __shfl_xor_sync(0xffffffffu, c, o);
    }
    if ((threadIdx.x & 31) == 0) {
      if (a) atomicAdd(&stats[2], (unsigned long long)a);
      if (b) atomicAdd(&stats[3], (unsigned long long)b);
      if (c) atomicAdd(&stats[4], (unsigned long long)c);
    }
  }
};

// One next() of the app on a transit with n > 0 neighbours; -1 = no vertex.
// Gathers from the big graph arrays (neighbour ids, weights, filter words) are used once per
// launch: they are loaded with the streaming policy (evict-first) so that they do not push the
// small per-sample and per-vertex arrays (maps, counters, staged output row, row offsets) out of L2.
// (Only the transit-parallel kernels do this; a sample-parallel walk revisits hub lists from the
// same thread step after step and is faster with the default policy: 60 vs 42 G edges/s measured.)
template <bool STREAM, typename T>
__device__ __forceinline__ T ld_graph(const T *p) { return STREAM ? __ldcs(p) : __ldg(p); }

template <int APP, bool STREAM = true>
__device__ __forceinline__ int32_t app_next(const NdGraphView &g, const WalkParams &wp, int step,
                                            int32_t transit, int32_t rs, int32_t n, int32_t &state_t,
                                            Rng &rng, int *status, Events &ev) {
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
    const float *__restrict__ weights = g.w + rs;
    const float max_w = __ldg(g.max_w + transit);
    int32_t x = rng.rand_int(n);
    float y = __fmul_rn(rng.uniform(), max_w);
    int it = 0;
    ev.weight_tries++;
    while (y > ld_graph<STREAM>(weights + x)) {
      if (++it > RETRY_CAP) { atomicOr(status, ND_DEV_RETRY_LIMIT); break; }
      x = rng.rand_int(n);
      y = __fmul_rn(rng.uniform(), max_w);
      ev.weight_tries++;
    }
    return ld_graph<STREAM>(edges + x);
  }
  if (APP == ND_APP_NODE2VEC) {  // randomWalks.cu:141-172
    if (n == 1 || step == 0) { state_t = transit; return ld_graph<STREAM>(edges); }
    const float inv_q = __fdiv_rn(1.0f, wp.q);
    float bound = wp.p > inv_q ? wp.p : inv_q;
    if (bound < 1.0f) bound = 1.0f;
    const int32_t t = state_t;
    const int32_t ts = __ldg(g.row_ptr + t);
    const int32_t tn = __ldg(g.row_ptr + t + 1) - ts;
    const int32_t *__restrict__ tedges = g.col + ts;
    for (int it = 0;; it++) {
      const int32_t x = rng.rand_int(n);
      const int32_t v = ld_graph<STREAM>(edges + x);
      const float y = __fmul_rn(rng.uniform(), bound);
      float h;
      ev.n2v_tries++;
      const bool is_ret = wp.n2v_compat ? (x == t) : (v == t);  // randomWalks.cu:159 compares the index
      if (is_ret) {
        h = wp.p;
      } else {
        // membership of v in the sorted list of t: the answer of utils::binarySearch
        // (src/utils.hpp:30-48), found with fewer dependent loads
        int32_t l = 0, r = tn;  // candidates in [l, r)
        bool found = false;
        if (wp.filter && tn >= FILTER_MIN_DEG) {
          uint32_t word;
          unsigned long long mask;
          filter_slot(v, (uint32_t)tn >> 2, word, mask);
          ev.n2v_probes += 2;  // one 8-byte load
          if ((ld_graph<STREAM>(wp.filter + ((uint32_t)ts >> 2) + word) & mask) != mask) r = 0;  // certainly not a neighbour
        }
        // 5-ary search: the four pivots of a level are loaded together, so a level costs one
        // memory latency and a 138K-entry list is searched in 8 levels instead of 17
        while (r - l > 4 && !found) {
          const int32_t q5 = (r - l) / 5;
          const int32_t p1 = l + q5, p2 = p1 + q5, p3 = p2 + q5, p4 = p3 + q5;
          const int32_t e1 = ld_graph<STREAM>(tedges + p1), e2 = ld_graph<STREAM>(tedges + p2), e3 = ld_graph<STREAM>(tedges + p3), e4 = ld_graph<STREAM>(tedges + p4);
          ev.n2v_probes += 4;
          if (v == e1 || v == e2 || v == e3 || v == e4) found = true;
          else if (v < e1) r = p1;
          else if (v < e2) { l = p1 + 1; r = p2; }
          else if (v < e3) { l = p2 + 1; r = p3; }
          else if (v < e4) { l = p3 + 1; r = p4; }
          else l = p4 + 1;
        }
        if (!found && r > l) {  // at most four left: load them together
          int32_t e[4];
#pragma unroll
          for (int k = 0; k < 4; k++) e[k] = l + k < r ? ld_graph<STREAM>(tedges + l + k) : -1;
          ev.n2v_probes += r - l;
          found = v == e[0] || v == e[1] || v == e[2] || v == e[3];
        }
        h = found ? inv_q : 1.0f;
      }
      if (y < h || it >= RETRY_CAP) {
        if (it >= RETRY_CAP) atomicOr(status, ND_DEV_RETRY_LIMIT);
        state_t = transit;
        return v;
      }
    }
  }
  return -1;
}

// ---------------------------------------------------------------- set-up kernels

// one warp per vertex: set the two bits of every neighbour in the vertex's filter region
__global__ void filter_build_kernel(NdGraphView g, unsigned long long *__restrict__ filter) {
  const int lane = threadIdx.x & 31;
  const int64_t warp_id = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t t = warp_id; t < g.V; t += n_warps) {
    const int32_t rs = g.row_ptr[t], deg = g.row_ptr[t + 1] - rs;
    if (deg < FILTER_MIN_DEG) continue;
    unsigned long long *region = filter + ((uint32_t)rs >> 2);
    for (int e = lane; e < deg; e += 32) {
      uint32_t word;
      unsigned long long mask;
      filter_slot(g.col[rs + e], (uint32_t)deg >> 2, word, mask);
      atomicOr(region + word, mask);
    }
  }
}

__global__ void walk_reset_kernel(const int32_t *__restrict__ initial, int32_t V, int64_t S, int steps,
                                  int32_t *__restrict__ len, int32_t *__restrict__ state,
                                  unsigned long long *__restrict__ stats) {
  const int64_t s = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (s < 8 && stats) stats[s] = 0ull;
  if (s >= S) return;
  const int32_t t = initial[s];
  len[s] = (t >= 0 && t < V) ? steps : -1;
  if (state) state[s] = 0;
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

constexpr int NEXT_THREADS = 512;

// One CTA per radix tile of the transit->sample map.  HIST: also count the first radix digit of the
// new keys (layout and digit as the radix scatter of pass 0 expects them).
template <int APP, bool HIST>
__global__ void __launch_bounds__(NEXT_THREADS)
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
          nbr = app_next<APP>(g, wp, step, t, rs, deg, st, rng, status, ev);
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
      for (int b = threadIdx.x; b < bins; b += NEXT_THREADS) {
        const uint32_t c = sh_hist[b];
        tile_hist[(int64_t)b * max_tiles + tile] = c;
        if (c) atomicAdd(&ghist[b], c);
      }
      __syncthreads();
    }
  }
  if (APP != ND_APP_UNIFORM_WALK) ev.flush(stats);
}

// ---------------------------------------------------------------- next() + counting inversion (load-balanced mode)
//
// The transit ids are a dense key space (< V) and the map holds at most one pair per walk, so
// the inversion does not need a multi-pass sort: next() takes a ticket on its new transit
// (atomicAdd on cnt[transit], the ticket is the pair's rank inside the transit's run), two small
// kernels turn the counters into run offsets (chunk sums, then per-chunk exclusive scan, which
// also clears the counters and publishes the live count), and one kernel moves every pair to
// offs[transit] + rank.  16 B read + 8 B written per pair beside 12 B per vertex of counter
// traffic, against 2-3 radix passes.  The order of the pairs inside one transit's run depends on
// the order the tickets were drawn; results do not, because every draw is keyed by the sample.

constexpr int CNT_THREADS = 256;
constexpr int CNT_PER_THREAD = 8;
constexpr int CNT_CHUNK = CNT_THREADS * CNT_PER_THREAD;  // counters per CTA

template <int APP, bool COUNT>
__global__ void __launch_bounds__(256)
walk_next_count_kernel(NdGraphView g, WalkParams wp, int step, int64_t first_sample,
                       const int32_t *__restrict__ in_key, const int32_t *__restrict__ in_val,
                       const int32_t *__restrict__ d_n, int32_t *__restrict__ out_key,
                       int32_t *__restrict__ out_val, int32_t *__restrict__ out_rank,
                       uint32_t *__restrict__ cnt, uint8_t *__restrict__ dirty, int32_t *__restrict__ tmp_step,
                       int32_t *__restrict__ len, int32_t *__restrict__ state, int *__restrict__ status,
                       unsigned long long *__restrict__ stats) {
  Events ev;
  const int n = *d_n;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int32_t t = in_key[i];
    const int32_t s = in_val[i];
    int32_t nbr = -1;
    if (t < 0 || t >= g.V) {
      atomicOr(status, ND_DEV_BAD_TRANSIT);
    } else {
      const int32_t rs = __ldg(g.row_ptr + t);
      const int32_t deg = __ldg(g.row_ptr + t + 1) - rs;
      if (deg > 0) {
        Rng rng(wp.seed, (uint32_t)(first_sample + s), (uint32_t)step, 0u);
        int32_t st = 0;
        if (APP == ND_APP_NODE2VEC && step > 0) st = state[s];
        nbr = app_next<APP>(g, wp, step, t, rs, deg, st, rng, status, ev);
        if (APP == ND_APP_NODE2VEC && nbr >= 0) state[s] = st;
      }
    }
    if (nbr >= 0) tmp_step[s] = nbr; else len[s] = step;
    if (COUNT) {
      out_key[i] = nbr >= 0 ? nbr : g.V;
      if (nbr >= 0) {
        out_val[i] = s;
        out_rank[i] = (int32_t)atomicAdd(&cnt[nbr], 1u);
        if (dirty) {  // this chunk of counters has work for the scan (test first: hub chunks are hit by everyone)
          uint8_t *d = dirty + nbr / CNT_CHUNK;
          if (__ldcg(d) == 0) *d = 1;
        }
      }
    }
  }
  if (APP != ND_APP_UNIFORM_WALK) ev.flush(stats);
}

__global__ void __launch_bounds__(CNT_THREADS)
cnt_chunk_sum_kernel(const uint32_t *__restrict__ cnt, int32_t V, const uint8_t *__restrict__ dirty,
                     uint32_t *__restrict__ bsum) {
  __shared__ uint32_t wsum[CNT_THREADS / 32];
  if (dirty && !dirty[blockIdx.x]) {  // no ticket was drawn in this chunk: its counters are all zero
    if (threadIdx.x == 0) bsum[blockIdx.x] = 0u;
    return;
  }
  const uint4 *src = reinterpret_cast<const uint4 *>(cnt + (size_t)blockIdx.x * CNT_CHUNK);
  uint32_t part = 0;
#pragma unroll
  for (int r = 0; r < CNT_PER_THREAD / 4; r++) {
    const uint4 a = src[r * CNT_THREADS + threadIdx.x];
    part += a.x + a.y + a.z + a.w;
  }
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = part;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t t = 0;
    for (int w = 0; w < CNT_THREADS / 32; w++) t += wsum[w];
    bsum[blockIdx.x] = t;
  }
}

// CTA b: start of its chunk = sum of the chunk sums before it; exclusive scan of its counters into
// offs; counters cleared for the next step; the last CTA publishes the number of live pairs.
__global__ void __launch_bounds__(CNT_THREADS)
cnt_scan_kernel(uint32_t *__restrict__ cnt, int32_t V, const uint32_t *__restrict__ bsum,
                uint8_t *__restrict__ dirty, uint32_t *__restrict__ offs, int32_t *__restrict__ d_n_out) {
  __shared__ uint32_t wsum[CNT_THREADS / 32];
  __shared__ uint32_t base_sh;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool is_dirty = !dirty || dirty[blockIdx.x] != 0;
  const bool is_last = blockIdx.x == gridDim.x - 1;
  // a chunk nobody drew a ticket in holds no transit of the next step: its offsets are never
  // read, so the CTA has nothing to do (the last CTA still publishes the live count)
  if (!is_dirty && !is_last) return;
  uint32_t part = 0;
  for (int i = threadIdx.x; i < (int)blockIdx.x; i += CNT_THREADS) part += bsum[i];
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  if (lane == 0) wsum[warp] = part;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t t = 0;
    for (int w = 0; w < CNT_THREADS / 32; w++) t += wsum[w];
    base_sh = t;
  }
  __syncthreads();
  // each thread owns 8 consecutive counters (one 32-byte sector)
  // (the arrays are padded to whole chunks, so the two 16-byte accesses never leave them)
  const int first = blockIdx.x * CNT_CHUNK + threadIdx.x * CNT_PER_THREAD;
  uint32_t c[CNT_PER_THREAD];
  uint32_t tsum = 0;
  {
    const uint4 a = *reinterpret_cast<const uint4 *>(cnt + first);
    const uint4 b = *reinterpret_cast<const uint4 *>(cnt + first + 4);
    c[0] = a.x; c[1] = a.y; c[2] = a.z; c[3] = a.w; c[4] = b.x; c[5] = b.y; c[6] = b.z; c[7] = b.w;
  }
#pragma unroll
  for (int r = 0; r < CNT_PER_THREAD; r++) tsum += c[r];
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
  uint32_t o[CNT_PER_THREAD];
#pragma unroll
  for (int r = 0; r < CNT_PER_THREAD; r++) { o[r] = run; run += c[r]; }
  *reinterpret_cast<uint4 *>(offs + first) = make_uint4(o[0], o[1], o[2], o[3]);
  *reinterpret_cast<uint4 *>(offs + first + 4) = make_uint4(o[4], o[5], o[6], o[7]);
  *reinterpret_cast<uint4 *>(cnt + first) = make_uint4(0u, 0u, 0u, 0u);
  *reinterpret_cast<uint4 *>(cnt + first + 4) = make_uint4(0u, 0u, 0u, 0u);
  if (is_last && threadIdx.x == CNT_THREADS - 1) *d_n_out = (int32_t)run;
  if (dirty && threadIdx.x == 0) dirty[blockIdx.x] = 0;
}

__global__ void __launch_bounds__(256)
walk_scatter_kernel(const int32_t *__restrict__ d_n, int32_t V, const int32_t *__restrict__ ukey,
                    const int32_t *__restrict__ uval, const int32_t *__restrict__ urank,
                    const uint32_t *__restrict__ offs, int32_t *__restrict__ okey, int32_t *__restrict__ oval) {
  const int n = *d_n;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int32_t k = ukey[i];
    if (k == V) continue;
    const uint32_t pos = __ldg(offs + k) + (uint32_t)urank[i];
    okey[pos] = k;
    oval[pos] = uval[i];
  }
}

// ---------------------------------------------------------------- sample-parallel: a thread owns a walk

template <int APP>
__global__ void __launch_bounds__(256)
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
        nbr = app_next<APP, false>(g, wp, step, cur, rs, deg, st, rng, status, ev);
      }
      if (nbr < 0) break;
      tmp[(int64_t)step * S + s] = nbr;
      cur = nbr;
    }
    if (step < wp.steps) len[s] = step;
  }
  if (APP != ND_APP_UNIFORM_WALK) ev.flush(stats);
}

// ---------------------------------------------------------------- finalize: step-major -> sample-major

constexpr int FIN_SAMPLES = 32;   // samples per CTA
constexpr int FIN_THREADS = 256;
constexpr int FIN_MAX_STEPS = 128;  // steps per smem chunk

__global__ void __launch_bounds__(FIN_THREADS)
walk_finalize_kernel(const int32_t *__restrict__ tmp, const int32_t *__restrict__ len, int64_t S,
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
      if (kc == steps) {
        int32_t *dst = out + s0 * steps;
        for (int j = threadIdx.x; j < ns * steps; j += FIN_THREADS) dst[j] = tile[j % steps][j / steps];
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

template <int APP>
int launch_next_tp(nd_sampler *s, const WalkParams &wp, int step, bool hist, int grid, const int32_t *in_key,
                   const int32_t *in_val, const int32_t *d_n, int32_t *out_key, int32_t *out_val) {
  const NdRadixPlan &pl = s->radix.plan;
  const int bins = 1 << pl.bits[0];
  NdGraphView gv = nd_view(s->g);
  int32_t *tmp_step = s->d_tmp + (int64_t)step * s->S;
  if (hist) {
    walk_next_tp_kernel<APP, true><<<grid, NEXT_THREADS, bins * sizeof(uint32_t), s->stream>>>(
        gv, wp, step, s->first, pl.tile, in_key, in_val, d_n, out_key, out_val, tmp_step, s->d_len,
        s->d_state, pl.shift[0], bins, s->radix.tile_hist, pl.max_tiles, s->radix.ghist, s->d_status, s->d_stats);
  } else {
    walk_next_tp_kernel<APP, false><<<grid, NEXT_THREADS, 0, s->stream>>>(
        gv, wp, step, s->first, pl.tile, in_key, in_val, d_n, out_key, out_val, tmp_step, s->d_len,
        s->d_state, 0, 1, nullptr, 0, nullptr, s->d_status, s->d_stats);
  }
  return ND_OK;
}

template <int APP>
int launch_sp(nd_sampler *s, const WalkParams &wp) {
  const int64_t blocks = (s->S + 255) / 256;
  const int grid = (int)(blocks < (int64_t)s->dev.sms * 32 ? blocks : (int64_t)s->dev.sms * 32);
  walk_sp_kernel<APP><<<grid, 256, 0, s->stream>>>(nd_view(s->g), wp, s->first, s->S, s->d_initial,
                                                    s->d_tmp, s->d_len, s->d_status, s->d_stats);
  return ND_OK;
}

}  // namespace

int nd_walk_alloc(nd_sampler *s) {
  const int64_t S = s->S;
  const int steps = s->p.steps;
  ND_REQUIRE(steps >= 1 && steps <= 4096, ND_ERR_ARG, "walk length %d out of range [1,4096]", steps);
  ND_CUDA(cudaMalloc(&s->d_tmp, sizeof(int32_t) * (size_t)S * steps));
  ND_CUDA(cudaMalloc(&s->d_len, sizeof(int32_t) * (size_t)S));
  if (s->p.app == ND_APP_NODE2VEC) {
    ND_CUDA(cudaMalloc(&s->d_state, sizeof(int32_t) * (size_t)S));
    // adjacency pre-filter: 2 bytes per CSR entry, built once per sampler
    const size_t words = (size_t)(s->g->E / 4) + 2;
    ND_CUDA(cudaMalloc(&s->d_filter, sizeof(unsigned long long) * words));
    ND_CUDA(cudaMemset(s->d_filter, 0, sizeof(unsigned long long) * words));
    filter_build_kernel<<<s->dev.sms * 16, 256>>>(nd_view(s->g), s->d_filter);
    ND_CUDA(cudaGetLastError());
  }
  s->map_cap = S;
  for (int i = 0; i < 2; i++) {
    ND_CUDA(cudaMalloc(&s->d_map_key[i], sizeof(int32_t) * (size_t)S));
    ND_CUDA(cudaMalloc(&s->d_map_val[i], sizeof(int32_t) * (size_t)S));
  }
  ND_CUDA(cudaMalloc(&s->d_init_key, sizeof(int32_t) * (size_t)S));
  ND_CUDA(cudaMalloc(&s->d_init_val, sizeof(int32_t) * (size_t)S));
  ND_CUDA(cudaMalloc(&s->d_nlive, sizeof(int32_t) * (size_t)(steps + 2)));
  const int key_bits = nd_bit_length((uint32_t)(s->g->V > 1 ? s->g->V - 1 : 1));
  ND_TRY(nd_radix_scratch_alloc(&s->radix, key_bits, S));
  // counting inversion (load-balanced mode)
  const size_t V = (size_t)s->g->V;
  const size_t chunks = (V + CNT_CHUNK - 1) / CNT_CHUNK;
  ND_CUDA(cudaMalloc(&s->d_cnt, sizeof(uint32_t) * chunks * CNT_CHUNK));   // padded to whole chunks
  ND_CUDA(cudaMalloc(&s->d_offs, sizeof(uint32_t) * chunks * CNT_CHUNK));
  ND_CUDA(cudaMalloc(&s->d_bsum, sizeof(uint32_t) * chunks));
  ND_CUDA(cudaMalloc(&s->d_dirty, chunks));
  ND_CUDA(cudaMemset(s->d_dirty, 0, chunks));
  ND_CUDA(cudaMalloc(&s->d_rank, sizeof(int32_t) * (size_t)(S > 0 ? S : 1)));
  ND_CUDA(cudaMemset(s->d_cnt, 0, sizeof(uint32_t) * chunks * CNT_CHUNK));
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
  WalkParams wp{s->p.seed, s->p.p, s->p.q, s->p.stop_prob, s->p.n2v_ref_compat, steps, s->d_filter};
  const int rblocks = (int)((S + 255) / 256);
  walk_reset_kernel<<<rblocks > 1 ? rblocks : 1, 256, 0, st>>>(s->d_initial, s->g->V, S, steps, s->d_len, s->d_state, s->d_stats);
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
    const int grid = (int)(tiles < (int64_t)s->dev.sms * 4 ? tiles : (int64_t)s->dev.sms * 4);
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
    const int chunks = (V + CNT_CHUNK - 1) / CNT_CHUNK;
    // Tracking which counter chunks were touched lets the scan skip the others; it pays when the
    // counter array is large against the live pairs (late PPR steps on 2^24 vertices).  On small
    // graphs every chunk is touched every step and the flag traffic would only add contention.
    uint8_t *dirty = chunks >= 2048 ? s->d_dirty : nullptr;
    const int64_t blocks = (S + 255) / 256;
    const int grid = (int)(blocks < (int64_t)s->dev.sms * 64 ? blocks : (int64_t)s->dev.sms * 64);
    NdGraphView gv = nd_view(s->g);
    const int32_t *in_key = s->d_init_key, *in_val = s->d_init_val;
    int32_t *ukey = s->d_map_key[0], *uval = s->d_map_val[0];   // unsorted pairs written by next()
    int32_t *skey = s->d_map_key[1], *sval = s->d_map_val[1];   // sorted map of the following step
    for (int step = 0; step < steps; step++) {
      const bool last = step == steps - 1;
      const int32_t *d_n = s->d_nlive + step;
      int32_t *tmp_step = s->d_tmp + (int64_t)step * S;
      nd_phase_begin(s, ND_PHASE_NEXT);
#define ND_LAUNCH_COUNT(APPID)                                                                                         \
  if (last) walk_next_count_kernel<APPID, false><<<grid, 256, 0, st>>>(gv, wp, step, s->first, in_key, in_val, d_n, ukey, uval, s->d_rank, s->d_cnt, dirty, tmp_step, s->d_len, s->d_state, s->d_status, s->d_stats); \
  else walk_next_count_kernel<APPID, true><<<grid, 256, 0, st>>>(gv, wp, step, s->first, in_key, in_val, d_n, ukey, uval, s->d_rank, s->d_cnt, dirty, tmp_step, s->d_len, s->d_state, s->d_status, s->d_stats);
      switch (app) {
        case ND_APP_UNIFORM_WALK: ND_LAUNCH_COUNT(ND_APP_UNIFORM_WALK) break;
        case ND_APP_DEEPWALK: ND_LAUNCH_COUNT(ND_APP_DEEPWALK) break;
        case ND_APP_PPR: ND_LAUNCH_COUNT(ND_APP_PPR) break;
        default: ND_LAUNCH_COUNT(ND_APP_NODE2VEC) break;
      }
#undef ND_LAUNCH_COUNT
      nd_phase_end(s);
      nd_count_launches(1);
      if (last) break;
      nd_phase_begin(s, ND_PHASE_INVERT);
      cnt_chunk_sum_kernel<<<chunks, CNT_THREADS, 0, st>>>(s->d_cnt, V, dirty, s->d_bsum);
      cnt_scan_kernel<<<chunks, CNT_THREADS, 0, st>>>(s->d_cnt, V, s->d_bsum, dirty, s->d_offs, s->d_nlive + step + 1);
      walk_scatter_kernel<<<grid, 256, 0, st>>>(d_n, V, ukey, uval, s->d_rank, s->d_offs, skey, sval);
      nd_phase_end(s);
      nd_count_launches(3);
      in_key = skey;
      in_val = sval;
    }
  }
  nd_phase_begin(s, ND_PHASE_FINALIZE);
  const int64_t groups = (S + FIN_SAMPLES - 1) / FIN_SAMPLES;
  const int fgrid = (int)(groups < (int64_t)s->dev.sms * 16 ? groups : (int64_t)s->dev.sms * 16);
  walk_finalize_kernel<<<fgrid > 0 ? fgrid : 1, FIN_THREADS, 0, st>>>(s->d_tmp, s->d_len, S, steps, s->g->V, s->d_out, s->d_stats);
  nd_phase_end(s);
  nd_count_launches(1);
  ND_CUDA(cudaGetLastError());
  return ND_OK;
}

int nd_walk_sample(nd_sampler *s, int mode) {
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
