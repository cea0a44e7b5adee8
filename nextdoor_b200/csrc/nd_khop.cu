// k-hop neighbourhood sampling (GraphSAGE): every sample expands each vertex of hop k-1 into
// stepSize(k) neighbours.  ND_APP_KHOP draws them independently with replacement (KHopApp::next,
// src/apps/khop/khop.cu:10-23); ND_APP_KHOP_DISTINCT draws without replacement (Floyd's algorithm,
// one keyed draw per slot; all neighbours when the list is not longer than the fan-out) and ends
// with a per-hop distinct pass.
//
// Transit-parallel execution (doTransitParallelSampling, src/nextdoor.cu:2191-3006).  A step works
// on the (transit, pair) map sorted by transit; pair q = sample*n_prev + parent slot.  With load
// balancing the sorted map is cut into runs of equal transit and every run is put into a bin, the
// job of partitionTransitsInKernels (src/nextdoor.cu:1520-1802, thresholds src/utils.hpp:491-497):
//   sub-warp bin : few samples on the transit -> one sub-warp per pair, neighbours gathered from
//                  global memory (the role of identityKernel, src/nextdoor.cu:338-504);
//   block bin    : one work item; grid bin: the run is cut into several work items.  A work item
//                  is executed by one CTA that stages the transit's adjacency list in shared
//                  memory once -- a 1-D bulk copy (TMA) completing on an mbarrier for long lists,
//                  16-byte vector loads for short ones -- and serves every (sample, slot) draw of
//                  its pairs from there (gridKernel + CachedArray, src/nextdoor.cu:976-1204, 76-124).
// Bins are decided by samples-on-transit x sub-warp width (the reference's measure) and by the
// list length (staging must cost fewer sectors than the gathers it replaces).  Nothing returns
// to the host between steps: counts and work lists stay on the device.
//
// Output layout: child j of parent slot i of hop k is written at prefix_k + i*stepSize(k) + j and
// its draws are keyed by slot i*stepSize(k) + j.  The reference hands out positions inside
// [prefix_k, prefix_k + n_k) with an atomic counter (src/nextdoor.cu:295-305), so any order
// within the hop is a legal outcome of it; this one is deterministic.
#include <cstdlib>

#include "nd_common.cuh"
#include "nd_philox.cuh"

namespace {

using ndrng::Rng;

constexpr int KTHREADS = 256;
constexpr int STAGE_CAP = 11776;         // ints of shared memory for a staged list (46 KB)
constexpr int TMA_MIN_INTS = 64;         // below this the list is staged with int4 loads
constexpr int WAIT_CAP = 1 << 22;        // iteration limit of the mbarrier wait
constexpr uint8_t FLAG_PLAIN = 1, FLAG_STAGED = 2;

struct KhopParams {
  uint64_t seed;
  int64_t first_sample;
  int32_t V;
  int32_t fs;        // final sample size
  int step, steps;
  int f;             // fan-out of this step
  int sw;            // sub-warp width: next power of two >= f (subWarpSizeAtStep, src/nextdoor.cu:133-160)
  int n_prev;        // parents per sample
  int prefix_prev, prefix;  // offsets of hop k-1 / hop k inside a sample's row
  int fan_after[ND_MAX_STEPS_FANOUT];  // fan-outs of the hops after this one (for the dead-slot fill)
  int n_after;
  bool distinct;
  bool write_map;
};

// ---- mbarrier / bulk-copy wrappers (no cluster launch: the CTA is its own cluster)

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_copy_g2s(void *dst_smem, const void *src, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst_smem)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok)
               : "r"(smem_u32(bar)), "r"(parity)
               : "memory");
  return ok != 0;
}
// bounded wait: false when the limit ran out
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity) {
  for (int it = 0; it < WAIT_CAP; it++)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}

// ---- one pair: f slots drawn by a sub-warp of `sw` lanes.  `edges` points at the transit's list
// (global memory or the staged copy); the slot's lane returns its neighbour or -1.
template <bool DISTINCT, typename EdgePtr>
__device__ __forceinline__ int32_t draw_slot(const KhopParams &kp, EdgePtr edges, int32_t deg, int64_t gs, int parent,
                                             int j, bool active, int sub_base, uint32_t sub_mask) {
  int32_t idx = -1;
  if (active && deg > 0) {
    if (!DISTINCT) {
      Rng rng(kp.seed, (uint32_t)gs, (uint32_t)kp.step, (uint32_t)(parent * kp.f + j));
      idx = rng.rand_int(deg);
    } else if (deg <= kp.f) {
      idx = j < deg ? j : -1;
    } else {
      Rng rng(kp.seed, (uint32_t)gs, (uint32_t)kp.step, (uint32_t)(parent * kp.f + j));
      idx = rng.rand_int(deg - kp.f + j + 1);  // Floyd candidate of slot j
    }
  }
  if (DISTINCT) {
    // Floyd's resolution, slot after slot: a candidate already picked by an earlier slot is
    // replaced by m_j = deg - f + j.  Every lane of the warp runs the loop (ballots), each
    // sub-warp only looks at its own lanes.
    const bool floyd = active && deg > kp.f;
    int32_t fin = -1;  // final pick of this lane once its turn has passed
    for (int jj = 0; jj < kp.f; jj++) {
      const int32_t cand = __shfl_sync(0xffffffffu, idx, sub_base + jj);
      const uint32_t hit = __ballot_sync(0xffffffffu, floyd && fin == cand) & sub_mask;
      if (floyd && j == jj) fin = hit ? (deg - kp.f + jj) : cand;
    }
    if (floyd) idx = fin;
  }
  return idx >= 0 ? edges[idx] : -1;
}

// A dead slot (no neighbour) leaves its whole subtree unsampled: write the invalid id there.
__device__ __forceinline__ void fill_descendants(const KhopParams &kp, int32_t *row, int slot) {
  int64_t cnt = 1;
  int base = kp.prefix + kp.n_prev * kp.f;  // offset of hop k+1
  int n_level = kp.n_prev * kp.f;
  for (int m = 0; m < kp.n_after; m++) {
    cnt *= kp.fan_after[m];
    for (int64_t i = 0; i < cnt; i++) row[base + (int64_t)slot * cnt + i] = kp.V;
    n_level *= kp.fan_after[m];
    base += n_level;
  }
}

template <bool DISTINCT, typename EdgePtr>
__device__ __forceinline__ void process_pair(const KhopParams &kp, EdgePtr edges, int32_t deg, int32_t q,
                                             int32_t *__restrict__ out, int32_t *__restrict__ mkey,
                                             int32_t *__restrict__ mval, int j, int sub_base, uint32_t sub_mask,
                                             bool pair_ok, uint32_t &edges_cnt) {
  const int32_t s = pair_ok ? q / kp.n_prev : 0;
  const int parent = pair_ok ? q - s * kp.n_prev : 0;
  const bool active = pair_ok && j < kp.f;
  const int32_t nbr = draw_slot<DISTINCT>(kp, edges, deg, kp.first_sample + s, parent, j, active, sub_base, sub_mask);
  if (active) {
    int32_t *row = out + (int64_t)s * kp.fs;
    const int slot = parent * kp.f + j;
    row[kp.prefix + slot] = nbr >= 0 ? nbr : kp.V;
    if (nbr >= 0) edges_cnt++;
    else if (kp.n_after) fill_descendants(kp, row, slot);
    if (kp.write_map) {
      const int64_t c = (int64_t)q * kp.f + j;
      mkey[c] = nbr >= 0 ? nbr : kp.V;
      mval[c] = (int32_t)c;
    }
  }
}

__device__ __forceinline__ void flush_counts(uint32_t edges_cnt, uint32_t pairs_cnt, unsigned long long *stats) {
  for (int o = 16; o > 0; o >>= 1) {
    edges_cnt += __shfl_xor_sync(0xffffffffu, edges_cnt, o);
    pairs_cnt += __shfl_xor_sync(0xffffffffu, pairs_cnt, o);
  }
  if ((threadIdx.x & 31) == 0) {
    if (edges_cnt) atomicAdd(&stats[0], (unsigned long long)edges_cnt);
    if (pairs_cnt) atomicAdd(&stats[1], (unsigned long long)pairs_cnt);
  }
}

// ---------------------------------------------------------------- sub-warp kernel (and the sample-parallel path)
// FROM_MAP: pair i of the transit-sorted map; otherwise pair i in sample order, transit read from
// the previous hop (sampleParallelKernel, src/nextdoor.cu:1402-1424).
template <bool DISTINCT, bool FROM_MAP>
__global__ void __launch_bounds__(KTHREADS)
khop_pairs_kernel(NdGraphView g, KhopParams kp, const int32_t *__restrict__ in_key, const int32_t *__restrict__ in_val,
                  const int32_t *__restrict__ d_n, int64_t n_host, const int32_t *__restrict__ initial,
                  const uint8_t *__restrict__ flags, int32_t *__restrict__ out, int32_t *__restrict__ mkey,
                  int32_t *__restrict__ mval, int *__restrict__ status, unsigned long long *__restrict__ stats) {
  const int64_t n = FROM_MAP ? (int64_t)*d_n : n_host;
  const int lane = threadIdx.x & 31;
  const int per_warp = 32 / kp.sw;
  const int sub = lane / kp.sw, j = lane % kp.sw;
  const int sub_base = sub * kp.sw;
  const uint32_t sub_mask = (kp.sw == 32 ? 0xffffffffu : ((1u << kp.sw) - 1u)) << sub_base;
  const int64_t warp_id = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  uint32_t edges_cnt = 0, pairs_cnt = 0;
  for (int64_t base = warp_id * per_warp; base < n; base += n_warps * per_warp) {
    const int64_t i = base + sub;
    bool ok = i < n;
    int32_t q = 0, t = -1;
    if (ok) {
      if (FROM_MAP) {
        t = in_key[i];
        q = in_val[i];
      } else {
        q = (int32_t)i;
        const int32_t s = q / kp.n_prev;
        t = kp.step == 0 ? initial[s] : out[(int64_t)s * kp.fs + kp.prefix_prev + (q - s * kp.n_prev)];
      }
      if (t < 0 || t >= g.V) {
        if (FROM_MAP) atomicOr(status, ND_DEV_BAD_TRANSIT);
        ok = false;  // sample-parallel: a dead parent; its subtree was filled when it died
      }
    }
    if (ok && FROM_MAP && flags && flags[t] == FLAG_STAGED) ok = false;  // served by the staged kernel
    int32_t rs = 0, deg = 0;
    if (ok) {
      rs = __ldg(g.row_ptr + t);
      deg = __ldg(g.row_ptr + t + 1) - rs;
      if (j == 0) pairs_cnt++;
    }
    process_pair<DISTINCT>(kp, g.col + rs, deg, q, out, mkey, mval, j, sub_base, sub_mask, ok, edges_cnt);
  }
  flush_counts(edges_cnt, pairs_cnt, stats);
}

// ---------------------------------------------------------------- binning
// One thread per map position; the head of a run of equal transits bisects for the run's end,
// classifies the transit and, for the block / grid bins, appends the run's work items.
struct BinCounts { int32_t subwarp_transits, block_transits, grid_transits, items; };

__global__ void __launch_bounds__(KTHREADS)
khop_bin_kernel(NdGraphView g, const int32_t *__restrict__ keys, const int32_t *__restrict__ d_n, int f, int sw,
                int item_pairs, int64_t items_cap, uint8_t *__restrict__ flags, int2 *__restrict__ items,
                BinCounts *__restrict__ bc, int *__restrict__ status) {
  const int n = *d_n;
  const int lane = threadIdx.x & 31;
  const int warp_id = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int n_warps = (gridDim.x * blockDim.x) >> 5;
  for (int base = warp_id * 32; base < n; base += n_warps * 32) {
    // a warp looks at 32 consecutive map positions; run heads are found with one ballot, and a
    // run that ends inside the window needs no search at all
    const int i = base + lane;
    const int32_t t = i < n ? keys[i] : -2;
    int32_t prev = __shfl_up_sync(0xffffffffu, t, 1);
    if (lane == 0) prev = base > 0 ? keys[base - 1] : -1;
    const bool head = i < n && (i == 0 || prev != t);
    const uint32_t heads = __ballot_sync(0xffffffffu, head);
    if (!head || t < 0 || t >= g.V) continue;
    const uint32_t later = lane == 31 ? 0u : (heads & ~((2u << lane) - 1u));
    int end;
    if (later) {
      end = base + __ffs(later) - 1;
    } else {
      const int wend = min(base + 32, n);
      end = wend;
      if (wend < n && keys[wend] == t) {  // the run leaves the window: bisect for its end
        int lo = wend + 1, hi = n;
        while (lo < hi) {
          const int mid = lo + (hi - lo) / 2;
          if (keys[mid] == t) lo = mid + 1; else hi = mid;
        }
        end = lo;
      }
    }
    const int count = end - i;
    const int32_t deg = __ldg(g.row_ptr + t + 1) - __ldg(g.row_ptr + t);
    const int64_t work = (int64_t)count * sw;  // threads the run occupies (src/nextdoor.cu:1565-1573)
    // staging reads deg/8 sectors once; gathering reads up to count*f sectors
    const bool worth = deg > 0 && (int64_t)deg <= 8ll * count * f;
    uint8_t flag = FLAG_PLAIN;
    if (work >= 256 && worth) {  // a CTA's worth of draws: LoadBalancingThreshold::GridLevel
      const int n_items = (count + item_pairs - 1) / item_pairs;
      const int at = atomicAdd(&bc->items, n_items);
      if ((int64_t)at + n_items <= items_cap) {
        for (int c = 0; c < n_items; c++) {
          const int st = i + c * item_pairs;
          items[at + c] = make_int2(st, min(item_pairs, end - st));
        }
        flag = FLAG_STAGED;
        atomicAdd(n_items > 1 ? &bc->grid_transits : &bc->block_transits, 1);
      } else {
        atomicOr(status, ND_DEV_OVERFLOW);
      }
    }
    if (flag == FLAG_PLAIN) atomicAdd(&bc->subwarp_transits, 1);
    flags[t] = flag;
  }
}

// ---------------------------------------------------------------- block / grid bins: staged adjacency list
template <bool DISTINCT>
__global__ void __launch_bounds__(KTHREADS)
khop_staged_kernel(NdGraphView g, KhopParams kp, const int32_t *__restrict__ in_key, const int32_t *__restrict__ in_val,
                   const int2 *__restrict__ items, const BinCounts *__restrict__ bc, int64_t items_cap,
                   int32_t *__restrict__ out, int32_t *__restrict__ mkey, int32_t *__restrict__ mval,
                   int *__restrict__ status, unsigned long long *__restrict__ stats) {
  __shared__ __align__(128) int32_t stage[STAGE_CAP];
  __shared__ __align__(8) uint64_t bar;
  __shared__ int32_t sh_q[KTHREADS];   // pair ids of the work item (item_pairs <= KTHREADS)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int per_warp = 32 / kp.sw;
  const int sub = lane / kp.sw, j = lane % kp.sw;
  const int sub_base = sub * kp.sw;
  const uint32_t sub_mask = (kp.sw == 32 ? 0xffffffffu : ((1u << kp.sw) - 1u)) << sub_base;
  const int subs_per_cta = (KTHREADS / 32) * per_warp;
  int n_items = bc->items;
  if ((int64_t)n_items > items_cap) n_items = (int)items_cap;
  if (threadIdx.x == 0) mbar_init(&bar, 1);
  __syncthreads();
  uint32_t parity = 0;
  bool tma_ok = true;   // cleared for good after a wait ran out
  uint32_t edges_cnt = 0, pairs_cnt = 0;
  for (int it = blockIdx.x; it < n_items; it += gridDim.x) {
    const int2 item = items[it];
    const int32_t t = in_key[item.x];
    const int32_t rs = __ldg(g.row_ptr + t);
    const int32_t deg = __ldg(g.row_ptr + t + 1) - rs;
    // 16-byte aligned window [a0, a1) around the list; the arrays carry padding past the last edge
    const int32_t a0 = rs & ~3;
    const int32_t a1 = (rs + deg + 3) & ~3;
    const int win = a1 - a0;
    // after a bulk copy whose wait ran out, the CTA stops using `stage` altogether: that copy may
    // still land there, so every later item gathers from global memory
    bool staged = win <= STAGE_CAP && tma_ok;
    sh_q[threadIdx.x] = threadIdx.x < item.y ? in_val[item.x + threadIdx.x] : 0;  // one coalesced load, overlaps the copy
    if (staged) {
      if (win >= TMA_MIN_INTS) {
        if (threadIdx.x == 0) {
          // the previous item's reads of `stage` are ordered before this async write
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          mbar_expect_tx(&bar, (uint32_t)win * 4u);
          bulk_copy_g2s(stage, g.col + a0, (uint32_t)win * 4u, &bar);
        }
        const bool done = mbar_wait_bounded(&bar, parity);
        parity ^= 1u;
        if (!done) {  // give up on bulk copies in this CTA; gather from global memory instead
          atomicOr(status, ND_DEV_WAIT_TIMEOUT);
          tma_ok = false;
          staged = false;
        }
        // every lane must agree (a lane that timed out later than another one)
        staged = __syncthreads_and(staged ? 1 : 0) != 0;
        if (!staged) tma_ok = false;
      } else {
        const int4 *src = reinterpret_cast<const int4 *>(g.col + a0);
        int4 *dst = reinterpret_cast<int4 *>(stage);
        for (int v = threadIdx.x; v < win / 4; v += KTHREADS) dst[v] = __ldg(src + v);
        __syncthreads();
      }
    } else {
      __syncthreads();  // list longer than the staging buffer: only sh_q needs publishing
    }
    const int32_t *sh_edges = stage + (rs - a0);
    const int32_t *gl_edges = g.col + rs;
    for (int p0 = 0; p0 < item.y; p0 += subs_per_cta) {
      const int p = p0 + warp * per_warp + sub;
      const bool ok = p < item.y;
      const int32_t q = ok ? sh_q[p] : 0;
      if (ok && j == 0) pairs_cnt++;
      if (staged) process_pair<DISTINCT>(kp, sh_edges, deg, q, out, mkey, mval, j, sub_base, sub_mask, ok, edges_cnt);
      else process_pair<DISTINCT>(kp, gl_edges, deg, q, out, mkey, mval, j, sub_base, sub_mask, ok, edges_cnt);
    }
    __syncthreads();  // all reads of `stage` done before the next item overwrites it
  }
  // a copy that never signalled may still be in flight: give it one more bounded wait before
  // the CTA's shared memory is released
  if (!tma_ok) mbar_wait_bounded(&bar, parity ^ 1u);
  flush_counts(edges_cnt, pairs_cnt, stats);
}

// ---------------------------------------------------------------- helpers

__global__ void fill_i32_kernel(int32_t *__restrict__ p, int64_t n, int32_t v) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) p[i] = v;
}

// zero the counters; samples whose seed is not a vertex get a row of invalid ids
__global__ void khop_reset_kernel(const int32_t *__restrict__ initial, int32_t V, int64_t S, int32_t fs,
                                  int32_t *__restrict__ out, unsigned long long *__restrict__ stats) {
  const int64_t s = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (s < 8) stats[s] = 0ull;
  if (s >= S) return;
  const int32_t t = initial[s];
  if (t < 0 || t >= V) for (int i = 0; i < fs; i++) out[s * fs + i] = V;
}

int grid_for(int64_t threads, int sms, int per_sm) {
  int64_t b = (threads + KTHREADS - 1) / KTHREADS;
  const int64_t cap = (int64_t)sms * per_sm;
  if (b > cap) b = cap;
  return (int)(b > 0 ? b : 1);
}

int next_pow2(int x) { int p = 1; while (p < x) p <<= 1; return p; }

}  // namespace

int nd_khop_alloc(nd_sampler *s) {
  const nd_app_params &p = s->p;
  int64_t n = 1, cap = 1;
  for (int k = 0; k < p.steps; k++) {
    ND_REQUIRE(p.fanout[k] >= 1 && p.fanout[k] <= 32, ND_ERR_ARG, "fan-out %d of hop %d outside [1,32]", p.fanout[k], k);
    if (k < p.steps - 1) { n *= p.fanout[k]; cap = n; }
  }
  if (p.app == ND_APP_KHOP_DISTINCT) {
    int64_t m = 1;
    for (int k = 0; k < p.steps; k++) { m *= p.fanout[k]; ND_REQUIRE(m <= 2048, ND_ERR_ARG, "distinct: hop %d holds %lld ids, limit 2048", k, (long long)m); }
  }
  const int64_t S = s->S;
  s->map_cap = S * cap;
  ND_REQUIRE(s->map_cap * 32 < ((int64_t)1 << 31), ND_ERR_RANGE, "%lld (transit, sample) pairs per step do not fit int32 pair ids", (long long)s->map_cap);
  const size_t mc = (size_t)(s->map_cap > 0 ? s->map_cap : 1);
  for (int i = 0; i < 2; i++) {
    ND_CUDA(cudaMalloc(&s->d_map_key[i], sizeof(int32_t) * mc));
    ND_CUDA(cudaMalloc(&s->d_map_val[i], sizeof(int32_t) * mc));
  }
  ND_CUDA(cudaMalloc(&s->d_init_key, sizeof(int32_t) * (size_t)(S > 0 ? S : 1)));
  ND_CUDA(cudaMalloc(&s->d_init_val, sizeof(int32_t) * (size_t)(S > 0 ? S : 1)));
  ND_CUDA(cudaMalloc(&s->d_nlive, sizeof(int32_t) * (size_t)(2 * p.steps + 4)));
  // work items of the block / grid bins: a staged run has >= 1 pair and is cut every 128+ pairs
  s->runs_cap = s->map_cap / 2 + s->map_cap / 128 + 1024;
  ND_CUDA(cudaMalloc(&s->d_runs, sizeof(int2) * (size_t)s->runs_cap));
  ND_CUDA(cudaMalloc(&s->d_bin_counts, sizeof(int32_t) * 4 * (size_t)p.steps));
  ND_CUDA(cudaMalloc(&s->d_state, (size_t)s->g->V + 16));  // per-transit bin flags (kernelTypeForTransit, src/nextdoor.cu:2309)
  if (p.app == ND_APP_KHOP_DISTINCT) ND_CUDA(cudaMalloc(&s->d_hop_counts, sizeof(int32_t) * (size_t)(S > 0 ? S : 1) * p.steps));
  const int key_bits = nd_bit_length((uint32_t)(s->g->V > 1 ? s->g->V - 1 : 1));
  ND_TRY(nd_radix_scratch_alloc(&s->radix, key_bits, s->map_cap > S ? s->map_cap : S));
  // host-known sizes of the unsorted child maps, kept on the device for the sort
  std::vector<int32_t> full((size_t)p.steps + 1, 0);
  int64_t m = S;
  for (int k = 0; k < p.steps; k++) { m *= p.fanout[k]; full[k] = (int32_t)(k < p.steps - 1 ? m : 0); }
  ND_CUDA(cudaMemcpy(s->d_nlive + p.steps + 2, full.data(), sizeof(int32_t) * (size_t)p.steps, cudaMemcpyHostToDevice));
  return ND_OK;
}

int nd_khop_sample(nd_sampler *s, int mode) {
  // Load balancing of k-hop = binning by run size + adjacency lists staged in shared memory.  On
  // B200 it measured slower than the plain pairs kernel in every configuration tried (2^21-vertex
  // R-MAT graph; 262,144 and 2,097,152 seeds; with and without replacement: 9-25 % slower): the
  // lists that are short enough to stage and hot enough to pay are served by the 126 MB L2 anyway.
  // So the load-balanced mode runs the plain transit-parallel kernels unless ND_KHOP_STAGING=1.
  if (mode == ND_MODE_TRANSIT_PARALLEL_LB) {
    const char *e = getenv("ND_KHOP_STAGING");
    if (!(e && e[0] == '1')) mode = ND_MODE_TRANSIT_PARALLEL;
  }
  const nd_app_params &p = s->p;
  const int64_t S = s->S;
  const bool distinct = p.app == ND_APP_KHOP_DISTINCT;
  NdGraphView gv = nd_view(s->g);
  cudaStream_t st = s->stream;
  khop_reset_kernel<<<grid_for(S > 8 ? S : 8, 1 << 20, 1 << 10), KTHREADS, 0, st>>>(s->d_initial, s->g->V, S, s->fs, s->d_out, s->d_stats);
  nd_count_launches(1);
  if (mode == ND_MODE_TRANSIT_PARALLEL_LB) {
    ND_CUDA(cudaMemsetAsync(s->d_bin_counts, 0, sizeof(int32_t) * 4 * (size_t)p.steps, st));
  }
  const int32_t *in_key = s->d_init_key, *in_val = s->d_init_val;
  int cur = 0;
  int n_prev = 1, prefix_prev = 0, prefix = 0;
  for (int k = 0; k < p.steps; k++) {
    KhopParams kp;
    kp.seed = p.seed; kp.first_sample = s->first; kp.V = s->g->V; kp.fs = s->fs;
    kp.step = k; kp.steps = p.steps; kp.f = p.fanout[k]; kp.sw = next_pow2(kp.f);
    kp.n_prev = n_prev; kp.prefix_prev = prefix_prev; kp.prefix = prefix;
    kp.n_after = 0;
    for (int m = k + 1; m < p.steps; m++) kp.fan_after[kp.n_after++] = p.fanout[m];
    kp.distinct = distinct;
    const bool last = k == p.steps - 1;
    kp.write_map = mode != ND_MODE_SAMPLE_PARALLEL && !last;
    const int64_t n_pairs_full = S * n_prev;
    int32_t *mk = s->d_map_key[cur], *mv = s->d_map_val[cur];
    const int32_t *d_n = s->d_nlive + k;
    const int grid = grid_for(n_pairs_full * kp.sw, s->dev.sms, 16);
    if (mode == ND_MODE_SAMPLE_PARALLEL) {
      nd_phase_begin(s, ND_PHASE_NEXT);
      if (distinct) khop_pairs_kernel<true, false><<<grid, KTHREADS, 0, st>>>(gv, kp, nullptr, nullptr, nullptr, n_pairs_full, s->d_initial, nullptr, s->d_out, mk, mv, s->d_status, s->d_stats);
      else khop_pairs_kernel<false, false><<<grid, KTHREADS, 0, st>>>(gv, kp, nullptr, nullptr, nullptr, n_pairs_full, s->d_initial, nullptr, s->d_out, mk, mv, s->d_status, s->d_stats);
      nd_phase_end(s);
      nd_count_launches(1);
    } else {
      if (kp.write_map) {  // children of pairs that died earlier are never visited: pre-mark them dead
        fill_i32_kernel<<<grid_for(n_pairs_full * kp.f, s->dev.sms, 16), KTHREADS, 0, st>>>(mk, n_pairs_full * kp.f, s->g->V);
        nd_count_launches(1);
      }
      const bool lb = mode == ND_MODE_TRANSIT_PARALLEL_LB;
      uint8_t *flags = lb ? (uint8_t *)s->d_state : nullptr;
      BinCounts *bc = (BinCounts *)s->d_bin_counts + k;
      // up to 16 rounds of a CTA's sub-warps (TRANSITS_PER_THREAD, src/nextdoor.cu:976), at most one pair per thread
      const int item_pairs = 16 * (KTHREADS / kp.sw) < KTHREADS ? 16 * (KTHREADS / kp.sw) : KTHREADS;
      if (lb) {
        nd_phase_begin(s, ND_PHASE_BIN);
        khop_bin_kernel<<<grid_for(n_pairs_full, s->dev.sms, 16), KTHREADS, 0, st>>>(gv, in_key, d_n, kp.f, kp.sw, item_pairs, s->runs_cap, flags, (int2 *)s->d_runs, bc, s->d_status);
        nd_phase_end(s);
        nd_count_launches(1);
      }
      nd_phase_begin(s, ND_PHASE_NEXT);
      if (distinct) khop_pairs_kernel<true, true><<<grid, KTHREADS, 0, st>>>(gv, kp, in_key, in_val, d_n, 0, s->d_initial, flags, s->d_out, mk, mv, s->d_status, s->d_stats);
      else khop_pairs_kernel<false, true><<<grid, KTHREADS, 0, st>>>(gv, kp, in_key, in_val, d_n, 0, s->d_initial, flags, s->d_out, mk, mv, s->d_status, s->d_stats);
      nd_count_launches(1);
      if (lb) {
        const int sgrid = s->dev.sms * 4;
        if (distinct) khop_staged_kernel<true><<<sgrid, KTHREADS, 0, st>>>(gv, kp, in_key, in_val, (const int2 *)s->d_runs, bc, s->runs_cap, s->d_out, mk, mv, s->d_status, s->d_stats);
        else khop_staged_kernel<false><<<sgrid, KTHREADS, 0, st>>>(gv, kp, in_key, in_val, (const int2 *)s->d_runs, bc, s->runs_cap, s->d_out, mk, mv, s->d_status, s->d_stats);
        nd_count_launches(1);
      }
      nd_phase_end(s);
      if (!last) {
        nd_phase_begin(s, ND_PHASE_INVERT);
        NdSortArrays arr;
        arr.nwords = 2;
        arr.a[0] = (uint32_t *)mk; arr.a[1] = (uint32_t *)mv; arr.a[2] = nullptr;
        arr.b[0] = (uint32_t *)s->d_map_key[cur ^ 1]; arr.b[1] = (uint32_t *)s->d_map_val[cur ^ 1]; arr.b[2] = nullptr;
        bool in_b = false;
        ND_TRY(nd_radix_sort(s->dev, st, &s->radix, s->radix.plan, arr, 0, s->d_nlive + p.steps + 2 + k, s->d_nlive + k + 1,
                             true, (uint32_t)s->g->V, false, &in_b));
        nd_phase_end(s);
        const int res = in_b ? (cur ^ 1) : cur;
        in_key = s->d_map_key[res];
        in_val = s->d_map_val[res];
        cur = res ^ 1;
      }
    }
    prefix_prev = prefix;
    prefix += n_prev * kp.f;
    n_prev *= kp.f;
  }
  if (distinct) {
    nd_phase_begin(s, ND_PHASE_DEDUP);
    int off = 0, n = 1;
    for (int k = 0; k < p.steps; k++) {
      n *= p.fanout[k];
      ND_TRY(nd_distinct_launch(st, s->d_out + off, S, n, s->fs, s->g->V, s->d_hop_counts + k, p.steps));
      nd_count_launches(1);
      off += n;
    }
    nd_phase_end(s);
  }
  ND_CUDA(cudaGetLastError());
  return ND_OK;
}
