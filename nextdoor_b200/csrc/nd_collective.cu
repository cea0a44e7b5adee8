// Collective-neighbourhood layer sampling: one sample is a batch of transits and every layer draws
// stepSize vertices for the whole batch.
//
// ND_APP_FASTGCN_REF / ND_APP_LADIES_REF follow the reference's shipped next()
// (src/apps/fastgcn/fastgcnSampling.cu:23-47, src/apps/ladies/ladiessampling.cu:23-47): a vertex
// drawn uniformly from the whole graph, then one has_edge_logn probe (src/csr.hpp:343-359) per
// transit to fill the layer's adjacency (row, col) entries.
//
// ND_APP_FASTGCN_IS / ND_APP_LADIES_IS are the importance samplers the reference does not have:
// the candidates of a layer are the sorted unique union of the transits' neighbours, weighted by
// degree^2 (FastGCN) or by the sum over transits of (w(i,v)/rowsum_i)^2 (LADIES); the weights are
// prefix-summed in candidate order and every slot inverts the CDF at u * total.  Pipeline per
// layer, the collective-neighbourhood construction of the reference made useful
// (collectiveNeighbrsSize / collectiveNeighborhood, src/nextdoor.cu:1206-1283, whose copied
// neighbourhood the shipped next() never reads):
//   sizes   : sum of degrees per sample                        (one warp per sample)
//   gather  : every neighbour id, its sample and its LADIES term into one flat array
//   sort    : by id, then stably by sample, with the in-house radix sort (3 words per element)
//   weigh   : the first element of every (sample, id) run carries the candidate's weight, the
//             rest carry 0, so no compaction pass is needed and the CDF is unchanged
//   sample  : one CTA per sample: block-wide prefix sum built from warp-shuffle scans, the
//             stepSize inverse-CDF draws, and the adjacency probes
// The per-layer sizes come back to the host once (the reference does the same before its
// per-step cudaMalloc, src/nextdoor.cu:2413-2429) so that samples can be processed in chunks that
// fit the candidate buffers whatever the hub sizes are.
#include <algorithm>
#include <cstdlib>
#include <vector>

#include "nd_common.cuh"
#include "nd_philox.cuh"

namespace {

using ndrng::Rng;
constexpr int CTHREADS = 256;

struct CollParams {
  uint64_t seed;
  int64_t first_sample;
  int32_t V, fs, L, B, stride, step, ntr;
  int app;
};

__device__ __forceinline__ const int32_t *transits_of(const CollParams &cp, const int32_t *initial, const int32_t *out, int64_t s) {
  return cp.step == 0 ? initial + s * cp.B : out + s * cp.fs + (int64_t)(cp.step - 1) * cp.L;
}

__device__ __forceinline__ bool has_edge_logn(const NdGraphView &g, int32_t src, int32_t dst) {
  int32_t l = __ldg(g.row_ptr + src), r = __ldg(g.row_ptr + src + 1) - 1;
  while (l <= r) {
    const int32_t m = l + (r - l) / 2;
    const int32_t e = __ldg(g.col + m);
    if (e == dst) return true;
    if (e < dst) l = m + 1; else r = m - 1;
  }
  return false;
}

// adjacency entries of one layer of one sample: (row,col) = (i,j) where transit i -- vertex j is an edge
__device__ __forceinline__ void emit_adjacency(const NdGraphView &g, const CollParams &cp, const int32_t *tr,
                                               const int32_t *layer, int32_t *arow, int32_t *acol) {
  for (int e = threadIdx.x; e < cp.stride; e += blockDim.x) {
    const int i = e / cp.L, j = e - i * cp.L;
    int32_t ri = -1, cj = -1;
    if (i < cp.ntr) {
      const int32_t t = tr[i], v = layer[j];
      if (t >= 0 && t < cp.V && v >= 0 && v < cp.V && has_edge_logn(g, t, v)) { ri = i; cj = j; }
    }
    arow[e] = ri;
    acol[e] = cj;
  }
}

// ---------------------------------------------------------------- reference semantics: uniform over V
__global__ void __launch_bounds__(CTHREADS)
coll_ref_kernel(NdGraphView g, CollParams cp, int steps, int64_t S, const int32_t *__restrict__ initial, int32_t *out,
                int32_t *__restrict__ adj_row, int32_t *__restrict__ adj_col, unsigned long long *__restrict__ stats) {
  __shared__ int32_t sh_tr[1024];
  __shared__ int32_t sh_layer[1024];
  for (int64_t s = blockIdx.x; s < S; s += gridDim.x) {
    for (int step = 0; step < steps; step++) {
      cp.step = step;
      cp.ntr = step == 0 ? cp.B : cp.L;
      const int32_t *tr = transits_of(cp, initial, out, s);
      for (int i = threadIdx.x; i < cp.ntr; i += CTHREADS) sh_tr[i] = tr[i];
      for (int j = threadIdx.x; j < cp.L; j += CTHREADS) {
        Rng rng(cp.seed, (uint32_t)(cp.first_sample + s), (uint32_t)step, (uint32_t)j);
        const int32_t id = rng.rand_int(cp.V);
        sh_layer[j] = id;
        out[s * cp.fs + (int64_t)step * cp.L + j] = id;
      }
      __syncthreads();
      const int64_t a = (s * steps + step) * (int64_t)cp.stride;
      emit_adjacency(g, cp, sh_tr, sh_layer, adj_row + a, adj_col + a);
      __syncthreads();
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    stats[0] = (unsigned long long)S * steps * cp.L;
    stats[1] = (unsigned long long)S * (cp.B + (unsigned long long)(steps - 1) * cp.L);
  }
}

// ---------------------------------------------------------------- importance sampling pipeline

// one warp per sample: sum of the transits' degrees
__global__ void __launch_bounds__(CTHREADS)
coll_sizes_kernel(NdGraphView g, CollParams cp, int64_t S, const int32_t *__restrict__ initial,
                  const int32_t *__restrict__ out, int32_t *__restrict__ sizes) {
  const int64_t s = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  if (s >= S) return;
  const int lane = threadIdx.x & 31;
  const int32_t *tr = transits_of(cp, initial, out, s);
  int64_t sum = 0;
  for (int i = lane; i < cp.ntr; i += 32) {
    const int32_t t = tr[i];
    if (t >= 0 && t < cp.V) sum += __ldg(g.row_ptr + t + 1) - __ldg(g.row_ptr + t);
  }
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane == 0) sizes[s] = (int32_t)(sum > 0x7fffffff ? 0x7fffffff : sum);
}

// one CTA per sample of the chunk: copy every transit's neighbours into the flat candidate arrays.
// Warp w takes transits w, w+8, ...; the start of transit i inside the sample's region is the
// running sum of the degrees before it (shared-memory scan by thread 0: ntr <= 1024).
__global__ void __launch_bounds__(CTHREADS)
coll_gather_kernel(NdGraphView g, CollParams cp, int64_t s0, int64_t s1, const int32_t *__restrict__ initial,
                   const int32_t *__restrict__ out, const int64_t *__restrict__ offs, uint32_t *__restrict__ c_id,
                   uint32_t *__restrict__ c_seg, uint32_t *__restrict__ c_w) {
  __shared__ int32_t sh_start[1025];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int64_t s = s0 + blockIdx.x; s < s1; s += gridDim.x) {
    const int32_t *tr = transits_of(cp, initial, out, s);
    if (threadIdx.x == 0) {
      int32_t run = 0;
      for (int i = 0; i < cp.ntr; i++) {
        sh_start[i] = run;
        const int32_t t = tr[i];
        if (t >= 0 && t < cp.V) run += __ldg(g.row_ptr + t + 1) - __ldg(g.row_ptr + t);
      }
      sh_start[cp.ntr] = run;
    }
    __syncthreads();
    const int64_t base = offs[s] - offs[s0];
    for (int i = warp; i < cp.ntr; i += CTHREADS / 32) {
      const int32_t t = tr[i];
      if (t < 0 || t >= cp.V) continue;
      const int32_t rs = __ldg(g.row_ptr + t), deg = __ldg(g.row_ptr + t + 1) - rs;
      float rowsum = 0.f;
      if (cp.app == ND_APP_LADIES_IS) {  // fp64 partial sums: the order of the adds does not matter
        double part = 0.0;
        for (int e = lane; e < deg; e += 32) part += (double)__ldg(g.w + rs + e);
        for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        rowsum = (float)part;
      }
      const int64_t dst = base + sh_start[i];
      for (int e = lane; e < deg; e += 32) {
        c_id[dst + e] = (uint32_t)__ldg(g.col + rs + e);
        c_seg[dst + e] = (uint32_t)(s - s0);
        float term = 0.f;
        if (cp.app == ND_APP_LADIES_IS) {
          const float r = __fdiv_rn(__ldg(g.w + rs + e), rowsum);
          term = __fmul_rn(r, r);
        }
        c_w[dst + e] = __float_as_uint(term);
      }
    }
    __syncthreads();
  }
}

// thread per element: the first element of a (sample, id) run gets the candidate's weight (for
// LADIES the run's terms summed in their stable order), the others get 0
__global__ void __launch_bounds__(CTHREADS)
coll_weigh_kernel(NdGraphView g, int app, int64_t n, const uint32_t *__restrict__ c_id, const uint32_t *__restrict__ c_seg,
                  const uint32_t *__restrict__ c_w, float *__restrict__ wt, unsigned long long *__restrict__ stats) {
  uint32_t heads = 0;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x) {
    const uint32_t id = c_id[e], seg = c_seg[e];
    const bool head = e == 0 || c_id[e - 1] != id || c_seg[e - 1] != seg;
    float w = 0.f;
    if (head) {
      heads++;
      if (app == ND_APP_FASTGCN_IS) {
        const float d = __int2float_rn(__ldg(g.row_ptr + id + 1) - __ldg(g.row_ptr + id));
        w = __fmul_rn(d, d);
      } else {
        for (int64_t k = e; k < n && c_id[k] == id && c_seg[k] == seg; k++) w = __fadd_rn(w, __uint_as_float(c_w[k]));
      }
    }
    wt[e] = w;
  }
  for (int o = 16; o > 0; o >>= 1) heads += __shfl_xor_sync(0xffffffffu, heads, o);
  if ((threadIdx.x & 31) == 0 && heads) atomicAdd(&stats[6], (unsigned long long)heads);
}

// one CTA per sample: inclusive prefix sum of the weights over the sample's region (warp-shuffle
// scans + carry), then the layer's draws and the adjacency entries
__global__ void __launch_bounds__(CTHREADS)
coll_sample_kernel(NdGraphView g, CollParams cp, int steps, int64_t s0, int64_t s1, const int32_t *__restrict__ initial,
                   int32_t *out, const int64_t *__restrict__ offs, const uint32_t *__restrict__ c_id,
                   const float *__restrict__ wt, double *__restrict__ cdf, int32_t *__restrict__ adj_row,
                   int32_t *__restrict__ adj_col, float *__restrict__ prob, unsigned long long *__restrict__ stats) {
  __shared__ double warp_tot[CTHREADS / 32];
  __shared__ double carry_sh;
  __shared__ int32_t sh_tr[1024];
  __shared__ int32_t sh_layer[1024];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int64_t s = s0 + blockIdx.x; s < s1; s += gridDim.x) {
    const int64_t base = offs[s] - offs[s0];
    const int64_t n = offs[s + 1] - offs[s];
    // fp64 accumulation of the fp32 weights (sums agree with any other order of addition to
    // ~1e-16; FastGCN's integer weights sum exactly)
    if (threadIdx.x == 0) carry_sh = 0.0;
    __syncthreads();
    for (int64_t c0 = 0; c0 < n; c0 += CTHREADS) {
      const int64_t i = c0 + threadIdx.x;
      double inc = i < n ? (double)wt[base + i] : 0.0;
      for (int o = 1; o < 32; o <<= 1) {
        const double t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
      }
      if (lane == 31) warp_tot[warp] = inc;
      __syncthreads();
      double woff = carry_sh;
      for (int w = 0; w < warp; w++) woff += warp_tot[w];
      if (i < n) cdf[base + i] = woff + inc;
      __syncthreads();
      if (threadIdx.x == CTHREADS - 1) carry_sh = woff + inc;
      __syncthreads();
    }
    const double total = carry_sh;
    const int32_t *tr = transits_of(cp, initial, out, s);
    for (int i = threadIdx.x; i < cp.ntr; i += CTHREADS) sh_tr[i] = tr[i];
    uint32_t valid = 0;
    for (int j = threadIdx.x; j < cp.L; j += CTHREADS) {
      int32_t pick = cp.V;
      float pr = 0.f;
      if (n > 0 && total > 0.0) {
        Rng rng(cp.seed, (uint32_t)(cp.first_sample + s), (uint32_t)cp.step, (uint32_t)j);
        const double target = (double)rng.uniform() * total;
        int64_t lo = 0, hi = n - 1;  // first index whose cdf reaches the target
        while (lo < hi) {
          const int64_t mid = lo + (hi - lo) / 2;
          if (cdf[base + mid] >= target) hi = mid; else lo = mid + 1;
        }
        pick = (int32_t)c_id[base + lo];
        pr = (float)((double)wt[base + lo] / total);
        valid++;
      }
      sh_layer[j] = pick;
      out[s * cp.fs + (int64_t)cp.step * cp.L + j] = pick;
      prob[s * cp.fs + (int64_t)cp.step * cp.L + j] = pr;
    }
    __syncthreads();
    const int64_t a = (s * steps + cp.step) * (int64_t)cp.stride;
    emit_adjacency(g, cp, sh_tr, sh_layer, adj_row + a, adj_col + a);
    for (int o = 16; o > 0; o >>= 1) valid += __shfl_xor_sync(0xffffffffu, valid, o);
    if (lane == 0 && valid) atomicAdd(&stats[0], (unsigned long long)valid);
    __syncthreads();
  }
}

// ---------------------------------------------------------------- importance sampling, bitmap path
//
// When a bit per vertex fits the CTA's shared memory (V up to about 1.4 M with 227 KB), the union
// of a sample's neighbour lists needs no sort: one CTA per sample streams the transits' lists and
// sets the neighbours' bits; a popcount scan over groups of BM_GROUP_WORDS words ranks every set
// bit, which is the candidate's index in the sorted unique union; the candidates' weights are
// summed per group and scanned in fp64, and a draw bisects the group sums and then walks the one
// group its target falls into.  FastGCN weights are recomputed from the row offsets where they are
// needed; LADIES accumulates its terms per candidate rank in a global fp64 array (one V-entry
// region per CTA) during a second pass over the lists.  No host round trip, no chunking: one
// launch per layer for all samples.  Sums are fp64, so they agree with the sorted sequential
// order to ~1e-16 (FastGCN's integer weights sum exactly).
constexpr int BM_THREADS = 1024;
constexpr int BM_GROUP_WORDS = 16;   // 512 candidates per group
constexpr int BM_BIG_LIST = 4096;    // lists at least this long are streamed by the whole CTA

// The bitmap, the group prefix counts and the group CDF make the "big" part (about V/8 + 3V/128
// bytes); it lives in shared memory when the whole layout fits the CTA's opt-in shared memory
// (graphs up to about 1.4 M vertices) and otherwise in a per-CTA slice of a global scratch array
// (glob_bytes > 0), where the same code runs on L2-resident words.  The small part (transits,
// layer, row sums, reduction scratch) is always in shared memory.
struct BmLayout {
  int words, groups;
  uint32_t off_gcdf, off_gpref;                        // inside the big part (the bitmap is at 0)
  uint32_t off_tr, off_layer, off_rowsum, off_red;     // inside shared memory
  uint32_t bytes;                                      // dynamic shared memory of the launch
  uint32_t glob_bytes;                                 // per-CTA slice of the global scratch, 0 = big part in shared memory
};

__device__ __forceinline__ void bm_mark(uint32_t *bm, int32_t v) {
  const uint32_t bit = 1u << (v & 31);
  uint32_t *wp = bm + ((uint32_t)v >> 5);
  if (!(*(volatile uint32_t *)wp & bit)) atomicOr(wp, bit);  // hub lists overlap: most bits are set already
}

__device__ __forceinline__ uint32_t bm_rank(const uint32_t *bm, const uint32_t *gpref, int32_t v) {
  const uint32_t word = (uint32_t)v >> 5, grp = word / BM_GROUP_WORDS;
  uint32_t r = gpref[grp];
  for (uint32_t k = grp * BM_GROUP_WORDS; k < word; k++) r += __popc(bm[k]);
  return r + __popc(bm[word] & ((1u << (v & 31)) - 1u));
}

// Streams one neighbour list with STRIDE cooperating threads: sets the neighbours' bits and, for
// LADIES, adds the weights to the caller's partial row sum.  The body of the list is read as
// 16-byte vectors (the arrays are 256-byte aligned, so entry rs + head is 16-byte aligned for
// head = (4 - rs % 4) % 4), BM_VEC vectors in flight per thread; head and tail entries one by one.
constexpr int BM_UNROLL = 8;   // scalar loads in flight per thread (second LADIES pass)
constexpr int BM_VEC = 4;      // 16-byte loads in flight per thread
template <bool LADIES, int STRIDE>
__device__ __forceinline__ void bm_stream(const NdGraphView &g, uint32_t *bm, int32_t rs, int32_t deg, int me, double &part) {
  const int32_t *__restrict__ col = g.col + rs;
  const float *__restrict__ wts = g.w + rs;
  int head = (4 - (rs & 3)) & 3;
  if (head > deg) head = deg;
  if (me < head) {
    bm_mark(bm, __ldg(col + me));
    if (LADIES) part += (double)__ldg(wts + me);
  }
  const int n4 = (deg - head) >> 2;
  const int4 *__restrict__ col4 = reinterpret_cast<const int4 *>(col + head);
  const float4 *__restrict__ w4 = reinterpret_cast<const float4 *>(wts + head);
  for (int e0 = me; e0 < n4; e0 += STRIDE * BM_VEC) {
    int4 v[BM_VEC];
    float4 w[BM_VEC];
#pragma unroll
    for (int k = 0; k < BM_VEC; k++) {
      const int e = e0 + k * STRIDE;
      v[k] = e < n4 ? __ldg(col4 + e) : make_int4(-1, -1, -1, -1);
      if (LADIES) w[k] = e < n4 ? __ldg(w4 + e) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int k = 0; k < BM_VEC; k++) {
      if (v[k].x >= 0) { bm_mark(bm, v[k].x); bm_mark(bm, v[k].y); bm_mark(bm, v[k].z); bm_mark(bm, v[k].w); }
      if (LADIES) part += ((double)w[k].x + (double)w[k].y) + ((double)w[k].z + (double)w[k].w);
    }
  }
  for (int e = head + (n4 << 2) + me; e < deg; e += STRIDE) {
    bm_mark(bm, __ldg(col + e));
    if (LADIES) part += (double)__ldg(wts + e);
  }
}

// LADIES second pass over one list: (w / rowsum)^2 of every entry added to its candidate's accumulator
template <int STRIDE>
__device__ __forceinline__ void bm_accumulate(const NdGraphView &g, const uint32_t *bm, const uint32_t *gpref, double *acc,
                                              int32_t rs, int32_t deg, int me, float rowsum) {
  for (int e0 = me; e0 < deg; e0 += STRIDE * BM_UNROLL) {
    int32_t v[BM_UNROLL];
    float w[BM_UNROLL];
#pragma unroll
    for (int k = 0; k < BM_UNROLL; k++) {
      const int e = e0 + k * STRIDE;
      v[k] = e < deg ? __ldg(g.col + rs + e) : -1;
      w[k] = e < deg ? __ldg(g.w + rs + e) : 0.f;
    }
#pragma unroll
    for (int k = 0; k < BM_UNROLL; k++) {
      if (v[k] >= 0) {
        const float r = __fdiv_rn(w[k], rowsum);
        atomicAdd(acc + bm_rank(bm, gpref, v[k]), (double)__fmul_rn(r, r));
      }
    }
  }
}

template <bool LADIES>
__device__ __forceinline__ float bm_weight(const NdGraphView &g, const double *acc, int32_t v, uint32_t rank) {
  if (LADIES) return (float)acc[rank];
  const float d = __int2float_rn(__ldg(g.row_ptr + v + 1) - __ldg(g.row_ptr + v));
  return __fmul_rn(d, d);
}

// exclusive (uint32) or inclusive (double) scan of a shared array by the whole CTA: every thread
// owns a contiguous chunk, the chunk totals are scanned through warp shuffles
__device__ __forceinline__ uint32_t bm_scan_u32(uint32_t *a, int n, uint32_t *red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int per = (n + BM_THREADS - 1) / BM_THREADS;
  const int b = threadIdx.x * per, e = b + per < n ? b + per : n;
  uint32_t sum = 0;
  for (int i = b; i < e; i++) sum += a[i];
  uint32_t inc = sum;
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) red[warp] = inc;
  __syncthreads();
  uint32_t base = inc - sum;
  for (int w = 0; w < warp; w++) base += red[w];
  uint32_t total = 0;
  for (int w = 0; w < BM_THREADS / 32; w++) total += red[w];
  for (int i = b; i < e; i++) { const uint32_t c = a[i]; a[i] = base; base += c; }
  __syncthreads();
  return total;
}

__device__ __forceinline__ void bm_scan_f64(double *a, int n, double *red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int per = (n + BM_THREADS - 1) / BM_THREADS;
  const int b = threadIdx.x * per, e = b + per < n ? b + per : n;
  double sum = 0.0;
  for (int i = b; i < e; i++) sum += a[i];
  double inc = sum;
  for (int o = 1; o < 32; o <<= 1) {
    const double t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) red[warp] = inc;
  __syncthreads();
  double base = inc - sum;
  for (int w = 0; w < warp; w++) base += red[w];
  for (int i = b; i < e; i++) { base += a[i]; a[i] = base; }
  __syncthreads();
}

template <bool LADIES>
__global__ void __launch_bounds__(BM_THREADS, 1)
coll_bitmap_kernel(NdGraphView g, CollParams cp, int steps, int64_t S, BmLayout lay, unsigned char *__restrict__ gscratch,
                   const int32_t *__restrict__ initial, int32_t *out, double *__restrict__ acc_all, int32_t *__restrict__ adj_row,
                   int32_t *__restrict__ adj_col, float *__restrict__ prob, unsigned long long *__restrict__ stats) {
  extern __shared__ __align__(16) unsigned char bm_smem[];
  unsigned char *big = lay.glob_bytes ? gscratch + (size_t)blockIdx.x * lay.glob_bytes : bm_smem;
  uint32_t *bm = reinterpret_cast<uint32_t *>(big);
  double *gcdf = reinterpret_cast<double *>(big + lay.off_gcdf);
  uint32_t *gpref = reinterpret_cast<uint32_t *>(big + lay.off_gpref);
  int32_t *sh_tr = reinterpret_cast<int32_t *>(bm_smem + lay.off_tr);
  int32_t *sh_layer = reinterpret_cast<int32_t *>(bm_smem + lay.off_layer);
  float *sh_rowsum = reinterpret_cast<float *>(bm_smem + lay.off_rowsum);
  double *red = reinterpret_cast<double *>(bm_smem + lay.off_red);   // 32 doubles
  uint32_t *red_u = reinterpret_cast<uint32_t *>(red + 32);           // 32 words
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  double *acc = LADIES ? acc_all + (size_t)blockIdx.x * (size_t)cp.V : nullptr;
  unsigned long long ids_sum = 0, uniq_sum = 0;  // thread 0
  uint32_t valid = 0;
  for (int64_t s = blockIdx.x; s < S; s += gridDim.x) {
    const int32_t *tr = transits_of(cp, initial, out, s);
    for (int i = tid; i < cp.ntr; i += BM_THREADS) sh_tr[i] = tr[i];
    for (int w = tid * 4; w < lay.words; w += BM_THREADS * 4) *reinterpret_cast<uint4 *>(bm + w) = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
    // ---- pass 1: the union as a bitmap (and the LADIES row sums)
    for (int i = warp; i < cp.ntr; i += BM_THREADS / 32) {  // short lists: a warp each
      const int32_t t = sh_tr[i];
      if (t < 0 || t >= cp.V) { if (LADIES && lane == 0) sh_rowsum[i] = 0.f; continue; }
      const int32_t rs = __ldg(g.row_ptr + t), deg = __ldg(g.row_ptr + t + 1) - rs;
      if (deg >= BM_BIG_LIST) continue;
      double part = 0.0;
      bm_stream<LADIES, 32>(g, bm, rs, deg, lane, part);
      if (LADIES) {
        for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        if (lane == 0) sh_rowsum[i] = (float)part;
      }
    }
    for (int i = 0; i < cp.ntr; i++) {  // long lists: the whole CTA
      const int32_t t = sh_tr[i];
      if (t < 0 || t >= cp.V) continue;
      const int32_t rs = __ldg(g.row_ptr + t), deg = __ldg(g.row_ptr + t + 1) - rs;
      if (tid == 0) ids_sum += (unsigned long long)deg;
      if (deg < BM_BIG_LIST) continue;
      double part = 0.0;
      bm_stream<LADIES, BM_THREADS>(g, bm, rs, deg, tid, part);
      if (LADIES) {
        for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        if (lane == 0) red[warp] = part;
        __syncthreads();
        if (tid == 0) {
          double tot = 0.0;
          for (int w = 0; w < BM_THREADS / 32; w++) tot += red[w];
          sh_rowsum[i] = (float)tot;
        }
        __syncthreads();
      }
    }
    __syncthreads();
    // ---- candidates per group, ranks
    for (int gi = tid; gi < lay.groups; gi += BM_THREADS) {
      uint32_t c = 0;
#pragma unroll
      for (int k = 0; k < BM_GROUP_WORDS; k += 4) {
        const uint4 q = *reinterpret_cast<const uint4 *>(bm + gi * BM_GROUP_WORDS + k);
        c += __popc(q.x) + __popc(q.y) + __popc(q.z) + __popc(q.w);
      }
      gpref[gi] = c;
    }
    __syncthreads();
    const uint32_t U = bm_scan_u32(gpref, lay.groups, red_u);
    if (tid == 0) uniq_sum += U;
    // ---- LADIES pass 2: the terms of every list entry, added to the candidate's accumulator
    if (LADIES) {
      for (uint32_t u = tid; u < U; u += BM_THREADS) acc[u] = 0.0;
      __syncthreads();
      for (int i = warp; i < cp.ntr; i += BM_THREADS / 32) {
        const int32_t t = sh_tr[i];
        if (t < 0 || t >= cp.V) continue;
        const int32_t rs = __ldg(g.row_ptr + t), deg = __ldg(g.row_ptr + t + 1) - rs;
        if (deg >= BM_BIG_LIST) continue;
        bm_accumulate<32>(g, bm, gpref, acc, rs, deg, lane, sh_rowsum[i]);
      }
      for (int i = 0; i < cp.ntr; i++) {
        const int32_t t = sh_tr[i];
        if (t < 0 || t >= cp.V) continue;
        const int32_t rs = __ldg(g.row_ptr + t), deg = __ldg(g.row_ptr + t + 1) - rs;
        if (deg < BM_BIG_LIST) continue;
        bm_accumulate<BM_THREADS>(g, bm, gpref, acc, rs, deg, tid, sh_rowsum[i]);
      }
      __syncthreads();
    }
    // ---- weight of every group, in candidate order; inclusive scan over the groups
    for (int gi = tid; gi < lay.groups; gi += BM_THREADS) {
      double sum = 0.0;
      uint32_t r = gpref[gi];
      for (int k = 0; k < BM_GROUP_WORDS; k++) {
        uint32_t bits = bm[gi * BM_GROUP_WORDS + k];
        while (bits) {
          const int b = __ffs(bits) - 1;
          bits &= bits - 1;
          sum += (double)bm_weight<LADIES>(g, acc, (int32_t)(((gi * BM_GROUP_WORDS + k) << 5) + b), r);
          r++;
        }
      }
      gcdf[gi] = sum;
    }
    __syncthreads();
    bm_scan_f64(gcdf, lay.groups, red);
    const double total = gcdf[lay.groups - 1];
    // ---- the layer's draws
    for (int j = tid; j < cp.L; j += BM_THREADS) {
      int32_t pick = cp.V;
      float pr = 0.f;
      if (U > 0 && total > 0.0) {
        Rng rng(cp.seed, (uint32_t)(cp.first_sample + s), (uint32_t)cp.step, (uint32_t)j);
        const double target = (double)rng.uniform() * total;
        int lo = 0, hi = lay.groups - 1;  // first group whose prefix reaches the target
        while (lo < hi) {
          const int mid = lo + (hi - lo) / 2;
          if (gcdf[mid] >= target) hi = mid; else lo = mid + 1;
        }
        double run = lo > 0 ? gcdf[lo - 1] : 0.0;
        uint32_t r = gpref[lo];
        int32_t last_v = cp.V;
        float pw = 0.f;
        bool found = false;
        for (int gi = lo; gi < lay.groups && !found; gi++) {
          for (int k = 0; k < BM_GROUP_WORDS && !found; k++) {
            uint32_t bits = bm[gi * BM_GROUP_WORDS + k];
            while (bits && !found) {
              const int b = __ffs(bits) - 1;
              bits &= bits - 1;
              last_v = (int32_t)(((gi * BM_GROUP_WORDS + k) << 5) + b);
              pw = bm_weight<LADIES>(g, acc, last_v, r);
              run += (double)pw;
              r++;
              found = run >= target;
            }
          }
        }
        pick = last_v;  // not found: rounding left the target above the last prefix, the last candidate takes it
        pr = (float)((double)pw / total);
        valid++;
      }
      sh_layer[j] = pick;
      out[s * cp.fs + (int64_t)cp.step * cp.L + j] = pick;
      prob[s * cp.fs + (int64_t)cp.step * cp.L + j] = pr;
    }
    __syncthreads();
    const int64_t a = (s * steps + cp.step) * (int64_t)cp.stride;
    emit_adjacency(g, cp, sh_tr, sh_layer, adj_row + a, adj_col + a);
    __syncthreads();
  }
  for (int o = 16; o > 0; o >>= 1) valid += __shfl_xor_sync(0xffffffffu, valid, o);
  if (lane == 0 && valid) atomicAdd(&stats[0], (unsigned long long)valid);
  if (tid == 0) {
    if (ids_sum) atomicAdd(&stats[5], ids_sum);
    if (uniq_sum) atomicAdd(&stats[6], uniq_sum);
  }
}

// shared memory the layout may use; ND_COLLECTIVE_BITMAP_GLOBAL=1 puts the big part into global
// scratch whatever the graph's size (the tests use it to cover that path on small graphs)
static int bm_smem_budget(const nd_sampler *s) {
  const char *e = getenv("ND_COLLECTIVE_BITMAP_GLOBAL");
  return e && e[0] == '1' ? 0 : s->dev.smem_optin;
}

static BmLayout bm_layout(int32_t V, int ntr_max, int L, int smem_optin) {
  BmLayout l;
  l.words = (int)((((int64_t)V + 31) / 32 + BM_GROUP_WORDS - 1) / BM_GROUP_WORDS * BM_GROUP_WORDS);
  l.groups = l.words / BM_GROUP_WORDS;
  uint32_t big = 4u * (uint32_t)l.words;       // a multiple of 64
  l.off_gcdf = big; big += 8u * (uint32_t)l.groups;
  l.off_gpref = big; big += 4u * (uint32_t)(l.groups + 1);
  big = (big + 255u) & ~255u;
  const uint32_t small = 8u * 32u + 4u * 32u + 4u * (uint32_t)ntr_max + 4u * (uint32_t)L + 4u * (uint32_t)ntr_max;
  const bool in_smem = (int64_t)big + small <= (int64_t)smem_optin;
  uint32_t off = in_smem ? big : 0u;
  l.off_red = off; off += 8u * 32u + 4u * 32u;
  l.off_tr = off; off += 4u * (uint32_t)ntr_max;
  l.off_layer = off; off += 4u * (uint32_t)L;
  l.off_rowsum = off; off += 4u * (uint32_t)ntr_max;
  l.bytes = off;
  l.glob_bytes = in_smem ? 0u : big;
  return l;
}

// clears the counters; stats[1] (live pairs) is known up front for these apps
__global__ void coll_reset_kernel(unsigned long long *stats, unsigned long long pairs) {
  if (threadIdx.x < 8) stats[threadIdx.x] = threadIdx.x == 1 ? pairs : 0ull;
}

}  // namespace

// candidate buffers: three 32-bit words per element (id, sample, LADIES term), double-buffered for
// the sort, plus weight and CDF
static int ensure_cand(nd_sampler *s, int64_t need) {
  if (need <= s->cand_cap) return ND_OK;
  int64_t cap = std::max<int64_t>(need, (int64_t)1 << 22);
  cudaFree(s->d_cand); cudaFree(s->d_cand_w);
  nd_radix_scratch_free(&s->radix);
  s->d_cand = nullptr; s->d_cand_w = nullptr; s->cand_cap = 0;
  ND_CUDA(cudaMalloc(&s->d_cand, sizeof(uint32_t) * 6 * (size_t)cap));
  ND_CUDA(cudaMalloc(&s->d_cand_w, (sizeof(float) + sizeof(double)) * (size_t)cap));  // cdf (fp64) first, then weights
  ND_TRY(nd_radix_scratch_alloc(&s->radix, 32, cap));
  s->cand_cap = cap;
  return ND_OK;
}

int nd_collective_alloc(nd_sampler *s) {
  const nd_app_params &p = s->p;
  const int L = p.fanout[0], B = p.batch;
  const size_t S1 = (size_t)(s->S > 0 ? s->S : 1);
  const size_t adj = S1 * p.steps * (size_t)(B > L ? B : L) * L;
  ND_CUDA(cudaMalloc(&s->d_adj_row, sizeof(int32_t) * adj));
  ND_CUDA(cudaMalloc(&s->d_adj_col, sizeof(int32_t) * adj));
  ND_CUDA(cudaMalloc(&s->d_prob, sizeof(float) * S1 * s->fs));
  ND_CUDA(cudaMemset(s->d_prob, 0, sizeof(float) * S1 * s->fs));
  ND_CUDA(cudaMalloc(&s->d_len, sizeof(int32_t) * (S1 + 1)));        // per-sample sizes of the layer
  ND_CUDA(cudaMalloc(&s->d_tmp, sizeof(int64_t) * (S1 + 1)));        // per-sample region offsets
  ND_CUDA(cudaMalloc(&s->d_nlive, sizeof(int32_t) * 4));
  if (p.app == ND_APP_FASTGCN_IS || p.app == ND_APP_LADIES_IS) {
    // the union is built as a bitmap with a bit per vertex: in shared memory when it fits the CTA's
    // opt-in shared memory, else in a per-CTA slice of global scratch; ND_COLLECTIVE_SORT=1 selects
    // the sort pipeline instead (kept for the tests, which compare the two)
    const BmLayout lay = bm_layout(s->g->V, B > L ? B : L, L, bm_smem_budget(s));
    const char *force = getenv("ND_COLLECTIVE_SORT");
    const bool ladies = p.app == ND_APP_LADIES_IS;
    if (B <= 1024 && L <= 1024 && !(force && force[0] == '1')) {
      s->coll_bitmap = true;
      s->coll_grid = (int)std::min<int64_t>(S1, (int64_t)s->dev.sms);
      if (lay.glob_bytes) ND_CUDA(cudaMalloc(&s->d_bm, (size_t)lay.glob_bytes * (size_t)s->coll_grid));
      if (ladies) {
        ND_CUDA(cudaFuncSetAttribute(coll_bitmap_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)lay.bytes));
        ND_CUDA(cudaMalloc(&s->d_acc, sizeof(double) * (size_t)s->coll_grid * (size_t)s->g->V));
      } else {
        ND_CUDA(cudaFuncSetAttribute(coll_bitmap_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)lay.bytes));
      }
    } else {
      ND_TRY(ensure_cand(s, (int64_t)1 << 22));
    }
  }
  return ND_OK;
}

const char *nd_collective_kernel_name(const nd_sampler *s) {
  if (!s->coll_bitmap) return "coll_sizes/gather/weigh/sample kernels + radix sort";
  return s->d_bm ? "coll_bitmap_kernel (bitmap in global scratch)" : "coll_bitmap_kernel (bitmap in shared memory)";
}

int nd_collective_sample(nd_sampler *s, int mode) {
  (void)mode;  // the reference runs next() of collective apps through sampleParallelKernel in every mode (src/nextdoor.cu:2900-2916)
  const nd_app_params &p = s->p;
  const int64_t S = s->S;
  cudaStream_t st = s->stream;
  NdGraphView gv = nd_view(s->g);
  CollParams cp;
  cp.seed = p.seed; cp.first_sample = s->first; cp.V = s->g->V; cp.fs = s->fs; cp.L = p.fanout[0]; cp.B = p.batch;
  cp.stride = (cp.B > cp.L ? cp.B : cp.L) * cp.L; cp.step = 0; cp.ntr = cp.B; cp.app = p.app;
  const bool ref_app = p.app == ND_APP_FASTGCN_REF || p.app == ND_APP_LADIES_REF;
  const unsigned long long pairs = (unsigned long long)(S * (cp.B + (int64_t)(p.steps - 1) * cp.L));
  coll_reset_kernel<<<1, 32, 0, st>>>(s->d_stats, s->coll_bitmap && !ref_app ? pairs : 0ull);
  nd_count_launches(1);
  const int grid = (int)std::min<int64_t>(S, (int64_t)s->dev.sms * 8);
  if (ref_app) {
    nd_phase_begin(s, ND_PHASE_NEXT);
    coll_ref_kernel<<<grid, CTHREADS, 0, st>>>(gv, cp, p.steps, S, s->d_initial, s->d_out, s->d_adj_row, s->d_adj_col, s->d_stats);
    nd_phase_end(s);
    nd_count_launches(1);
    ND_CUDA(cudaGetLastError());
    return ND_OK;
  }
  if (s->coll_bitmap) {  // one launch per layer, nothing comes back to the host: asynchronous like the walk and k-hop jobs
    const BmLayout lay = bm_layout(cp.V, cp.B > cp.L ? cp.B : cp.L, cp.L, bm_smem_budget(s));
    for (int step = 0; step < p.steps; step++) {
      cp.step = step;
      cp.ntr = step == 0 ? cp.B : cp.L;
      nd_phase_begin(s, ND_PHASE_NEXT);
      if (p.app == ND_APP_LADIES_IS)
        coll_bitmap_kernel<true><<<s->coll_grid, BM_THREADS, lay.bytes, st>>>(gv, cp, p.steps, S, lay, s->d_bm, s->d_initial, s->d_out, s->d_acc,
                                                                             s->d_adj_row, s->d_adj_col, s->d_prob, s->d_stats);
      else
        coll_bitmap_kernel<false><<<s->coll_grid, BM_THREADS, lay.bytes, st>>>(gv, cp, p.steps, S, lay, s->d_bm, s->d_initial, s->d_out, nullptr,
                                                                              s->d_adj_row, s->d_adj_col, s->d_prob, s->d_stats);
      nd_phase_end(s);
      nd_count_launches(1);
    }
    ND_CUDA(cudaGetLastError());
    return ND_OK;
  }
  std::vector<int32_t> sizes((size_t)S);
  std::vector<int64_t> offs((size_t)S + 1);
  int64_t union_ids = 0;
  int64_t *d_offs = (int64_t *)s->d_tmp;
  for (int step = 0; step < p.steps; step++) {
    cp.step = step;
    cp.ntr = step == 0 ? cp.B : cp.L;
    nd_phase_begin(s, ND_PHASE_COLLECT);
    coll_sizes_kernel<<<(int)((S * 32 + CTHREADS - 1) / CTHREADS), CTHREADS, 0, st>>>(gv, cp, S, s->d_initial, s->d_out, s->d_len);
    nd_count_launches(1);
    ND_CUDA(cudaMemcpyAsync(sizes.data(), s->d_len, sizeof(int32_t) * (size_t)S, cudaMemcpyDeviceToHost, st));
    ND_CUDA(cudaStreamSynchronize(st));
    offs[0] = 0;
    int64_t biggest = 0;
    for (int64_t i = 0; i < S; i++) { offs[i + 1] = offs[i] + sizes[i]; biggest = std::max<int64_t>(biggest, sizes[i]); }
    union_ids += offs[S];
    ND_REQUIRE(biggest < ((int64_t)1 << 30), ND_ERR_RANGE, "a collective neighbourhood of %lld ids does not fit", (long long)biggest);
    ND_TRY(ensure_cand(s, biggest));
    ND_CUDA(cudaMemcpyAsync(d_offs, offs.data(), sizeof(int64_t) * ((size_t)S + 1), cudaMemcpyHostToDevice, st));
    nd_phase_end(s);
    const int64_t cap = s->cand_cap;
    uint32_t *c_a[3] = {(uint32_t *)s->d_cand, (uint32_t *)s->d_cand + cap, (uint32_t *)s->d_cand + 2 * cap};
    uint32_t *c_b[3] = {(uint32_t *)s->d_cand + 3 * cap, (uint32_t *)s->d_cand + 4 * cap, (uint32_t *)s->d_cand + 5 * cap};
    double *cdf = (double *)s->d_cand_w;
    float *wt = (float *)(cdf + cap);
    int64_t s0 = 0;
    while (s0 < S) {  // chunk of samples whose neighbourhoods fit the buffers together
      int64_t s1 = s0 + 1;
      while (s1 < S && offs[s1 + 1] - offs[s0] <= cap) s1++;
      const int64_t n = offs[s1] - offs[s0];
      const int cgrid = (int)std::min<int64_t>(s1 - s0, (int64_t)s->dev.sms * 8);
      if (n > 0) {
        nd_phase_begin(s, ND_PHASE_COLLECT);
        const int32_t n32 = (int32_t)n;
        ND_CUDA(cudaMemcpyAsync(s->d_nlive, &n32, sizeof(int32_t), cudaMemcpyHostToDevice, st));
        coll_gather_kernel<<<cgrid, CTHREADS, 0, st>>>(gv, cp, s0, s1, s->d_initial, s->d_out, d_offs, c_a[0], c_a[1], c_a[2]);
        nd_count_launches(1);
        uint32_t *cur[3] = {c_a[0], c_a[1], c_a[2]}, *oth[3] = {c_b[0], c_b[1], c_b[2]};
        const int key_word[2] = {0, 1};
        const int key_bits[2] = {nd_bit_length((uint32_t)(cp.V > 1 ? cp.V - 1 : 1)), nd_bit_length((uint32_t)(s1 - s0 > 1 ? s1 - s0 - 1 : 1))};
        for (int k = 0; k < 2; k++) {
          NdSortArrays arr;
          arr.nwords = 3;
          for (int w = 0; w < 3; w++) { arr.a[w] = cur[w]; arr.b[w] = oth[w]; }
          NdRadixPlan pl = nd_radix_plan(key_bits[k], cap);
          bool in_b = false;
          ND_TRY(nd_radix_sort(s->dev, st, &s->radix, pl, arr, key_word[k], s->d_nlive, nullptr, false, 0u, false, &in_b));
          if (in_b) for (int w = 0; w < 3; w++) std::swap(cur[w], oth[w]);
        }
        const int wgrid = (int)std::min<int64_t>((n + CTHREADS - 1) / CTHREADS, (int64_t)s->dev.sms * 16);
        coll_weigh_kernel<<<wgrid, CTHREADS, 0, st>>>(gv, p.app, n, cur[0], cur[1], cur[2], wt, s->d_stats);
        nd_count_launches(1);
        nd_phase_end(s);
        nd_phase_begin(s, ND_PHASE_NEXT);
        coll_sample_kernel<<<cgrid, CTHREADS, 0, st>>>(gv, cp, p.steps, s0, s1, s->d_initial, s->d_out, d_offs, cur[0], wt, cdf,
                                                     s->d_adj_row, s->d_adj_col, s->d_prob, s->d_stats);
        nd_count_launches(1);
        nd_phase_end(s);
        // the next chunk reuses the buffers and the host copy of its size
        ND_CUDA(cudaStreamSynchronize(st));
      } else {
        coll_sample_kernel<<<cgrid, CTHREADS, 0, st>>>(gv, cp, p.steps, s0, s1, s->d_initial, s->d_out, d_offs, c_a[0], wt, cdf,
                                                     s->d_adj_row, s->d_adj_col, s->d_prob, s->d_stats);
        nd_count_launches(1);
      }
      s0 = s1;
    }
  }
  const unsigned long long h[2] = {(unsigned long long)(S * (cp.B + (int64_t)(p.steps - 1) * cp.L)), (unsigned long long)union_ids};
  ND_CUDA(cudaMemcpyAsync(s->d_stats + 1, &h[0], sizeof(unsigned long long), cudaMemcpyHostToDevice, st));
  ND_CUDA(cudaMemcpyAsync(s->d_stats + 5, &h[1], sizeof(unsigned long long), cudaMemcpyHostToDevice, st));
  ND_CUDA(cudaStreamSynchronize(st));
  ND_CUDA(cudaGetLastError());
  return ND_OK;
}
