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
  for (int e = threadIdx.x; e < cp.stride; e += CTHREADS) {
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

__global__ void coll_reset_kernel(unsigned long long *stats) { if (threadIdx.x < 8) stats[threadIdx.x] = 0ull; }

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
  if (p.app == ND_APP_FASTGCN_IS || p.app == ND_APP_LADIES_IS) ND_TRY(ensure_cand(s, (int64_t)1 << 22));
  return ND_OK;
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
  coll_reset_kernel<<<1, 32, 0, st>>>(s->d_stats);
  nd_count_launches(1);
  const int grid = (int)std::min<int64_t>(S, (int64_t)s->dev.sms * 8);
  if (p.app == ND_APP_FASTGCN_REF || p.app == ND_APP_LADIES_REF) {
    nd_phase_begin(s, ND_PHASE_NEXT);
    coll_ref_kernel<<<grid, CTHREADS, 0, st>>>(gv, cp, p.steps, S, s->d_initial, s->d_out, s->d_adj_row, s->d_adj_col, s->d_stats);
    nd_phase_end(s);
    nd_count_launches(1);
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
