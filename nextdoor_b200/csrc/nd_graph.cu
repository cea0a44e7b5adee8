// Graph side of the path on the device: CSR construction from edge records, the synthetic R-MAT
// generator, per-vertex max weight, and the byte-budget range partitioner.
//
// Replaces Graph::load_from_edge_list_binary + csr_from_graph (src/graph.hpp:106-159,
// src/csr.hpp:399-424: per-vertex std::vector, OpenMP std::sort, serial fill), transferCSRToGPUs
// (src/nextdoor.cu:1893-1911) and create_csr_partitions (src/graph_partitioner.cuh:1-173).
// The records are sorted by (src, dst, weight) with three stable LSD sorts of the in-house radix
// sort (weight bits, then dst, then src), row offsets come from the boundaries of the sorted src
// array, and the sorted dst / weight arrays become col / w in place.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <string>
#include <vector>

#include "nd_common.cuh"
#include "nd_philox.cuh"

namespace {

// order-preserving map of fp32 onto uint32 (negative weights sort below positive ones)
__device__ __forceinline__ uint32_t float_to_key(float f) {
  const uint32_t b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

struct Rec12 { int32_t s, d; float w; };

__global__ void unpack_records_kernel(const Rec12 *__restrict__ rec, int64_t n, uint32_t *__restrict__ src,
                                      uint32_t *__restrict__ dst, uint32_t *__restrict__ wk,
                                      int32_t *__restrict__ max_id, int *__restrict__ status) {
  int32_t m = -1;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const Rec12 r = rec[i];
    if (r.s < 0 || r.d < 0) atomicOr(status, ND_DEV_BAD_TRANSIT);
    src[i] = (uint32_t)r.s; dst[i] = (uint32_t)r.d; wk[i] = float_to_key(r.w);
    m = max(m, max(r.s, r.d));
  }
  for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0 && m >= 0) atomicMax(max_id, m);
}

// R-MAT (a,b,c,d) = (.57,.19,.19,.05).  Undirected edge e, attempt t: Philox counter
// (e_lo, e_hi, t, level/4), key = seed ^ "RMAT"; level l consumes draw l with integer quadrant
// thresholds; an attempt with an endpoint >= V or src == dst is retried; the weight is draw
// `scale` of the accepted attempt, 1 + 4 * (x>>8) * 2^-24.  Both directions are emitted.
__global__ void rmat_kernel(int32_t V, int scale, int64_t M, uint64_t seed, uint32_t *__restrict__ src,
                            uint32_t *__restrict__ dst, uint32_t *__restrict__ wk) {
  const uint32_t T1 = 2448131358u, T2 = 3264175144u, T3 = 4080218931u;
  const uint32_t k0 = (uint32_t)seed ^ 0x524D4154u, k1 = (uint32_t)(seed >> 32);
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < M; e += (int64_t)gridDim.x * blockDim.x) {
    int32_t s = 0, d = 0;
    float w = 0.f;
    for (uint32_t attempt = 0; attempt < (1u << 20); attempt++) {
      uint32_t o[4];
      s = 0; d = 0;
      bool ok = false;
      for (int l = 0; l <= scale; l++) {
        if ((l & 3) == 0) ndrng::philox4x32_10((uint32_t)e, (uint32_t)((uint64_t)e >> 32), attempt, (uint32_t)(l >> 2), k0, k1, o);
        const uint32_t x = (l & 3) == 0 ? o[0] : ((l & 3) == 1 ? o[1] : ((l & 3) == 2 ? o[2] : o[3]));
        if (l == scale) {
          if (s < V && d < V && s != d) {
            ok = true;
            w = __fadd_rn(1.0f, __fmul_rn(4.0f, __fmul_rn(__uint2float_rn(x >> 8), 5.9604644775390625e-08f)));
          }
          break;
        }
        int sb, db;
        if (x < T1) { sb = 0; db = 0; }
        else if (x < T2) { sb = 0; db = 1; }
        else if (x < T3) { sb = 1; db = 0; }
        else { sb = 1; db = 1; }
        s = (s << 1) | sb;
        d = (d << 1) | db;
      }
      if (ok) break;
    }
    const uint32_t key = float_to_key(w);
    src[2 * e] = s; dst[2 * e] = d; wk[2 * e] = key;
    src[2 * e + 1] = d; dst[2 * e + 1] = s; wk[2 * e + 1] = key;
  }
}

// row_ptr from the sorted src array: element i closes the rows (src[i-1], src[i]]
__global__ void row_ptr_kernel(const uint32_t *__restrict__ src, int64_t n, int32_t V, int32_t *__restrict__ row_ptr) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i <= n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t lo = i == 0 ? 0 : (int64_t)src[i - 1] + 1;
    const int64_t hi = i == n ? V : (int64_t)src[i];
    for (int64_t v = lo; v <= hi; v++) row_ptr[v] = (int32_t)i;
  }
}

__global__ void weights_back_kernel(uint32_t *__restrict__ wk, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    wk[i] = __float_as_uint(key_to_float(wk[i]));
}

// Vertex::max_weight (src/graph.hpp:71-80) starts from 0, so only positive weights can raise it
// and their bit patterns order like ints.  Thread per edge; the owner row comes from the sorted
// src array when the CSR was just built here, else from a bisection of row_ptr; a warp whose 32
// edges share one row reduces first and issues a single atomic.
__global__ void max_weight_kernel(const int32_t *__restrict__ row_ptr, const uint32_t *__restrict__ src,
                                  const float *__restrict__ w, int32_t V, int64_t E,
                                  int32_t *__restrict__ max_w_bits) {
  for (int64_t base = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) & ~31ll; base < E;
       base += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = base + (threadIdx.x & 31);
    const bool in = i < E;
    const float x = in ? w[i] : 0.f;
    int32_t v = -1;
    if (in) {
      if (src) {
        v = (int32_t)src[i];
      } else {  // largest v with row_ptr[v] <= i
        int32_t lo = 0, hi = V;
        while (hi - lo > 1) {
          const int32_t mid = lo + (hi - lo) / 2;
          if ((int64_t)row_ptr[mid] <= i) lo = mid; else hi = mid;
        }
        v = lo;
      }
    }
    const uint32_t peers = __match_any_sync(0xffffffffu, v);
    float m = x;
    if (peers == 0xffffffffu) {
      for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      if ((threadIdx.x & 31) == 0 && in && m > 0.f) atomicMax(max_w_bits + v, __float_as_int(m));
    } else if (in && m > 0.f) {
      atomicMax(max_w_bits + v, __float_as_int(m));
    }
  }
}

__global__ void max_degree_kernel(const int32_t *__restrict__ row_ptr, int32_t V, int32_t *__restrict__ out) {
  int32_t m = 0;
  for (int64_t v = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; v < V; v += (int64_t)gridDim.x * blockDim.x)
    m = max(m, row_ptr[v + 1] - row_ptr[v]);
  for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) atomicMax(out, m);
}

// Greedy byte-budget partitioner.  Partition k starts at (u, e_start); with
// G(v) = 4*(row_ptr[v+1] - max(e_start,row_ptr[u])) + 16*(v-u+1) (strictly increasing in v) it is
// closed at the first v with G(v) >= budget, found by bisection.  One thread: the work is
// n_parts * log2(V) dependent loads.
__global__ void partition_kernel(const int32_t *__restrict__ row_ptr, int32_t V, long long budget, int max_parts,
                                 int32_t *__restrict__ first_v, int32_t *__restrict__ last_v,
                                 long long *__restrict__ first_e, long long *__restrict__ last_e,
                                 int32_t *__restrict__ n_parts) {
  if (blockIdx.x != 0 || threadIdx.x != 0) return;
  int np = 0;
  int32_t u = 0;
  long long e_start = 0;
  const long long E = row_ptr[V];
  while (u < V && np < max_parts) {
    const long long es = e_start > row_ptr[u] ? e_start : (long long)row_ptr[u];
    // first v in [u, V) with G(v) >= budget
    int32_t lo = u, hi = V;  // answer in [lo, hi]; hi == V means none
    while (lo < hi) {
      const int32_t mid = lo + (hi - lo) / 2;
      const long long G = 4 * ((long long)row_ptr[mid + 1] - es) + 16 * (long long)(mid - u + 1);
      if (G >= budget) hi = mid; else lo = mid + 1;
    }
    int32_t u_end;
    long long e_end;
    bool closed = lo < V;
    if (!closed) {
      u_end = V - 1; e_end = E - 1;
    } else {
      const int32_t v = lo;
      const long long s = v == u ? es : (long long)row_ptr[v];
      const long long edges = (long long)row_ptr[v + 1] - s;
      const long long n_edges = s - es;
      const long long nv = v - u + 1;
      long long room = (budget - nv * 16) / 4 - n_edges;
      if (room < 0) room = 0;
      if (room >= edges) { u_end = v; e_end = s + edges - 1; }
      else if (v > u) { u_end = v - 1; e_end = s - 1; }
      else { if (room == 0) room = 1; u_end = v; e_end = s + room - 1; }
    }
    first_v[np] = u; last_v[np] = u_end; first_e[np] = e_start; last_e[np] = e_end;
    np++;
    if (!closed) break;
    e_start = e_end + 1;
    u = e_start >= row_ptr[u_end + 1] ? u_end + 1 : u_end;
  }
  *n_parts = np;
}

int grid_for(int64_t n, int threads, int sms) {
  int64_t b = (n + threads - 1) / threads;
  const int64_t cap = (int64_t)sms * 16;
  if (b > cap) b = cap;
  return (int)(b > 0 ? b : 1);
}

// sorted SoA records (device, already (src,dst,wkey) in a[]) -> graph
int build_from_soa(int device, int64_t n, int32_t V, uint32_t *a[3], uint32_t *b[3], cudaStream_t st, nd_graph **out) {
  NdDeviceInfo dev;
  ND_TRY(nd_device_info(device, &dev));
  ND_REQUIRE(n < ((int64_t)1 << 31), ND_ERR_RANGE, "%lld edges do not fit the int32 edge index of the CSR", (long long)n);
  NdRadixScratch scr;
  ND_TRY(nd_radix_scratch_alloc(&scr, 32, n));
  int32_t *d_n = nullptr;
  ND_CUDA(cudaMalloc(&d_n, sizeof(int32_t)));
  const int32_t n32 = (int32_t)n;
  ND_CUDA(cudaMemcpyAsync(d_n, &n32, sizeof(int32_t), cudaMemcpyHostToDevice, st));
  const int vbits = nd_bit_length((uint32_t)(V > 1 ? V - 1 : 1));
  const int key_word[3] = {2, 1, 0};
  const int key_bits[3] = {32, vbits, vbits};
  uint32_t *cur[3] = {a[0], a[1], a[2]}, *oth[3] = {b[0], b[1], b[2]};
  for (int k = 0; k < 3; k++) {
    NdSortArrays arr;
    arr.nwords = 3;
    for (int w = 0; w < 3; w++) { arr.a[w] = cur[w]; arr.b[w] = oth[w]; }
    bool in_b = false;
    const NdRadixPlan pl = nd_radix_plan(key_bits[k], n);
    ND_TRY(nd_radix_sort(dev, st, &scr, pl, arr, key_word[k], d_n, nullptr, false, 0u, false, &in_b));
    if (in_b) for (int w = 0; w < 3; w++) { uint32_t *t = cur[w]; cur[w] = oth[w]; oth[w] = t; }
  }
  nd_graph *g = new nd_graph();
  g->device = device; g->V = V; g->E = n;
  ND_CUDA(cudaMalloc(&g->row_ptr, sizeof(int32_t) * ((size_t)V + 1)));
  row_ptr_kernel<<<grid_for(n + 1, 256, dev.sms), 256, 0, st>>>(cur[0], n, V, g->row_ptr);
  weights_back_kernel<<<grid_for(n, 256, dev.sms), 256, 0, st>>>(cur[2], n);
  ND_CUDA(cudaMalloc(&g->max_w, sizeof(float) * (size_t)V));
  ND_CUDA(cudaMemsetAsync(g->max_w, 0, sizeof(float) * (size_t)V, st));
  if (n > 0)
    max_weight_kernel<<<grid_for(n, 256, dev.sms), 256, 0, st>>>(g->row_ptr, cur[0], (const float *)cur[2], V, n, (int32_t *)g->max_w);
  ND_CUDA(cudaGetLastError());
  ND_CUDA(cudaStreamSynchronize(st));
  // keep the buffers that hold the sorted dst / weights as col / w (they carry 32 bytes of
  // padding for the 16-byte staging windows); release the rest
  g->col = (int32_t *)cur[1];
  g->w = (float *)cur[2];
  ND_CUDA(cudaMemset(g->col + n, 0, sizeof(int32_t) * 8));
  ND_CUDA(cudaMemset(g->w + n, 0, sizeof(float) * 8));
  cudaFree(cur[0]);
  for (int w = 0; w < 3; w++) cudaFree(oth[w]);
  nd_radix_scratch_free(&scr);
  cudaFree(d_n);
  ND_TRY(nd_graph_finish(g, st));
  *out = g;
  return ND_OK;
}

}  // namespace

int nd_graph_finish(nd_graph *g, cudaStream_t st) {
  NdDeviceInfo dev;
  ND_TRY(nd_device_info(g->device, &dev));
  if (!g->max_w) {
    ND_CUDA(cudaMalloc(&g->max_w, sizeof(float) * (size_t)(g->V > 0 ? g->V : 1)));
    ND_CUDA(cudaMemsetAsync(g->max_w, 0, sizeof(float) * (size_t)g->V, st));
    if (g->E > 0)
      max_weight_kernel<<<grid_for(g->E, 256, dev.sms), 256, 0, st>>>(g->row_ptr, nullptr, g->w, g->V, g->E, (int32_t *)g->max_w);
  }
  int32_t *d_m = nullptr;
  ND_CUDA(cudaMalloc(&d_m, sizeof(int32_t)));
  ND_CUDA(cudaMemsetAsync(d_m, 0, sizeof(int32_t), st));
  max_degree_kernel<<<grid_for(g->V, 256, dev.sms), 256, 0, st>>>(g->row_ptr, g->V, d_m);
  ND_CUDA(cudaMemcpyAsync(&g->max_degree, d_m, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
  ND_CUDA(cudaStreamSynchronize(st));
  cudaFree(d_m);
  return ND_OK;
}

extern "C" {

int nd_graph_from_csr(int device, int32_t V, int64_t E, const int32_t *row_ptr, const int32_t *col,
                      const float *w, const float *max_w, nd_graph **out) {
  ND_REQUIRE(out && row_ptr && (E == 0 || (col && w)) && V >= 1 && E >= 0, ND_ERR_ARG, "nd_graph_from_csr: bad argument");
  ND_REQUIRE(E < ((int64_t)1 << 31), ND_ERR_RANGE, "%lld edges do not fit the int32 edge index of the CSR", (long long)E);
  ND_REQUIRE(row_ptr[0] == 0 && row_ptr[V] == E, ND_ERR_ARG, "row_ptr must run from 0 to E");
  ND_CUDA(cudaSetDevice(device));
  nd_graph *g = new nd_graph();
  g->device = device; g->V = V; g->E = E;
  ND_CUDA(cudaMalloc(&g->row_ptr, sizeof(int32_t) * ((size_t)V + 1)));
  // 32 bytes of padding: staging copies read whole 16-byte windows around a list
  ND_CUDA(cudaMalloc(&g->col, sizeof(int32_t) * ((size_t)E + 8)));
  ND_CUDA(cudaMalloc(&g->w, sizeof(float) * ((size_t)E + 8)));
  ND_CUDA(cudaMemset(g->col + E, 0, sizeof(int32_t) * 8));
  ND_CUDA(cudaMemset(g->w + E, 0, sizeof(float) * 8));
  ND_CUDA(cudaMemcpy(g->row_ptr, row_ptr, sizeof(int32_t) * ((size_t)V + 1), cudaMemcpyHostToDevice));
  if (E > 0) {
    ND_CUDA(cudaMemcpy(g->col, col, sizeof(int32_t) * (size_t)E, cudaMemcpyHostToDevice));
    ND_CUDA(cudaMemcpy(g->w, w, sizeof(float) * (size_t)E, cudaMemcpyHostToDevice));
  }
  if (max_w) {
    ND_CUDA(cudaMalloc(&g->max_w, sizeof(float) * (size_t)V));
    ND_CUDA(cudaMemcpy(g->max_w, max_w, sizeof(float) * (size_t)V, cudaMemcpyHostToDevice));
  }
  ND_TRY(nd_graph_finish(g, nullptr));
  *out = g;
  return ND_OK;
}

static int from_edge_records_min_v(int device, int64_t n, const void *records, int32_t min_v, nd_graph **out);

int nd_graph_from_edge_records(int device, int64_t n, const void *records, nd_graph **out) {
  return from_edge_records_min_v(device, n, records, 0, out);
}

// min_v: lower bound of the vertex count (the adjacency-list format numbers vertices by line,
// including lines without edges)
static int from_edge_records_min_v(int device, int64_t n, const void *records, int32_t min_v, nd_graph **out) {
  ND_REQUIRE(out && (records || n == 0) && n >= 0, ND_ERR_ARG, "nd_graph_from_edge_records: bad argument");
  ND_REQUIRE(n < ((int64_t)1 << 31), ND_ERR_RANGE, "%lld edges do not fit the int32 edge index of the CSR", (long long)n);
  ND_CUDA(cudaSetDevice(device));
  NdDeviceInfo dev;
  ND_TRY(nd_device_info(device, &dev));
  const size_t cap = (size_t)(n > 0 ? n : 1);
  Rec12 *d_rec = nullptr;
  uint32_t *a[3], *b[3];
  ND_CUDA(cudaMalloc(&d_rec, sizeof(Rec12) * cap));
  for (int w = 0; w < 3; w++) { ND_CUDA(cudaMalloc(&a[w], 4 * (cap + 8))); ND_CUDA(cudaMalloc(&b[w], 4 * (cap + 8))); }
  int32_t *d_max = nullptr;
  int *d_status = nullptr;
  ND_CUDA(cudaMalloc(&d_max, sizeof(int32_t)));
  ND_CUDA(cudaMalloc(&d_status, sizeof(int)));
  ND_CUDA(cudaMemset(d_max, 0xff, sizeof(int32_t)));
  ND_CUDA(cudaMemset(d_status, 0, sizeof(int)));
  ND_CUDA(cudaMemcpy(d_rec, records, sizeof(Rec12) * (size_t)n, cudaMemcpyHostToDevice));
  unpack_records_kernel<<<grid_for(n, 256, dev.sms), 256>>>(d_rec, n, a[0], a[1], a[2], d_max, d_status);
  int32_t max_id = -1;
  int status = 0;
  ND_CUDA(cudaMemcpy(&max_id, d_max, sizeof(int32_t), cudaMemcpyDeviceToHost));
  ND_CUDA(cudaMemcpy(&status, d_status, sizeof(int), cudaMemcpyDeviceToHost));
  cudaFree(d_rec); cudaFree(d_max); cudaFree(d_status);
  if (status != 0 || max_id == 0x7fffffff) {
    for (int w = 0; w < 3; w++) { cudaFree(a[w]); cudaFree(b[w]); }
    nd_set_error("edge records hold a negative or out-of-range vertex id");
    return ND_ERR_RANGE;
  }
  int32_t V = max_id + 1 > 0 ? max_id + 1 : 1;  // vertex count = max id + 1 (src/graph.hpp:131-142)
  if (V < min_v) V = min_v;
  return build_from_soa(device, n, V, a, b, nullptr, out);
}

int nd_graph_load_edge_list_binary(int device, const char *path, nd_graph **out) {
  ND_REQUIRE(path && out, ND_ERR_ARG, "nd_graph_load_edge_list_binary: bad argument");
  FILE *fp = fopen(path, "rb");
  if (!fp) { nd_set_error("File '%s' not found", path); return ND_ERR_IO; }
  fseek(fp, 0, SEEK_END);
  const long fsize = ftell(fp);
  fseek(fp, 0, SEEK_SET);
  const int64_t n = fsize / 12;
  std::vector<char> buf((size_t)(n * 12 > 0 ? n * 12 : 1));
  const size_t got = fread(buf.data(), 1, (size_t)(n * 12), fp);
  fclose(fp);
  if (got != (size_t)(n * 12)) { nd_set_error("short read on '%s'", path); return ND_ERR_IO; }
  return nd_graph_from_edge_records(device, n, buf.data(), out);
}

// Text edge list (Graph::load_from_edge_list_txt, src/graph.hpp:162-254): whitespace-separated
// "src dst weight" triples, reading stops at the first zero (or missing) weight, and -- as the
// reference does (:210) -- every edge is stored with weight 0: this format carries topology only.
static int load_edge_list_text(int device, const char *path, nd_graph **out) {
  FILE *fp = fopen(path, "r");
  if (!fp) { nd_set_error("File '%s' not found", path); return ND_ERR_IO; }
  std::vector<Rec12> recs;
  long long a = 0, b = 0;
  double w = 0;
  while (fscanf(fp, "%lld %lld %lf", &a, &b, &w) == 3) {
    if (w == 0.0) break;
    if (a < 0 || b < 0 || a > 0x7ffffffe || b > 0x7ffffffe) { fclose(fp); nd_set_error("vertex id out of range in '%s'", path); return ND_ERR_RANGE; }
    recs.push_back(Rec12{(int32_t)a, (int32_t)b, 0.0f});
  }
  fclose(fp);
  return from_edge_records_min_v(device, (int64_t)recs.size(), recs.data(), 0, out);
}

// Text adjacency list (Graph::load_from_adjacency_list, src/graph.hpp:256-326): one vertex per
// line, "id nbr weight nbr weight ..."; vertices are renumbered by line order and neighbour ids
// are translated through that numbering (an id that never heads a line maps to 0, as the
// reference's unordered_map lookup does).
static int load_adjacency_list_text(int device, const char *path, nd_graph **out) {
  FILE *fp = fopen(path, "r");
  if (!fp) { nd_set_error("File '%s' cannot open", path); return ND_ERR_IO; }
  std::vector<Rec12> recs;
  std::vector<long long> ids;
  std::string line;
  std::vector<char> buf(1 << 20);
  while (fgets(buf.data(), (int)buf.size(), fp)) {
    line.assign(buf.data());
    while (!line.empty() && line.back() != '\n' && fgets(buf.data(), (int)buf.size(), fp)) line += buf.data();
    const char *p = line.c_str();
    char *end = nullptr;
    const long long id = strtoll(p, &end, 10);
    if (end == p) continue;  // blank line
    const int32_t row = (int32_t)ids.size();
    ids.push_back(id);
    p = end;
    for (;;) {
      const long long nb = strtoll(p, &end, 10);
      if (end == p) break;
      p = end;
      const float wt = strtof(p, &end);
      if (end == p) break;
      p = end;
      recs.push_back(Rec12{row, (int32_t)nb, wt});  // dst still holds the file's id
    }
  }
  fclose(fp);
  std::vector<std::pair<long long, int32_t>> order(ids.size());
  for (size_t i = 0; i < ids.size(); i++) order[i] = {ids[i], (int32_t)i};
  std::sort(order.begin(), order.end());
  for (Rec12 &r : recs) {
    auto it = std::lower_bound(order.begin(), order.end(), std::make_pair((long long)r.d, (int32_t)-1));
    // several lines with one id: the last one wins, like repeated assignment into the reference's map
    int32_t to = 0;
    while (it != order.end() && it->first == r.d) { to = it->second; ++it; }
    r.d = to;
  }
  return from_edge_records_min_v(device, (int64_t)recs.size(), recs.data(), (int32_t)ids.size(), out);
}

int nd_graph_load(int device, const char *path, const char *graph_type, const char *graph_format, nd_graph **out) {
  ND_REQUIRE(path && graph_type && graph_format && out, ND_ERR_ARG, "nd_graph_load: null argument");
  const bool edge_list = strcmp(graph_type, "edge-list") == 0, adj_list = strcmp(graph_type, "adj-list") == 0;
  ND_REQUIRE(edge_list || adj_list, ND_ERR_ARG, "Incorrect graph file type '%s'", graph_type);
  if (edge_list && strcmp(graph_format, "binary") == 0) return nd_graph_load_edge_list_binary(device, path, out);
  if (edge_list && strcmp(graph_format, "text") == 0) return load_edge_list_text(device, path, out);
  if (adj_list && strcmp(graph_format, "text") == 0) return load_adjacency_list_text(device, path, out);
  nd_set_error("graph_format '%s' not supported for graph_type '%s'", graph_format, graph_type);
  return ND_ERR_ARG;
}

int nd_graph_rmat(int device, int32_t V, int64_t M, uint64_t seed, nd_graph **out) {
  ND_REQUIRE(out && V >= 2 && M >= 1, ND_ERR_ARG, "nd_graph_rmat: bad argument");
  ND_REQUIRE(2 * M < ((int64_t)1 << 31), ND_ERR_RANGE, "%lld CSR entries do not fit the int32 edge index", (long long)(2 * M));
  ND_CUDA(cudaSetDevice(device));
  NdDeviceInfo dev;
  ND_TRY(nd_device_info(device, &dev));
  const size_t cap = (size_t)(2 * M);
  uint32_t *a[3], *b[3];
  for (int w = 0; w < 3; w++) { ND_CUDA(cudaMalloc(&a[w], 4 * (cap + 8))); ND_CUDA(cudaMalloc(&b[w], 4 * (cap + 8))); }
  int scale = 0;
  while (((int64_t)1 << scale) < V) scale++;
  rmat_kernel<<<grid_for(M, 256, dev.sms), 256>>>(V, scale, M, seed, a[0], a[1], a[2]);
  ND_CUDA(cudaGetLastError());
  return build_from_soa(device, 2 * M, V, a, b, nullptr, out);
}

int nd_graph_info(const nd_graph *g, int32_t *V, int64_t *E, int32_t *max_degree, int *device) {
  ND_REQUIRE(g, ND_ERR_ARG, "null graph");
  if (V) *V = g->V;
  if (E) *E = g->E;
  if (max_degree) *max_degree = g->max_degree;
  if (device) *device = g->device;
  return ND_OK;
}

int nd_graph_to_host(const nd_graph *g, int32_t *row_ptr, int32_t *col, float *w, float *max_w) {
  ND_REQUIRE(g, ND_ERR_ARG, "null graph");
  ND_CUDA(cudaSetDevice(g->device));
  if (row_ptr) ND_CUDA(cudaMemcpy(row_ptr, g->row_ptr, sizeof(int32_t) * ((size_t)g->V + 1), cudaMemcpyDeviceToHost));
  if (col && g->E) ND_CUDA(cudaMemcpy(col, g->col, sizeof(int32_t) * (size_t)g->E, cudaMemcpyDeviceToHost));
  if (w && g->E) ND_CUDA(cudaMemcpy(w, g->w, sizeof(float) * (size_t)g->E, cudaMemcpyDeviceToHost));
  if (max_w) ND_CUDA(cudaMemcpy(max_w, g->max_w, sizeof(float) * (size_t)g->V, cudaMemcpyDeviceToHost));
  return ND_OK;
}

int nd_graph_device_ptrs(const nd_graph *g, const int32_t **row_ptr, const int32_t **col, const float **w,
                         const float **max_w) {
  ND_REQUIRE(g, ND_ERR_ARG, "null graph");
  if (row_ptr) *row_ptr = g->row_ptr;
  if (col) *col = g->col;
  if (w) *w = g->w;
  if (max_w) *max_w = g->max_w;
  return ND_OK;
}

int nd_graph_destroy(nd_graph *g) {
  if (!g) return ND_OK;
  cudaSetDevice(g->device);
  cudaFree(g->row_ptr); cudaFree(g->col); cudaFree(g->w); cudaFree(g->max_w);
  cudaFree(g->colw); cudaFree(g->vrec); cudaFree(g->adjset);
  delete g;
  return ND_OK;
}

int nd_graph_partition(const nd_graph *g, int64_t budget_bytes, int32_t max_parts, int32_t *first_v,
                       int32_t *last_v, int64_t *first_e, int64_t *last_e, int32_t *n_parts) {
  ND_REQUIRE(g && first_v && last_v && first_e && last_e && n_parts && max_parts >= 1, ND_ERR_ARG, "nd_graph_partition: bad argument");
  ND_REQUIRE(budget_bytes >= 20, ND_ERR_ARG, "partition budget of %lld bytes cannot hold one vertex and one edge", (long long)budget_bytes);
  ND_CUDA(cudaSetDevice(g->device));
  int32_t *d_fv, *d_lv, *d_n;
  long long *d_fe, *d_le;
  ND_CUDA(cudaMalloc(&d_fv, 4 * (size_t)max_parts)); ND_CUDA(cudaMalloc(&d_lv, 4 * (size_t)max_parts));
  ND_CUDA(cudaMalloc(&d_fe, 8 * (size_t)max_parts)); ND_CUDA(cudaMalloc(&d_le, 8 * (size_t)max_parts));
  ND_CUDA(cudaMalloc(&d_n, 4));
  partition_kernel<<<1, 32>>>(g->row_ptr, g->V, budget_bytes, max_parts, d_fv, d_lv, d_fe, d_le, d_n);
  ND_CUDA(cudaMemcpy(n_parts, d_n, 4, cudaMemcpyDeviceToHost));
  const size_t k = (size_t)*n_parts;
  ND_CUDA(cudaMemcpy(first_v, d_fv, 4 * k, cudaMemcpyDeviceToHost));
  ND_CUDA(cudaMemcpy(last_v, d_lv, 4 * k, cudaMemcpyDeviceToHost));
  ND_CUDA(cudaMemcpy(first_e, d_fe, 8 * k, cudaMemcpyDeviceToHost));
  ND_CUDA(cudaMemcpy(last_e, d_le, 8 * k, cudaMemcpyDeviceToHost));
  cudaFree(d_fv); cudaFree(d_lv); cudaFree(d_fe); cudaFree(d_le); cudaFree(d_n);
  return ND_OK;
}

}  // extern "C"
