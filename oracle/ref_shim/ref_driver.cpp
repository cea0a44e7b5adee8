/*
 * ref_driver.cpp -- drives the reference's OWN next() bodies and host graph loader on the CPU.
 * TEST INFRASTRUCTURE ONLY (validates oracle/nd_oracle.c, generates golden fixtures, and is the
 * "reference" CPU baseline).  Built by oracle/Makefile into oracle/_ref/libnd_ref.so with the
 * reference sources included from their own tree; none of them is copied here.
 *
 * The step loop around next() is a restatement: which transit feeds which slot follows
 * sampleParallelKernel (src/nextdoor.cu:1390-1500) and next() is invoked as at :1445-1446,
 * only when the transit has edges (:255, :412, :1143); output slots use the deterministic
 * layout prefix_k + parent*stepSize + j.  Draws are the keyed Philox draws of the oracle.
 */
#include "ref_shim.h"

#include <omp.h>

#include "apps/randomwalks/randomWalks.cu"
#undef VERTICES_PER_SAMPLE
#include "apps/khop/khop.cu"
#undef VERTICES_PER_SAMPLE
#include "apps/fastgcn/fastgcnSampling.cu"
#undef VERTICES_PER_SAMPLE
#undef NUM_LAYERS
#undef NUM_SAMPLED_VERTICES
#undef NUM_SAMPLES
#include "apps/ladies/ladiessampling.cu"
#define REF_LAYERS NUM_LAYERS
#define REF_LAYER_SIZE NUM_SAMPLED_VERTICES
#undef VERTICES_PER_SAMPLE
#define main ref_example_main
#include "uniformRandWalk.cu" /* example/, found through -I<reference>/example */
#undef main

namespace {

struct HostCSR {
  std::vector<CSR::Vertex> verts;
  CSRPartition *part = nullptr;
  int32_t V = 0;
  HostCSR(int32_t V_, const int32_t *row_ptr, const int32_t *col, const float *w, const float *max_w)
      : verts(V_), V(V_) {
    for (int32_t v = 0; v < V; v++) {
      verts[v].id = v;
      verts[v].start_edge_id = row_ptr[v];
      verts[v].end_edge_id = row_ptr[v + 1] > row_ptr[v] ? row_ptr[v + 1] - 1 : -1;
      verts[v].max_weight = max_w[v];
    }
    part = new CSRPartition(0, V - 1, 0, row_ptr[V] - 1, verts.data(), col, w);
  }
  ~HostCSR() { delete part; }
};

template <class App, class SampleType>
void run_walk(HostCSR &g, int steps, int64_t S, int64_t first, uint64_t seed, const int32_t *initial,
              int32_t *out, int64_t *edges_out) {
  const int32_t INV = g.V;
  int64_t total = 0;
#pragma omp parallel for schedule(dynamic, 256) reduction(+ : total)
  for (int64_t s = 0; s < S; s++) {
    SampleType sample = SampleType();
    VertexID cur = initial[s];
    for (int step = 0; step < steps; step++) {
      VertexID nbr = -1;
      if (cur != INV && cur != -1) {
        EdgePos_t n = g.part->get_n_edges_for_vertex(cur);
        if (n != 0) {
          const CSR::Edge *edges = g.part->get_edges(cur);
          const float *weights = g.part->get_weights(cur);
          const float mw = g.part->get_max_weight(cur);
          curandState st{seed, (uint32_t)(first + s), (uint32_t)step, 0u, 0u};
          nbr = App().template next<SampleType, const CSR::Edge *, const float *>(
              step, g.part, &cur, (VertexID)(first + s), &sample, mw, edges, weights, n, 0, &st);
        }
      }
      if (nbr != -1) { out[s * steps + step] = nbr; cur = nbr; total++; }
      else { out[s * steps + step] = INV; cur = INV; }
    }
  }
  *edges_out = total;
}

void run_khop(HostCSR &g, int64_t S, int64_t first, uint64_t seed, const int32_t *initial,
              int32_t *out, int64_t *edges_out) {
  const int32_t INV = g.V;
  KHopApp app;
  const int steps = app.steps();
  int fs = 0, n = 1;
  for (int k = 0; k < steps; k++) { n *= app.stepSize(k); fs += n; }
  int64_t total = 0;
#pragma omp parallel for schedule(dynamic, 64) reduction(+ : total)
  for (int64_t s = 0; s < S; s++) {
    KHopSample sample;
    int32_t *o = out + s * fs;
    int prefix_prev = 0, n_prev = 1, prefix = 0;
    for (int step = 0; step < steps; step++) {
      const int k = app.stepSize(step);
      for (int i = 0; i < n_prev; i++) {
        VertexID transit = step == 0 ? initial[s] : o[prefix_prev + i];
        for (int j = 0; j < k; j++) {
          VertexID nbr = -1;
          if (transit != INV && transit != -1) {
            EdgePos_t ne = g.part->get_n_edges_for_vertex(transit);
            if (ne != 0) {
              const CSR::Edge *edges = g.part->get_edges(transit);
              const float *weights = g.part->get_weights(transit);
              curandState st{seed, (uint32_t)(first + s), (uint32_t)step, (uint32_t)(i * k + j), 0u};
              nbr = app.next<KHopSample, const CSR::Edge *, const float *>(
                  step, g.part, &transit, (VertexID)(first + s), &sample, g.part->get_max_weight(transit),
                  edges, weights, ne, j, &st);
            }
          }
          o[prefix + i * k + j] = nbr != -1 ? nbr : INV;
          total += nbr != -1;
        }
      }
      prefix_prev = prefix; prefix += n_prev * k; n_prev *= k;
    }
  }
  *edges_out = total;
}

template <class App, class SampleType>
void run_collective(HostCSR &g, int steps, int64_t S, int64_t first, uint64_t seed,
                    const int32_t *initial, int32_t *out, int32_t *adj_row, int32_t *adj_col,
                    int64_t *edges_out) {
  const int L = REF_LAYER_SIZE;
  const int fs = steps * L;
  const int stride = L * L;
  int64_t total = 0;
#pragma omp parallel for schedule(dynamic, 4) reduction(+ : total)
  for (int64_t s = 0; s < S; s++) {
    SampleType *sample = new SampleType();
    std::memset(sample, 0xff, sizeof(SampleType)); /* untouched entries read as (-1,-1) */
    for (int step = 0; step < steps; step++) {
      const VertexID *transits = step == 0 ? initial + s * L : out + s * fs + (step - 1) * L;
      for (int j = 0; j < L; j++) {
        EdgePos_t ne = 0;
        for (int i = 0; i < L; i++) ne += g.part->get_n_edges_for_vertex(transits[i]);
        const CSR::Edge *edges = nullptr;
        const float *weights = nullptr;
        curandState st{seed, (uint32_t)(first + s), (uint32_t)step, (uint32_t)j, 0u};
        VertexID nbr = App().template next<SampleType, const CSR::Edge *, const float *>(
            step, g.part, transits, (VertexID)(first + s), sample, 0.0f, edges, weights, ne, j, &st);
        out[s * fs + step * L + j] = nbr;
        total++;
      }
      if (adj_row) {
        std::memcpy(adj_row + (s * steps + step) * (int64_t)stride, sample->adjacencyMatrixRow[step], sizeof(int) * stride);
        std::memcpy(adj_col + (s * steps + step) * (int64_t)stride, sample->adjacencyMatrixCol[step], sizeof(int) * stride);
      }
    }
    delete sample;
  }
  *edges_out = total;
}

}  // namespace

extern "C" {

int ref_layers(void) { return REF_LAYERS; }
int ref_layer_size(void) { return REF_LAYER_SIZE; }
int ref_max_threads(void) { return omp_get_max_threads(); }

/* app ids as in nd_oracle.h; steps is honoured for walks and (<= REF_LAYERS) for collective apps */
int ref_sample(int32_t V, const int32_t *row_ptr, const int32_t *col, const float *w, const float *max_w,
               int app, int steps, int64_t S, int64_t first, uint64_t seed, const int32_t *initial,
               int32_t *out, int32_t *adj_row, int32_t *adj_col, int64_t *edges_out, int threads) {
  HostCSR g(V, row_ptr, col, w, max_w);
  if (threads > 0) omp_set_num_threads(threads);
  int64_t e = 0;
  switch (app) {
    case 0: run_walk<UniformRandomWalkApp, UniformRandomWalkSample>(g, steps, S, first, seed, initial, out, &e); break;
    case 1: run_walk<DeepWalkApp, DummySample>(g, steps, S, first, seed, initial, out, &e); break;
    case 2: run_walk<PPRApp, DummySample>(g, steps, S, first, seed, initial, out, &e); break;
    case 3: run_walk<Node2VecApp, Node2VecSample>(g, steps, S, first, seed, initial, out, &e); break;
    case 4: run_khop(g, S, first, seed, initial, out, &e); break;
    case 6: if (steps > REF_LAYERS) return -2;
      run_collective<FastGCNSamplingApp, FastGCNSample>(g, steps, S, first, seed, initial, out, adj_row, adj_col, &e); break;
    case 7: if (steps > REF_LAYERS) return -2;
      run_collective<ImportanceSampleApp, ImportanceSample>(g, steps, S, first, seed, initial, out, adj_row, adj_col, &e); break;
    default: return -1;
  }
  if (edges_out) *edges_out = e;
  return 0;
}

/* The reference's host loader end to end: Graph::load_from_edge_list_binary (src/graph.hpp:106-159)
 * then csr_from_graph (src/csr.hpp:399-424).  Call once with row_ptr == NULL for the sizes. */
int ref_load_edge_list_binary(const char *path, int32_t *V_out, int64_t *E_out, int32_t *row_ptr,
                              int32_t *col, float *w, float *max_w) {
  Graph graph;
  graph.load_from_edge_list_binary(path, true);
  int32_t V = (int32_t)graph.get_vertices().size();
  int64_t E = graph.get_n_edges();
  *V_out = V; *E_out = E;
  if (!row_ptr) return 0;
  CSR *csr = new CSR(V, (EdgePos_t)E);
  csr_from_graph(csr, graph);
  for (int32_t v = 0; v < V; v++) {
    const CSR::Vertex &x = csr->get_vertices()[v];
    row_ptr[v] = x.start_edge_id;
    max_w[v] = x.max_weight;
  }
  row_ptr[V] = (int32_t)E;
  std::memcpy(col, csr->get_edges(), sizeof(int32_t) * E);
  std::memcpy(w, csr->get_weights(), sizeof(float) * E);
  return 0;
}

/* The reference's two text loaders, Graph::load_from_edge_list_txt (src/graph.hpp:162-254) and
 * Graph::load_from_adjacency_list (:256-326), followed by csr_from_graph.  kind: 1 = text edge
 * list, 2 = text adjacency list.  Call once with row_ptr == NULL for the sizes. */
int ref_load_text(const char *path, int kind, int32_t *V_out, int64_t *E_out, int32_t *row_ptr,
                  int32_t *col, float *w, float *max_w) {
  Graph graph;
  if (kind == 1) {
    FILE *fp = fopen(path, "r");
    if (!fp) return -1;
    graph.load_from_edge_list_txt(fp, true);
    fclose(fp);
  } else {
    graph.load_from_adjacency_list((char *)path);
  }
  int32_t V = (int32_t)graph.get_vertices().size();
  int64_t E = graph.get_n_edges();
  *V_out = V; *E_out = E;
  if (!row_ptr) return 0;
  CSR *csr = new CSR(V, (EdgePos_t)E);
  csr_from_graph(csr, graph);
  for (int32_t v = 0; v < V; v++) {
    row_ptr[v] = csr->get_vertices()[v].start_edge_id;
    max_w[v] = csr->get_vertices()[v].max_weight;
  }
  row_ptr[V] = (int32_t)E;
  std::memcpy(col, csr->get_edges(), sizeof(int32_t) * E);
  std::memcpy(w, csr->get_weights(), sizeof(float) * E);
  return 0;
}

}  // extern "C"
