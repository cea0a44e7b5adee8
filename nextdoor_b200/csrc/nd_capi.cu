// extern "C" boundary of the library: error text, sampler life cycle, result access, phase
// timers and the single-operator entry points.  The reference's counterparts are named in
// include/nextdoor_b200.h beside each declaration.
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include "nd_common.cuh"
#include "nd_philox.cuh"

#include <atomic>

static thread_local char g_err[512] = "";
static std::atomic<long long> g_launches{0};

void nd_count_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

void nd_set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int nd_device_info(int device, NdDeviceInfo *info) {
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0) {
    nd_set_error("no CUDA device: %s", e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0");
    return ND_ERR_CUDA;
  }
  ND_REQUIRE(device >= 0 && device < n, ND_ERR_ARG, "device %d out of range [0,%d)", device, n);
  info->device = device;
  ND_CUDA(cudaDeviceGetAttribute(&info->sms, cudaDevAttrMultiProcessorCount, device));
  ND_CUDA(cudaDeviceGetAttribute(&info->smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
  return ND_OK;
}

void nd_phase_begin(nd_sampler *s, int phase) {
  if (!s->timer.on) return;
  cudaEvent_t a, b;
  cudaEventCreate(&a);
  cudaEventCreate(&b);
  s->timer.ev.push_back(a);
  s->timer.ev.push_back(b);
  s->timer.phase_of_pair.push_back(phase);
  cudaEventRecord(a, s->stream);
}

void nd_phase_end(nd_sampler *s) {
  if (!s->timer.on) return;
  cudaEventRecord(s->timer.ev.back(), s->stream);
}

namespace {

__global__ void philox_uniform_kernel(uint64_t seed, int64_t n, const uint32_t *__restrict__ t4, float *__restrict__ out) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= n) return;
  ndrng::Rng rng(seed, t4[4 * i], t4[4 * i + 1], t4[4 * i + 2]);
  const uint32_t draw = t4[4 * i + 3];
  float u = 0.f;
  for (uint32_t d = 0; d <= draw; d++) u = rng.uniform();
  out[i] = u;
}

__global__ void default_initial_kernel(int64_t first, int64_t S, int isz, int32_t V, int32_t *__restrict__ initial) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= S * isz) return;
  const int64_t s = first + i / isz;
  const int j = (int)(i % isz);
  // walks / k-hop: sample i starts at vertex i % V (randomWalks.cu:34, khop.cu:47);
  // collective: batch b holds ids b*isz + j (fastgcnSampling.cu:80-82)
  initial[i] = isz == 1 ? (int32_t)(s % V) : (int32_t)((s * isz + j) % V);
}

void free_sampler(nd_sampler *s) {
  nd_hostrows_free(s);
  cudaFree(s->d_initial); cudaFree(s->d_out); cudaFree(s->d_tmp); cudaFree(s->d_len); cudaFree(s->d_plen); cudaFree(s->d_state);
  for (int i = 0; i < 2; i++) { cudaFree(s->d_map_key[i]); cudaFree(s->d_map_val[i]); }
  cudaFree(s->d_init_key); cudaFree(s->d_init_val); cudaFree(s->d_nlive); cudaFree(s->d_stats); cudaFree(s->d_status);
  cudaFree(s->d_runs); cudaFree(s->d_bin_counts); cudaFree(s->d_hop_counts);
  cudaFree(s->d_adj_row); cudaFree(s->d_adj_col); cudaFree(s->d_prob); cudaFree(s->d_cand); cudaFree(s->d_cand_w); cudaFree(s->d_acc); cudaFree(s->d_bm);
  cudaFree(s->d_cnt); cudaFree(s->d_offs); cudaFree(s->d_bsum); cudaFree(s->d_rank);
  for (int i = 0; i < 2; i++) cudaFree(s->d_srec[i]);
  cudaFree(s->d_init_rec); cudaFree(s->d_uext);
  for (int i = 0; i < 3; i++) if (s->graph_exec[i]) cudaGraphExecDestroy(s->graph_exec[i]);
  if (s->copy_event) cudaEventDestroy(s->copy_event);
  if (s->copy_done) cudaEventDestroy(s->copy_done);
  if (s->side_fork) cudaEventDestroy(s->side_fork);
  if (s->side_join) cudaEventDestroy(s->side_join);
  if (s->side) cudaStreamDestroy(s->side);
  if (s->active_done) cudaEventDestroy(s->active_done);
  if (s->h_active) cudaFreeHost(s->h_active);
  nd_radix_scratch_free(&s->radix);
  for (cudaEvent_t e : s->timer.ev) cudaEventDestroy(e);
  delete s;
}

int check_params(const nd_app_params *p) {
  ND_REQUIRE(p, ND_ERR_ARG, "null app parameters");
  ND_REQUIRE(p->app >= ND_APP_UNIFORM_WALK && p->app <= ND_APP_LADIES_IS, ND_ERR_ARG, "unknown app id %d", p->app);
  ND_REQUIRE(p->steps >= 1, ND_ERR_ARG, "steps must be >= 1 (got %d)", p->steps);
  if (nd_is_khop(p->app)) {
    ND_REQUIRE(p->steps <= ND_MAX_STEPS_FANOUT, ND_ERR_ARG, "k-hop supports at most %d hops", ND_MAX_STEPS_FANOUT);
    int64_t n = 1, tot = 0;
    for (int k = 0; k < p->steps; k++) {
      ND_REQUIRE(p->fanout[k] >= 1 && p->fanout[k] <= 64, ND_ERR_ARG, "fan-out %d of hop %d outside [1,64]", p->fanout[k], k);
      n *= p->fanout[k];
      tot += n;
      ND_REQUIRE(tot < (1 << 24), ND_ERR_ARG, "final sample size too large");
    }
  }
  if (nd_is_collective(p->app)) {
    ND_REQUIRE(p->fanout[0] >= 1 && p->fanout[0] <= 1024, ND_ERR_ARG, "layer size %d outside [1,1024]", p->fanout[0]);
    ND_REQUIRE(p->batch >= 1 && p->batch <= 1024, ND_ERR_ARG, "batch %d outside [1,1024]", p->batch);
  }
  if (p->app == ND_APP_NODE2VEC) ND_REQUIRE(p->p > 0.f && p->q > 0.f, ND_ERR_ARG, "node2vec needs p, q > 0");
  return ND_OK;
}

}  // namespace

extern "C" {

const char *nd_last_error(void) { return g_err; }
int nd_version(void) { return 100; }
int64_t nd_launch_count(void) { return (int64_t)g_launches.load(); }

int nd_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
  return n;
}

int nd_initial_sample_size(const nd_app_params *p) { return (p && nd_is_collective(p->app)) ? p->batch : 1; }

int nd_final_sample_size(const nd_app_params *p) {
  if (!p) return 0;
  if (nd_is_walk(p->app)) return p->steps;
  if (nd_is_khop(p->app)) {
    int64_t n = 1, tot = 0;
    for (int k = 0; k < p->steps && k < ND_MAX_STEPS_FANOUT; k++) { n *= p->fanout[k]; tot += n; }
    return (int)tot;
  }
  return p->steps * p->fanout[0];
}

int nd_shard_range(int64_t total, int idx, int parts, int64_t *first, int64_t *count) {
  ND_REQUIRE(parts >= 1 && idx >= 0 && idx < parts && total >= 0 && first && count, ND_ERR_ARG, "nd_shard_range: bad argument");
  const int64_t per = total / parts;
  *first = idx * per;
  *count = idx < parts - 1 ? per : total - (int64_t)(parts - 1) * per;
  return ND_OK;
}

int nd_sampler_create(const nd_graph *g, const nd_app_params *p, int64_t num_samples, int64_t first_sample,
                      const int32_t *initial, nd_sampler **out) {
  ND_REQUIRE(g && out, ND_ERR_ARG, "nd_sampler_create: null graph or output");
  ND_TRY(check_params(p));
  ND_REQUIRE(num_samples >= 0 && first_sample >= 0, ND_ERR_ARG, "negative sample count or offset");
  ND_REQUIRE(first_sample + num_samples <= 0xffffffffll, ND_ERR_RANGE, "global sample index exceeds 32 bits");
  ND_REQUIRE(num_samples * (int64_t)nd_final_sample_size(p) < ((int64_t)1 << 40), ND_ERR_RANGE, "output too large");
  ND_CUDA(cudaSetDevice(g->device));
  nd_sampler *s = new nd_sampler();
  s->g = g;
  s->p = *p;
  s->S = num_samples;
  s->first = first_sample;
  s->fs = nd_final_sample_size(p);
  s->isz = nd_initial_sample_size(p);
  int rc = nd_device_info(g->device, &s->dev);
  if (rc != ND_OK) { delete s; return rc; }
  const size_t S1 = (size_t)(num_samples > 0 ? num_samples : 1);
  auto fail = [&](int code) { free_sampler(s); return code; };
#define ND_TRY_S(call) do { int c__ = (call); if (c__ != ND_OK) return fail(c__); } while (0)
#define ND_CUDA_S(call) do { cudaError_t e__ = (call); if (e__ != cudaSuccess) { nd_set_error("%s failed: %s", #call, cudaGetErrorString(e__)); return fail(ND_ERR_CUDA); } } while (0)
  ND_CUDA_S(cudaMalloc(&s->d_initial, sizeof(int32_t) * S1 * s->isz));
  ND_CUDA_S(cudaMalloc(&s->d_out, sizeof(int32_t) * S1 * s->fs));
  ND_CUDA_S(cudaMalloc(&s->d_stats, sizeof(unsigned long long) * 8));
  ND_CUDA_S(cudaMalloc(&s->d_status, sizeof(int)));
  ND_CUDA_S(cudaMemset(s->d_stats, 0, sizeof(unsigned long long) * 8));
  ND_CUDA_S(cudaMemset(s->d_status, 0, sizeof(int)));
  if (nd_is_walk(p->app)) ND_TRY_S(nd_walk_alloc(s));
  else if (nd_is_khop(p->app)) ND_TRY_S(nd_khop_alloc(s));
  else ND_TRY_S(nd_collective_alloc(s));
  if (initial) {
    ND_CUDA_S(cudaMemcpy(s->d_initial, initial, sizeof(int32_t) * (size_t)num_samples * s->isz, cudaMemcpyHostToDevice));
  } else if (num_samples > 0) {
    const int64_t n = num_samples * s->isz;
    default_initial_kernel<<<(int)((n + 255) / 256), 256>>>(first_sample, num_samples, s->isz, g->V, s->d_initial);
    ND_CUDA_S(cudaGetLastError());
  }
  if (!nd_is_collective(p->app)) ND_TRY_S(nd_sampler_build_initial_map(s));
  ND_CUDA_S(cudaDeviceSynchronize());
#undef ND_TRY_S
#undef ND_CUDA_S
  *out = s;
  return ND_OK;
}

int nd_sampler_set_initial(nd_sampler *s, const int32_t *initial) {
  ND_REQUIRE(s && initial, ND_ERR_ARG, "nd_sampler_set_initial: null argument");
  ND_CUDA(cudaSetDevice(s->g->device));
  ND_CUDA(cudaMemcpyAsync(s->d_initial, initial, sizeof(int32_t) * (size_t)s->S * s->isz, cudaMemcpyHostToDevice, s->stream));
  if (!nd_is_collective(s->p.app)) ND_TRY(nd_sampler_build_initial_map(s));
  return ND_OK;
}

int nd_sampler_set_stream(nd_sampler *s, void *stream) {
  ND_REQUIRE(s, ND_ERR_ARG, "null sampler");
  s->stream = (cudaStream_t)stream;
  return ND_OK;
}

int nd_sampler_sample(nd_sampler *s, int mode) {
  ND_REQUIRE(s, ND_ERR_ARG, "null sampler");
  ND_REQUIRE(mode >= ND_MODE_TRANSIT_PARALLEL && mode <= ND_MODE_SAMPLE_PARALLEL, ND_ERR_ARG, "unknown mode %d", mode);
  ND_CUDA(cudaSetDevice(s->g->device));
  if (s->timer.on) {
    for (cudaEvent_t e : s->timer.ev) cudaEventDestroy(e);
    s->timer.ev.clear();
    s->timer.phase_of_pair.clear();
  }
  s->sampled = true;
  if (s->S == 0) return ND_OK;
  if (s->copy_pending) {  // a result copy on another stream still reads the buffers this job overwrites
    ND_CUDA(cudaStreamWaitEvent(s->stream, s->copy_done, 0));
    s->copy_pending = false;
  }
  if (nd_is_walk(s->p.app)) return nd_walk_sample(s, mode);
  if (nd_is_khop(s->p.app)) return nd_khop_sample(s, mode);
  return nd_collective_sample(s, mode);
}

int nd_sampler_sync(nd_sampler *s) {
  ND_REQUIRE(s, ND_ERR_ARG, "null sampler");
  ND_CUDA(cudaSetDevice(s->g->device));
  ND_CUDA(cudaStreamSynchronize(s->stream));
  int status = 0;
  ND_CUDA(cudaMemcpy(&status, s->d_status, sizeof(int), cudaMemcpyDeviceToHost));
  if (status != 0) {
    ND_CUDA(cudaMemset(s->d_status, 0, sizeof(int)));
    nd_set_error("device status word 0x%x:%s%s%s%s", status, status & ND_DEV_BAD_TRANSIT ? " transit id out of range" : "",
                 status & ND_DEV_WAIT_TIMEOUT ? " bounded wait gave up" : "", status & ND_DEV_OVERFLOW ? " buffer overflow avoided" : "",
                 status & ND_DEV_RETRY_LIMIT ? " rejection loop hit its cap" : "");
    return ND_ERR_DEVICE;
  }
  return ND_OK;
}

int nd_sampler_final_samples(nd_sampler *s, int32_t *out) {
  ND_REQUIRE(s && (out || s->S == 0), ND_ERR_ARG, "nd_sampler_final_samples: null argument");
  ND_REQUIRE(s->sampled, ND_ERR_STATE, "final samples requested before sample()");
  ND_TRY(nd_sampler_sync(s));
  if (s->S > 0) ND_CUDA(cudaMemcpy(out, s->d_out, sizeof(int32_t) * (size_t)s->S * s->fs, cudaMemcpyDeviceToHost));
  return ND_OK;
}

int nd_sampler_final_samples_async(nd_sampler *s, int32_t *out, void *copy_stream) {
  ND_REQUIRE(s && (out || s->S == 0), ND_ERR_ARG, "nd_sampler_final_samples_async: null argument");
  ND_REQUIRE(s->sampled, ND_ERR_STATE, "final samples requested before sample()");
  ND_CUDA(cudaSetDevice(s->g->device));
  cudaStream_t cs = copy_stream ? (cudaStream_t)copy_stream : s->stream;
  if (cs != s->stream) {  // the copy waits for the sampling enqueued so far, the sampling stream does not wait for the copy
    if (!s->copy_event) ND_CUDA(cudaEventCreateWithFlags(&s->copy_event, cudaEventDisableTiming));
    ND_CUDA(cudaEventRecord(s->copy_event, s->stream));
    ND_CUDA(cudaStreamWaitEvent(cs, s->copy_event, 0));
  }
  if (s->S > 0) ND_CUDA(cudaMemcpyAsync(out, s->d_out, sizeof(int32_t) * (size_t)s->S * s->fs, cudaMemcpyDeviceToHost, cs));
  if (cs != s->stream) {
    if (!s->copy_done) ND_CUDA(cudaEventCreateWithFlags(&s->copy_done, cudaEventDisableTiming));
    ND_CUDA(cudaEventRecord(s->copy_done, cs));
    s->copy_pending = true;
  }
  return ND_OK;
}

int nd_stream_sync(int device, void *stream) {
  ND_CUDA(cudaSetDevice(device));
  ND_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  return ND_OK;
}

int nd_sampler_final_samples_device(nd_sampler *s, const int32_t **out) {
  ND_REQUIRE(s && out, ND_ERR_ARG, "nd_sampler_final_samples_device: null argument");
  *out = s->d_out;
  return ND_OK;
}

int nd_sampler_aux(nd_sampler *s, int32_t *adj_row, int32_t *adj_col, float *prob, int32_t *hop_counts) {
  ND_REQUIRE(s, ND_ERR_ARG, "null sampler");
  ND_REQUIRE(s->sampled, ND_ERR_STATE, "auxiliary outputs requested before sample()");
  ND_TRY(nd_sampler_sync(s));
  if (nd_is_collective(s->p.app)) {
    const int L = s->p.fanout[0], B = s->p.batch;
    const size_t n = (size_t)s->S * s->p.steps * (B > L ? B : L) * L;
    if (adj_row) ND_CUDA(cudaMemcpy(adj_row, s->d_adj_row, 4 * n, cudaMemcpyDeviceToHost));
    if (adj_col) ND_CUDA(cudaMemcpy(adj_col, s->d_adj_col, 4 * n, cudaMemcpyDeviceToHost));
    if (prob && s->d_prob) ND_CUDA(cudaMemcpy(prob, s->d_prob, 4 * (size_t)s->S * s->fs, cudaMemcpyDeviceToHost));
  }
  if (hop_counts && s->d_hop_counts)
    ND_CUDA(cudaMemcpy(hop_counts, s->d_hop_counts, 4 * (size_t)s->S * s->p.steps, cudaMemcpyDeviceToHost));
  return ND_OK;
}

int nd_sampler_stats(nd_sampler *s, int64_t *stats, int n) {
  ND_REQUIRE(s && stats && n >= 1 && n <= 8, ND_ERR_ARG, "nd_sampler_stats: bad argument");
  ND_TRY(nd_sampler_sync(s));
  unsigned long long h[8];
  ND_CUDA(cudaMemcpy(h, s->d_stats, sizeof(h), cudaMemcpyDeviceToHost));
  for (int i = 0; i < n; i++) stats[i] = (int64_t)h[i];
  return ND_OK;
}

int nd_sampler_live_pairs(nd_sampler *s, int32_t *live, int n) {
  ND_REQUIRE(s && live && n >= 1, ND_ERR_ARG, "nd_sampler_live_pairs: bad argument");
  ND_REQUIRE(nd_is_walk(s->p.app), ND_ERR_ARG, "nd_sampler_live_pairs: walk applications only");
  ND_TRY(nd_sampler_sync(s));
  const int m = n < s->p.steps ? n : s->p.steps;
  ND_CUDA(cudaMemcpy(live, s->d_nlive, sizeof(int32_t) * (size_t)m, cudaMemcpyDeviceToHost));
  for (int i = m; i < n; i++) live[i] = 0;
  return ND_OK;
}

int nd_sampler_set_profiling(nd_sampler *s, int on) {
  ND_REQUIRE(s, ND_ERR_ARG, "null sampler");
  s->timer.on = on != 0;
  return ND_OK;
}

int nd_sampler_phase_ms(nd_sampler *s, float *ms, int32_t *launches, int n) {
  ND_REQUIRE(s && ms && n >= 1 && n <= ND_PHASE_COUNT, ND_ERR_ARG, "nd_sampler_phase_ms: bad argument");
  ND_TRY(nd_sampler_sync(s));
  float acc[ND_PHASE_COUNT] = {0};
  int cnt[ND_PHASE_COUNT] = {0};
  for (size_t i = 0; i < s->timer.phase_of_pair.size(); i++) {
    float t = 0.f;
    ND_CUDA(cudaEventElapsedTime(&t, s->timer.ev[2 * i], s->timer.ev[2 * i + 1]));
    acc[s->timer.phase_of_pair[i]] += t;
    cnt[s->timer.phase_of_pair[i]]++;
  }
  for (int i = 0; i < n; i++) { ms[i] = acc[i]; if (launches) launches[i] = cnt[i]; }
  return ND_OK;
}

int nd_sampler_next_kernel(const nd_sampler *s, int mode, char *name, int n) {
  ND_REQUIRE(s && name && n > 0, ND_ERR_ARG, "nd_sampler_next_kernel: bad argument");
  ND_REQUIRE(mode >= ND_MODE_TRANSIT_PARALLEL && mode <= ND_MODE_SAMPLE_PARALLEL, ND_ERR_ARG, "unknown mode %d", mode);
  static const char *const walk_app[] = {"uniform walk", "DeepWalk", "PPR", "node2vec"};
  const int app = s->p.app;
  if (nd_is_walk(app)) {
    const char *k = mode == ND_MODE_TRANSIT_PARALLEL ? "walk_next_tp_kernel"
                    : mode == ND_MODE_TRANSIT_PARALLEL_LB ? "walk_next_count_kernel"
                    : (app == ND_APP_UNIFORM_WALK || getenv("ND_SP_PLAIN")) ? "walk_sp_kernel" : "walk_sp_rounds_kernel";
    snprintf(name, (size_t)n, "%s<%s>", k, walk_app[app]);
  } else if (nd_is_khop(app)) {
    const char *e = getenv("ND_KHOP_STAGING");
    const bool staged = mode == ND_MODE_TRANSIT_PARALLEL_LB && e && e[0] == '1';
    snprintf(name, (size_t)n, "%s", staged ? "khop_bin_kernel + khop_pairs_kernel + khop_staged_kernel" : "khop_pairs_kernel");
  } else if (app == ND_APP_FASTGCN_REF || app == ND_APP_LADIES_REF) {
    snprintf(name, (size_t)n, "coll_ref_kernel");
  } else {
    snprintf(name, (size_t)n, "%s", nd_collective_kernel_name(s));
  }
  return ND_OK;
}

int nd_sampler_destroy(nd_sampler *s) {
  if (!s) return ND_OK;
  cudaSetDevice(s->g->device);
  cudaStreamSynchronize(s->stream);
  free_sampler(s);
  return ND_OK;
}

// ---------------------------------------------------------------- single operators

int nd_invert_map(int device, int64_t n, int32_t *keys_in, int32_t *vals_in, int32_t invalid,
                  int32_t *keys_out, int32_t *vals_out, int64_t *n_live_out) {
  ND_REQUIRE(n >= 0 && n < ((int64_t)1 << 31) && invalid >= 1, ND_ERR_ARG, "nd_invert_map: bad size or invalid id");
  ND_REQUIRE(n == 0 || (keys_in && vals_in && keys_out && vals_out), ND_ERR_ARG, "nd_invert_map: null pointer");
  ND_CUDA(cudaSetDevice(device));
  if (n == 0) { if (n_live_out) *n_live_out = 0; return ND_OK; }
  NdDeviceInfo dev;
  ND_TRY(nd_device_info(device, &dev));
  NdRadixScratch scr;
  ND_TRY(nd_radix_scratch_alloc(&scr, nd_bit_length((uint32_t)(invalid > 1 ? invalid - 1 : 1)), n));
  int32_t *d_n = nullptr;
  ND_CUDA(cudaMalloc(&d_n, 2 * sizeof(int32_t)));
  const int32_t n32 = (int32_t)n;
  ND_CUDA(cudaMemcpy(d_n, &n32, sizeof(int32_t), cudaMemcpyHostToDevice));
  NdSortArrays arr;
  arr.nwords = 2;
  arr.a[0] = (uint32_t *)keys_in; arr.a[1] = (uint32_t *)vals_in; arr.a[2] = nullptr;
  arr.b[0] = (uint32_t *)keys_out; arr.b[1] = (uint32_t *)vals_out; arr.b[2] = nullptr;
  bool in_b = false;
  int rc = nd_radix_sort(dev, nullptr, &scr, scr.plan, arr, 0, d_n, d_n + 1, true, (uint32_t)invalid, false, &in_b);
  int32_t live = 0;
  if (rc == ND_OK) {
    ND_CUDA(cudaMemcpy(&live, d_n + 1, sizeof(int32_t), cudaMemcpyDeviceToHost));
    if (!in_b && live > 0) {
      ND_CUDA(cudaMemcpy(keys_out, keys_in, sizeof(int32_t) * (size_t)live, cudaMemcpyDeviceToDevice));
      ND_CUDA(cudaMemcpy(vals_out, vals_in, sizeof(int32_t) * (size_t)live, cudaMemcpyDeviceToDevice));
    }
  }
  ND_CUDA(cudaDeviceSynchronize());
  nd_radix_scratch_free(&scr);
  cudaFree(d_n);
  if (n_live_out) *n_live_out = live;
  return rc;
}

// ---- the inversion with its scratch kept between calls

struct nd_inverter {
  int device = 0;
  NdDeviceInfo dev;
  int64_t max_pairs = 0;
  int32_t invalid = 0;
  NdRadixScratch scr;
  int32_t *d_n = nullptr;   // [2]: pairs in, live pairs out
};

int nd_inverter_create(int device, int64_t max_pairs, int32_t invalid, nd_inverter **out) {
  ND_REQUIRE(out && max_pairs >= 1 && max_pairs < ((int64_t)1 << 31) && invalid >= 1, ND_ERR_ARG, "nd_inverter_create: bad argument");
  ND_CUDA(cudaSetDevice(device));
  nd_inverter *inv = new nd_inverter();
  inv->device = device;
  inv->max_pairs = max_pairs;
  inv->invalid = invalid;
  int rc = nd_device_info(device, &inv->dev);
  if (rc == ND_OK) rc = nd_radix_scratch_alloc(&inv->scr, nd_bit_length((uint32_t)(invalid > 1 ? invalid - 1 : 1)), max_pairs);
  if (rc == ND_OK && cudaMalloc(&inv->d_n, 2 * sizeof(int32_t)) != cudaSuccess) { nd_set_error("nd_inverter_create: cudaMalloc failed"); rc = ND_ERR_CUDA; }
  if (rc != ND_OK) { nd_radix_scratch_free(&inv->scr); cudaFree(inv->d_n); delete inv; return rc; }
  *out = inv;
  return ND_OK;
}

int nd_inverter_run(nd_inverter *inv, void *stream, int64_t n, int32_t *keys_in, int32_t *vals_in, int32_t *keys_out,
                    int32_t *vals_out, const int32_t **d_n_live) {
  ND_REQUIRE(inv && n >= 0 && n <= inv->max_pairs, ND_ERR_ARG, "nd_inverter_run: %lld pairs exceed the inverter's capacity", (long long)n);
  ND_REQUIRE(n == 0 || (keys_in && vals_in && keys_out && vals_out), ND_ERR_ARG, "nd_inverter_run: null pointer");
  ND_CUDA(cudaSetDevice(inv->device));
  cudaStream_t st = (cudaStream_t)stream;
  const int32_t n32[2] = {(int32_t)n, 0};
  ND_CUDA(cudaMemcpyAsync(inv->d_n, n32, sizeof(n32), cudaMemcpyHostToDevice, st));  // pageable source: staged before the call returns
  if (d_n_live) *d_n_live = inv->d_n + 1;
  if (n == 0) return ND_OK;
  NdSortArrays arr;
  arr.nwords = 2;
  arr.a[0] = (uint32_t *)keys_in; arr.a[1] = (uint32_t *)vals_in; arr.a[2] = nullptr;
  arr.b[0] = (uint32_t *)keys_out; arr.b[1] = (uint32_t *)vals_out; arr.b[2] = nullptr;
  bool in_b = false;
  ND_TRY(nd_radix_sort(inv->dev, st, &inv->scr, inv->scr.plan, arr, 0, inv->d_n, inv->d_n + 1, true, (uint32_t)inv->invalid, false, &in_b));
  if (!in_b) {  // an even number of passes: the result sits in the input arrays
    ND_CUDA(cudaMemcpyAsync(keys_out, keys_in, sizeof(int32_t) * (size_t)n, cudaMemcpyDeviceToDevice, st));
    ND_CUDA(cudaMemcpyAsync(vals_out, vals_in, sizeof(int32_t) * (size_t)n, cudaMemcpyDeviceToDevice, st));
  }
  return ND_OK;
}

int nd_inverter_destroy(nd_inverter *inv) {
  if (!inv) return ND_OK;
  cudaSetDevice(inv->device);
  nd_radix_scratch_free(&inv->scr);
  cudaFree(inv->d_n);
  delete inv;
  return ND_OK;
}

int nd_distinct_segments(int device, int32_t *data, int64_t n_segments, int32_t seg_len, int32_t invalid, int32_t *counts) {
  ND_REQUIRE(n_segments >= 0 && seg_len >= 1 && (data || n_segments == 0), ND_ERR_ARG, "nd_distinct_segments: bad argument");
  ND_CUDA(cudaSetDevice(device));
  if (n_segments == 0) return ND_OK;
  ND_TRY(nd_distinct_launch(nullptr, data, n_segments, seg_len, seg_len, invalid, counts, 1));
  ND_CUDA(cudaDeviceSynchronize());
  return ND_OK;
}

int nd_walk_step(const nd_graph *g, const nd_app_params *p, int step, int64_t n, const int32_t *d_transits,
                 const int64_t *d_samples, int32_t *d_next, void *stream) {
  ND_REQUIRE(g && p && n >= 0 && step >= 0 && (n == 0 || (d_transits && d_samples && d_next)), ND_ERR_ARG, "nd_walk_step: bad argument");
  ND_REQUIRE(p->app == ND_APP_UNIFORM_WALK || p->app == ND_APP_DEEPWALK || p->app == ND_APP_PPR, ND_ERR_ARG,
             "nd_walk_step: app %d needs the adjacency of another vertex than the transit (node2vec) or is not a walk", p->app);
  ND_CUDA(cudaSetDevice(g->device));
  if (n == 0) return ND_OK;
  return nd_walk_step_launch(g, p, step, n, d_transits, d_samples, d_next, (cudaStream_t)stream);
}

int nd_walk_step_packed(const nd_graph *g, const nd_app_params *p, int step, int64_t n, const uint64_t *d_walkers_in,
                        uint64_t *d_walkers_out, void *stream) {
  ND_REQUIRE(g && p && n >= 0 && step >= 0 && (n == 0 || (d_walkers_in && d_walkers_out)), ND_ERR_ARG, "nd_walk_step_packed: bad argument");
  ND_REQUIRE(p->app == ND_APP_UNIFORM_WALK || p->app == ND_APP_DEEPWALK || p->app == ND_APP_PPR, ND_ERR_ARG,
             "nd_walk_step_packed: app %d needs the adjacency of another vertex than the transit (node2vec) or is not a walk", p->app);
  ND_CUDA(cudaSetDevice(g->device));
  if (n == 0) return ND_OK;
  return nd_walk_step_packed_launch(g, p, step, n, d_walkers_in, d_walkers_out, (cudaStream_t)stream);
}

int nd_walk_step_status(int device, void *stream, int *status) {
  ND_REQUIRE(status, ND_ERR_ARG, "nd_walk_step_status: null argument");
  ND_CUDA(cudaSetDevice(device));
  return nd_walk_step_status_read((cudaStream_t)stream, status);
}

int nd_philox_uniform(int device, uint64_t seed, int64_t n, const uint32_t *tuples4, float *out) {
  ND_REQUIRE(n >= 0 && (n == 0 || (tuples4 && out)), ND_ERR_ARG, "nd_philox_uniform: bad argument");
  ND_CUDA(cudaSetDevice(device));
  if (n == 0) return ND_OK;
  philox_uniform_kernel<<<(int)((n + 255) / 256), 256>>>(seed, n, tuples4, out);
  ND_CUDA(cudaGetLastError());
  ND_CUDA(cudaDeviceSynchronize());
  return ND_OK;
}

}  // extern "C"
