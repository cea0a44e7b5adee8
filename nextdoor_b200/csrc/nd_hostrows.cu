// Walk results into a caller's dense host array without moving the empty slots.
//
// getFinalSamples (src/nextdoor.cu:3211-3237) hands the caller a dense [samples, steps] array.
// For walks that end early almost all of it is the invalid id (PPR with a stop probability of
// 0.15: 3 vertices on average in rows of 100), and copying it over PCIe takes twenty times longer
// than sampling it.  A walk's vertices are a prefix of its row, and the sampler knows each row's
// length (d_plen), so this path moves only the prefixes: the rows are packed on the device, the
// lengths and the packed vertices are copied, and host threads write them into the caller's
// array.  The caller's array keeps its contents from call to call like the device array does:
// `row_len` holds for every row how many leading slots may hold a vertex (everything behind is
// the invalid id), so an update rewrites only the slots a walk fills now or filled in the
// previous update of that array.  Three calls, so that the caller can overlap them with the next
// job's sampling: begin (enqueue) -> fetch (lengths have landed: enqueue the vertices) -> finish
// (vertices have landed: write the rows).
#include <stdlib.h>

#include <thread>
#include <vector>

#include "nd_common.cuh"

struct NdHostRows {
  int32_t *h_len = nullptr;     // pinned [S]: the rows' lengths of the job being copied
  int32_t *h_vals = nullptr;    // pinned: packed vertices
  size_t vals_cap = 0;
  uint32_t *d_chunk = nullptr;  // per chunk of PACK_ROWS rows: sum of lengths, then exclusive prefix
  int n_chunks = 0;
  cudaEvent_t packed = nullptr, len_done = nullptr, vals_done = nullptr, total_done = nullptr;
  uint32_t *h_total = nullptr;  // pinned: number of packed vertices (nd_sampler_pack_rows)
  cudaStream_t cs = nullptr;
  int32_t *out = nullptr, *row_len = nullptr;
  int64_t total = 0;
  bool dense = false;           // most slots are in use: the dense array is copied as it is
  int stage = 0;                // 0 idle, 1 begun, 2 fetched
  int threads = 1;
};

namespace {

constexpr int PACK_THREADS = 256, PACK_PER_THREAD = 16, PACK_ROWS = PACK_THREADS * PACK_PER_THREAD;

__global__ void __launch_bounds__(PACK_THREADS)
pack_sum_kernel(const int32_t *__restrict__ plen, int64_t S, uint32_t *__restrict__ chunk) {
  __shared__ uint32_t wsum[PACK_THREADS / 32];
  const int64_t first = (int64_t)blockIdx.x * PACK_ROWS;
  uint32_t t = 0;
  for (int r = threadIdx.x; r < PACK_ROWS; r += PACK_THREADS)
    if (first + r < S) t += (uint32_t)plen[first + r];
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = t;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t a = 0;
    for (int w = 0; w < PACK_THREADS / 32; w++) a += wsum[w];
    chunk[blockIdx.x] = a;
  }
}

// one CTA: chunk sums -> exclusive prefix in place, the grand total in chunk[n]
__global__ void __launch_bounds__(1024) pack_scan_kernel(uint32_t *__restrict__ chunk, int n) {
  __shared__ uint32_t wsum[32];
  __shared__ uint32_t carry_sh;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_sh = 0;
  __syncthreads();
  for (int base = 0; base < n; base += 1024) {
    const int i = base + threadIdx.x;
    const uint32_t v = i < n ? chunk[i] : 0u;
    uint32_t inc = v;
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += t;
    }
    if (lane == 31) wsum[warp] = inc;
    __syncthreads();
    uint32_t before = carry_sh;
    for (int w = 0; w < warp; w++) before += wsum[w];
    if (i < n) chunk[i] = before + inc - v;
    __syncthreads();
    if (threadIdx.x == 1023) carry_sh = before + inc;
    __syncthreads();
  }
  if (threadIdx.x == 0) chunk[n] = carry_sh;
}

// the inverse of pack_rows_kernel on the receiving side: row r of `out` takes its len[r] vertices
// from vals, the slots it held before beyond that (row_len[r]) go back to the invalid id
__global__ void __launch_bounds__(PACK_THREADS)
unpack_rows_kernel(const int32_t *__restrict__ len, const int32_t *__restrict__ vals, const uint32_t *__restrict__ chunk_base,
                   int64_t S, int steps, int32_t invalid, int32_t *__restrict__ out, int32_t *__restrict__ row_len) {
  __shared__ uint32_t wsum[PACK_THREADS / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t first = (int64_t)blockIdx.x * PACK_ROWS + (int64_t)threadIdx.x * PACK_PER_THREAD;
  int32_t l[PACK_PER_THREAD];
  uint32_t t = 0;
#pragma unroll
  for (int r = 0; r < PACK_PER_THREAD; r++) {
    l[r] = first + r < S ? len[first + r] : 0;
    t += (uint32_t)l[r];
  }
  uint32_t inc = t;
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t u = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += u;
  }
  if (lane == 31) wsum[warp] = inc;
  __syncthreads();
  size_t pos = (size_t)chunk_base[blockIdx.x] + inc - t;
  for (int w = 0; w < warp; w++) pos += wsum[w];
#pragma unroll
  for (int r = 0; r < PACK_PER_THREAD; r++) {
    if (first + r >= S) break;
    int32_t *row = out + (first + r) * steps;
    const int32_t had = row_len[first + r];
    for (int k = 0; k < l[r]; k++) row[k] = vals[pos + k];
    for (int k = l[r]; k < had; k++) row[k] = invalid;
    if (had != l[r]) row_len[first + r] = l[r];
    pos += (size_t)l[r];
  }
}

// a thread owns PACK_PER_THREAD consecutive rows; their prefixes go to vals back to back
__global__ void __launch_bounds__(PACK_THREADS)
pack_rows_kernel(const int32_t *__restrict__ plen, const int32_t *__restrict__ out, int64_t S, int steps,
                 const uint32_t *__restrict__ chunk_base, int32_t *__restrict__ vals) {
  __shared__ uint32_t wsum[PACK_THREADS / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t first = (int64_t)blockIdx.x * PACK_ROWS + (int64_t)threadIdx.x * PACK_PER_THREAD;
  int32_t l[PACK_PER_THREAD];
  uint32_t t = 0;
#pragma unroll
  for (int r = 0; r < PACK_PER_THREAD; r++) {
    l[r] = first + r < S ? plen[first + r] : 0;
    t += (uint32_t)l[r];
  }
  uint32_t inc = t;
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t u = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += u;
  }
  if (lane == 31) wsum[warp] = inc;
  __syncthreads();
  size_t pos = (size_t)chunk_base[blockIdx.x] + inc - t;
  for (int w = 0; w < warp; w++) pos += wsum[w];
#pragma unroll
  for (int r = 0; r < PACK_PER_THREAD; r++) {
    const int32_t *row = out + (first + r) * steps;
    for (int k = 0; k < l[r]; k++) vals[pos + k] = row[k];
    pos += (size_t)l[r];
  }
}

// positions in the packed array are 32-bit
bool packable(const nd_sampler *s) { return s->S * (int64_t)s->fs < ((int64_t)1 << 32); }

int host_threads() {
  if (const char *e = getenv("ND_HOST_THREADS")) {
    const int n = atoi(e);
    if (n >= 1) return n < 256 ? n : 256;
  }
  const unsigned hc = std::thread::hardware_concurrency();
  return hc == 0 ? 4 : (hc > 32 ? 32 : (int)hc);
}

// runs fn(t, first_row, end_row) on `threads` contiguous row ranges; a range whose thread cannot be
// started (the process is out of threads) is run by the caller, so nothing escapes the C boundary
template <class F>
void for_row_ranges(int64_t S, int threads, F fn) {
  if (threads > S) threads = S > 0 ? (int)S : 1;
  std::vector<std::thread> pool;
  pool.reserve((size_t)threads);
  int started = 1;
  for (; started < threads; started++) {
    try {
      pool.emplace_back(fn, started, S * started / threads, S * (started + 1) / threads);
    } catch (...) {
      break;
    }
  }
  fn(0, (int64_t)0, S / threads);
  for (int t = started; t < threads; t++) fn(t, S * t / threads, S * (t + 1) / threads);
  for (auto &th : pool) th.join();
}

// staging state of a sampler, made at the first use
int hostrows_init(nd_sampler *s) {
  if (s->hostrows) return ND_OK;
  s->hostrows = new NdHostRows();   // a creation that fails half way is taken down again, so the next call starts over
  NdHostRows *h = s->hostrows;
  const size_t S1 = (size_t)(s->S > 0 ? s->S : 1);
  h->n_chunks = (int)((S1 + PACK_ROWS - 1) / PACK_ROWS);
  h->threads = host_threads();
  cudaError_t e = cudaMallocHost(&h->h_len, sizeof(int32_t) * S1);
  if (e == cudaSuccess) e = cudaMallocHost(&h->h_total, sizeof(uint32_t));
  if (e == cudaSuccess) e = cudaMalloc(&h->d_chunk, sizeof(uint32_t) * ((size_t)h->n_chunks + 1));
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->packed, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->len_done, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->vals_done, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->total_done, cudaEventDisableTiming);
  if (e != cudaSuccess) {
    nd_hostrows_free(s);
    nd_set_error("staging buffers of the packed result: %s", cudaGetErrorString(e));
    cudaGetLastError();
    return ND_ERR_CUDA;
  }
  return ND_OK;
}

// the rows' prefixes packed into the staging array of the walk (free between two passes), on the sampler's stream
int pack_enqueue(nd_sampler *s) {
  NdHostRows *h = s->hostrows;
  pack_sum_kernel<<<h->n_chunks, PACK_THREADS, 0, s->stream>>>(s->d_plen, s->S, h->d_chunk);
  pack_scan_kernel<<<1, 1024, 0, s->stream>>>(h->d_chunk, h->n_chunks);
  pack_rows_kernel<<<h->n_chunks, PACK_THREADS, 0, s->stream>>>(s->d_plen, s->d_out, s->S, s->fs, h->d_chunk, s->d_tmp);
  nd_count_launches(3);
  ND_CUDA(cudaGetLastError());
  return ND_OK;
}

}  // namespace

void nd_hostrows_free(nd_sampler *s);

void nd_hostrows_free(nd_sampler *s) {
  NdHostRows *h = s->hostrows;
  if (!h) return;
  if (h->h_len) cudaFreeHost(h->h_len);
  if (h->h_vals) cudaFreeHost(h->h_vals);
  cudaFree(h->d_chunk);
  if (h->packed) cudaEventDestroy(h->packed);
  if (h->len_done) cudaEventDestroy(h->len_done);
  if (h->vals_done) cudaEventDestroy(h->vals_done);
  if (h->total_done) cudaEventDestroy(h->total_done);
  if (h->h_total) cudaFreeHost(h->h_total);
  delete h;
  s->hostrows = nullptr;
}

extern "C" {

int nd_host_fill_int32(int32_t *dst, int64_t n, int32_t value) {
  ND_REQUIRE(dst || n == 0, ND_ERR_ARG, "nd_host_fill_int32: null destination");
  ND_REQUIRE(n >= 0, ND_ERR_ARG, "nd_host_fill_int32: negative length");
  for_row_ranges(n, host_threads(), [=](int, int64_t a, int64_t b) {
    for (int64_t i = a; i < b; i++) dst[i] = value;
  });
  return ND_OK;
}

int nd_sampler_host_update_begin(nd_sampler *s, int32_t *out, int32_t *row_len, void *copy_stream) {
  ND_REQUIRE(s && ((out && row_len) || s->S == 0), ND_ERR_ARG, "nd_sampler_host_update_begin: null argument");
  ND_REQUIRE(nd_is_walk(s->p.app), ND_ERR_ARG, "host row updates exist for the walk apps (their rows are prefixes)");
  ND_REQUIRE(s->sampled, ND_ERR_STATE, "host update requested before sample()");
  ND_CUDA(cudaSetDevice(s->g->device));
  ND_TRY(hostrows_init(s));
  NdHostRows *h = s->hostrows;
  ND_REQUIRE(h->stage == 0, ND_ERR_STATE, "the previous host update of this sampler was not finished");
  h->out = out;
  h->row_len = row_len;
  h->cs = copy_stream ? (cudaStream_t)copy_stream : s->stream;
  if (s->S == 0) { h->stage = 1; return ND_OK; }
  // (an error below leaves stage 0: nothing was begun as far as the caller is concerned)
  if (packable(s)) ND_TRY(pack_enqueue(s));   // (larger arrays take the dense copy in fetch)
  if (h->cs != s->stream) {
    ND_CUDA(cudaEventRecord(h->packed, s->stream));
    ND_CUDA(cudaStreamWaitEvent(h->cs, h->packed, 0));
  }
  ND_CUDA(cudaMemcpyAsync(h->h_len, s->d_plen, sizeof(int32_t) * (size_t)s->S, cudaMemcpyDeviceToHost, h->cs));
  ND_CUDA(cudaEventRecord(h->len_done, h->cs));
  if (h->cs != s->stream) {  // the next sampling of this sampler waits for the copies that read its buffers
    if (!s->copy_done) ND_CUDA(cudaEventCreateWithFlags(&s->copy_done, cudaEventDisableTiming));
    ND_CUDA(cudaEventRecord(s->copy_done, h->cs));
    s->copy_pending = true;
  }
  h->stage = 1;
  return ND_OK;
}

int nd_sampler_host_update_fetch(nd_sampler *s) {
  ND_REQUIRE(s && s->hostrows && s->hostrows->stage == 1, ND_ERR_STATE, "nd_sampler_host_update_fetch without a begun update");
  NdHostRows *h = s->hostrows;
  h->stage = 0;   // an error below abandons the update; stage 2 is set once the copy is enqueued
  h->total = 0;
  h->dense = false;
  if (s->S == 0) { h->stage = 2; return ND_OK; }
  ND_CUDA(cudaSetDevice(s->g->device));
  ND_CUDA(cudaEventSynchronize(h->len_done));
  std::vector<int64_t> part((size_t)h->threads, 0);
  const int32_t *len = h->h_len;
  for_row_ranges(s->S, h->threads, [&](int t, int64_t a, int64_t b) {
    int64_t sum = 0;
    for (int64_t i = a; i < b; i++) sum += len[i];
    part[(size_t)t] = sum;
  });
  for (int64_t v : part) h->total += v;
  h->dense = 2 * h->total > s->S * (int64_t)s->fs || !packable(s);
  if (h->dense) {
    ND_CUDA(cudaMemcpyAsync(h->out, s->d_out, sizeof(int32_t) * (size_t)s->S * s->fs, cudaMemcpyDeviceToHost, h->cs));
  } else if (h->total > 0) {
    if ((size_t)h->total > h->vals_cap) {
      if (h->h_vals) ND_CUDA(cudaFreeHost(h->h_vals));
      h->h_vals = nullptr;
      h->vals_cap = (size_t)h->total + (size_t)h->total / 4 + 4096;
      ND_CUDA(cudaMallocHost(&h->h_vals, sizeof(int32_t) * h->vals_cap));
    }
    ND_CUDA(cudaMemcpyAsync(h->h_vals, s->d_tmp, sizeof(int32_t) * (size_t)h->total, cudaMemcpyDeviceToHost, h->cs));
  }
  ND_CUDA(cudaEventRecord(h->vals_done, h->cs));
  if (h->cs != s->stream) {
    ND_CUDA(cudaEventRecord(s->copy_done, h->cs));
    s->copy_pending = true;
  }
  h->stage = 2;
  return ND_OK;
}

int nd_sampler_host_update_finish(nd_sampler *s, int64_t *values_copied) {
  ND_REQUIRE(s && s->hostrows && s->hostrows->stage >= 1, ND_ERR_STATE, "nd_sampler_host_update_finish without a begun update");
  NdHostRows *h = s->hostrows;
  if (h->stage == 1) ND_TRY(nd_sampler_host_update_fetch(s));
  ND_REQUIRE(h->stage == 2, ND_ERR_STATE, "nd_sampler_host_update_finish: the update was abandoned after an error");
  h->stage = 0;
  if (values_copied) *values_copied = h->dense ? s->S * (int64_t)s->fs : h->total;
  if (s->S == 0) return ND_OK;
  ND_CUDA(cudaSetDevice(s->g->device));
  ND_CUDA(cudaEventSynchronize(h->vals_done));
  const int32_t *len = h->h_len, *vals = h->h_vals;
  int32_t *out = h->out, *row_len = h->row_len;
  const int steps = s->fs;
  const int32_t invalid = s->g->V;
  if (h->dense) {  // the whole array came over as it is: only the lengths are left to note
    for_row_ranges(s->S, h->threads, [=](int, int64_t a, int64_t b) {
      for (int64_t i = a; i < b; i++) row_len[i] = len[i];
    });
    return ND_OK;
  }
  // every thread needs the position of its first row in the packed array: the ranges' sums again
  std::vector<int64_t> part((size_t)h->threads + 1, 0);
  for_row_ranges(s->S, h->threads, [&](int t, int64_t a, int64_t b) {
    int64_t sum = 0;
    for (int64_t i = a; i < b; i++) sum += len[i];
    part[(size_t)t + 1] = sum;
  });
  for (size_t t = 1; t < part.size(); t++) part[t] += part[t - 1];
  for_row_ranges(s->S, h->threads, [&, out, row_len, len, vals](int t, int64_t a, int64_t b) {
    const int32_t *src = vals + part[(size_t)t];
    for (int64_t i = a; i < b; i++) {
      const int32_t now = len[i], had = row_len[i];
      int32_t *row = out + i * steps;
      for (int k = 0; k < now; k++) row[k] = src[k];
      for (int k = now; k < had; k++) row[k] = invalid;
      src += now;
      if (now != had) row_len[i] = now;
    }
  });
  return ND_OK;
}

// ---- the same packing between GPUs: the sender packs, the receiver unpacks into its dense array

int nd_sampler_pack_rows(nd_sampler *s, const int32_t **d_row_len, const int32_t **d_vals) {
  ND_REQUIRE(s && d_row_len && d_vals, ND_ERR_ARG, "nd_sampler_pack_rows: null argument");
  ND_REQUIRE(nd_is_walk(s->p.app), ND_ERR_ARG, "packed rows exist for the walk apps (their rows are prefixes)");
  ND_REQUIRE(s->sampled, ND_ERR_STATE, "packed rows requested before sample()");
  ND_REQUIRE(packable(s), ND_ERR_RANGE, "result array too large for 32-bit positions in the packed form");
  ND_CUDA(cudaSetDevice(s->g->device));
  ND_TRY(hostrows_init(s));
  NdHostRows *h = s->hostrows;
  ND_REQUIRE(h->stage == 0, ND_ERR_STATE, "a host update of this sampler is using the staging array");
  *d_row_len = s->d_plen;
  *d_vals = s->d_tmp;
  *h->h_total = 0;
  if (s->S > 0) {
    ND_TRY(pack_enqueue(s));
    ND_CUDA(cudaMemcpyAsync(h->h_total, h->d_chunk + h->n_chunks, sizeof(uint32_t), cudaMemcpyDeviceToHost, s->stream));
  }
  ND_CUDA(cudaEventRecord(h->total_done, s->stream));
  return ND_OK;
}

int nd_sampler_pack_rows_total(nd_sampler *s, int64_t *total) {
  ND_REQUIRE(s && total && s->hostrows && s->hostrows->total_done, ND_ERR_STATE, "nd_sampler_pack_rows_total before nd_sampler_pack_rows");
  ND_CUDA(cudaSetDevice(s->g->device));
  ND_CUDA(cudaEventSynchronize(s->hostrows->total_done));
  *total = (int64_t)*s->hostrows->h_total;
  return ND_OK;
}

int64_t nd_rows_scratch_words(int64_t n_rows) { return (n_rows + PACK_ROWS - 1) / PACK_ROWS + 1; }

int nd_rows_unpack(int device, void *stream, int64_t n_rows, int steps, int32_t invalid, const int32_t *d_len,
                   const int32_t *d_vals, int32_t *d_out, int32_t *d_row_len, uint32_t *d_scratch) {
  ND_REQUIRE(n_rows >= 0 && steps >= 1, ND_ERR_ARG, "nd_rows_unpack: bad size");
  if (n_rows == 0) return ND_OK;
  ND_REQUIRE(d_len && d_out && d_row_len && d_scratch, ND_ERR_ARG, "nd_rows_unpack: null argument");
  ND_REQUIRE(n_rows * (int64_t)steps < ((int64_t)1 << 32), ND_ERR_RANGE, "nd_rows_unpack: array too large for 32-bit positions");
  ND_CUDA(cudaSetDevice(device));
  cudaStream_t st = (cudaStream_t)stream;
  const int n_chunks = (int)((n_rows + PACK_ROWS - 1) / PACK_ROWS);
  pack_sum_kernel<<<n_chunks, PACK_THREADS, 0, st>>>(d_len, n_rows, d_scratch);
  pack_scan_kernel<<<1, 1024, 0, st>>>(d_scratch, n_chunks);
  unpack_rows_kernel<<<n_chunks, PACK_THREADS, 0, st>>>(d_len, d_vals, d_scratch, n_rows, steps, invalid, d_out, d_row_len);
  nd_count_launches(3);
  ND_CUDA(cudaGetLastError());
  return ND_OK;
}

}  // extern "C"
