// Per-segment dedup: sort ascending, drop equal neighbours, compact to the front, pad with the
// invalid id, report the unique count.
//
// Semantics of remove_duplicates_in_hop_per_block (src/distinct.cuh:1-111, dead code in the
// reference: one CTA per root, cub BlockRadixSort, a single thread compacting, segments above
// 1024 entries skipped).  Here a segment (one hop of one sample: 25 or 250 ids for GraphSAGE) is
// owned by a thread group sized to it; the group runs a bitonic network over the padded segment
// in shared memory, flags the first element of every run of equal ids, ranks the flags with a
// shared-memory scan and writes the survivors back in one coalesced pass.
#include "nd_common.cuh"

namespace {

constexpr int DTHREADS = 256;
constexpr int MAX_SEG = 2048;

// P = padded (power of two) segment length, G = threads per segment (P/2 capped at DTHREADS).
template <int P>
__global__ void __launch_bounds__(DTHREADS)
distinct_kernel(int32_t *__restrict__ data, int64_t n_segments, int32_t seg_len, int32_t seg_stride,
                int32_t invalid, int32_t *__restrict__ counts, int32_t counts_stride) {
  constexpr int G = (P / 2 < 32) ? 32 : ((P / 2 > DTHREADS) ? DTHREADS : P / 2);
  constexpr int SEGS_PER_CTA = DTHREADS / G;
  __shared__ int32_t keys[SEGS_PER_CTA][P];
  __shared__ int32_t rank[SEGS_PER_CTA][P];
  const int grp = threadIdx.x / G, t = threadIdx.x % G;
  const int64_t seg0 = (int64_t)blockIdx.x * SEGS_PER_CTA;
  // every group runs the same number of barriers, so groups past the end just idle on a dummy
  const int64_t seg = seg0 + grp;
  const bool active = seg < n_segments;
  int32_t *k = keys[grp];
  int32_t *r = rank[grp];
  int32_t *base = data + seg * (int64_t)seg_stride;
  for (int i = t; i < P; i += G) {
    int32_t v = 0x7fffffff;
    if (active && i < seg_len) {
      v = base[i];
      if (v == invalid || v < 0) v = 0x7fffffff;
    }
    k[i] = v;
  }
  auto gsync = [&]() { if (G <= 32) __syncwarp(); else __syncthreads(); };
  gsync();
  for (int size = 2; size <= P; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = t; i < P / 2; i += G) {
        const int lo = 2 * i - (i & (stride - 1));
        const int hi = lo + stride;
        const bool up = (lo & size) == 0;
        const int32_t a = k[lo], b = k[hi];
        if ((a > b) == up) { k[lo] = b; k[hi] = a; }
      }
      gsync();
    }
  }
  // flags, then inclusive Hillis-Steele scan in shared memory
  for (int i = t; i < P; i += G) r[i] = (k[i] != 0x7fffffff && (i == 0 || k[i] != k[i - 1])) ? 1 : 0;
  gsync();
  for (int off = 1; off < P; off <<= 1) {
    int32_t add[(P + G - 1) / G];
    int c = 0;
    for (int i = t; i < P; i += G, c++) add[c] = i >= off ? r[i - off] : 0;
    gsync();
    c = 0;
    for (int i = t; i < P; i += G, c++) r[i] += add[c];
    gsync();
  }
  const int32_t uniq = r[P - 1];
  // survivors to the front (positions only ever move left, and reads come from shared memory)
  if (active) {
    for (int i = t; i < seg_len; i += G) {
      const bool head = k[i] != 0x7fffffff && (i == 0 || k[i] != k[i - 1]);
      if (head) base[r[i] - 1] = k[i];
    }
    for (int i = uniq + t; i < seg_len; i += G) base[i] = invalid;
    if (t == 0 && counts) counts[seg * (int64_t)counts_stride] = uniq;
  }
}

// Segments of up to 256 ids: one warp per segment, the whole segment in registers (E ids per
// lane, lane l owns positions l*E .. l*E+E-1).  The bitonic network exchanges inside a lane for
// strides below E and with warp shuffles above; run heads are ranked with a shuffle scan.  No shared
// memory and no block barrier.
template <int E>
__global__ void __launch_bounds__(DTHREADS)
distinct_warp_kernel(int32_t *__restrict__ data, int64_t n_segments, int32_t seg_len, int32_t seg_stride,
                     int32_t invalid, int32_t *__restrict__ counts, int32_t counts_stride) {
  constexpr int P = 32 * E;
  const int lane = threadIdx.x & 31;
  const int64_t seg = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  if (seg >= n_segments) return;  // whole warps leave together
  int32_t *base = data + seg * (int64_t)seg_stride;
  int32_t v[E];
#pragma unroll
  for (int e = 0; e < E; e++) {
    const int g = lane * E + e;
    int32_t x = 0x7fffffff;
    if (g < seg_len) {
      x = base[g];
      if (x == invalid || x < 0) x = 0x7fffffff;
    }
    v[e] = x;
  }
#pragma unroll
  for (int size = 2; size <= P; size <<= 1) {
#pragma unroll
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      if (stride >= E) {
        const int ls = stride / E;
        const bool lower = (lane & ls) == 0;
#pragma unroll
        for (int e = 0; e < E; e++) {
          const int32_t other = __shfl_xor_sync(0xffffffffu, v[e], ls);
          const bool up = (((lane * E + e) & size) == 0);
          v[e] = (lower == up) ? min(v[e], other) : max(v[e], other);
        }
      } else {
#pragma unroll
        for (int e = 0; e < E; e++) {
          if ((e & stride) == 0) {
            const bool up = (((lane * E + e) & size) == 0);
            const int32_t a = v[e], b = v[e + stride];
            if ((a > b) == up) { v[e] = b; v[e + stride] = a; }
          }
        }
      }
    }
  }
  int32_t before = __shfl_up_sync(0xffffffffu, v[E - 1], 1);  // last id of the lane to the left
  bool head[E];
  int cnt = 0;
#pragma unroll
  for (int e = 0; e < E; e++) {
    const int32_t prev = e == 0 ? before : v[e - 1];
    head[e] = v[e] != 0x7fffffff && ((lane == 0 && e == 0) || v[e] != prev);
    cnt += head[e] ? 1 : 0;
  }
  int inc = cnt;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  const int uniq = __shfl_sync(0xffffffffu, inc, 31);
  int pos = inc - cnt;
#pragma unroll
  for (int e = 0; e < E; e++)
    if (head[e]) base[pos++] = v[e];
  for (int i = uniq + lane; i < seg_len; i += 32) base[i] = invalid;
  if (lane == 0 && counts) counts[seg * (int64_t)counts_stride] = uniq;
}

}  // namespace

int nd_distinct_launch(cudaStream_t st, int32_t *data, int64_t n_segments, int32_t seg_len, int32_t seg_stride,
                       int32_t invalid, int32_t *counts, int32_t counts_stride) {
  ND_REQUIRE(seg_len >= 1 && seg_len <= MAX_SEG, ND_ERR_ARG, "distinct: segment length %d outside [1,%d]", seg_len, MAX_SEG);
  int P = 32;
  while (P < seg_len) P <<= 1;
  if (P <= 256) {  // a warp per segment, ids in registers
    const int64_t blocks = (n_segments * 32 + DTHREADS - 1) / DTHREADS;
    switch (P) {
      case 32: distinct_warp_kernel<1><<<(unsigned)blocks, DTHREADS, 0, st>>>(data, n_segments, seg_len, seg_stride, invalid, counts, counts_stride); break;
      case 64: distinct_warp_kernel<2><<<(unsigned)blocks, DTHREADS, 0, st>>>(data, n_segments, seg_len, seg_stride, invalid, counts, counts_stride); break;
      case 128: distinct_warp_kernel<4><<<(unsigned)blocks, DTHREADS, 0, st>>>(data, n_segments, seg_len, seg_stride, invalid, counts, counts_stride); break;
      default: distinct_warp_kernel<8><<<(unsigned)blocks, DTHREADS, 0, st>>>(data, n_segments, seg_len, seg_stride, invalid, counts, counts_stride); break;
    }
    ND_CUDA(cudaGetLastError());
    return ND_OK;
  }
#define LAUNCH(PP)                                                                                       \
  {                                                                                                      \
    constexpr int G = ((PP) / 2 < 32) ? 32 : (((PP) / 2 > DTHREADS) ? DTHREADS : (PP) / 2);              \
    const int64_t blocks = (n_segments + (DTHREADS / G) - 1) / (DTHREADS / G);                           \
    distinct_kernel<PP><<<(unsigned)blocks, DTHREADS, 0, st>>>(data, n_segments, seg_len, seg_stride, invalid, counts, counts_stride); \
  }
  switch (P) {
    case 32: LAUNCH(32) break;
    case 64: LAUNCH(64) break;
    case 128: LAUNCH(128) break;
    case 256: LAUNCH(256) break;
    case 512: LAUNCH(512) break;
    case 1024: LAUNCH(1024) break;
    default: LAUNCH(2048) break;
  }
#undef LAUNCH
  ND_CUDA(cudaGetLastError());
  return ND_OK;
}
