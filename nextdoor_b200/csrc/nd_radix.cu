// In-house LSD radix sort for the transit-map inversion and the CSR build.
//
// Replaces cub::DeviceRadixSort::SortPairs / DeviceRunLengthEncode / DeviceScan of the reference's
// step loop (src/nextdoor.cu:2930-2933, 2535-2567) and its host-side std::sort of adjacency lists
// (src/graph.hpp:154-157).  One pass = three kernels with no inter-block waits:
//   hist    : per-tile digit counts -> tile_hist[bin][tile], global digit counts -> ghist[bin]
//   scan    : one CTA per bin: base of the bin (sum of lower bins) + exclusive scan over tiles
//   scatter : stable in-tile ranking (warp match + per-warp counters) and the permuted store
// The element count lives on the device (*d_n), so a whole multi-step job needs no host
// round trip; pairs carrying the drop key (dead walks) vanish in the first pass and the
// surviving count is written next to the data.  The first hist can be fused into the kernel
// that produces the keys (the next() kernels do that).
#include "nd_common.cuh"

namespace {

constexpr int THREADS = ND_RADIX_THREADS;
constexpr int WARPS = THREADS / 32;
constexpr int IPT = 8;                 // items per thread
constexpr int TILE = THREADS * IPT;    // 2048 pairs per tile

__device__ __forceinline__ uint32_t warp_incl_scan(uint32_t v) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  return v;
}

__global__ void __launch_bounds__(THREADS)
radix_hist_kernel(const uint32_t *__restrict__ keys, const int32_t *__restrict__ d_n, int shift, int bins,
                  bool drop, uint32_t drop_key, uint32_t *__restrict__ tile_hist, int64_t max_tiles,
                  uint32_t *__restrict__ ghist) {
  extern __shared__ uint32_t sh[];   // [bins] counts of the current tile, [bins] counts of all tiles of this CTA
  uint32_t *acc = sh + bins;
  const int n = *d_n;
  const int tiles = (n + TILE - 1) / TILE;
  const uint32_t mask = bins - 1;
  for (int b = threadIdx.x; b < bins; b += THREADS) acc[b] = 0;
  for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    for (int b = threadIdx.x; b < bins; b += THREADS) sh[b] = 0;
    __syncthreads();
    const int base = tile * TILE;
    uint32_t k[IPT];
#pragma unroll
    for (int r = 0; r < IPT; r++) {  // all loads of the tile first
      const int i = base + r * THREADS + threadIdx.x;
      k[r] = i < n ? keys[i] : drop_key;
    }
#pragma unroll
    for (int r = 0; r < IPT; r++) {
      const int i = base + r * THREADS + threadIdx.x;
      if (i < n && !(drop && k[r] == drop_key)) atomicAdd(&sh[(k[r] >> shift) & mask], 1u);
    }
    __syncthreads();
    for (int b = threadIdx.x; b < bins; b += THREADS) {  // a bin is always handled by the same thread
      const uint32_t c = sh[b];
      tile_hist[(int64_t)b * max_tiles + tile] = c;
      acc[b] += c;
    }
    __syncthreads();
  }
  // one global atomic per bin and CTA instead of one per bin and tile
  for (int b = threadIdx.x; b < bins; b += THREADS)
    if (acc[b]) atomicAdd(&ghist[b], acc[b]);
}

// grid = bins.  CTA b turns row b of tile_hist into global start offsets.
__global__ void __launch_bounds__(THREADS)
radix_scan_kernel(const int32_t *__restrict__ d_n, int bins, uint32_t *__restrict__ tile_hist,
                  int64_t max_tiles, const uint32_t *__restrict__ ghist, int32_t *__restrict__ d_n_out) {
  __shared__ uint32_t warp_tot[WARPS];
  __shared__ uint32_t carry_sh;
  const int n = *d_n;
  const int tiles = (n + TILE - 1) / TILE;
  const int b = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // base = sum of ghist[0..b)
  uint32_t part = 0;
  for (int i = threadIdx.x; i < b; i += THREADS) part += ghist[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  if (lane == 0) warp_tot[warp] = part;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t t = 0;
    for (int w = 0; w < WARPS; w++) t += warp_tot[w];
    carry_sh = t;
  }
  __syncthreads();
  uint32_t *row = tile_hist + (int64_t)b * max_tiles;
  for (int t0 = 0; t0 < tiles; t0 += THREADS) {
    const int t = t0 + threadIdx.x;
    const uint32_t v = t < tiles ? row[t] : 0u;
    uint32_t inc = warp_incl_scan(v);
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    uint32_t woff = 0;
    for (int w = 0; w < warp; w++) woff += warp_tot[w];
    const uint32_t carry = carry_sh;
    if (t < tiles) row[t] = carry + woff + inc - v;
    __syncthreads();
    if (threadIdx.x == THREADS - 1) carry_sh = carry + woff + inc;
    __syncthreads();
  }
  if (b == bins - 1 && threadIdx.x == 0 && d_n_out) *d_n_out = (int32_t)carry_sh;
}

template <int NW>
__global__ void __launch_bounds__(THREADS)
radix_scatter_kernel(NdSortArrays arr, int key_word, const int32_t *__restrict__ d_n, int shift, int bins,
                     bool drop, uint32_t drop_key, const uint32_t *__restrict__ tile_hist,
                     int64_t max_tiles, uint32_t *__restrict__ ghist_to_clear) {
  extern __shared__ uint32_t cnt[];  // [WARPS][bins]
  const int n = *d_n;
  const int tiles = (n + TILE - 1) / TILE;
  const uint32_t mask = bins - 1;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t lt = (1u << lane) - 1u;
  uint32_t *my = cnt + warp * bins;
  const uint32_t *__restrict__ keys = arr.a[key_word];

  for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    for (int i = threadIdx.x; i < WARPS * bins; i += THREADS) cnt[i] = 0;
    __syncthreads();
    const int wbase = tile * TILE + warp * (32 * IPT);
    uint32_t k[IPT];
    uint32_t rank[IPT];
    uint32_t dig[IPT];
#pragma unroll
    for (int r = 0; r < IPT; r++) {
      const int i = wbase + r * 32 + lane;
      bool live = i < n;
      if (live) {
        k[r] = keys[i];
        if (drop && k[r] == drop_key) live = false;
      }
      dig[r] = live ? ((k[r] >> shift) & mask) : 0xffffffffu;
    }
#pragma unroll
    for (int r = 0; r < IPT; r++) {
      const uint32_t d = dig[r];
      const uint32_t peers = __match_any_sync(0xffffffffu, d);
      const int leader = __ffs(peers) - 1;
      uint32_t old = 0;
      if (d != 0xffffffffu && lane == leader) {
        old = my[d];
        my[d] = old + __popc(peers);
      }
      old = __shfl_sync(0xffffffffu, old, leader);
      rank[r] = old + __popc(peers & lt);
      __syncwarp();
    }
    __syncthreads();
    // per bin: exclusive scan over the warps, seeded with the tile's global start of the bin
    for (int b = threadIdx.x; b < bins; b += THREADS) {
      uint32_t run = tile_hist[(int64_t)b * max_tiles + tile];
#pragma unroll
      for (int w = 0; w < WARPS; w++) {
        const uint32_t c = cnt[w * bins + b];
        cnt[w * bins + b] = run;
        run += c;
      }
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < IPT; r++) {
      if (dig[r] != 0xffffffffu) {
        const int i = wbase + r * 32 + lane;
        const uint32_t pos = my[dig[r]] + rank[r];
#pragma unroll
        for (int w = 0; w < NW; w++) arr.b[w][pos] = (w == key_word) ? k[r] : arr.a[w][i];
      }
    }
    __syncthreads();
  }
  if (ghist_to_clear && blockIdx.x == 0)
    for (int b = threadIdx.x; b < bins; b += THREADS) ghist_to_clear[b] = 0;
}

// Scatter for large maps (256 bins): the tile is first permuted into shared memory in its sorted
// order, then written out, so that consecutive threads store to consecutive addresses inside a
// bin's run instead of every lane of a warp storing to a different sector.  Same stable order as
// radix_scatter_kernel.  Shared memory: [WARPS][bins] counters, [bins] tile-local starts, [bins]
// global starts, [NW][TILE] staged words.
template <int NW>
__global__ void __launch_bounds__(THREADS)
radix_scatter_staged_kernel(NdSortArrays arr, int key_word, const int32_t *__restrict__ d_n, int shift, int bins,
                            bool drop, uint32_t drop_key, const uint32_t *__restrict__ tile_hist,
                            int64_t max_tiles, uint32_t *__restrict__ ghist_to_clear) {
  extern __shared__ uint32_t sm[];
  uint32_t *cnt = sm;                          // [WARPS][bins]
  uint32_t *lstart = cnt + WARPS * bins;       // [bins] first slot of the bin inside the staged tile
  uint32_t *gbase = lstart + bins;             // [bins] first slot of the bin's run of this tile in the output
  uint32_t *stage = gbase + bins;              // [NW][TILE]
  __shared__ uint32_t warp_tot[WARPS];
  const int n = *d_n;
  const int tiles = (n + TILE - 1) / TILE;
  const uint32_t mask = bins - 1;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t lt = (1u << lane) - 1u;
  uint32_t *my = cnt + warp * bins;
  const uint32_t *__restrict__ keys = arr.a[key_word];

  for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    for (int i = threadIdx.x; i < WARPS * bins; i += THREADS) cnt[i] = 0;
    __syncthreads();
    const int wbase = tile * TILE + warp * (32 * IPT);
    uint32_t k[IPT], rank[IPT], dig[IPT];
#pragma unroll
    for (int r = 0; r < IPT; r++) {
      const int i = wbase + r * 32 + lane;
      bool live = i < n;
      if (live) {
        k[r] = keys[i];
        if (drop && k[r] == drop_key) live = false;
      }
      dig[r] = live ? ((k[r] >> shift) & mask) : 0xffffffffu;
    }
#pragma unroll
    for (int r = 0; r < IPT; r++) {
      const uint32_t d = dig[r];
      const uint32_t peers = __match_any_sync(0xffffffffu, d);
      const int leader = __ffs(peers) - 1;
      uint32_t old = 0;
      if (d != 0xffffffffu && lane == leader) {
        old = my[d];
        my[d] = old + __popc(peers);
      }
      old = __shfl_sync(0xffffffffu, old, leader);
      rank[r] = old + __popc(peers & lt);
      __syncwarp();
    }
    __syncthreads();
    // per bin: exclusive scan over the warps (kept in cnt), tile count of the bin -> lstart (scanned below)
    for (int b = threadIdx.x; b < bins; b += THREADS) {
      uint32_t run = 0;
#pragma unroll
      for (int w = 0; w < WARPS; w++) {
        const uint32_t c = cnt[w * bins + b];
        cnt[w * bins + b] = run;
        run += c;
      }
      lstart[b] = run;
      gbase[b] = tile_hist[(int64_t)b * max_tiles + tile];
    }
    __syncthreads();
    // exclusive scan of the tile counts over the bins (bins is a multiple of THREADS or smaller)
    uint32_t carry = 0;
    for (int b0 = 0; b0 < bins; b0 += THREADS) {
      const int b = b0 + threadIdx.x;
      const uint32_t v = b < bins ? lstart[b] : 0u;
      const uint32_t inc = warp_incl_scan(v);
      if (lane == 31) warp_tot[warp] = inc;
      __syncthreads();
      uint32_t woff = carry;
      for (int w = 0; w < warp; w++) woff += warp_tot[w];
      if (b < bins) lstart[b] = woff + inc - v;
      uint32_t tot = 0;
      for (int w = 0; w < WARPS; w++) tot += warp_tot[w];
      carry += tot;
      __syncthreads();
    }
    const uint32_t n_live = carry;
#pragma unroll
    for (int r = 0; r < IPT; r++) {
      if (dig[r] != 0xffffffffu) {
        const int i = wbase + r * 32 + lane;
        const uint32_t lp = lstart[dig[r]] + my[dig[r]] + rank[r];
#pragma unroll
        for (int w = 0; w < NW; w++) stage[w * TILE + lp] = (w == key_word) ? k[r] : arr.a[w][i];
      }
    }
    __syncthreads();
    for (uint32_t j = threadIdx.x; j < n_live; j += THREADS) {
      const uint32_t key = stage[key_word * TILE + j];
      const uint32_t d = (key >> shift) & mask;
      const uint32_t pos = gbase[d] + (j - lstart[d]);
#pragma unroll
      for (int w = 0; w < NW; w++) arr.b[w][pos] = stage[w * TILE + j];
    }
    __syncthreads();
  }
  if (ghist_to_clear && blockIdx.x == 0)
    for (int b = threadIdx.x; b < bins; b += THREADS) ghist_to_clear[b] = 0;
}

}  // namespace

static int nd_radix_max_digit(int64_t max_n) { return max_n <= ((int64_t)4 << 20) ? 10 : 8; }

NdRadixPlan nd_radix_plan(int key_bits, int64_t max_n) {
  NdRadixPlan p;
  if (key_bits < 1) key_bits = 1;
  p.key_bits = key_bits;
  // Small maps stay L2-resident, where the scattered stores of a wide digit cost nothing extra
  // and every pass saved is three launches saved; large maps need 256-bin passes so that each
  // tile still writes runs of full sectors.
  const int max_digit = nd_radix_max_digit(max_n);
  p.passes = (key_bits + max_digit - 1) / max_digit;
  int left = key_bits, sh = 0;
  p.max_bins = 0;
  for (int i = 0; i < p.passes; i++) {
    const int b = (left + (p.passes - i) - 1) / (p.passes - i);
    p.bits[i] = b;
    p.shift[i] = sh;
    sh += b;
    left -= b;
    if ((1 << b) > p.max_bins) p.max_bins = 1 << b;
  }
  p.tile = TILE;
  p.max_n = max_n;
  p.max_tiles = (max_n + TILE - 1) / TILE;
  if (p.max_tiles < 1) p.max_tiles = 1;
  return p;
}

// The scratch is sized for the widest digit any plan over max_n pairs may pick, so one allocation
// serves sorts on keys of different widths (transit ids, edge endpoints, weight bits).
int nd_radix_scratch_alloc(NdRadixScratch *s, int key_bits, int64_t max_n) {
  s->plan = nd_radix_plan(key_bits, max_n);
  s->cap_bins = 1 << nd_radix_max_digit(max_n);
  s->bytes = sizeof(uint32_t) * ((size_t)s->cap_bins * s->plan.max_tiles + 8 * (size_t)s->cap_bins);
  void *p = nullptr;
  ND_CUDA(cudaMalloc(&p, s->bytes));
  s->tile_hist = (uint32_t *)p;
  s->ghist = s->tile_hist + (size_t)s->cap_bins * s->plan.max_tiles;
  ND_CUDA(cudaMemset(s->ghist, 0, sizeof(uint32_t) * 8 * s->cap_bins));
  return ND_OK;
}

void nd_radix_scratch_free(NdRadixScratch *s) {
  if (s->tile_hist) cudaFree(s->tile_hist);
  s->tile_hist = nullptr;
  s->ghist = nullptr;
}

int nd_radix_sort(const NdDeviceInfo &dev, cudaStream_t st, NdRadixScratch *scr, const NdRadixPlan &pl,
                  NdSortArrays arr, int key_word, const int32_t *d_n, int32_t *d_n_out, bool drop_enable,
                  uint32_t drop_key, bool first_hist_done, bool *result_in_b) {
  ND_REQUIRE(pl.max_tiles == scr->plan.max_tiles && pl.max_bins <= scr->cap_bins && pl.passes <= 8, ND_ERR_ARG,
             "radix plan does not fit the scratch it was given");
  ND_REQUIRE(!drop_enable || d_n_out, ND_ERR_ARG, "dropping keys needs a place for the surviving count");
  const int64_t tiles = pl.max_tiles;
  const int grid = (int)(tiles < (int64_t)dev.sms * 8 ? tiles : (int64_t)dev.sms * 8);
  bool in_b = false;
  for (int p = 0; p < pl.passes; p++) {
    const int bins = 1 << pl.bits[p];
    const bool drop = drop_enable && p == 0;
    const int32_t *n_ptr = (p == 0 || !drop_enable) ? d_n : d_n_out;
    uint32_t *gh = scr->ghist + (size_t)p * scr->cap_bins;
    NdSortArrays cur = arr;
    if (in_b) for (int w = 0; w < arr.nwords; w++) { cur.a[w] = arr.b[w]; cur.b[w] = arr.a[w]; }
    if (!(p == 0 && first_hist_done)) {
      radix_hist_kernel<<<grid, THREADS, 2 * bins * sizeof(uint32_t), st>>>(
          cur.a[key_word], n_ptr, pl.shift[p], bins, drop, drop_key, scr->tile_hist, pl.max_tiles, gh);
    }
    radix_scan_kernel<<<bins, THREADS, 0, st>>>(n_ptr, bins, scr->tile_hist, pl.max_tiles, gh,
                                                  p == 0 ? d_n_out : nullptr);
    if (bins <= 256 && pl.max_n > ((int64_t)4 << 20)) {  // large maps: coalesced stores through a staged tile
      const size_t sms = sizeof(uint32_t) * ((size_t)WARPS * bins + 2 * (size_t)bins + (size_t)arr.nwords * TILE);
      switch (arr.nwords) {
        case 1: radix_scatter_staged_kernel<1><<<grid, THREADS, sms, st>>>(cur, key_word, n_ptr, pl.shift[p], bins, drop, drop_key, scr->tile_hist, pl.max_tiles, gh); break;
        case 2: radix_scatter_staged_kernel<2><<<grid, THREADS, sms, st>>>(cur, key_word, n_ptr, pl.shift[p], bins, drop, drop_key, scr->tile_hist, pl.max_tiles, gh); break;
        default: radix_scatter_staged_kernel<3><<<grid, THREADS, sms, st>>>(cur, key_word, n_ptr, pl.shift[p], bins, drop, drop_key, scr->tile_hist, pl.max_tiles, gh); break;
      }
      in_b = !in_b;
      nd_count_launches((p == 0 && first_hist_done) ? 2 : 3);
      continue;
    }
    const size_t sm = (size_t)WARPS * bins * sizeof(uint32_t);
    switch (arr.nwords) {
      case 1: radix_scatter_kernel<1><<<grid, THREADS, sm, st>>>(cur, key_word, n_ptr, pl.shift[p], bins, drop, drop_key, scr->tile_hist, pl.max_tiles, gh); break;
      case 2: radix_scatter_kernel<2><<<grid, THREADS, sm, st>>>(cur, key_word, n_ptr, pl.shift[p], bins, drop, drop_key, scr->tile_hist, pl.max_tiles, gh); break;
      default: radix_scatter_kernel<3><<<grid, THREADS, sm, st>>>(cur, key_word, n_ptr, pl.shift[p], bins, drop, drop_key, scr->tile_hist, pl.max_tiles, gh); break;
    }
    in_b = !in_b;
    nd_count_launches((p == 0 && first_hist_done) ? 2 : 3);
  }
  ND_CUDA(cudaGetLastError());
  if (result_in_b) *result_in_b = in_b;
  return ND_OK;
}
