// Device-wide building blocks shared by the transposition and the graph-construction kernels:
// an exclusive scan of uint32 and one pass of a stable least-significant-digit radix sort
// (8-bit digits) of uint32 keys with a uint32 payload.  Every translation unit that includes
// this header gets its own copy of the kernels (internal linkage).
#pragma once
#include "common.cuh"

namespace gnn {

constexpr int kRadixBits = 8;
constexpr int kRadix = 1 << kRadixBits;
constexpr int kSortThreads = 256;
constexpr int kSortItems = 16;
constexpr int kSortTile = kSortThreads * kSortItems;  // 4096 keys per CTA
constexpr int kSortWarps = kSortThreads / 32;

constexpr int kScanThreads = 512;
constexpr int kScanItems = 8;
constexpr int kScanTile = kScanThreads * kScanItems;

// ---- exclusive scan of uint32 ------------------------------------------------

__device__ __forceinline__ unsigned block_exclusive_scan(unsigned v, unsigned* total) {
  __shared__ unsigned warp_tot[32];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  unsigned inc = v;
#pragma unroll
  for (int s = 1; s < 32; s <<= 1) {
    unsigned t = __shfl_up_sync(kFull, inc, s);
    if (lane >= s) inc += t;
  }
  if (lane == 31) warp_tot[w] = inc;
  __syncthreads();
  if (w == 0) {
    const int nw = blockDim.x >> 5;
    unsigned x = lane < nw ? warp_tot[lane] : 0u;
    unsigned xi = x;
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
      unsigned t = __shfl_up_sync(kFull, xi, s);
      if (lane >= s) xi += t;
    }
    warp_tot[lane] = xi - x;  // exclusive warp offsets
    if (lane == 31) *total = xi;
  }
  __syncthreads();
  const unsigned r = warp_tot[w] + inc - v;
  __syncthreads();
  return r;
}

static __global__ void __launch_bounds__(kScanThreads)
scan_tiles_kernel(unsigned* data, int64_t n, unsigned* tile_sums) {
  __shared__ unsigned total;
  const int64_t base = (int64_t)blockIdx.x * kScanTile + (int64_t)threadIdx.x * kScanItems;
  unsigned v[kScanItems];
  unsigned sum = 0;
#pragma unroll
  for (int j = 0; j < kScanItems; ++j) {
    v[j] = base + j < n ? data[base + j] : 0u;
    sum += v[j];
  }
  unsigned off = block_exclusive_scan(sum, &total);
#pragma unroll
  for (int j = 0; j < kScanItems; ++j) {
    if (base + j < n) data[base + j] = off;
    off += v[j];
  }
  if (threadIdx.x == 0) tile_sums[blockIdx.x] = total;
}

static __global__ void __launch_bounds__(kScanThreads)
scan_sums_kernel(unsigned* sums, int n) {
  __shared__ unsigned total;
  unsigned carry = 0;
  for (int base = 0; base < n; base += kScanThreads) {
    const int i = base + threadIdx.x;
    const unsigned v = i < n ? sums[i] : 0u;
    const unsigned off = block_exclusive_scan(v, &total);
    if (i < n) sums[i] = carry + off;
    carry += total;
    __syncthreads();
  }
}

static __global__ void __launch_bounds__(kScanThreads)
scan_add_kernel(unsigned* data, int64_t n, const unsigned* tile_sums) {
  const unsigned add = tile_sums[blockIdx.x];
  const int64_t base = (int64_t)blockIdx.x * kScanTile + (int64_t)threadIdx.x * kScanItems;
#pragma unroll
  for (int j = 0; j < kScanItems; ++j)
    if (base + j < n) data[base + j] += add;
}

inline void exclusive_scan_inplace(unsigned* data, int64_t n, unsigned* tile_sums, cudaStream_t st) {
  if (n <= 0) return;
  const int tiles = (int)((n + kScanTile - 1) / kScanTile);
  scan_tiles_kernel<<<tiles, kScanThreads, 0, st>>>(data, n, tile_sums);
  if (tiles > 1) {
    scan_sums_kernel<<<1, kScanThreads, 0, st>>>(tile_sums, tiles);
    scan_add_kernel<<<tiles, kScanThreads, 0, st>>>(data, n, tile_sums);
  }
}

// ---- radix passes --------------------------------------------------------------

static __global__ void __launch_bounds__(kSortThreads)
radix_hist_kernel(const unsigned* __restrict__ keys, int n, int shift,
                  unsigned* __restrict__ counts, int num_tiles) {
  __shared__ unsigned h[kRadix];
  h[threadIdx.x] = 0;
  __syncthreads();
  const int base = blockIdx.x * kSortTile;
#pragma unroll
  for (int i = 0; i < kSortItems; ++i) {
    const int idx = base + i * kSortThreads + threadIdx.x;
    if (idx < n) atomicAdd(&h[(keys[idx] >> shift) & (kRadix - 1)], 1u);
  }
  __syncthreads();
  counts[(size_t)threadIdx.x * num_tiles + blockIdx.x] = h[threadIdx.x];
}

// Stable scatter.  Tile order is (warp, iteration, lane); keys with equal digit
// keep that order: earlier warps first, then earlier iterations, then lower
// lanes (rank inside one iteration from match_any).
static __global__ void __launch_bounds__(kSortThreads)
radix_scatter_kernel(const unsigned* __restrict__ keys_in, const unsigned* __restrict__ vals_in,
                     unsigned* __restrict__ keys_out, unsigned* __restrict__ vals_out, int n,
                     int shift, const unsigned* __restrict__ bases, int num_tiles) {
  __shared__ unsigned wh[kSortWarps][kRadix];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < kSortWarps * kRadix; i += kSortThreads) (&wh[0][0])[i] = 0;
  __syncthreads();
  const int wbase = blockIdx.x * kSortTile + w * (kSortTile / kSortWarps);
  unsigned key[kSortItems];
  unsigned rank[kSortItems];
#pragma unroll
  for (int i = 0; i < kSortItems; ++i) {
    const int idx = wbase + i * 32 + lane;
    const bool valid = idx < n;
    key[i] = valid ? keys_in[idx] : 0u;
    const unsigned d = valid ? ((key[i] >> shift) & (kRadix - 1)) : (unsigned)(kRadix + lane);
    const unsigned peers = __match_any_sync(kFull, d);
    const unsigned below = __popc(peers & ((1u << lane) - 1u));
    const unsigned prev = valid ? wh[w][d] : 0u;
    __syncwarp();
    if (valid && below == 0) wh[w][d] = prev + __popc(peers);
    __syncwarp();
    rank[i] = prev + below;
  }
  __syncthreads();
  {
    const int d = threadIdx.x;  // kSortThreads == kRadix
    unsigned run = bases[(size_t)d * num_tiles + blockIdx.x];
#pragma unroll
    for (int ww = 0; ww < kSortWarps; ++ww) {
      const unsigned c = wh[ww][d];
      wh[ww][d] = run;
      run += c;
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < kSortItems; ++i) {
    const int idx = wbase + i * 32 + lane;
    if (idx < n) {
      const unsigned d = (key[i] >> shift) & (kRadix - 1);
      const unsigned dst = wh[w][d] + rank[i];
      keys_out[dst] = key[i];
      vals_out[dst] = vals_in ? vals_in[idx] : (unsigned)idx;
    }
  }
}

// Sorts (keys, vals) by the low `bits` bits of the keys with ceil(bits / 8) stable passes.
// keys_in / vals_in are read only (vals_in == nullptr: the payload is the position); the buffers
// a / b of each kind alternate, and the sorted arrays end up in *keys_sorted / *vals_sorted.
// counts: 256 * num_tiles words, sums: scan scratch (see sort_scratch_words).
inline void radix_sort_pairs(const unsigned* keys_in, const unsigned* vals_in, int n, int bits,
                             unsigned* keys_a, unsigned* keys_b, unsigned* vals_a, unsigned* vals_b,
                             unsigned* counts, unsigned* sums, const unsigned** keys_sorted,
                             const unsigned** vals_sorted, cudaStream_t stream) {
  const int num_tiles = n > 0 ? (n + kSortTile - 1) / kSortTile : 1;
  const size_t counts_elems = (size_t)kRadix * num_tiles;
  const int passes = (bits + kRadixBits - 1) / kRadixBits;
  for (int p = 0; p < passes && n > 0; ++p) {
    unsigned* keys_out = (p % 2 == 0) ? keys_a : keys_b;
    unsigned* vals_out = (p % 2 == 0) ? vals_a : vals_b;
    const int shift = p * kRadixBits;
    radix_hist_kernel<<<num_tiles, kSortThreads, 0, stream>>>(keys_in, n, shift, counts, num_tiles);
    exclusive_scan_inplace(counts, (int64_t)counts_elems, sums, stream);
    radix_scatter_kernel<<<num_tiles, kSortThreads, 0, stream>>>(keys_in, vals_in, keys_out, vals_out, n, shift,
                                                                 counts, num_tiles);
    keys_in = keys_out;
    vals_in = vals_out;
  }
  *keys_sorted = keys_in;
  *vals_sorted = vals_in;
}

inline int bits_for(int64_t n_values) {
  int bits = 1;
  while (bits < 31 && ((int64_t)1 << bits) < n_values) ++bits;
  return bits;
}

}  // namespace gnn
