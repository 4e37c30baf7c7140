// CSR -> CSC transpose as a stable least-significant-digit radix sort of the
// edges by column id, carrying the CSR edge position as int32 payload.
// Replaces the cuSPARSE call of the reference (src/csr2csc/csr2csc.cu:7-43,
// which carries the permutation as float32 and is exact only below 2^24 edges)
// and the host SciPy path of its scripts
// (script/train/train_gatconv_our.py:107-121).  Stability makes row ids ascend
// inside every column, i.e. the result equals scipy's csr_matrix.tocsc().
#include "../../include/gnn_b200.h"
#include "common.cuh"

using namespace gnn;

namespace {

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

__global__ void __launch_bounds__(kScanThreads)
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

__global__ void __launch_bounds__(kScanThreads)
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

__global__ void __launch_bounds__(kScanThreads)
scan_add_kernel(unsigned* data, int64_t n, const unsigned* tile_sums) {
  const unsigned add = tile_sums[blockIdx.x];
  const int64_t base = (int64_t)blockIdx.x * kScanTile + (int64_t)threadIdx.x * kScanItems;
#pragma unroll
  for (int j = 0; j < kScanItems; ++j)
    if (base + j < n) data[base + j] += add;
}

void exclusive_scan_inplace(unsigned* data, int64_t n, unsigned* tile_sums, cudaStream_t st) {
  if (n <= 0) return;
  const int tiles = (int)((n + kScanTile - 1) / kScanTile);
  scan_tiles_kernel<<<tiles, kScanThreads, 0, st>>>(data, n, tile_sums);
  if (tiles > 1) {
    scan_sums_kernel<<<1, kScanThreads, 0, st>>>(tile_sums, tiles);
    scan_add_kernel<<<tiles, kScanThreads, 0, st>>>(data, n, tile_sums);
  }
}

// ---- radix passes --------------------------------------------------------------

__global__ void __launch_bounds__(kSortThreads)
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
__global__ void __launch_bounds__(kSortThreads)
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

// ---- segment ids, column pointers, row gather ------------------------------------

__global__ void __launch_bounds__(kThreadsPerCta)
expand_seg_ids_kernel(ChunkGeom g, int* __restrict__ seg_of) {
  const int lane = threadIdx.x & 31;
  const int chunk_id = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (chunk_id >= g.num_chunks) return;
  for_each_piece(g, chunk_id, [&](int s, int a, int b, bool, bool) {
    for (int e = a + lane; e < b; e += 32) seg_of[e] = s;
  });
}

__global__ void build_ptr_from_sorted_kernel(const unsigned* __restrict__ sorted, int n,
                                             int ncols, int* __restrict__ col_ptr) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i > n) return;
  int prev = i == 0 ? -1 : (int)sorted[i - 1];
  int cur = i == n ? ncols : (int)sorted[i];
  if (cur > ncols) cur = ncols;
  if (prev >= ncols) prev = ncols - 1;
  for (int c = prev + 1; c <= cur; ++c) col_ptr[c] = i;
}

__global__ void gather_rows_kernel(const int* __restrict__ seg_of, const int* __restrict__ permute,
                                   int n, int* __restrict__ row_ind) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) row_ind[i] = seg_of[permute[i]];
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

struct SortLayout {
  int num_tiles;
  size_t counts_elems;
  int scan_tiles;
  size_t off_keys_a, off_keys_b, off_vals_t, off_seg, off_counts, off_sums, total;
};

SortLayout layout_for(int64_t nnz) {
  SortLayout L;
  L.num_tiles = (int)((nnz + kSortTile - 1) / kSortTile);
  if (L.num_tiles < 1) L.num_tiles = 1;
  L.counts_elems = (size_t)kRadix * L.num_tiles;
  L.scan_tiles = (int)((L.counts_elems + kScanTile - 1) / kScanTile);
  size_t o = 0;
  const size_t eb = align_up((size_t)(nnz > 0 ? nnz : 1) * 4, 256);
  L.off_keys_a = o; o += eb;
  L.off_keys_b = o; o += eb;
  L.off_vals_t = o; o += eb;
  L.off_seg = o; o += eb;
  L.off_counts = o; o += align_up(L.counts_elems * 4, 256);
  L.off_sums = o; o += align_up((size_t)L.scan_tiles * 4, 256);
  L.total = o + 256;
  return L;
}

int bad(const char* m) {
  set_last_error(m);
  return GNN_ERR_INVALID_ARG;
}

}  // namespace

extern "C" int gnn_csr2csc_workspace_bytes(int64_t nnz, size_t* bytes) {
  if (!bytes || nnz < 0) return bad("gnn_csr2csc_workspace_bytes: bad argument");
  *bytes = layout_for(nnz).total;
  return GNN_OK;
}

extern "C" int gnn_csr2csc(const int* row_ptr, const int* col_ind, int64_t n_rows,
                           int64_t n_cols, int64_t nnz, int* col_ptr, int* row_ind,
                           int* permute, void* workspace, size_t workspace_bytes,
                           cudaStream_t stream) {
  if (n_rows < 0 || n_cols < 0 || nnz < 0) return bad("gnn_csr2csc: negative size");
  if (n_rows > INT32_MAX - 1 || n_cols > INT32_MAX - 1 || nnz > INT32_MAX - 4096)
    return bad("gnn_csr2csc: size exceeds int32 indexing");
  if (!row_ptr || !col_ptr || (nnz && (!col_ind || !row_ind || !permute)))
    return bad("gnn_csr2csc: null pointer");
  const SortLayout L = layout_for(nnz);
  if (!workspace || workspace_bytes < L.total) {
    set_last_error("gnn_csr2csc: workspace too small");
    return GNN_ERR_WORKSPACE;
  }
  char* base = (char*)align_up((uintptr_t)workspace, 256);
  unsigned* keys_a = (unsigned*)(base + L.off_keys_a);
  unsigned* keys_b = (unsigned*)(base + L.off_keys_b);
  unsigned* vals_t = (unsigned*)(base + L.off_vals_t);
  int* seg_of = (int*)(base + L.off_seg);
  unsigned* counts = (unsigned*)(base + L.off_counts);
  unsigned* sums = (unsigned*)(base + L.off_sums);
  const int n = (int)nnz;

  int bits = 1;
  while (bits < 31 && ((int64_t)1 << bits) < n_cols) ++bits;
  const int passes = (bits + kRadixBits - 1) / kRadixBits;

  const unsigned* keys_in = (const unsigned*)col_ind;
  const unsigned* vals_in = nullptr;
  const unsigned* sorted = keys_in;
  if (n > 0) {
    for (int p = 0; p < passes; ++p) {
      unsigned* keys_out = (p % 2 == 0) ? keys_a : keys_b;
      unsigned* vals_out = ((passes - 1 - p) % 2 == 0) ? (unsigned*)permute : vals_t;
      const int shift = p * kRadixBits;
      radix_hist_kernel<<<L.num_tiles, kSortThreads, 0, stream>>>(keys_in, n, shift, counts, L.num_tiles);
      exclusive_scan_inplace(counts, (int64_t)L.counts_elems, sums, stream);
      radix_scatter_kernel<<<L.num_tiles, kSortThreads, 0, stream>>>(
          keys_in, vals_in, keys_out, vals_out, n, shift, counts, L.num_tiles);
      keys_in = keys_out;
      vals_in = vals_out;
    }
    sorted = keys_in;
    const int chunk = pick_chunk(nnz);
    ChunkGeom g{row_ptr, col_ind, (int)n_rows, n, chunk, num_chunks_for(nnz, chunk)};
    expand_seg_ids_kernel<<<(g.num_chunks + kWarpsPerCta - 1) / kWarpsPerCta, kThreadsPerCta, 0, stream>>>(g, seg_of);
    gather_rows_kernel<<<(n + 255) / 256, 256, 0, stream>>>(seg_of, permute, n, row_ind);
  }
  build_ptr_from_sorted_kernel<<<(n + 1 + 255) / 256, 256, 0, stream>>>(sorted, n, (int)n_cols, col_ptr);
  return check_launch("gnn_csr2csc");
}
