// CSR -> CSC transpose as a stable least-significant-digit radix sort of the
// edges by column id, carrying the CSR edge position as int32 payload.
// Replaces the cuSPARSE call of the reference (src/csr2csc/csr2csc.cu:7-43,
// which carries the permutation as float32 and is exact only below 2^24 edges)
// and the host SciPy path of its scripts
// (script/train/train_gatconv_our.py:107-121).  Stability makes row ids ascend
// inside every column, i.e. the result equals scipy's csr_matrix.tocsc().
#include "../../include/gnn_b200.h"
#include "radix_sort.cuh"

using namespace gnn;

namespace {

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
