// Graph construction on the device: the steps in front of the fused kernels that the
// reference's scripts do on the host with DGL and SciPy
// (script/train/train_gatconv_our.py:82-95: remove_self_loop / add_self_loop, edges ->
// scipy.sparse.csr_matrix -> indptr / indices; train_gmmconv_our.py:80-93,124-130), and the
// bookkeeping of the row-block partition that has no counterpart there (single GPU).
//
//   gnn_coo_to_csr            (dst, src) pairs -> in-edge CSR sorted by (dst, src), duplicates
//                             removed, optionally self-loops replaced by exactly one per node:
//                             two stable radix sorts (by src, then by dst), head flags, scan,
//                             compaction.  The result equals scipy's csr_matrix(...) with
//                             sum_duplicates() / sorted indices, bit for bit.
//   gnn_edge_balanced_bounds  row-block boundaries with about nnz / parts edges per block.
//   gnn_halo_needs            for every block q the set of ids its edges reference outside the
//                             block, as flags scanned into positions (one pass over the edges).
//   gnn_compact_flagged       the sorted id lists behind those flags.
//   gnn_halo_remap            ids of one block's edges -> [own rows | halo rows] index space.
#include "../../include/gnn_b200.h"
#include "radix_sort.cuh"

using namespace gnn;

namespace {

int bad(const char* m) {
  set_last_error(m);
  return GNN_ERR_INVALID_ARG;
}
size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Pairs to sort: the m given ones (dropped, i.e. given the sentinel destination n that sorts
// last, when an endpoint is out of range or -- with self_loops -- when dst == src) followed by
// one (i, i) per node when self_loops is set.
__global__ void stage_pairs_kernel(const int* __restrict__ dst, const int* __restrict__ src, int64_t m, int n,
                                   int self_loops, unsigned* __restrict__ kd, unsigned* __restrict__ ks) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = m + (self_loops ? n : 0);
  if (i >= total) return;
  if (i < m) {
    const int d = dst[i], s = src[i];
    const bool ok = d >= 0 && d < n && s >= 0 && s < n && !(self_loops && d == s);
    kd[i] = ok ? (unsigned)d : (unsigned)n;
    ks[i] = ok ? (unsigned)s : 0u;
  } else {
    kd[i] = ks[i] = (unsigned)(i - m);
  }
}

// flag[i] = 1 for the first of every run of equal (dst, src) among the valid pairs.
__global__ void head_flags_kernel(const unsigned* __restrict__ kd, const unsigned* __restrict__ ks, int64_t total,
                                  int n, unsigned* __restrict__ flag) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i > total) return;
  if (i == total) { flag[i] = 0; return; }  // one extra slot: the scan leaves the count there
  const bool valid = kd[i] < (unsigned)n;
  flag[i] = (valid && (i == 0 || kd[i] != kd[i - 1] || ks[i] != ks[i - 1])) ? 1u : 0u;
}

// pos = exclusive scan of the head flags (pos[total] = number of unique edges).
__global__ void compact_edges_kernel(const unsigned* __restrict__ kd, const unsigned* __restrict__ ks,
                                     const unsigned* __restrict__ pos, int64_t total, int n,
                                     int* __restrict__ col_ind, int* __restrict__ row_ptr,
                                     long long* __restrict__ nnz_out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i > total) return;
  if (i == total) {
    *nnz_out = (long long)pos[total];  // the extra slot of the scan: number of unique edges
    return;
  }
  const unsigned d = kd[i];
  if (d >= (unsigned)n) return;
  const bool head = pos[i + 1] != pos[i];
  if (!head) return;
  const unsigned p = pos[i];
  col_ind[p] = (int)ks[i];
  // row_ptr[r] = number of unique edges with destination < r: this head is the first edge of
  // row d exactly when the previous valid pair has a smaller destination
  const int prev = i == 0 ? -1 : (int)kd[i - 1];
  if (prev != (int)d)
    for (int r = prev + 1; r <= (int)d; ++r) row_ptr[r] = (int)p;
}

// Rows behind the last non-empty one (and row n) point at the end.
__global__ void finish_row_ptr_kernel(const unsigned* __restrict__ kd, const unsigned* __restrict__ pos,
                                      int64_t total, int n, int* __restrict__ row_ptr) {
  // last valid destination: binary search for the first sentinel in the sorted keys
  int64_t lo = 0, hi = total;
  while (lo < hi) {
    const int64_t mid = (lo + hi) >> 1;
    if (kd[mid] < (unsigned)n) lo = mid + 1; else hi = mid;
  }
  const int last = lo == 0 ? -1 : (int)kd[lo - 1];
  const int cnt = (int)pos[total];
  for (int r = last + 1 + (int)threadIdx.x + (int)blockIdx.x * (int)blockDim.x; r <= n;
       r += (int)(blockDim.x * gridDim.x))
    row_ptr[r] = cnt;
}

struct CooLayout {
  size_t off_kd_a, off_kd_b, off_ks_a, off_ks_b, off_flag, off_counts, off_sums, total;
};

CooLayout coo_layout(int64_t total) {
  CooLayout L;
  const size_t eb = align_up((size_t)(total + 1) * 4, 256);
  const int num_tiles = (int)((total + kSortTile - 1) / kSortTile) + 1;
  const size_t counts_elems = (size_t)kRadix * num_tiles;
  const size_t scan_elems = counts_elems > (size_t)(total + 1) ? counts_elems : (size_t)(total + 1);
  const int scan_tiles = (int)((scan_elems + kScanTile - 1) / kScanTile) + 1;
  size_t o = 0;
  L.off_kd_a = o; o += eb;
  L.off_kd_b = o; o += eb;
  L.off_ks_a = o; o += eb;
  L.off_ks_b = o; o += eb;
  L.off_flag = o; o += eb;
  L.off_counts = o; o += align_up(counts_elems * 4, 256);
  L.off_sums = o; o += align_up((size_t)scan_tiles * 4, 256);
  L.total = o + 256;
  return L;
}

__global__ void bounds_kernel(const int* __restrict__ row_ptr, int n, int parts, int* __restrict__ bounds) {
  const int g = threadIdx.x;
  if (g > parts) return;
  const long long nnz = row_ptr[n];
  int cut;
  if (g == 0) cut = 0;
  else if (g == parts) cut = n;
  else {
    const long long target = (g * nnz) / parts;
    int lo = 0, hi = n;  // first row whose start is at or after the target
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if ((long long)row_ptr[mid] < target) lo = mid + 1; else hi = mid;
    }
    cut = lo;
  }
  bounds[g] = cut;
}

__device__ __forceinline__ int block_of(const int* __restrict__ bounds, int world, int row) {
  int q = 0;
  for (int k = 1; k < world; ++k)
    if (row >= bounds[k]) q = k;
  return q;
}

__global__ void __launch_bounds__(kThreadsPerCta)
halo_mark_kernel(ChunkGeom g, const int* __restrict__ bounds, int world, unsigned* __restrict__ flags) {
  const int lane = threadIdx.x & 31;
  const int chunk_id = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (chunk_id >= g.num_chunks) return;
  for_each_piece(g, chunk_id, [&](int s, int a, int b, bool, bool) {
    const int q = block_of(bounds, world, s);
    const int lo = bounds[q], hi = bounds[q + 1];
    for (int e = a + lane; e < b; e += 32) {
      const int v = __ldg(g.idx + e);
      if (v < lo || v >= hi) flags[(size_t)q * g.nseg + v] = 1u;  // racing writers store the same value
    }
  });
}

__global__ void compact_flagged_kernel(const unsigned* __restrict__ pos, int64_t n, int64_t period,
                                       int* __restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  if (pos[i + 1] != pos[i]) out[pos[i]] = (int)(i % period);
}

__global__ void halo_remap_kernel(const int* __restrict__ idx, int64_t nnz, int lo, int hi,
                                  const unsigned* __restrict__ pos, int* __restrict__ ext) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= nnz) return;
  const int v = idx[e];
  ext[e] = (v >= lo && v < hi) ? v - lo : (hi - lo) + (int)(pos[v] - pos[0]);
}

}  // namespace

extern "C" int gnn_coo_to_csr_workspace_bytes(int64_t n_pairs, int64_t n_nodes, size_t* bytes) {
  if (!bytes || n_pairs < 0 || n_nodes < 0) return bad("gnn_coo_to_csr_workspace_bytes: bad argument");
  *bytes = coo_layout(n_pairs + n_nodes).total;
  return GNN_OK;
}

extern "C" int gnn_coo_to_csr(const int* dst, const int* src, int64_t n_pairs, int64_t n_nodes, int self_loops,
                              int* row_ptr, int* col_ind, long long* nnz_out, void* workspace,
                              size_t workspace_bytes, cudaStream_t stream) {
  if (n_pairs < 0 || n_nodes < 0) return bad("gnn_coo_to_csr: negative size");
  const int64_t total = n_pairs + (self_loops ? n_nodes : 0);
  if (n_nodes > INT32_MAX - 2 || total > INT32_MAX - 4096) return bad("gnn_coo_to_csr: size exceeds int32 indexing");
  if (!row_ptr || !nnz_out || (n_pairs && (!dst || !src)) || (total && !col_ind))
    return bad("gnn_coo_to_csr: null pointer");
  const CooLayout L = coo_layout(n_pairs + n_nodes);
  if (!workspace || workspace_bytes < L.total) {
    set_last_error("gnn_coo_to_csr: workspace too small");
    return GNN_ERR_WORKSPACE;
  }
  char* base = (char*)align_up((uintptr_t)workspace, 256);
  unsigned* kd_a = (unsigned*)(base + L.off_kd_a);
  unsigned* kd_b = (unsigned*)(base + L.off_kd_b);
  unsigned* ks_a = (unsigned*)(base + L.off_ks_a);
  unsigned* ks_b = (unsigned*)(base + L.off_ks_b);
  unsigned* flag = (unsigned*)(base + L.off_flag);
  unsigned* counts = (unsigned*)(base + L.off_counts);
  unsigned* sums = (unsigned*)(base + L.off_sums);
  const int n = (int)n_nodes;
  const int T = (int)total;
  const unsigned grid = (unsigned)((total + 1 + 255) / 256);
  if (total > 0)
    stage_pairs_kernel<<<grid, 256, 0, stream>>>(dst, src, n_pairs, n, self_loops ? 1 : 0, kd_a, ks_a);
  const int bits = bits_for(n_nodes + 1);  // the sentinel destination n is a key value too
  // stable sort by source (payload: destination), then by destination (payload: source)
  const unsigned *k1, *v1, *k2, *v2;
  radix_sort_pairs(ks_a, kd_a, T, bits, ks_b, ks_a, kd_b, kd_a, counts, sums, &k1, &v1, stream);
  // k1 = sources sorted, v1 = their destinations; the buffers not holding them are free
  unsigned* free_k = (k1 == ks_a) ? ks_b : ks_a;
  unsigned* free_v = (v1 == kd_a) ? kd_b : kd_a;
  // second sort: keys = destinations (v1), payload = sources (k1)
  unsigned* kdo_a = free_v;                       // destinations ping
  unsigned* kdo_b = const_cast<unsigned*>(v1);    // destinations pong (overwritten from pass 2 on: v1 is consumed by pass 1)
  unsigned* kso_a = free_k;
  unsigned* kso_b = const_cast<unsigned*>(k1);
  radix_sort_pairs(v1, k1, T, bits, kdo_a, kdo_b, kso_a, kso_b, counts, sums, &k2, &v2, stream);
  // k2 = destinations ascending, v2 = sources ascending inside a destination
  head_flags_kernel<<<grid, 256, 0, stream>>>(k2, v2, total, n, flag);
  exclusive_scan_inplace(flag, total + 1, sums, stream);
  compact_edges_kernel<<<grid, 256, 0, stream>>>(k2, v2, flag, total, n, col_ind, row_ptr, nnz_out);
  finish_row_ptr_kernel<<<(unsigned)((n_nodes + 1 + 255) / 256 < 1024 ? (n_nodes + 1 + 255) / 256 : 1024), 256, 0, stream>>>(
      k2, flag, total, n, row_ptr);
  return check_launch("gnn_coo_to_csr");
}

extern "C" int gnn_edge_balanced_bounds(const int* row_ptr, int64_t n_rows, int parts, int* bounds,
                                        cudaStream_t stream) {
  if (n_rows < 0 || parts < 1 || parts > 1023) return bad("gnn_edge_balanced_bounds: bad argument");
  if (n_rows > INT32_MAX - 1) return bad("gnn_edge_balanced_bounds: size exceeds int32 indexing");
  if (!row_ptr || !bounds) return bad("gnn_edge_balanced_bounds: null pointer");
  bounds_kernel<<<1, 1024, 0, stream>>>(row_ptr, (int)n_rows, parts, bounds);
  return check_launch("gnn_edge_balanced_bounds");
}

extern "C" int gnn_halo_needs_workspace_bytes(int64_t n_nodes, int world, size_t* bytes) {
  if (!bytes || n_nodes < 0 || world < 1) return bad("gnn_halo_needs_workspace_bytes: bad argument");
  const size_t elems = (size_t)n_nodes * world + 1;
  *bytes = align_up(((elems + kScanTile - 1) / kScanTile + 1) * 4, 256) + 256;
  return GNN_OK;
}

extern "C" int gnn_halo_needs(const int* ptr, const int* idx, int64_t n_nodes, int64_t nnz, const int* bounds,
                              int world, unsigned* positions, void* workspace, size_t workspace_bytes,
                              cudaStream_t stream) {
  if (n_nodes < 0 || nnz < 0 || world < 1) return bad("gnn_halo_needs: bad argument");
  if (n_nodes > INT32_MAX - 1 || nnz > INT32_MAX - 4096 || (int64_t)n_nodes * world > INT32_MAX - 4096)
    return bad("gnn_halo_needs: size exceeds int32 indexing");
  if (!ptr || (!idx && nnz) || !bounds || !positions) return bad("gnn_halo_needs: null pointer");
  size_t need = 0;
  gnn_halo_needs_workspace_bytes(n_nodes, world, &need);
  if (!workspace || workspace_bytes < need) {
    set_last_error("gnn_halo_needs: workspace too small");
    return GNN_ERR_WORKSPACE;
  }
  const int64_t elems = n_nodes * world + 1;
  if (cudaMemsetAsync(positions, 0, (size_t)elems * 4, stream) != cudaSuccess) {
    set_last_error("gnn_halo_needs: memset failed");
    return GNN_ERR_CUDA;
  }
  if (nnz > 0) {
    const int chunk = pick_chunk(nnz);
    ChunkGeom g{ptr, idx, (int)n_nodes, (int)nnz, chunk, num_chunks_for(nnz, chunk)};
    halo_mark_kernel<<<(g.num_chunks + kWarpsPerCta - 1) / kWarpsPerCta, kThreadsPerCta, 0, stream>>>(
        g, bounds, world, positions);
  }
  exclusive_scan_inplace(positions, elems, (unsigned*)align_up((uintptr_t)workspace, 256), stream);
  return check_launch("gnn_halo_needs");
}

extern "C" int gnn_compact_flagged(const unsigned* positions, int64_t n, int64_t period, int* out,
                                   cudaStream_t stream) {
  if (n < 0 || period <= 0) return bad("gnn_compact_flagged: bad argument");
  if (n == 0) return GNN_OK;
  if (!positions || !out) return bad("gnn_compact_flagged: null pointer");
  compact_flagged_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(positions, n, period, out);
  return check_launch("gnn_compact_flagged");
}

extern "C" int gnn_halo_remap(const int* idx, int64_t nnz, int lo, int hi, const unsigned* positions_of_rank,
                              int* ext, cudaStream_t stream) {
  if (nnz < 0 || lo < 0 || hi < lo) return bad("gnn_halo_remap: bad argument");
  if (nnz == 0) return GNN_OK;
  if (!idx || !positions_of_rank || !ext) return bad("gnn_halo_remap: null pointer");
  halo_remap_kernel<<<(unsigned)((nnz + 255) / 256), 256, 0, stream>>>(idx, nnz, lo, hi, positions_of_rank, ext);
  return check_launch("gnn_halo_remap");
}
