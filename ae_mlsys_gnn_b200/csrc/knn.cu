// k-nearest-neighbour graph of a batch of point clouds, the step in front of EdgeConv.
//
// The reference builds it with DGL's KNNGraph(k) on the host side of every layer
// (script/train/train_edgeconv_our.py:20,52); a framework formulation (pairwise distance
// matrix + top-k) writes B x P x P distances.  Here one thread owns one query point, walks
// the points of its cloud through shared-memory tiles and keeps its k best candidates in a
// sorted list: nothing of size P x P is ever stored.
//
// Contract (what the CPU oracle restates): squared Euclidean distance accumulated in float64
// over the coordinates in ascending order, each term rounded separately
// (d += (a-b)*(a-b), no fused multiply-add); neighbours sorted by (distance, index), i.e. among
// equal distances the lower point index comes first, so the point itself is its own first
// neighbour; src_ind[(b*P + i)*k + j] = b*P + (index of the j-th nearest point of cloud b),
// the layout gnn_edgeconv_fwd reads (src/fused_edgeconv/fused_edgeconv.cu:29-30).
#include "../../include/gnn_b200.h"
#include "common.cuh"

using namespace gnn;

namespace {

constexpr int kKnnThreads = 128;
constexpr int kKnnMaxK = 64;
constexpr int kKnnTileFloats = 6144;  // 24 KB of candidate coordinates per tile

int bad(const char* m) {
  set_last_error(m);
  return GNN_ERR_INVALID_ARG;
}

// CREG > 0: the query's coordinates stay in registers (C == CREG); 0: read from memory.
template <int CREG>
__global__ void __launch_bounds__(kKnnThreads)
knn_kernel(const float* __restrict__ pts, int P, int C, int k, int tile_pts, int* __restrict__ src_ind) {
  extern __shared__ float tile[];  // [tile_pts][C]
  const int cloud = blockIdx.y;
  const int i = blockIdx.x * kKnnThreads + threadIdx.x;  // query point inside the cloud
  const bool active = i < P;
  const float* cp = pts + (size_t)cloud * P * C;
  const float* qrow = cp + (size_t)(active ? i : 0) * C;
  float qreg[CREG > 0 ? CREG : 1];
  if (CREG > 0) {
#pragma unroll
    for (int c = 0; c < CREG; ++c) qreg[c] = __ldg(qrow + c);
  }
  double bd[kKnnMaxK];
  int bi[kKnnMaxK];
  int cnt = 0;
  double worst = 0.0;

  for (int base = 0; base < P; base += tile_pts) {
    const int np = min(tile_pts, P - base);
    __syncthreads();
    for (int t = threadIdx.x; t < np * C; t += kKnnThreads) tile[t] = __ldg(cp + (size_t)base * C + t);
    __syncthreads();
    if (!active) continue;
    for (int j = 0; j < np; ++j) {
      const float* cand = tile + j * C;
      double d = 0.0;
      if (CREG > 0) {
#pragma unroll
        for (int c = 0; c < CREG; ++c) {
          const double df = (double)qreg[c] - (double)cand[c];
          d = __dadd_rn(d, __dmul_rn(df, df));
        }
      } else {
        for (int c = 0; c < C; ++c) {
          const double df = (double)__ldg(qrow + c) - (double)cand[c];
          d = __dadd_rn(d, __dmul_rn(df, df));
        }
      }
      if (cnt == k && !(d < worst)) continue;  // candidates come in index order: ties keep the earlier one
      int pos = cnt < k ? cnt : k - 1;
      while (pos > 0 && bd[pos - 1] > d) {
        bd[pos] = bd[pos - 1];
        bi[pos] = bi[pos - 1];
        --pos;
      }
      bd[pos] = d;
      bi[pos] = base + j;
      if (cnt < k) ++cnt;
      worst = bd[cnt - 1];
    }
  }
  if (active) {
    int* out = src_ind + ((size_t)cloud * P + i) * k;
    for (int j = 0; j < k; ++j) out[j] = cloud * P + bi[j];
  }
}

}  // namespace

extern "C" int gnn_knn_graph(const float* points, int64_t n_clouds, int64_t n_points, int n_coords, int k,
                             int* src_ind, cudaStream_t stream) {
  if (n_clouds < 0 || n_points < 0 || n_coords <= 0 || k <= 0) return bad("gnn_knn_graph: bad size");
  if (k > kKnnMaxK) {
    set_last_error("gnn_knn_graph: k > 64 is not supported");
    return GNN_ERR_UNSUPPORTED;
  }
  if (k > n_points && n_clouds > 0) return bad("gnn_knn_graph: k exceeds the number of points of a cloud");
  if (n_clouds == 0 || n_points == 0) return GNN_OK;
  if (!points || !src_ind) return bad("gnn_knn_graph: null pointer");
  if (n_clouds > 65535 || n_clouds * n_points > INT32_MAX || n_coords > kKnnTileFloats)
    return bad("gnn_knn_graph: size exceeds the supported range");
  const int P = (int)n_points, C = n_coords;
  int tile_pts = kKnnTileFloats / C;
  if (tile_pts > P) tile_pts = P;
  const size_t smem = (size_t)tile_pts * C * sizeof(float);
  dim3 grid((P + kKnnThreads - 1) / kKnnThreads, (unsigned)n_clouds);
#define GNN_KNN(CR) knn_kernel<CR><<<grid, kKnnThreads, smem, stream>>>(points, P, C, k, tile_pts, src_ind)
  switch (C) {
    case 2: GNN_KNN(2); break;
    case 3: GNN_KNN(3); break;
    case 4: GNN_KNN(4); break;
    default: GNN_KNN(0); break;
  }
#undef GNN_KNN
  return check_launch("gnn_knn_graph");
}
