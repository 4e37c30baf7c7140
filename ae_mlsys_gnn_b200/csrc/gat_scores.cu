// Attention scores of a GAT layer and their backward, each as ONE pass over the
// projected features instead of the chain of elementwise / reduction kernels the
// reference layer leaves to the framework (layers/gatconv_layer.py:52-53:
// attn_row = (attn_l * h).sum(-1), attn_col = (attn_r * h).sum(-1), and autograd's
// backward of those two lines).
//
//  forward : attn_row[n,h] = <attn_l[h,:], feat[n,h,:]>, attn_col[n,h] = <attn_r[h,:], feat[n,h,:]>
//  backward: grad_feat[n,h,:] += grad_attn_row[n,h] * attn_l[h,:] + grad_attn_col[n,h] * attn_r[h,:]
//            grad_attn_l[h,:] = sum_n grad_attn_row[n,h] * feat[n,h,:]   (same for r / col)
// The sums over nodes are reduced per CTA in a fixed order and then over CTAs in
// block order by a second kernel: deterministic, no atomics.
#include "../../include/gnn_b200.h"
#include "wgather.cuh"

using namespace gnn;

namespace {

constexpr int kScoreBlocks = 148 * 4;

template <int HP, int Q, bool VEC>
__global__ void __launch_bounds__(kThreadsPerCta)
gat_scores_fwd_kernel(int64_t n, int H, int F, const float* __restrict__ feat,
                      const float* __restrict__ attn_l, const float* __restrict__ attn_r,
                      float* __restrict__ attn_row, float* __restrict__ attn_col) {
  constexpr int VW = VEC ? 4 : 1;
  constexpr int V = 2 * HP;
  constexpr int LPV = 32 / V;
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerCta;
  const int width = H * F;
  RowTile<Q, VEC> t;
  t.init(lane, width, F, H);
  float al[Q][VW], ar[Q][VW];
  t.load(attn_l, lane, al);
  t.load(attn_r, lane, ar);
  for (int64_t r = warp; r < n; r += nwarps) {
    float v[Q][VW];
    t.load(feat + r * width, lane, v);
    float p[V];
#pragma unroll
    for (int i = 0; i < V; ++i) p[i] = 0.f;
#pragma unroll
    for (int q = 0; q < Q; ++q) {
      float dl = 0.f, dr = 0.f;
#pragma unroll
      for (int i = 0; i < VW; ++i) {
        dl = fmaf(al[q][i], v[q][i], dl);
        dr = fmaf(ar[q][i], v[q][i], dr);
      }
#pragma unroll
      for (int h = 0; h < HP; ++h)
        if (t.head[q] == h) { p[h] += dl; p[HP + h] += dr; }
    }
    warp_multi_sum<V>(p, lane);
    if ((lane & (LPV - 1)) == 0) {
      const int idx = lane / LPV;
      if (idx < HP) { if (idx < H) attn_row[r * H + idx] = p[0]; }
      else if (idx - HP < H) attn_col[r * H + (idx - HP)] = p[0];
    }
  }
}

template <int HP, int Q, bool VEC>
__global__ void __launch_bounds__(kThreadsPerCta)
gat_scores_bwd_kernel(int64_t n, int H, int F, const float* __restrict__ feat,
                      const float* __restrict__ attn_l, const float* __restrict__ attn_r,
                      const float* __restrict__ grad_attn_row, const float* __restrict__ grad_attn_col,
                      float* __restrict__ grad_feat, float* __restrict__ partial) {
  constexpr int VW = VEC ? 4 : 1;
  constexpr int TW = Q * 32 * VW;  // floats covered by one tile
  __shared__ float red[kWarpsPerCta][2 * TW];
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  const int64_t warp = (int64_t)blockIdx.x * kWarpsPerCta + wib;
  const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerCta;
  const int width = H * F;
  RowTile<Q, VEC> t;
  t.init(lane, width, F, H);
  float accl[Q][VW], accr[Q][VW];
  t.zero(accl);
  t.zero(accr);
  for (int64_t r = warp; r < n; r += nwarps) {
    float v[Q][VW], gf[Q][VW], al[Q][VW], ar[Q][VW];
    t.load(feat + r * width, lane, v);
    t.load(grad_feat + r * width, lane, gf);
    t.load(attn_l, lane, al);
    t.load(attn_r, lane, ar);
#pragma unroll
    for (int q = 0; q < Q; ++q) {
      const float gr = __ldg(grad_attn_row + r * H + t.head[q]);
      const float gc = __ldg(grad_attn_col + r * H + t.head[q]);
#pragma unroll
      for (int i = 0; i < VW; ++i) {
        gf[q][i] = fmaf(gr, al[q][i], fmaf(gc, ar[q][i], gf[q][i]));
        accl[q][i] = fmaf(gr, v[q][i], accl[q][i]);
        accr[q][i] = fmaf(gc, v[q][i], accr[q][i]);
      }
    }
    t.store(grad_feat + r * width, lane, gf);
  }
  // CTA reduction in warp order, then one partial row per CTA
#pragma unroll
  for (int q = 0; q < Q; ++q)
#pragma unroll
    for (int i = 0; i < VW; ++i) {
      const int e = (lane + 32 * q) * VW + i;
      red[wib][e] = accl[q][i];
      red[wib][TW + e] = accr[q][i];
    }
  __syncthreads();
  for (int e = threadIdx.x; e < 2 * TW; e += kThreadsPerCta) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kWarpsPerCta; ++w) s += red[w][e];
    const int which = e / TW, pos = e % TW;
    if (pos < width) partial[((size_t)blockIdx.x * 2 + which) * width + pos] = s;
  }
}

__global__ void gat_scores_reduce_kernel(int nblocks, int width, const float* __restrict__ partial,
                                         float* __restrict__ grad_attn_l, float* __restrict__ grad_attn_r) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= 2 * width) return;
  const int which = e / width, pos = e % width;
  float s = 0.f;
  for (int b = 0; b < nblocks; ++b) s += partial[((size_t)b * 2 + which) * width + pos];
  (which == 0 ? grad_attn_l : grad_attn_r)[pos] = s;
}

int bad(const char* m) {
  set_last_error(m);
  return GNN_ERR_INVALID_ARG;
}

int score_blocks(int64_t n) {
  int64_t b = (n + kWarpsPerCta - 1) / kWarpsPerCta;
  if (b > kScoreBlocks) b = kScoreBlocks;
  if (b < 1) b = 1;
  return (int)b;
}

bool shape_ok(int H, int F, bool vec) { return H <= 8 && (int64_t)H * F <= max_tile_width(vec); }

}  // namespace

extern "C" int gnn_gat_scores_fwd(const float* feat, const float* attn_l, const float* attn_r,
                                  int64_t n, int H, int F, float* attn_row, float* attn_col,
                                  cudaStream_t stream) {
  if (n < 0 || H <= 0 || F <= 0) return bad("gnn_gat_scores_fwd: bad size");
  if (n == 0) return GNN_OK;
  if (!feat || !attn_l || !attn_r || !attn_row || !attn_col) return bad("gnn_gat_scores_fwd: null pointer");
  const bool vec = F % 4 == 0 && aligned16(feat) && aligned16(attn_l) && aligned16(attn_r);
  if (!shape_ok(H, F, vec)) {
    set_last_error("gnn_gat_scores_fwd: H > 8 or H*F beyond the largest tile");
    return GNN_ERR_UNSUPPORTED;
  }
  const int blocks = score_blocks(n);
  dispatch_tile(next_pow2(H), H * F, vec, [&](auto hp, auto q, auto v) {
    gat_scores_fwd_kernel<decltype(hp)::value, decltype(q)::value, decltype(v)::value>
        <<<blocks, kThreadsPerCta, 0, stream>>>(n, H, F, feat, attn_l, attn_r, attn_row, attn_col);
  });
  return check_launch("gnn_gat_scores_fwd");
}

extern "C" int gnn_gat_scores_bwd_workspace_bytes(int64_t n, int H, int F, size_t* bytes) {
  if (!bytes || n < 0 || H <= 0 || F <= 0) return bad("gnn_gat_scores_bwd_workspace_bytes: bad argument");
  *bytes = (size_t)kScoreBlocks * 2 * H * F * sizeof(float) + 256;
  return GNN_OK;
}

extern "C" int gnn_gat_scores_bwd(const float* feat, const float* attn_l, const float* attn_r,
                                  const float* grad_attn_row, const float* grad_attn_col, int64_t n,
                                  int H, int F, float* grad_feat, float* grad_attn_l,
                                  float* grad_attn_r, void* workspace, size_t workspace_bytes,
                                  cudaStream_t stream) {
  if (n < 0 || H <= 0 || F <= 0) return bad("gnn_gat_scores_bwd: bad size");
  if (!attn_l || !attn_r || !grad_attn_l || !grad_attn_r || (n && (!feat || !grad_attn_row || !grad_attn_col || !grad_feat)))
    return bad("gnn_gat_scores_bwd: null pointer");
  const bool vec = F % 4 == 0 && aligned16(feat) && aligned16(attn_l) && aligned16(attn_r) && aligned16(grad_feat);
  if (!shape_ok(H, F, vec)) {
    set_last_error("gnn_gat_scores_bwd: H > 8 or H*F beyond the largest tile");
    return GNN_ERR_UNSUPPORTED;
  }
  size_t need = 0;
  gnn_gat_scores_bwd_workspace_bytes(n, H, F, &need);
  if (!workspace || workspace_bytes < need) {
    set_last_error("gnn_gat_scores_bwd: workspace too small");
    return GNN_ERR_WORKSPACE;
  }
  float* partial = (float*)(((uintptr_t)workspace + 255) / 256 * 256);
  const int blocks = score_blocks(n);
  const int width = H * F;
  dispatch_tile(next_pow2(H), width, vec, [&](auto hp, auto q, auto v) {
    gat_scores_bwd_kernel<decltype(hp)::value, decltype(q)::value, decltype(v)::value>
        <<<blocks, kThreadsPerCta, 0, stream>>>(n, H, F, feat, attn_l, attn_r, grad_attn_row,
                                                 grad_attn_col, grad_feat, partial);
  });
  gat_scores_reduce_kernel<<<(2 * width + 127) / 128, 128, 0, stream>>>(blocks, width, partial,
                                                                        grad_attn_l, grad_attn_r);
  return check_launch("gnn_gat_scores_bwd");
}
