// Fused EdgeConv max-aggregation with arg-max capture and its scatter backward
// (reference: src/fused_edgeconv/fused_edgeconv.cu:21-73 forward, :175-200
// backward).
//
// The reference maps lanes to neighbours, so every warp load touches 32
// different rows.  Here lanes map to features: a group of GS lanes owns one
// destination node and reads each neighbour row with contiguous 128-bit loads;
// all k neighbour rows of the node are in flight together.
//
// Tie rule (bit-exact arg-max): the reference reduces each block of 32
// neighbours with an xor butterfly that takes the partner on `>=`, and takes a
// later block of 32 on `>=`.  Among equal maxima that selects, inside a block,
// the neighbour whose 5-bit position has the largest bit-reversed value, and
// across blocks the later block; padding positions behave as (-1e38, id -1).
// Visiting the candidates block by block in increasing bit-reversed position
// with a `>=` update reproduces exactly that choice.
#include "../../include/gnn_b200.h"
#include "common.cuh"

#include <string>

using namespace gnn;

namespace {

// ACT: the stored maximum goes through LeakyReLU(slope) first (the activation the DGCNN
// model applies to every EdgeConv output, script/train/train_edgeconv_our.py:44-52); the
// arg-max is that of the raw values, which LeakyReLU (monotone for slope > 0) preserves.
template <int Q, bool VEC, bool ACT>
__global__ void __launch_bounds__(256)
edgeconv_fwd_kernel(int n, int F, int k, int gs, const int* __restrict__ src_ind,
                    const float* __restrict__ h_src, const float* __restrict__ h_dst,
                    float* __restrict__ out, int* __restrict__ max_idx, float slope) {
  constexpr int VW = VEC ? 4 : 1;
  const int lane = threadIdx.x & 31;
  const int warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int per_warp = 32 / gs;
  const int node = warp * per_warp + lane / gs;
  const int fl = lane % gs;
  if (node >= n) return;

  bool valid[Q];
  float dst[Q][VW], best[Q][VW];
  int bid[Q][VW];
  const float* drow = h_dst + (size_t)node * F;
#pragma unroll
  for (int q = 0; q < Q; ++q) {
    const int e0 = (fl + gs * q) * VW;
    valid[q] = e0 < F;
#pragma unroll
    for (int i = 0; i < VW; ++i) {
      dst[q][i] = 0.f;
      best[q][i] = -INFINITY;
      bid[q][i] = -1;
    }
    if (valid[q]) {
      if constexpr (VEC) {
        float4 t = __ldg(reinterpret_cast<const float4*>(drow) + fl + gs * q);
        dst[q][0] = t.x; dst[q][1] = t.y; dst[q][2] = t.z; dst[q][3] = t.w;
      } else {
        dst[q][0] = __ldg(drow + fl + gs * q);
      }
    }
  }
  const int* nb = src_ind + (size_t)node * k;
  for (int cb = 0; cb < k; cb += 32) {
#pragma unroll 8
    for (int t = 0; t < 32; ++t) {
      const int pos = (int)(__brev((unsigned)t) >> 27);
      const int j = cb + pos;
      if (j < k) {
        const int c = __ldg(nb + j);
        const float* srow = h_src + (size_t)c * F;
#pragma unroll
        for (int q = 0; q < Q; ++q) {
          if (valid[q]) {
            float v[VW];
            if constexpr (VEC) {
              float4 t4 = __ldg(reinterpret_cast<const float4*>(srow) + fl + gs * q);
              v[0] = t4.x; v[1] = t4.y; v[2] = t4.z; v[3] = t4.w;
            } else {
              v[0] = __ldg(srow + fl + gs * q);
            }
#pragma unroll
            for (int i = 0; i < VW; ++i) {
              const float val = dst[q][i] + v[i];
              if (val >= best[q][i]) { best[q][i] = val; bid[q][i] = c; }
            }
          }
        }
      } else {
#pragma unroll
        for (int q = 0; q < Q; ++q)
#pragma unroll
          for (int i = 0; i < VW; ++i)
            if (kNegBig >= best[q][i]) { best[q][i] = kNegBig; bid[q][i] = -1; }
      }
    }
  }
  float* orow = out + (size_t)node * F;
  int* irow = max_idx + (size_t)node * F;
#pragma unroll
  for (int q = 0; q < Q; ++q) {
    if (valid[q]) {
      if constexpr (ACT) {
#pragma unroll
        for (int i = 0; i < VW; ++i) best[q][i] = best[q][i] > 0.f ? best[q][i] : best[q][i] * slope;
      }
      if constexpr (VEC) {
        reinterpret_cast<float4*>(orow)[fl + gs * q] =
            make_float4(best[q][0], best[q][1], best[q][2], best[q][3]);
        reinterpret_cast<int4*>(irow)[fl + gs * q] =
            make_int4(bid[q][0], bid[q][1], bid[q][2], bid[q][3]);
      } else {
        orow[fl + gs * q] = best[q][0];
        irow[fl + gs * q] = bid[q][0];
      }
    }
  }
}

__global__ void edgeconv_bwd_kernel(int64_t total, int F, const int* __restrict__ max_idx,
                                    const float* __restrict__ grad_out,
                                    float* __restrict__ grad_src) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= total) return;
  const int c = max_idx[t];
  if (c >= 0) atomicAdd(grad_src + (size_t)c * F + (t % F), grad_out[t]);
}

// Backward of the activated forward: the gradient first passes LeakyReLU' (decided by the
// sign of the stored output, which is the sign of the raw maximum), is written out as the
// gradient of h_dst, and is scattered to the arg-max source row.
__global__ void edgeconv_bwd_act_kernel(int64_t total, int F, const int* __restrict__ max_idx,
                                        const float* __restrict__ grad_out,
                                        const float* __restrict__ out, float slope,
                                        float* __restrict__ grad_src,
                                        float* __restrict__ grad_dst) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= total) return;
  const float g = out[t] > 0.f ? grad_out[t] : grad_out[t] * slope;
  grad_dst[t] = g;
  const int c = max_idx[t];
  if (c >= 0) atomicAdd(grad_src + (size_t)c * F + (t % F), g);
}

int bad(const char* m) {
  set_last_error(m);
  return GNN_ERR_INVALID_ARG;
}

int bad2(const char* who, const char* m) {
  set_last_error((std::string(who) + ": " + m).c_str());
  return GNN_ERR_INVALID_ARG;
}

template <int Q, bool VEC>
void launch_fwd(int n, int F, int k, int gs, const int* src, const float* hs, const float* hd,
                float* out, int* idx, bool act, float slope, cudaStream_t st) {
  const int per_warp = 32 / gs;
  const int warps = (n + per_warp - 1) / per_warp;
  const int blocks = (warps + 7) / 8;
  if (act)
    edgeconv_fwd_kernel<Q, VEC, true><<<blocks, 256, 0, st>>>(n, F, k, gs, src, hs, hd, out, idx, slope);
  else
    edgeconv_fwd_kernel<Q, VEC, false><<<blocks, 256, 0, st>>>(n, F, k, gs, src, hs, hd, out, idx, 1.f);
}

}  // namespace

namespace {
int edgeconv_fwd_impl(const char* who, int k, const int* src_ind, const float* h_src,
                      const float* h_dst, int64_t n, int F, bool act, float slope, float* out,
                      int* max_idx, cudaStream_t stream) {
  if (n < 0 || F <= 0 || k <= 0) return bad2(who, "bad size");
  if (n * (int64_t)k > INT32_MAX) return bad2(who, "n*k exceeds int32 indexing");
  if (n == 0) return GNN_OK;
  if (!src_ind || !h_src || !h_dst || !out || !max_idx) return bad2(who, "null pointer");
  const bool vec = F % 4 == 0 && aligned16(h_src) && aligned16(h_dst) && aligned16(out) && aligned16(max_idx);
  const int units = vec ? F / 4 : F;
  int gs = 1;
  while (gs < 32 && gs < units) gs <<= 1;
  const int q = (units + gs - 1) / gs;
  if (q > 8) {
    set_last_error((std::string(who) + ": feature width beyond 1024 (aligned) / 256 floats").c_str());
    return GNN_ERR_UNSUPPORTED;
  }
#define GNN_EC(QQ)                                                                        \
  if (vec) launch_fwd<QQ, true>((int)n, F, k, gs, src_ind, h_src, h_dst, out, max_idx, act, slope, stream); \
  else launch_fwd<QQ, false>((int)n, F, k, gs, src_ind, h_src, h_dst, out, max_idx, act, slope, stream);
  if (q == 1) { GNN_EC(1) }
  else if (q == 2) { GNN_EC(2) }
  else if (q <= 4) { GNN_EC(4) }
  else { GNN_EC(8) }
#undef GNN_EC
  return check_launch(who);
}
}  // namespace

extern "C" int gnn_edgeconv_fwd(int k, const int* src_ind, const float* h_src,
                                const float* h_dst, int64_t n, int F, float* out,
                                int* max_idx, cudaStream_t stream) {
  return edgeconv_fwd_impl("gnn_edgeconv_fwd", k, src_ind, h_src, h_dst, n, F, false, 1.f, out,
                           max_idx, stream);
}

extern "C" int gnn_edgeconv_fwd_act(int k, const int* src_ind, const float* h_src,
                                    const float* h_dst, int64_t n, int F, float slope,
                                    float* out, int* max_idx, cudaStream_t stream) {
  if (!(slope > 0.f)) return bad("gnn_edgeconv_fwd_act: slope must be positive");
  return edgeconv_fwd_impl("gnn_edgeconv_fwd_act", k, src_ind, h_src, h_dst, n, F, true, slope,
                           out, max_idx, stream);
}

extern "C" int gnn_edgeconv_bwd(const float* grad_out, const int* max_idx, int64_t n,
                                int64_t n_src, int F, float* grad_src, cudaStream_t stream) {
  if (n < 0 || n_src < 0 || F <= 0) return bad("gnn_edgeconv_bwd: bad size");
  if (n_src == 0) return GNN_OK;
  if (!grad_src || (n && (!grad_out || !max_idx))) return bad("gnn_edgeconv_bwd: null pointer");
  cudaError_t e = cudaMemsetAsync(grad_src, 0, (size_t)n_src * F * sizeof(float), stream);
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return GNN_ERR_CUDA;
  }
  const int64_t total = n * F;
  if (total > 0) {
    const int64_t blocks = (total + 255) / 256;
    edgeconv_bwd_kernel<<<(unsigned)blocks, 256, 0, stream>>>(total, F, max_idx, grad_out, grad_src);
  }
  return check_launch("gnn_edgeconv_bwd");
}

extern "C" int gnn_edgeconv_bwd_act(const float* grad_out, const float* out, float slope,
                                    const int* max_idx, int64_t n, int64_t n_src, int F,
                                    float* grad_src, float* grad_dst, cudaStream_t stream) {
  if (n < 0 || n_src < 0 || F <= 0) return bad("gnn_edgeconv_bwd_act: bad size");
  if (!(slope > 0.f)) return bad("gnn_edgeconv_bwd_act: slope must be positive");
  if ((n_src && !grad_src) || (n && (!grad_out || !out || !max_idx || !grad_dst)))
    return bad("gnn_edgeconv_bwd_act: null pointer");
  if (n_src) {
    cudaError_t e = cudaMemsetAsync(grad_src, 0, (size_t)n_src * F * sizeof(float), stream);
    if (e != cudaSuccess) {
      set_last_error(cudaGetErrorString(e));
      return GNN_ERR_CUDA;
    }
  }
  const int64_t total = n * F;
  if (total > 0) {
    const int64_t blocks = (total + 255) / 256;
    edgeconv_bwd_act_kernel<<<(unsigned)blocks, 256, 0, stream>>>(total, F, max_idx, grad_out, out,
                                                                  slope, grad_src, grad_dst);
  }
  return check_launch("gnn_edgeconv_bwd_act");
}
