// GMMConv: fused Gaussian edge weighting + multi-kernel SpMM, the Gaussian
// weights alone, and their (mathematically correct) backward.
// Reference: src/fused_gmmconv/gmmconv.cu:48-80 fuseGmm, :34-46 gaussian,
// :154-184 gaussian_bp (the reference backward reduces nothing because its
// AllReduce takes the value by copy, src/util/computeUtil.h:154-160, and adds
// into uninitialised memory; the gradients here are the analytic ones).
#include "../../include/gnn_b200.h"
#include "wgather.cuh"

using namespace gnn;

namespace {

constexpr int kMaxDim = 8;  // pseudo-coordinate dimensions kept in registers

__global__ void gaussian_fwd_kernel(int64_t E, int K, int D, const float* __restrict__ pseudo,
                                    const float* __restrict__ mu,
                                    const float* __restrict__ inv_sigma,
                                    float* __restrict__ out) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= E * K) return;
  const int64_t e = t / K;
  const int k = (int)(t % K);
  float acc = 0.f;
  for (int d = 0; d < D; ++d) {
    const float x = (pseudo[e * D + d] - mu[k * D + d]) * inv_sigma[k * D + d];
    acc = fmaf(x, x, acc);
  }
  out[t] = expf(-0.5f * acc);
}

// One block accumulates, for every mixture kernel k in turn, its edges'
// contributions to grad_mu[k,:] and grad_inv_sigma[k,:] and writes them to
// partial[block][k][2][D]; a second kernel sums the partials in block order, so
// the result does not depend on scheduling.  grad_pseudo[e,:] is owned by the
// thread that owns edge e.
//   w      = exp(-0.5 sum_d ((p_d - mu_d) s_d)^2)
//   dw/dp_d  = -w (p_d - mu_d) s_d^2
//   dw/dmu_d = +w (p_d - mu_d) s_d^2
//   dw/ds_d  = -w (p_d - mu_d)^2 s_d
__global__ void __launch_bounds__(256)
gaussian_bwd_kernel(int64_t E, int K, int D, const float* __restrict__ pseudo,
                    const float* __restrict__ mu, const float* __restrict__ inv_sigma,
                    const float* __restrict__ grad_w, float* __restrict__ grad_pseudo,
                    float* __restrict__ partial) {
  __shared__ float red[8][2 * kMaxDim];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int k = 0; k < K; ++k) {
    float m[kMaxDim], s[kMaxDim], am[kMaxDim], as[kMaxDim];
#pragma unroll
    for (int d = 0; d < kMaxDim; ++d) {
      m[d] = d < D ? mu[k * D + d] : 0.f;
      s[d] = d < D ? inv_sigma[k * D + d] : 0.f;
      am[d] = 0.f;
      as[d] = 0.f;
    }
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < E; e += stride) {
      float diff[kMaxDim];
      float acc = 0.f;
#pragma unroll
      for (int d = 0; d < kMaxDim; ++d) {
        diff[d] = d < D ? pseudo[e * D + d] - m[d] : 0.f;
        const float x = diff[d] * s[d];
        acc = fmaf(x, x, acc);
      }
      const float gw = grad_w[e * K + k] * expf(-0.5f * acc);
#pragma unroll
      for (int d = 0; d < kMaxDim; ++d) {
        if (d < D) {
          const float t = gw * diff[d] * s[d] * s[d];
          am[d] += t;
          as[d] -= gw * diff[d] * diff[d] * s[d];
          if (k == 0) grad_pseudo[e * D + d] = -t;
          else grad_pseudo[e * D + d] -= t;
        }
      }
    }
#pragma unroll
    for (int d = 0; d < kMaxDim; ++d) {
      am[d] = warp_sum(am[d]);
      as[d] = warp_sum(as[d]);
    }
    __syncthreads();
    if (lane == 0) {
#pragma unroll
      for (int d = 0; d < kMaxDim; ++d) { red[w][d] = am[d]; red[w][kMaxDim + d] = as[d]; }
    }
    __syncthreads();
    if (threadIdx.x < 2 * kMaxDim) {
      float tot = 0.f;
      for (int ww = 0; ww < 8; ++ww) tot += red[ww][threadIdx.x];
      const int which = threadIdx.x / kMaxDim, d = threadIdx.x % kMaxDim;
      if (d < D) partial[(((size_t)blockIdx.x * K + k) * 2 + which) * D + d] = tot;
    }
  }
}

__global__ void gaussian_bwd_reduce_kernel(int nblocks, int K, int D,
                                           const float* __restrict__ partial,
                                           float* __restrict__ grad_mu,
                                           float* __restrict__ grad_sigma) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= K * 2 * D) return;
  const int k = t / (2 * D), which = (t / D) % 2, d = t % D;
  float tot = 0.f;
  for (int b = 0; b < nblocks; ++b) tot += partial[(((size_t)b * K + k) * 2 + which) * D + d];
  (which == 0 ? grad_mu : grad_sigma)[k * D + d] = tot;
}

int bad(const char* m) {
  set_last_error(m);
  return GNN_ERR_INVALID_ARG;
}
size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

int bwd_blocks(int64_t E) {
  int64_t b = (E + 255) / 256;
  if (b > 148 * 4) b = 148 * 4;
  if (b < 1) b = 1;
  return (int)b;
}

}  // namespace

extern "C" int gnn_gmm_fwd_workspace_bytes(int64_t nnz, int K, int F, size_t* bytes) {
  if (!bytes || nnz < 0 || K <= 0 || F <= 0) return bad("gnn_gmm_fwd_workspace_bytes: bad argument");
  const int HP = K <= 8 ? next_pow2(K) : 1;
  int64_t w = K <= 8 ? (int64_t)K * F : F;
  if (w > 512) w = 512;
  *bytes = wgather_scratch_floats(nnz, HP, (int)w) * sizeof(float) + 256;
  return GNN_OK;
}

extern "C" int gnn_gmm_fwd(const int* ptr, const int* idx, int64_t n_seg, int64_t nnz,
                           const float* node_feat, const float* pseudo, const int* perm,
                           const float* mu, const float* inv_sigma, int K, int D, int F,
                           float* out, void* workspace, size_t workspace_bytes,
                           cudaStream_t stream) {
  if (n_seg < 0 || nnz < 0 || K <= 0 || D <= 0 || F <= 0) return bad("gnn_gmm_fwd: bad size");
  if (n_seg > INT32_MAX - 1 || nnz > INT32_MAX - 4096) return bad("gnn_gmm_fwd: size exceeds int32 indexing");
  if (n_seg == 0) return GNN_OK;
  if (!ptr || (!idx && nnz) || !node_feat || (!pseudo && nnz) || !mu || !inv_sigma || !out)
    return bad("gnn_gmm_fwd: null pointer");
  const int64_t KF = (int64_t)K * F;
  const bool vec = F % 4 == 0 && aligned16(node_feat) && aligned16(out);
  if (K > 8 || KF > max_tile_width(vec)) {
    set_last_error("gnn_gmm_fwd: K > 8 or K*F beyond the largest tile (512 aligned / 256 floats)");
    return GNN_ERR_UNSUPPORTED;
  }
  size_t need = 0;
  gnn_gmm_fwd_workspace_bytes(nnz, K, F, &need);
  if (nnz > 0 && (!workspace || workspace_bytes < need)) {
    set_last_error("gnn_gmm_fwd: workspace too small");
    return GNN_ERR_WORKSPACE;
  }
  const int chunk = pick_chunk(nnz);
  WGatherParams p;
  p.g = ChunkGeom{ptr, idx, (int)n_seg, (int)nnz, chunk, num_chunks_for(nnz, chunk)};
  p.feat = node_feat; p.ld_feat = KF;
  p.out = out; p.ld_out = KF;
  p.H = K; p.F = F; p.width = (int)KF;
  p.scratch = (float*)align_up((uintptr_t)workspace, 256);
  p.aux_off = round_up4((int)KF);
  const int HPv = next_pow2(K);
  p.slot_stride = p.aux_off + round_up4(2 * HPv);
  bool ok = dispatch_tile(HPv, (int)KF, vec, [&](auto hp, auto q, auto v) {
    constexpr int HP = decltype(hp)::value;
    GaussPolicy<HP> pol{pseudo, mu, inv_sigma, perm, D};
    launch_wgather<GaussPolicy, HP, decltype(q)::value, decltype(v)::value>(p, pol, stream);
  });
  if (!ok) {
    set_last_error("gnn_gmm_fwd: no tile for this shape");
    return GNN_ERR_UNSUPPORTED;
  }
  return check_launch("gnn_gmm_fwd");
}

extern "C" int gnn_gaussian_fwd(const float* pseudo, const float* mu, const float* inv_sigma,
                                int64_t E, int K, int D, float* out, cudaStream_t stream) {
  if (E < 0 || K <= 0 || D <= 0) return bad("gnn_gaussian_fwd: bad size");
  if (E == 0) return GNN_OK;
  if (!pseudo || !mu || !inv_sigma || !out) return bad("gnn_gaussian_fwd: null pointer");
  const int64_t total = E * K;
  gaussian_fwd_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(E, K, D, pseudo, mu, inv_sigma, out);
  return check_launch("gnn_gaussian_fwd");
}

extern "C" int gnn_gaussian_bwd_workspace_bytes(int64_t E, int K, int D, size_t* bytes) {
  if (!bytes || E < 0 || K <= 0 || D <= 0) return bad("gnn_gaussian_bwd_workspace_bytes: bad argument");
  *bytes = (size_t)bwd_blocks(E) * K * 2 * D * sizeof(float) + 256;
  return GNN_OK;
}

extern "C" int gnn_gaussian_bwd(const float* pseudo, const float* mu, const float* inv_sigma,
                                const float* grad_w, int64_t E, int K, int D,
                                float* grad_pseudo, float* grad_mu, float* grad_inv_sigma,
                                void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  if (E < 0 || K <= 0 || D <= 0) return bad("gnn_gaussian_bwd: bad size");
  if (D > kMaxDim) {
    set_last_error("gnn_gaussian_bwd: more than 8 pseudo-coordinate dimensions");
    return GNN_ERR_UNSUPPORTED;
  }
  if (!mu || !inv_sigma || !grad_mu || !grad_inv_sigma || (E && (!pseudo || !grad_w || !grad_pseudo)))
    return bad("gnn_gaussian_bwd: null pointer");
  size_t need = 0;
  gnn_gaussian_bwd_workspace_bytes(E, K, D, &need);
  if (!workspace || workspace_bytes < need) {
    set_last_error("gnn_gaussian_bwd: workspace too small");
    return GNN_ERR_WORKSPACE;
  }
  float* partial = (float*)align_up((uintptr_t)workspace, 256);
  const int nb = bwd_blocks(E);
  gaussian_bwd_kernel<<<nb, 256, 0, stream>>>(E, K, D, pseudo, mu, inv_sigma, grad_w, grad_pseudo, partial);
  gaussian_bwd_reduce_kernel<<<(K * 2 * D + 127) / 128, 128, 0, stream>>>(nb, K, D, partial, grad_mu, grad_inv_sigma);
  return check_launch("gnn_gaussian_bwd");
}

// ---- the layer's tail: sum over the K kernels, residual, bias (layers/gmmconv_layer.py:69-75) ----
namespace {

// One thread per VW consecutive output floats: out[n,f] = ((sum_k x[n,k,f]) + res[n,f]) + bias[f].
template <int VW>
__global__ void kernels_sum_fwd_kernel(int64_t total, int K, int F, const float* __restrict__ x,
                                       const float* __restrict__ res, const float* __restrict__ bias,
                                       float* __restrict__ out) {
  const int64_t t = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * VW;
  if (t >= total) return;
  const int64_t n = t / F;
  const int f = (int)(t - n * F);
  const float* xr = x + (size_t)n * K * F + f;
  float acc[VW];
#pragma unroll
  for (int i = 0; i < VW; ++i) acc[i] = 0.f;
  for (int k = 0; k < K; ++k) {
    if constexpr (VW == 4) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(xr + (size_t)k * F));
      acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
    } else {
      acc[0] += __ldg(xr + (size_t)k * F);
    }
  }
#pragma unroll
  for (int i = 0; i < VW; ++i) {
    if (res) acc[i] += __ldg(res + t + i);
    if (bias) acc[i] += __ldg(bias + f + i);
  }
  if constexpr (VW == 4) *reinterpret_cast<float4*>(out + t) = make_float4(acc[0], acc[1], acc[2], acc[3]);
  else out[t] = acc[0];
}

// grad_x[n,k,:] = grad_out[n,:] for every k.
template <int VW>
__global__ void kernels_sum_bwd_kernel(int64_t total, int K, int F, const float* __restrict__ grad_out,
                                       float* __restrict__ grad_x) {
  const int64_t t = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * VW;
  if (t >= total) return;
  const int64_t n = t / F;
  const int f = (int)(t - n * F);
  float* gx = grad_x + (size_t)n * K * F + f;
  if constexpr (VW == 4) {
    const float4 g = __ldg(reinterpret_cast<const float4*>(grad_out + t));
    for (int k = 0; k < K; ++k) *reinterpret_cast<float4*>(gx + (size_t)k * F) = g;
  } else {
    const float g = __ldg(grad_out + t);
    for (int k = 0; k < K; ++k) gx[(size_t)k * F] = g;
  }
}

}  // namespace

extern "C" int gnn_gmm_sum_fwd(const float* x, const float* residual, const float* bias, int64_t n,
                               int K, int F, float* out, cudaStream_t stream) {
  if (n < 0 || K <= 0 || F <= 0) return bad("gnn_gmm_sum_fwd: bad size");
  if (n == 0) return GNN_OK;
  if (!x || !out) return bad("gnn_gmm_sum_fwd: null pointer");
  const int64_t total = n * F;
  const bool vec = F % 4 == 0 && aligned16(x) && aligned16(out) && (!residual || aligned16(residual)) &&
                   (!bias || aligned16(bias));
  if (vec)
    kernels_sum_fwd_kernel<4><<<(unsigned)((total / 4 + 255) / 256), 256, 0, stream>>>(total, K, F, x, residual, bias, out);
  else
    kernels_sum_fwd_kernel<1><<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(total, K, F, x, residual, bias, out);
  return check_launch("gnn_gmm_sum_fwd");
}

extern "C" int gnn_gmm_sum_bwd(const float* grad_out, int64_t n, int K, int F, float* grad_x,
                               cudaStream_t stream) {
  if (n < 0 || K <= 0 || F <= 0) return bad("gnn_gmm_sum_bwd: bad size");
  if (n == 0) return GNN_OK;
  if (!grad_out || !grad_x) return bad("gnn_gmm_sum_bwd: null pointer");
  const int64_t total = n * F;
  const bool vec = F % 4 == 0 && aligned16(grad_out) && aligned16(grad_x);
  if (vec)
    kernels_sum_bwd_kernel<4><<<(unsigned)((total / 4 + 255) / 256), 256, 0, stream>>>(total, K, F, grad_out, grad_x);
  else
    kernels_sum_bwd_kernel<1><<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(total, K, F, grad_out, grad_x);
  return check_launch("gnn_gmm_sum_bwd");
}
