// The unfused sparse operators that share the reference API: multi-head SpMM,
// single-head SpMM, (multi-head) SDDMM on CSR and COO, permutation of edge
// values, u_add_v, CSR edge softmax, and the per-edge attention values of the
// "stash" GAT variants.
#include "../../include/gnn_b200.h"
#include "wgather.cuh"

using namespace gnn;

namespace {

int bad(const char* m) {
  set_last_error(m);
  return GNN_ERR_INVALID_ARG;
}
size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// ---- SDDMM -------------------------------------------------------------------
// out[e,h] = <A[seg(e),h,:], B[idx[e],h,:]>   (src/sddmm/mhsddmm.cu:5-81,
// src/sddmm/sddmm.cu:5-359).  The segment's A row stays in registers while the
// warp walks the segment's edges; dot products of U edges x HP heads are
// reduced together with warp_multi_sum.
struct SddmmParams {
  ChunkGeom g;
  const float* A; int64_t ld_a;
  const float* B; int64_t ld_b;
  int H, F, width;
  float* out; int ld_out;  // out[e*ld_out + h]
};

template <int HP, int Q, bool VEC>
__global__ void __launch_bounds__(kThreadsPerCta)
sddmm_csr_kernel(SddmmParams p) {
  constexpr int VW = VEC ? 4 : 1;
  constexpr int U0 = Unroll<Q, VEC>::U;
  constexpr int U = (U0 * HP > 32) ? 32 / HP : U0;
  constexpr int V = U * HP;
  __shared__ int cs_all[kWarpsPerCta][32];
  __shared__ float gs_all[kWarpsPerCta][32 * HP];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int chunk_id = blockIdx.x * kWarpsPerCta + wib;
  if (chunk_id >= p.g.num_chunks) return;
  int* cs = cs_all[wib];
  float* gs = gs_all[wib];
  RowTile<Q, VEC> t;
  t.init(lane, p.width, p.F, p.H);
  for_each_piece(p.g, chunk_id, [&](int s, int a, int b, bool, bool) {
    float aq[Q][VW];
    t.load(p.A + (size_t)s * p.ld_a, lane, aq);
    for (int base = a; base < b; base += 32) {
      const int e = base + lane;
      const bool ok = e < b;
      const int c = __ldg(p.g.idx + (ok ? e : a));
      __syncwarp();
      cs[lane] = c;
      __syncwarp();
      const int nb = min(32, b - base);
      const int nbr = (nb + U - 1) / U * U;
#pragma unroll 1
      for (int jj = 0; jj < nbr; jj += U) {
        float v[U][Q][VW];
#pragma unroll
        for (int u = 0; u < U; ++u) t.load(p.B + (size_t)cs[jj + u] * p.ld_b, lane, v[u]);
        float pv[V];
#pragma unroll
        for (int i = 0; i < V; ++i) pv[i] = 0.f;
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
          for (int q = 0; q < Q; ++q) {
            float d = 0.f;
#pragma unroll
            for (int i = 0; i < VW; ++i) d = fmaf(aq[q][i], v[u][q][i], d);
#pragma unroll
            for (int h = 0; h < HP; ++h)
              if (t.head[q] == h) pv[u * HP + h] += d;
          }
        warp_multi_sum<V>(pv, lane);
        if ((lane & (32 / V - 1)) == 0) gs[jj * HP + lane / (32 / V)] = pv[0];
      }
      __syncwarp();
      if (ok) {
#pragma unroll
        for (int h = 0; h < HP; ++h)
          if (h < p.H) p.out[(size_t)e * p.ld_out + h] = gs[lane * HP + h];
      }
    }
  });
}

// COO: one warp per 32 consecutive edges, both rows gathered.
template <int Q, bool VEC>
__global__ void __launch_bounds__(kThreadsPerCta)
sddmm_coo_kernel(const int* __restrict__ row, const int* __restrict__ col, int64_t nnz,
                 const float* __restrict__ A, const float* __restrict__ B, int F,
                 float* __restrict__ out) {
  constexpr int VW = VEC ? 4 : 1;
  const int lane = threadIdx.x & 31;
  const int64_t base = ((int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5)) * 32;
  if (base >= nnz) return;
  RowTile<Q, VEC> t;
  t.init(lane, F, F, 1);
  const int64_t e = base + lane;
  const bool ok = e < nnz;
  const int r = __ldg(row + (ok ? e : base));
  const int c = __ldg(col + (ok ? e : base));
  float mine = 0.f;
  const int nb = (int)min((int64_t)32, nnz - base);
  for (int jj = 0; jj < nb; ++jj) {
    const int rr = __shfl_sync(kFull, r, jj);
    const int cc = __shfl_sync(kFull, c, jj);
    float x[Q][VW], y[Q][VW];
    t.load(A + (size_t)rr * F, lane, x);
    t.load(B + (size_t)cc * F, lane, y);
    float d = 0.f;
#pragma unroll
    for (int q = 0; q < Q; ++q)
#pragma unroll
      for (int i = 0; i < VW; ++i) d = fmaf(x[q][i], y[q][i], d);
    d = warp_sum(d);
    if (lane == jj) mine = d;
  }
  if (ok) out[e] = mine;
}

// ---- small per-edge kernels -----------------------------------------------------

__global__ void permute_rows_kernel(const int* __restrict__ perm, const float* __restrict__ vals,
                                    int64_t E, int H, float* __restrict__ out) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= E * H) return;
  const int64_t i = t / H;
  const int h = (int)(t % H);
  out[t] = vals[(size_t)perm[i] * H + h];
}

// out[e,f] = row_val[seg(e),f] + col_val[idx[e],f]   (src/u_add_v/u_add_v.cu:4-28)
__global__ void __launch_bounds__(kThreadsPerCta)
u_add_v_fwd_kernel(ChunkGeom g, int F, const float* __restrict__ row_val,
                   const float* __restrict__ col_val, float* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int chunk_id = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (chunk_id >= g.num_chunks) return;
  for_each_piece(g, chunk_id, [&](int s, int a, int b, bool, bool) {
    const int64_t total = (int64_t)(b - a) * F;
    for (int64_t t = lane; t < total; t += 32) {
      const int e = a + (int)(t / F);
      const int f = (int)(t % F);
      out[(size_t)e * F + f] =
          __ldg(row_val + (size_t)s * F + f) + __ldg(col_val + (size_t)__ldg(g.idx + e) * F + f);
    }
  });
}

// grad_row[s,f] = sum_{e in s} g[e,f];  grad_col[c,f] = sum_{e: idx[e]=c} g[e,f]
// (src/u_add_v/u_add_v.cu:43-78; both outputs are zero-filled first, which the
// reference forgets for grad_col).  The lanes walk a piece's (edge, feature) pairs in memory
// order, so all 32 are busy whatever F is; grad_col is scattered with atomics (the signature
// carries no transposed graph to gather over), grad_row is summed in registers and only the
// pieces of rows cut by a chunk boundary meet through atomics.
__global__ void __launch_bounds__(kThreadsPerCta)
u_add_v_bwd_kernel(ChunkGeom g, int F, const float* __restrict__ grad,
                   float* __restrict__ grad_row, float* __restrict__ grad_col) {
  const int lane = threadIdx.x & 31;
  const int chunk_id = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (chunk_id >= g.num_chunks) return;
  const bool lanes_own_feature = F <= 32 && 32 % F == 0;  // lane l always sees feature l % F
  for_each_piece(g, chunk_id, [&](int s, int a, int b, bool first, bool last) {
    const int64_t total = (int64_t)(b - a) * F;
    float acc = 0.f;
    for (int64_t t = lane; t < total; t += 32) {
      const int e = a + (int)(t / F);
      const int f = (int)(t % F);
      const float v = __ldg(grad + (size_t)a * F + t);
      acc += v;
      atomicAdd(grad_col + (size_t)__ldg(g.idx + e) * F + f, v);
    }
    if (lanes_own_feature) {
      for (int o = 16; o >= F; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (lane < F) {
        if (first && last) grad_row[(size_t)s * F + lane] = acc;
        else atomicAdd(grad_row + (size_t)s * F + lane, acc);
      }
    } else {
      for (int f = lane; f < F; f += 32) {
        float r = 0.f;
        for (int e = a; e < b; ++e) r += __ldg(grad + (size_t)e * F + f);
        if (first && last) grad_row[(size_t)s * F + f] = r;
        else atomicAdd(grad_row + (size_t)s * F + f, r);
      }
    }
  });
}

// CSR edge softmax over (E,H) values (src/edge_softmax/edge_softmax.cu:7-60 forward, :63-98
// backward).  One warp per segment; a segment of kHeavySegment edges or more is left to all
// the warps of its CTA together, so a hub does not hang on 32 lanes.  When H divides 32 the
// threads walk the segment's E x H block in memory order (thread t always sees head t % H)
// and the per-head reductions run across the threads of equal head; other H take one head
// at a time.
constexpr int kHeavySegment = 2048;

template <bool BLOCK, class Op>
__device__ __forceinline__ float group_reduce(float v, int stride, Op op, float* red) {
  // combines the values of the threads whose index is equal modulo `stride` (a power of two
  // <= 32): inside the warp by butterflies, across the warps of the CTA through `red`
  for (int o = 16; o >= stride; o >>= 1) v = op(v, __shfl_xor_sync(0xffffffffu, v, o));
  if constexpr (BLOCK) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    __syncthreads();  // the previous use of `red` is over
    if (lane < stride) red[w * 32 + lane] = v;
    __syncthreads();
    v = red[lane & (stride - 1)];
    for (int k = 1; k < kWarpsPerCta; ++k) v = op(v, red[k * 32 + (lane & (stride - 1))]);
  }
  return v;
}

template <bool BLOCK>
__device__ __forceinline__ void edge_softmax_fwd_segment(int a, int b, int H, const float* __restrict__ in,
                                                         float* __restrict__ out, float* red) {
  const int tid = BLOCK ? threadIdx.x : (threadIdx.x & 31);
  const int nthr = BLOCK ? kThreadsPerCta : 32;
  auto fmax2 = [](float x, float y) { return fmaxf(x, y); };
  auto add2 = [](float x, float y) { return x + y; };
  if (H <= 32 && 32 % H == 0) {
    const float* x = in + (size_t)a * H;
    float* y = out + (size_t)a * H;
    const int64_t total = (int64_t)(b - a) * H;
    float m = kNegBig;
    for (int64_t t = tid; t < total; t += nthr) m = fmaxf(m, __ldg(x + t));
    m = group_reduce<BLOCK>(m, H, fmax2, red);
    float sum = 0.f;
    for (int64_t t = tid; t < total; t += nthr) sum += expf(__ldg(x + t) - m);
    sum = group_reduce<BLOCK>(sum, H, add2, red);
    for (int64_t t = tid; t < total; t += nthr) y[t] = expf(__ldg(x + t) - m) / sum;
  } else {
    for (int h = 0; h < H; ++h) {
      float m = kNegBig;
      for (int e = a + tid; e < b; e += nthr) m = fmaxf(m, __ldg(in + (size_t)e * H + h));
      m = group_reduce<BLOCK>(m, 1, fmax2, red);
      float sum = 0.f;
      for (int e = a + tid; e < b; e += nthr) sum += expf(__ldg(in + (size_t)e * H + h) - m);
      sum = group_reduce<BLOCK>(sum, 1, add2, red);
      for (int e = a + tid; e < b; e += nthr)
        out[(size_t)e * H + h] = expf(__ldg(in + (size_t)e * H + h) - m) / sum;
    }
  }
}

template <bool BLOCK>
__device__ __forceinline__ void edge_softmax_bwd_segment(int a, int b, int H, const float* __restrict__ y,
                                                         const float* __restrict__ gy, float* __restrict__ gx,
                                                         float* red) {
  const int tid = BLOCK ? threadIdx.x : (threadIdx.x & 31);
  const int nthr = BLOCK ? kThreadsPerCta : 32;
  auto add2 = [](float x, float y) { return x + y; };
  if (H <= 32 && 32 % H == 0) {
    const size_t off = (size_t)a * H;
    const int64_t total = (int64_t)(b - a) * H;
    float dot = 0.f;
    for (int64_t t = tid; t < total; t += nthr) dot = fmaf(__ldg(y + off + t), __ldg(gy + off + t), dot);
    dot = group_reduce<BLOCK>(dot, H, add2, red);
    for (int64_t t = tid; t < total; t += nthr) gx[off + t] = __ldg(y + off + t) * (__ldg(gy + off + t) - dot);
  } else {
    for (int h = 0; h < H; ++h) {
      float dot = 0.f;
      for (int e = a + tid; e < b; e += nthr)
        dot = fmaf(__ldg(y + (size_t)e * H + h), __ldg(gy + (size_t)e * H + h), dot);
      dot = group_reduce<BLOCK>(dot, 1, add2, red);
      for (int e = a + tid; e < b; e += nthr)
        gx[(size_t)e * H + h] = __ldg(y + (size_t)e * H + h) * (__ldg(gy + (size_t)e * H + h) - dot);
    }
  }
}

__global__ void __launch_bounds__(kThreadsPerCta)
edge_softmax_fwd_kernel(const int* __restrict__ ptr, int nseg, int H,
                        const float* __restrict__ in, float* __restrict__ out) {
  __shared__ float red[kWarpsPerCta * 32];
  const int s0 = blockIdx.x * kWarpsPerCta;
  const int s = s0 + (threadIdx.x >> 5);
  if (s < nseg) {
    const int a = __ldg(ptr + s), b = __ldg(ptr + s + 1);
    if (b - a < kHeavySegment) edge_softmax_fwd_segment<false>(a, b, H, in, out, red);
  }
  for (int k = 0; k < kWarpsPerCta && s0 + k < nseg; ++k) {  // uniform over the CTA
    const int a = __ldg(ptr + s0 + k), b = __ldg(ptr + s0 + k + 1);
    if (b - a >= kHeavySegment) edge_softmax_fwd_segment<true>(a, b, H, in, out, red);
  }
}

__global__ void __launch_bounds__(kThreadsPerCta)
edge_softmax_bwd_kernel(const int* __restrict__ ptr, int nseg, int H,
                        const float* __restrict__ y, const float* __restrict__ gy,
                        float* __restrict__ gx) {
  __shared__ float red[kWarpsPerCta * 32];
  const int s0 = blockIdx.x * kWarpsPerCta;
  const int s = s0 + (threadIdx.x >> 5);
  if (s < nseg) {
    const int a = __ldg(ptr + s), b = __ldg(ptr + s + 1);
    if (b - a < kHeavySegment) edge_softmax_bwd_segment<false>(a, b, H, y, gy, gx, red);
  }
  for (int k = 0; k < kWarpsPerCta && s0 + k < nseg; ++k) {
    const int a = __ldg(ptr + s0 + k), b = __ldg(ptr + s0 + k + 1);
    if (b - a >= kHeavySegment) edge_softmax_bwd_segment<true>(a, b, H, y, gy, gx, red);
  }
}

// Per-edge activated logit and normalised attention of the GAT forward, the
// two E x H tensors the "stash" and "fusescatter" variants keep
// (src/fused_gat/fused_gat_stash.cu:193-288).
__global__ void __launch_bounds__(kThreadsPerCta)
gat_edge_alpha_kernel(ChunkGeom g, int H, float slope, const float* __restrict__ attn_row,
                      const float* __restrict__ attn_col, const float* __restrict__ edge_max,
                      const float* __restrict__ edge_sum, float* __restrict__ edge_relu,
                      float* __restrict__ edge_alpha) {
  const int lane = threadIdx.x & 31;
  const int chunk_id = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (chunk_id >= g.num_chunks) return;
  for_each_piece(g, chunk_id, [&](int s, int a, int b, bool, bool) {
    const int64_t total = (int64_t)(b - a) * H;
    for (int64_t t = lane; t < total; t += 32) {
      const int e = a + (int)(t / H);
      const int h = (int)(t % H);
      const float x = leaky_relu(__ldg(attn_row + (size_t)s * H + h) +
                                 __ldg(attn_col + (size_t)__ldg(g.idx + e) * H + h), slope);
      edge_relu[(size_t)e * H + h] = x;
      edge_alpha[(size_t)e * H + h] =
          expf(x - __ldg(edge_max + (size_t)s * H + h)) / __ldg(edge_sum + (size_t)s * H + h);
    }
  });
}

int check_sizes(const char* who, int64_t nseg, int64_t nnz) {
  if (nseg < 0 || nnz < 0) return bad(who);
  if (nseg > INT32_MAX - 1 || nnz > INT32_MAX - 4096) return bad(who);
  return GNN_OK;
}

ChunkGeom geom(const int* ptr, const int* idx, int64_t nseg, int64_t nnz) {
  const int chunk = pick_chunk(nnz);
  return ChunkGeom{ptr, idx, (int)nseg, (int)nnz, chunk, num_chunks_for(nnz, chunk)};
}

}  // namespace

// ---- weighted SpMM ---------------------------------------------------------------

extern "C" int gnn_mhspmm_workspace_bytes(int64_t nnz, int H, int F, size_t* bytes) {
  if (!bytes || nnz < 0 || H <= 0 || F <= 0) return bad("gnn_mhspmm_workspace_bytes: bad argument");
  const bool fused = H <= 8 && (int64_t)H * F <= 256;
  int64_t w = fused ? (int64_t)H * F : F;
  if (w > 512) w = 512;
  const size_t a = wgather_scratch_floats(nnz, 8, 512);
  (void)w;
  *bytes = a * sizeof(float) + 256;
  return GNN_OK;
}

// out[s,h,:] = sum_e att[pe,h] * feat[idx[e],h,:]; att == nullptr means weight 1
// (src/spmm/mhspmm.cu:4-42; operators/spmm.py:35-41 for the single-head form).
extern "C" int gnn_mhspmm(const int* ptr, const int* idx, int64_t n_seg, int64_t nnz,
                          const float* att, const int* perm, const float* feat, int H, int F,
                          float* out, void* workspace, size_t workspace_bytes,
                          cudaStream_t stream) {
  if (check_sizes("gnn_mhspmm: bad size", n_seg, nnz) || H <= 0 || F <= 0) return bad("gnn_mhspmm: bad size");
  if (n_seg == 0) return GNN_OK;
  if (!ptr || (!idx && nnz) || !feat || !out) return bad("gnn_mhspmm: null pointer");
  size_t need = 0;
  gnn_mhspmm_workspace_bytes(nnz, H, F, &need);
  if (nnz > 0 && (!workspace || workspace_bytes < need)) {
    set_last_error("gnn_mhspmm: workspace too small");
    return GNN_ERR_WORKSPACE;
  }
  const int64_t HF = (int64_t)H * F;
  const bool vec = F % 4 == 0 && aligned16(feat) && aligned16(out);
  const int cap = max_tile_width(vec);
  const bool fused = H <= 8 && HF <= cap;
  const ChunkGeom g = geom(ptr, idx, n_seg, nnz);
  const int HPv = fused ? next_pow2(H) : 1;
  const int slab = fused ? (int)HF : (F < cap ? F : cap);
  for (int h = 0; h < (fused ? 1 : H); ++h) {
    for (int f0 = 0; f0 < (fused ? 1 : F); f0 += slab) {
      const int w = fused ? (int)HF : (F - f0 < slab ? F - f0 : slab);
      const int64_t off = fused ? 0 : (int64_t)h * F + f0;
      WGatherParams p;
      p.g = g;
      p.feat = feat + off; p.ld_feat = HF;
      p.out = out + off; p.ld_out = HF;
      p.H = fused ? H : 1; p.F = fused ? F : w; p.width = w;
      p.scratch = (float*)align_up((uintptr_t)workspace, 256);
      p.aux_off = round_up4(w);
      p.slot_stride = p.aux_off + round_up4(2 * HPv);
      bool ok = dispatch_tile(HPv, w, vec, [&](auto hp, auto q, auto v) {
        constexpr int HP = decltype(hp)::value;
        EdgeValuePolicy<HP> pol{att ? att + (fused ? 0 : h) : nullptr, perm, H};
        launch_wgather<EdgeValuePolicy, HP, decltype(q)::value, decltype(v)::value>(p, pol, stream);
      });
      if (!ok) {
        set_last_error("gnn_mhspmm: no tile for this shape");
        return GNN_ERR_UNSUPPORTED;
      }
    }
  }
  return check_launch("gnn_mhspmm");
}

// ---- SDDMM -------------------------------------------------------------------------

extern "C" int gnn_mhsddmm(const int* ptr, const int* idx, int64_t n_seg, int64_t nnz,
                           const float* A, const float* B, int H, int F, float* out,
                           cudaStream_t stream) {
  if (check_sizes("gnn_mhsddmm: bad size", n_seg, nnz) || H <= 0 || F <= 0) return bad("gnn_mhsddmm: bad size");
  if (n_seg == 0 || nnz == 0) return GNN_OK;
  if (!ptr || !idx || !A || !B || !out) return bad("gnn_mhsddmm: null pointer");
  const int64_t HF = (int64_t)H * F;
  const bool vec = F % 4 == 0 && aligned16(A) && aligned16(B);
  const int cap = max_tile_width(vec);
  if (F > cap) {
    set_last_error("gnn_mhsddmm: per-head width beyond the largest tile (512 aligned / 256 floats)");
    return GNN_ERR_UNSUPPORTED;
  }
  const bool fused = H <= 8 && HF <= cap;
  const ChunkGeom g = geom(ptr, idx, n_seg, nnz);
  const int HPv = fused ? next_pow2(H) : 1;
  for (int h = 0; h < (fused ? 1 : H); ++h) {
    SddmmParams p;
    p.g = g;
    p.A = A + (fused ? 0 : (int64_t)h * F); p.ld_a = HF;
    p.B = B + (fused ? 0 : (int64_t)h * F); p.ld_b = HF;
    p.H = fused ? H : 1; p.F = F; p.width = fused ? (int)HF : F;
    p.out = out + (fused ? 0 : h); p.ld_out = H;
    bool ok = dispatch_tile(HPv, p.width, vec, [&](auto hp, auto q, auto v) {
      const int blocks = (g.num_chunks + kWarpsPerCta - 1) / kWarpsPerCta;
      sddmm_csr_kernel<decltype(hp)::value, decltype(q)::value, decltype(v)::value>
          <<<blocks, kThreadsPerCta, 0, stream>>>(p);
    });
    if (!ok) {
      set_last_error("gnn_mhsddmm: no tile for this shape");
      return GNN_ERR_UNSUPPORTED;
    }
  }
  return check_launch("gnn_mhsddmm");
}

extern "C" int gnn_sddmm_coo(const int* row_ind, const int* col_ind, int64_t nnz, const float* A,
                             const float* B, int F, float* out, cudaStream_t stream) {
  if (nnz < 0 || F <= 0) return bad("gnn_sddmm_coo: bad size");
  if (nnz == 0) return GNN_OK;
  if (!row_ind || !col_ind || !A || !B || !out) return bad("gnn_sddmm_coo: null pointer");
  const bool vec = F % 4 == 0 && aligned16(A) && aligned16(B);
  const int units = vec ? F / 4 : F;
  const int q = (units + 31) / 32;
  if (q > 8) {
    set_last_error("gnn_sddmm_coo: feature width beyond 1024 (aligned) / 256 floats");
    return GNN_ERR_UNSUPPORTED;
  }
  const int64_t warps = (nnz + 31) / 32;
  const unsigned blocks = (unsigned)((warps + kWarpsPerCta - 1) / kWarpsPerCta);
#define GNN_COO(QQ)                                                                              \
  if (vec) sddmm_coo_kernel<QQ, true><<<blocks, kThreadsPerCta, 0, stream>>>(row_ind, col_ind, nnz, A, B, F, out); \
  else sddmm_coo_kernel<QQ, false><<<blocks, kThreadsPerCta, 0, stream>>>(row_ind, col_ind, nnz, A, B, F, out);
  if (q == 1) { GNN_COO(1) }
  else if (q == 2) { GNN_COO(2) }
  else if (q <= 4) { GNN_COO(4) }
  else { GNN_COO(8) }
#undef GNN_COO
  return check_launch("gnn_sddmm_coo");
}

// ---- small operators -------------------------------------------------------------------

extern "C" int gnn_mhtranspose(const int* permute, const float* vals, int64_t E, int H,
                               float* out, cudaStream_t stream) {
  if (E < 0 || H <= 0) return bad("gnn_mhtranspose: bad size");
  if (E == 0) return GNN_OK;
  if (!permute || !vals || !out) return bad("gnn_mhtranspose: null pointer");
  const int64_t total = E * H;
  permute_rows_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(permute, vals, E, H, out);
  return check_launch("gnn_mhtranspose");
}

extern "C" int gnn_u_add_v_fwd(const int* row_ptr, const int* col_ind, int64_t n_rows, int64_t nnz,
                               const float* row_val, const float* col_val, int F, float* out,
                               cudaStream_t stream) {
  if (check_sizes("gnn_u_add_v_fwd: bad size", n_rows, nnz) || F <= 0) return bad("gnn_u_add_v_fwd: bad size");
  if (nnz == 0 || n_rows == 0) return GNN_OK;
  if (!row_ptr || !col_ind || !row_val || !col_val || !out) return bad("gnn_u_add_v_fwd: null pointer");
  const ChunkGeom g = geom(row_ptr, col_ind, n_rows, nnz);
  u_add_v_fwd_kernel<<<(g.num_chunks + kWarpsPerCta - 1) / kWarpsPerCta, kThreadsPerCta, 0, stream>>>(
      g, F, row_val, col_val, out);
  return check_launch("gnn_u_add_v_fwd");
}

extern "C" int gnn_u_add_v_bwd(const int* row_ptr, const int* col_ind, int64_t n_rows,
                               int64_t n_cols, int64_t nnz, const float* grad_out, int F,
                               float* grad_row, float* grad_col, cudaStream_t stream) {
  if (check_sizes("gnn_u_add_v_bwd: bad size", n_rows, nnz) || n_cols < 0 || F <= 0)
    return bad("gnn_u_add_v_bwd: bad size");
  if (!grad_row || !grad_col) return bad("gnn_u_add_v_bwd: null pointer");
  cudaError_t e1 = cudaMemsetAsync(grad_row, 0, (size_t)n_rows * F * sizeof(float), stream);
  cudaError_t e2 = cudaMemsetAsync(grad_col, 0, (size_t)n_cols * F * sizeof(float), stream);
  if (e1 != cudaSuccess || e2 != cudaSuccess) {
    set_last_error("gnn_u_add_v_bwd: memset failed");
    return GNN_ERR_CUDA;
  }
  if (nnz == 0 || n_rows == 0) return GNN_OK;
  if (!row_ptr || !col_ind || !grad_out) return bad("gnn_u_add_v_bwd: null pointer");
  const ChunkGeom g = geom(row_ptr, col_ind, n_rows, nnz);
  u_add_v_bwd_kernel<<<(g.num_chunks + kWarpsPerCta - 1) / kWarpsPerCta, kThreadsPerCta, 0, stream>>>(
      g, F, grad_out, grad_row, grad_col);
  return check_launch("gnn_u_add_v_bwd");
}

extern "C" int gnn_edge_softmax_fwd(const int* row_ptr, int64_t n_rows, int64_t nnz, const float* in,
                                    int H, float* out, cudaStream_t stream) {
  if (check_sizes("gnn_edge_softmax_fwd: bad size", n_rows, nnz) || H <= 0) return bad("gnn_edge_softmax_fwd: bad size");
  if (nnz == 0 || n_rows == 0) return GNN_OK;
  if (!row_ptr || !in || !out) return bad("gnn_edge_softmax_fwd: null pointer");
  edge_softmax_fwd_kernel<<<(unsigned)((n_rows + kWarpsPerCta - 1) / kWarpsPerCta), kThreadsPerCta, 0, stream>>>(
      row_ptr, (int)n_rows, H, in, out);
  return check_launch("gnn_edge_softmax_fwd");
}

extern "C" int gnn_edge_softmax_bwd(const int* row_ptr, int64_t n_rows, int64_t nnz, const float* y,
                                    const float* grad_y, int H, float* grad_x, cudaStream_t stream) {
  if (check_sizes("gnn_edge_softmax_bwd: bad size", n_rows, nnz) || H <= 0) return bad("gnn_edge_softmax_bwd: bad size");
  if (nnz == 0 || n_rows == 0) return GNN_OK;
  if (!row_ptr || !y || !grad_y || !grad_x) return bad("gnn_edge_softmax_bwd: null pointer");
  edge_softmax_bwd_kernel<<<(unsigned)((n_rows + kWarpsPerCta - 1) / kWarpsPerCta), kThreadsPerCta, 0, stream>>>(
      row_ptr, (int)n_rows, H, y, grad_y, grad_x);
  return check_launch("gnn_edge_softmax_bwd");
}

extern "C" int gnn_gat_edge_alpha(const int* row_ptr, const int* col_ind, int64_t n_rows, int64_t nnz,
                                  const float* attn_row, const float* attn_col, const float* edge_max,
                                  const float* edge_sum, int H, float negative_slope, float* edge_relu,
                                  float* edge_alpha, cudaStream_t stream) {
  if (check_sizes("gnn_gat_edge_alpha: bad size", n_rows, nnz) || H <= 0) return bad("gnn_gat_edge_alpha: bad size");
  if (nnz == 0 || n_rows == 0) return GNN_OK;
  if (!row_ptr || !col_ind || !attn_row || !attn_col || !edge_max || !edge_sum || !edge_relu || !edge_alpha)
    return bad("gnn_gat_edge_alpha: null pointer");
  const ChunkGeom g = geom(row_ptr, col_ind, n_rows, nnz);
  gat_edge_alpha_kernel<<<(g.num_chunks + kWarpsPerCta - 1) / kWarpsPerCta, kThreadsPerCta, 0, stream>>>(
      g, H, negative_slope, attn_row, attn_col, edge_max, edge_sum, edge_relu, edge_alpha);
  return check_launch("gnn_gat_edge_alpha");
}
