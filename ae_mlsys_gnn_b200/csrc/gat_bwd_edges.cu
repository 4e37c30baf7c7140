// One-gather backward of the fused GAT.
//
// The two-pass backward (gat_bwd.cuh) gathers h[c] over all edges once more just to form
//     S[r,h] = sum_j a_j <G[r,h,:], h[c_j,h,:]>      and      grad_attn_row.
// With the forward output out[r,h,:] = sum_j a_j h[c_j,h,:] at hand, S needs no edge at all:
//     S[r,h] = <G[r,h,:], out[r,h,:]>.
// The column pass (one gather of G[r] over the CSC) then knows the gradient of every edge
// logit, stores it (E x H floats, CSC order: gnn_gat_bwd_col_edges) while it forms grad_feat
// and grad_attn_col, and grad_attn_row[r] is the sum of those values over row r's edges --
// a pass over E x H scalars instead of E x H x F features.  The map from a CSR edge to its
// position in the CSC is the inverse of csr2csc's permutation, a property of the graph.
//
//   gnn_gat_bwd_pack      rowpack[r] = {attn_row[r], max[r], 1/sum[r], S[r]}   (node-wise)
//   gnn_gat_bwd_pack_elu  the same, with the backward of an ELU on the layer's output folded in
//   gnn_gat_bwd_row_sum   grad_attn_row[r,h] = sum over CSR edges e of row r of
//                         edge_grad[csr_pos[e], h]   (edge-balanced, deterministic)
//   gnn_invert_permutation
//
// Replaces, for callers that keep `out`, the row pass that stands in for the reference's
// mhspmm_backward_kernel + mhsddmm (src/fused_gat/fused_gat_SM.cu:560-607, :656-732).
#include "wgather.cuh"

using namespace gnn;

namespace {

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

int bad(const char* m) {
  set_last_error(m);
  return GNN_ERR_INVALID_ARG;
}

__global__ void invert_permutation_kernel(const int* __restrict__ perm, int64_t n, int* __restrict__ inv) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) inv[perm[i]] = (int)i;
}

// One warp per row.  VEC: H*F is a multiple of 4 and the matrices are 16-byte aligned.
// ELU: `gout` is the gradient with respect to elu(out) (the activation a model applies to the
// layer's output); the kernel first turns it into the gradient with respect to out,
//     g = gout * (out > 0 ? 1 : alpha * exp(out)),
// stores it in grad_pre (the operand the column pass gathers) and uses it for S -- the
// framework's separate elu-backward pass over the same two matrices disappears.
template <bool VEC, bool ELU>
__global__ void __launch_bounds__(kThreadsPerCta)
pack_kernel(int64_t n_rows, const float* __restrict__ out, const float* __restrict__ gout,
            const float* __restrict__ attn_row, const float* __restrict__ edge_max,
            const float* __restrict__ edge_sum, int H, int F, float alpha, float* __restrict__ grad_pre,
            float* __restrict__ rowpack) {
  const int lane = threadIdx.x & 31;
  const int64_t r = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  const float* o = out + (size_t)r * H * F;
  const float* g = gout + (size_t)r * H * F;
  float* gp = ELU ? grad_pre + (size_t)r * H * F : nullptr;
  float* rp = rowpack + (size_t)r * 4 * H;
  auto pre = [&](float ov, float gv) { return ELU ? gv * (ov > 0.f ? 1.f : alpha * expf(ov)) : gv; };
  for (int h = 0; h < H; ++h) {
    float acc = 0.f;
    if (VEC && F % 4 == 0) {
      const float4* o4 = reinterpret_cast<const float4*>(o + (size_t)h * F);
      const float4* g4 = reinterpret_cast<const float4*>(g + (size_t)h * F);
      for (int i = lane; i < F / 4; i += 32) {
        const float4 a = __ldg(o4 + i);
        float4 b = __ldg(g4 + i);
        b.x = pre(a.x, b.x); b.y = pre(a.y, b.y); b.z = pre(a.z, b.z); b.w = pre(a.w, b.w);
        if (ELU) reinterpret_cast<float4*>(gp + (size_t)h * F)[i] = b;
        acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc);
        acc = fmaf(a.z, b.z, acc); acc = fmaf(a.w, b.w, acc);
      }
    } else {
      for (int i = lane; i < F; i += 32) {
        const float a = __ldg(o + (size_t)h * F + i);
        const float b = pre(a, __ldg(g + (size_t)h * F + i));
        if (ELU) gp[(size_t)h * F + i] = b;
        acc = fmaf(a, b, acc);
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) {
      const float sum = __ldg(edge_sum + (size_t)r * H + h);
      const bool empty = !(sum > 0.f);  // a row without edges: same record as the two-pass backward writes
      rp[h] = __ldg(attn_row + (size_t)r * H + h);
      rp[H + h] = empty ? kNegBig : __ldg(edge_max + (size_t)r * H + h);
      rp[2 * H + h] = empty ? 0.f : 1.f / sum;
      rp[3 * H + h] = empty ? 0.f : acc;
    }
  }
}

// The same for rows of up to 512 floats read with 128-bit loads: the whole row of both
// matrices is requested at once (2 Q loads per lane in flight instead of two per head), the
// per-head sums come out of one combined butterfly, and the lanes that end up holding a head's
// sum write that head's record side by side.
template <int HP, int Q, bool ELU>
__global__ void __launch_bounds__(kThreadsPerCta)
pack_tile_kernel(int64_t n_rows, const float* __restrict__ out, const float* __restrict__ gout,
                 const float* __restrict__ attn_row, const float* __restrict__ edge_max,
                 const float* __restrict__ edge_sum, int H, int F, float alpha, float* __restrict__ grad_pre,
                 float* __restrict__ rowpack) {
  const int lane = threadIdx.x & 31;
  const int64_t r = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  RowTile<Q, true> t;
  t.init(lane, H * F, F, H);
  float ov[Q][4], gv[Q][4];
  t.load(out + (size_t)r * H * F, lane, ov);
  t.load(gout + (size_t)r * H * F, lane, gv);
  float pv[HP];
#pragma unroll
  for (int h = 0; h < HP; ++h) pv[h] = 0.f;
#pragma unroll
  for (int q = 0; q < Q; ++q) {
    float d = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if constexpr (ELU) gv[q][i] *= ov[q][i] > 0.f ? 1.f : alpha * expf(ov[q][i]);
      d = fmaf(ov[q][i], gv[q][i], d);
    }
#pragma unroll
    for (int h = 0; h < HP; ++h)
      if (t.head[q] == h && t.valid[q]) pv[h] += d;
  }
  if constexpr (ELU) t.store(grad_pre + (size_t)r * H * F, lane, gv);
  warp_multi_sum<HP>(pv, lane);  // head h on lanes [h*32/HP, (h+1)*32/HP)
  constexpr int LPH = 32 / HP;
  const int h = lane / LPH;
  if ((lane & (LPH - 1)) == 0 && h < H) {
    float* rp = rowpack + (size_t)r * 4 * H;
    const float sum = __ldg(edge_sum + (size_t)r * H + h);
    const bool empty = !(sum > 0.f);  // a row without edges: same record as the two-pass backward writes
    rp[h] = __ldg(attn_row + (size_t)r * H + h);
    rp[H + h] = empty ? kNegBig : __ldg(edge_max + (size_t)r * H + h);
    rp[2 * H + h] = empty ? 0.f : 1.f / sum;
    rp[3 * H + h] = empty ? 0.f : pv[0];
  }
}

struct RowSumParams {
  ChunkGeom g;             // CSR: ptr = row_ptr, idx = csr_pos (position of the edge in the CSC)
  const float* edge_grad;  // [nnz][H], CSC position order
  int H;
  float* grad_attn_row;    // [nseg][H]
  float* scratch;          // 2 * num_chunks slots of HP floats
};

// One warp per chunk of consecutive CSR positions.  The chunk is consumed in windows of 32
// positions: every lane gathers the value of its own edge (32 independent gathers in flight,
// the next window's requested before the current one is reduced), then the rows that
// overlap the window are summed one after the other with masked warp reductions.  Rows
// average a few dozen edges, so gathering per row instead would leave most lanes idle and
// expose one gather latency per row.
template <int HP>
__global__ void __launch_bounds__(kThreadsPerCta)
row_sum_kernel(RowSumParams p) {
  const int lane = threadIdx.x & 31;
  const int chunk_id = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (chunk_id >= p.g.num_chunks) return;
  const int lo = chunk_id * p.g.chunk;
  const int hi = min(lo + p.g.chunk, p.g.nnz);
  constexpr int LPH = 32 / HP;  // after warp_multi_sum head h sits on lanes [h*LPH, (h+1)*LPH)

  auto gather = [&](int e, float (&v)[HP]) {
#pragma unroll
    for (int h = 0; h < HP; ++h) v[h] = 0.f;
    if (e < hi) {
      const float* eg = p.edge_grad + (size_t)__ldg(p.g.idx + e) * p.H;
      if (HP == 4 && p.H == 4) {
        const float4 t = __ldg(reinterpret_cast<const float4*>(eg));
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
      } else {
#pragma unroll
        for (int h = 0; h < HP; ++h)
          if (h < p.H) v[h] = __ldg(eg + h);
      }
    }
  };
  // this lane's head of the finished (or cut) row s goes to the output or to a scratch slot
  auto emit = [&](int s, float total, bool first, bool last) {
    if ((lane & (LPH - 1)) == 0 && lane / LPH < p.H) {
      float* dst = (first && last) ? p.grad_attn_row + (size_t)s * p.H
                                   : p.scratch + slot_index(chunk_id, first) * HP;
      dst[lane / LPH] = total;
    }
  };

  int s = find_seg(p.g.ptr, p.g.nseg, lo);
  int beg = __ldg(p.g.ptr + s);
  float acc = 0.f;  // running sum of row s, head lane / LPH
  float cur[HP], nxt[HP];
  int empties = 0;
  gather(lo + lane, cur);
  for (int base = lo; base < hi; base += 32) {
    gather(base + 32 + lane, nxt);
    const int wend = min(base + 32, hi);
    while (s < p.g.nseg) {
      const int end = __ldg(p.g.ptr + s + 1);
      if (end == beg) {  // rows without edges: walk a few, then jump over the rest of the run
        if (++empties > kEmptyRunWalk) {
          s = find_seg(p.g.ptr, p.g.nseg, beg);
          empties = 0;
        } else {
          ++s;
        }
        continue;
      }
      empties = 0;
      const int a = max(beg, base), b = min(end, wend);
      if (b > a) {
        const bool mine = lane >= a - base && lane < b - base;
        float t[HP];
#pragma unroll
        for (int h = 0; h < HP; ++h) t[h] = mine ? cur[h] : 0.f;
        warp_multi_sum<HP>(t, lane);
        acc += t[0];
      }
      if (end > wend) break;  // the row goes on in the next window (or the next chunk)
      emit(s, acc, beg >= lo, true);
      acc = 0.f;
      beg = end;
      ++s;
      if (beg >= wend) break;
    }
#pragma unroll
    for (int h = 0; h < HP; ++h) cur[h] = nxt[h];
  }
  // a row that runs past the end of the chunk leaves its piece in a slot
  if (s < p.g.nseg && beg < hi && __ldg(p.g.ptr + s + 1) > hi) emit(s, acc, beg >= lo, false);
}

// Merges the pieces of rows that cross chunk boundaries (in chunk order) and zeroes rows
// without edges.
template <int HP>
__global__ void __launch_bounds__(kThreadsPerCta)
row_sum_fixup_kernel(RowSumParams p, int boundary_blocks) {
  const int tid = blockIdx.x * kThreadsPerCta + threadIdx.x;
  if ((int)blockIdx.x < boundary_blocks) {
    const int bnd = 1 + tid;
    if (bnd >= p.g.num_chunks) return;
    const int x = bnd * p.g.chunk;
    const int s = find_seg(p.g.ptr, p.g.nseg, x);
    const int beg = __ldg(p.g.ptr + s);
    if (!(beg < x && beg >= x - p.g.chunk)) return;  // no row starts in chunk bnd-1 and crosses x
    const int end = __ldg(p.g.ptr + s + 1);
    const int c0 = bnd - 1;
    const int c1 = (end - 1) / p.g.chunk;
    float tot[HP];
#pragma unroll
    for (int h = 0; h < HP; ++h) tot[h] = 0.f;
    for (int c = c0; c <= c1; ++c) {
      const float* slot = p.scratch + slot_index(c, c == c0) * HP;
#pragma unroll
      for (int h = 0; h < HP; ++h)
        if (h < p.H) tot[h] += slot[h];
    }
#pragma unroll
    for (int h = 0; h < HP; ++h)
      if (h < p.H) p.grad_attn_row[(size_t)s * p.H + h] = tot[h];
  } else {
    const int s = tid - boundary_blocks * kThreadsPerCta;
    if (s < p.g.nseg && __ldg(p.g.ptr + s) == __ldg(p.g.ptr + s + 1))
      for (int h = 0; h < p.H; ++h) p.grad_attn_row[(size_t)s * p.H + h] = 0.f;
  }
}

template <int HP>
void launch_row_sum(const RowSumParams& p, cudaStream_t stream) {
  if (p.g.num_chunks > 0) {
    const int blocks = (p.g.num_chunks + kWarpsPerCta - 1) / kWarpsPerCta;
    row_sum_kernel<HP><<<blocks, kThreadsPerCta, 0, stream>>>(p);
  }
  const int nbound = p.g.num_chunks > 1 ? p.g.num_chunks - 1 : 0;
  const int bblocks = (nbound + kThreadsPerCta - 1) / kThreadsPerCta;
  const int sblocks = (p.g.nseg + kThreadsPerCta - 1) / kThreadsPerCta;
  if (bblocks + sblocks > 0) row_sum_fixup_kernel<HP><<<bblocks + sblocks, kThreadsPerCta, 0, stream>>>(p, bblocks);
}

}  // namespace

extern "C" int gnn_invert_permutation(const int* perm, int64_t n, int* inv, cudaStream_t stream) {
  if (n < 0) return bad("gnn_invert_permutation: negative size");
  if (n == 0) return GNN_OK;
  if (!perm || !inv) return bad("gnn_invert_permutation: null pointer");
  if (n > INT32_MAX) return bad("gnn_invert_permutation: size exceeds int32 indexing");
  invert_permutation_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(perm, n, inv);
  return check_launch("gnn_invert_permutation");
}

namespace {
int launch_pack(const char* what, int64_t n_rows, const float* out, const float* grad_out, const float* attn_row,
                const float* edge_max, const float* edge_sum, int H, int F, bool elu, float alpha,
                float* grad_pre, float* rowpack, cudaStream_t stream) {
  if (n_rows < 0 || H <= 0 || F <= 0) return bad("gnn_gat_bwd_pack: bad size");
  if (n_rows == 0) return GNN_OK;
  if (!out || !grad_out || !attn_row || !edge_max || !edge_sum || !rowpack || (elu && !grad_pre))
    return bad("gnn_gat_bwd_pack: null pointer");
  const unsigned blocks = (unsigned)((n_rows + kWarpsPerCta - 1) / kWarpsPerCta);
  const bool vec = aligned16(out) && aligned16(grad_out) && (!elu || aligned16(grad_pre)) &&
                   ((int64_t)H * F) % 4 == 0;
  if (vec && F % 4 == 0 && H <= 8 && (int64_t)H * F <= 512) {
    const bool ok = dispatch_tile(next_pow2(H), H * F, true, [&](auto hp, auto q, auto) {
      constexpr int HP = decltype(hp)::value, Q = decltype(q)::value;
      if (elu)
        pack_tile_kernel<HP, Q, true><<<blocks, kThreadsPerCta, 0, stream>>>(n_rows, out, grad_out, attn_row, edge_max,
                                                                           edge_sum, H, F, alpha, grad_pre, rowpack);
      else
        pack_tile_kernel<HP, Q, false><<<blocks, kThreadsPerCta, 0, stream>>>(n_rows, out, grad_out, attn_row, edge_max,
                                                                            edge_sum, H, F, alpha, grad_pre, rowpack);
    });
    if (ok) return check_launch(what);
  }
#define GNN_PACK(V, E)                                                                                     \
  pack_kernel<V, E><<<blocks, kThreadsPerCta, 0, stream>>>(n_rows, out, grad_out, attn_row, edge_max,       \
                                                          edge_sum, H, F, alpha, grad_pre, rowpack)
  if (elu) {
    if (vec) GNN_PACK(true, true); else GNN_PACK(false, true);
  } else {
    if (vec) GNN_PACK(true, false); else GNN_PACK(false, false);
  }
#undef GNN_PACK
  return check_launch(what);
}
}  // namespace

extern "C" int gnn_gat_bwd_pack(int64_t n_rows, const float* out, const float* grad_out,
                                const float* attn_row, const float* edge_max, const float* edge_sum,
                                int H, int F, float* rowpack, cudaStream_t stream) {
  return launch_pack("gnn_gat_bwd_pack", n_rows, out, grad_out, attn_row, edge_max, edge_sum, H, F, false, 0.f,
                     nullptr, rowpack, stream);
}

extern "C" int gnn_gat_bwd_pack_elu(int64_t n_rows, const float* out, const float* grad_act,
                                    const float* attn_row, const float* edge_max, const float* edge_sum,
                                    int H, int F, float alpha, float* grad_pre, float* rowpack,
                                    cudaStream_t stream) {
  return launch_pack("gnn_gat_bwd_pack_elu", n_rows, out, grad_act, attn_row, edge_max, edge_sum, H, F, true,
                     alpha, grad_pre, rowpack, stream);
}

extern "C" int gnn_gat_bwd_row_sum_workspace_bytes(int64_t nnz, int H, size_t* bytes) {
  if (!bytes || nnz < 0 || H <= 0) return bad("gnn_gat_bwd_row_sum_workspace_bytes: bad argument");
  const int chunk = pick_chunk(nnz);
  *bytes = (size_t)num_chunks_for(nnz, chunk) * 2 * 8 * sizeof(float) + 256;
  return GNN_OK;
}

extern "C" int gnn_gat_bwd_row_sum(const int* row_ptr, const int* csr_pos, int64_t n_rows, int64_t nnz,
                                   const float* edge_grad, int H, float* grad_attn_row, void* workspace,
                                   size_t workspace_bytes, cudaStream_t stream) {
  if (n_rows < 0 || nnz < 0 || H <= 0) return bad("gnn_gat_bwd_row_sum: bad size");
  if (H > 8) {
    set_last_error("gnn_gat_bwd_row_sum: H > 8 is not supported");
    return GNN_ERR_UNSUPPORTED;
  }
  if (n_rows > INT32_MAX - 1 || nnz > INT32_MAX - 4096) return bad("gnn_gat_bwd_row_sum: size exceeds int32 indexing");
  if (n_rows == 0) return GNN_OK;
  if (!row_ptr || !grad_attn_row || (nnz && (!csr_pos || !edge_grad))) return bad("gnn_gat_bwd_row_sum: null pointer");
  if (nnz && !aligned16(edge_grad)) return bad("gnn_gat_bwd_row_sum: edge_grad must be 16-byte aligned");
  size_t need = 0;
  gnn_gat_bwd_row_sum_workspace_bytes(nnz, H, &need);
  if (nnz > 0 && (!workspace || workspace_bytes < need)) {
    set_last_error("gnn_gat_bwd_row_sum: workspace too small");
    return GNN_ERR_WORKSPACE;
  }
  const int chunk = pick_chunk(nnz);
  RowSumParams p;
  p.g = ChunkGeom{row_ptr, csr_pos, (int)n_rows, (int)nnz, chunk, num_chunks_for(nnz, chunk)};
  p.edge_grad = edge_grad;
  p.H = H;
  p.grad_attn_row = grad_attn_row;
  p.scratch = (float*)align_up((uintptr_t)workspace, 256);
  if (H == 1) launch_row_sum<1>(p, stream);
  else if (H == 2) launch_row_sum<2>(p, stream);
  else if (H <= 4) launch_row_sum<4>(p, stream);
  else launch_row_sum<8>(p, stream);
  return check_launch("gnn_gat_bwd_row_sum");
}
