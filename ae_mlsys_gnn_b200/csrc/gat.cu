// C-ABI entry points of the fused GAT forward / backward.
#include <stdlib.h>
#include "../../include/gnn_b200.h"
#include "gat_narrow.cuh"

using namespace gnn;

namespace {

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// One head, rows of at most 64 floats that cannot be read with 128-bit accesses: the
// sub-warp tiles of gat_narrow.cuh (several rows per warp instruction).
// (GNN_B200_NARROW=0 in the environment keeps the general tile: for A/B timing of the two.)
bool narrow_shape(const HeadPlan& pl, int H, int64_t width) {
  static const bool enabled = [] {
    const char* e = getenv("GNN_B200_NARROW");
    return !(e && e[0] == '0');
  }();
  return enabled && pl.fused && H == 1 && width <= 64;
}

// Calls fn(integral_constant<LPR>, integral_constant<Q>, bool_constant<VEC>) for the sub-warp tile covering
// `width` floats: VEC (rows of whole 16-byte units) gives every lane four consecutive floats.
template <bool VEC, class Fn>
void dispatch_narrow(int width, Fn&& fn) {
  using std::integral_constant;
  if constexpr (VEC) {
    using V = std::bool_constant<true>;
    if (width <= 16) fn(integral_constant<int, 4>{}, integral_constant<int, 4>{}, V{});
    else if (width <= 32) fn(integral_constant<int, 8>{}, integral_constant<int, 4>{}, V{});
    else fn(integral_constant<int, 16>{}, integral_constant<int, 4>{}, V{});
  } else {
    using V = std::bool_constant<false>;
    if (width <= 8) fn(integral_constant<int, 8>{}, integral_constant<int, 1>{}, V{});
    else if (width <= 16) fn(integral_constant<int, 16>{}, integral_constant<int, 1>{}, V{});
    else if (width <= 32) fn(integral_constant<int, 16>{}, integral_constant<int, 2>{}, V{});
    else if (width <= 48) fn(integral_constant<int, 16>{}, integral_constant<int, 3>{}, V{});
    else fn(integral_constant<int, 16>{}, integral_constant<int, 4>{}, V{});
  }
}

int bad(const char* msg) {
  set_last_error(msg);
  return GNN_ERR_INVALID_ARG;
}

}  // namespace

extern "C" int gnn_gat_fwd_workspace_bytes(int64_t nnz, int H, int F, size_t* bytes) {
  if (!bytes || nnz < 0 || H <= 0 || F <= 0) return bad("gnn_gat_fwd_workspace_bytes: bad argument");
  HeadPlan pl;
  plan_heads(H, F, true, false, &pl);
  const size_t a = wgather_scratch_floats(nnz, pl.HP, pl.slab);
  HeadPlan ps;
  plan_heads(H, F, false, false, &ps);
  const size_t b = wgather_scratch_floats(nnz, ps.HP, ps.slab);
  *bytes = (a > b ? a : b) * sizeof(float) + 256;
  return GNN_OK;
}

extern "C" int gnn_gat_fwd(const int* row_ptr, const int* col_ind, int64_t n_rows,
                           int64_t nnz, const float* attn_row, const float* attn_col,
                           const float* in_feat, int H, int F, float negative_slope,
                           float* out, float* edge_max, float* edge_sum,
                           void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  return gnn_gat_fwd_part(row_ptr, col_ind, n_rows, nnz, attn_row, attn_col, in_feat, H, F,
                          negative_slope, out, edge_max, edge_sum, 0, 1, workspace, workspace_bytes,
                          stream);
}

extern "C" int gnn_gat_fwd_part(const int* row_ptr, const int* col_ind, int64_t n_rows,
                                int64_t nnz, const float* attn_row, const float* attn_col,
                                const float* in_feat, int H, int F, float negative_slope,
                                float* out, float* edge_max, float* edge_sum, int accumulate,
                                int finalize, void* workspace, size_t workspace_bytes,
                                cudaStream_t stream) {
  if (n_rows < 0 || nnz < 0 || H <= 0 || F <= 0) return bad("gnn_gat_fwd: negative size");
  if (n_rows > INT32_MAX - 1 || nnz > INT32_MAX - 4096) return bad("gnn_gat_fwd: size exceeds int32 indexing");
  if (n_rows == 0) return GNN_OK;
  if (!row_ptr || (!col_ind && nnz) || !attn_row || !attn_col || !in_feat || !out || !edge_max || !edge_sum)
    return bad("gnn_gat_fwd: null pointer");
  const int64_t HF = (int64_t)H * F;
  const bool aligned = aligned16(in_feat) && aligned16(out) && HF % 4 == 0;
  HeadPlan pl;
  if (!plan_heads(H, F, aligned, false, &pl)) {
    set_last_error("gnn_gat_fwd: unsupported shape");
    return GNN_ERR_UNSUPPORTED;
  }
  if (!pl.fused && F > pl.slab && (accumulate || !finalize)) {
    // every column slab of a head re-derives the head's softmax state from its own launch; a
    // second slab would merge against state the first slab of the same call already merged
    set_last_error("gnn_gat_fwd_part: launches over column blocks need the per-head width within one tile "
                   "(512 floats aligned / 256 otherwise)");
    return GNN_ERR_UNSUPPORTED;
  }
  size_t need = 0;
  gnn_gat_fwd_workspace_bytes(nnz, H, F, &need);
  if (nnz > 0 && (!workspace || workspace_bytes < need)) {
    set_last_error("gnn_gat_fwd: workspace too small");
    return GNN_ERR_WORKSPACE;
  }
  float* scratch = (float*)align_up((uintptr_t)workspace, 256);

  const int chunk = pick_chunk(nnz);
  ChunkGeom g{row_ptr, col_ind, (int)n_rows, (int)nnz, chunk, num_chunks_for(nnz, chunk)};
  const int nh = pl.fused ? 1 : H;
  for (int h = 0; h < nh; ++h) {
    const int Hh = pl.fused ? H : 1;
    for (int f0 = 0; f0 < (pl.fused ? 1 : F); f0 += pl.slab) {
      const int w = pl.fused ? (int)HF : (F - f0 < pl.slab ? F - f0 : pl.slab);
      const int64_t off = pl.fused ? 0 : (int64_t)h * F + f0;
      WGatherParams p;
      p.g = g;
      p.feat = in_feat + off; p.ld_feat = HF;
      p.out = out + off; p.ld_out = HF;
      p.H = Hh; p.F = pl.fused ? F : w; p.width = w;
      p.scratch = scratch;
      p.aux_off = round_up4(w);
      p.slot_stride = p.aux_off + round_up4(2 * pl.HP);
      p.accumulate = accumulate ? 1 : 0;
      p.finalize = finalize ? 1 : 0;
      const bool narrow = narrow_shape(pl, H, w);
      bool ok = dispatch_tile(pl.HP, w, pl.vec, [&](auto hp, auto q, auto v) {
        constexpr int HP = decltype(hp)::value;
        GatSoftmaxPolicy<HP> pol;
        pol.attn_seg = attn_row + (pl.fused ? 0 : h);
        pol.attn_idx = attn_col + (pl.fused ? 0 : h);
        pol.ld_attn = H;
        pol.slope = negative_slope;
        pol.seg_max = edge_max + (pl.fused ? 0 : h);
        pol.seg_sum = edge_sum + (pl.fused ? 0 : h);
        if constexpr (HP == 1) {
          if (narrow) {  // sub-warp main kernel; the merge kernel of the general tile reads its slots
            if (p.g.num_chunks > 0) {
              const int blocks = (p.g.num_chunks + kWarpsPerCta - 1) / kWarpsPerCta;
              dispatch_narrow<decltype(v)::value>(w, [&](auto lpr, auto nq, auto nv) {
                gat_fwd_narrow_kernel<decltype(lpr)::value, decltype(nq)::value, decltype(nv)::value>
                    <<<blocks, kThreadsPerCta, 0, stream>>>(p, pol);
              });
            }
            launch_wgather_fixup<GatSoftmaxPolicy, HP, decltype(q)::value, decltype(v)::value>(p, pol, stream);
            return;
          }
        }
        launch_wgather<GatSoftmaxPolicy, HP, decltype(q)::value, decltype(v)::value>(p, pol, stream);
      });
      if (!ok) {
        set_last_error("gnn_gat_fwd: no tile for this shape");
        return GNN_ERR_UNSUPPORTED;
      }
    }
  }
  return check_launch("gnn_gat_fwd");
}

// ---------------------------------------------------------------------------

namespace {

size_t bwd_scratch_floats(int64_t nnz, int HP, int width) {
  const size_t col = wgather_scratch_floats(nnz, HP, width);
  const int chunk = pick_chunk(nnz);
  const size_t row = (size_t)num_chunks_for(nnz, chunk) * 2 * 4 * HP;
  return col > row ? col : row;
}

template <int HP, int Q, bool VEC>
void launch_row(const GatBwdRowParams& p, cudaStream_t stream) {
  if (p.g.num_chunks > 0) {
    const int blocks = (p.g.num_chunks + kWarpsPerCta - 1) / kWarpsPerCta;
    bool done = false;
    if constexpr (VEC) {
      if (p.width == 128 * Q) {  // every slot fully used: heads are aligned with the tile slots
        if constexpr (Q <= HP) {
          if (p.F == 128) { gat_bwd_row_kernel<HP, Q, VEC, 1><<<blocks, kThreadsPerCta, 0, stream>>>(p); done = true; }
        }
        if constexpr (2 * Q <= HP) {
          if (p.F == 64) { gat_bwd_row_kernel<HP, Q, VEC, 2><<<blocks, kThreadsPerCta, 0, stream>>>(p); done = true; }
        }
      }
    }
    if (!done) gat_bwd_row_kernel<HP, Q, VEC><<<blocks, kThreadsPerCta, 0, stream>>>(p);
  }
  const int nbound = p.g.num_chunks > 1 ? p.g.num_chunks - 1 : 0;
  const int bblocks = (nbound + kWarpsPerCta - 1) / kWarpsPerCta;
  const int sblocks = (p.g.nseg + kThreadsPerCta - 1) / kThreadsPerCta;
  if (bblocks + sblocks > 0)
    gat_bwd_row_fixup_kernel<HP><<<bblocks + sblocks, kThreadsPerCta, 0, stream>>>(p, bblocks);
}

template <int HP, int Q, bool VEC, bool ACC, bool EDGES>
void launch_col_main(const GatBwdColParams& p, cudaStream_t stream) {
  const int blocks = (p.g.num_chunks + kWarpsPerCta - 1) / kWarpsPerCta;
  if constexpr (VEC && Q >= 3 && Q <= HP) {  // the widest tiles (rows of more than 256 floats): rows in flight in shared memory
    static const bool ring = [] {
      const char* e = getenv("GNN_B200_COL_RING");
      return e ? atoi(e) != 0 : true;
    }();
    if (ring && p.width == 128 * Q && p.F == 128) {
      auto kernel = gat_bwd_col_kernel<HP, Q, VEC, 1, ACC, EDGES, true>;
      // more than 48 KB of dynamic shared memory needs this opt-in once per device and kernel
      static bool opted[64] = {};
      int dev = 0;
      cudaGetDevice(&dev);
      bool ready = dev >= 0 && dev < 64 && opted[dev];
      if (!ready && cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)gather_ring_bytes<Q>()) == cudaSuccess) {
        ready = true;
        if (dev >= 0 && dev < 64) opted[dev] = true;
      }
      if (ready) {
        kernel<<<blocks, kThreadsPerCta, gather_ring_bytes<Q>(), stream>>>(p);
        return;
      }
    }
  }
  if constexpr (VEC) {
    if (p.width == 128 * Q) {  // every slot fully used: heads are aligned with the tile slots
      if constexpr (Q <= HP) {
        if (p.F == 128) { gat_bwd_col_kernel<HP, Q, VEC, 1, ACC, EDGES><<<blocks, kThreadsPerCta, 0, stream>>>(p); return; }
      }
      if constexpr (2 * Q <= HP) {
        if (p.F == 64) { gat_bwd_col_kernel<HP, Q, VEC, 2, ACC, EDGES><<<blocks, kThreadsPerCta, 0, stream>>>(p); return; }
      }
    }
  }
  gat_bwd_col_kernel<HP, Q, VEC, 0, ACC, EDGES><<<blocks, kThreadsPerCta, 0, stream>>>(p);
}

template <bool ACC, bool EDGES, bool VEC>
void launch_col_narrow(const GatBwdColParams& p, cudaStream_t stream) {
  const int blocks = (p.g.num_chunks + kWarpsPerCta - 1) / kWarpsPerCta;
  dispatch_narrow<VEC>(p.width, [&](auto lpr, auto nq, auto nv) {
    if constexpr (decltype(nv)::value) {
      static const bool ring = [] {
        const char* e = getenv("GNN_B200_NARROW_RING");
        return e ? atoi(e) != 0 : true;
      }();
      if (ring) {  // 32 KB of dynamic shared memory: within the default limit, no opt-in needed
        gat_bwd_col_narrow_kernel<decltype(lpr)::value, decltype(nq)::value, ACC, EDGES, true, true>
            <<<blocks, kThreadsPerCta, kNarrowRingBytes, stream>>>(p);
        return;
      }
    }
    gat_bwd_col_narrow_kernel<decltype(lpr)::value, decltype(nq)::value, ACC, EDGES, decltype(nv)::value>
        <<<blocks, kThreadsPerCta, 0, stream>>>(p);
  });
}

template <int HP, int Q, bool VEC>
void launch_col(const GatBwdColParams& p, cudaStream_t stream, bool narrow = false) {
  if (p.g.num_chunks > 0 && narrow) {
    if (p.edge_grad) {
      if (p.accumulate) launch_col_narrow<true, true, VEC>(p, stream);
      else launch_col_narrow<false, true, VEC>(p, stream);
    } else {
      if (p.accumulate) launch_col_narrow<true, false, VEC>(p, stream);
      else launch_col_narrow<false, false, VEC>(p, stream);
    }
  } else if (p.g.num_chunks > 0) {
    if (p.edge_grad) {
      if (p.accumulate) launch_col_main<HP, Q, VEC, true, true>(p, stream);
      else launch_col_main<HP, Q, VEC, false, true>(p, stream);
    } else {
      if (p.accumulate) launch_col_main<HP, Q, VEC, true, false>(p, stream);
      else launch_col_main<HP, Q, VEC, false, false>(p, stream);
    }
  }
  const int nbound = p.g.num_chunks > 1 ? p.g.num_chunks - 1 : 0;
  const int bblocks = (nbound + kWarpsPerCta - 1) / kWarpsPerCta;
  const int sblocks = (p.g.nseg + kThreadsPerCta - 1) / kThreadsPerCta;
  if (bblocks + sblocks > 0)
    gat_bwd_col_fixup_kernel<HP, Q, VEC><<<bblocks + sblocks, kThreadsPerCta, 0, stream>>>(p, bblocks);
}

}  // namespace

extern "C" int gnn_gat_bwd_row_workspace_bytes(int64_t nnz, int H, int F, size_t* bytes) {
  if (!bytes || nnz < 0 || H <= 0 || F <= 0) return bad("gnn_gat_bwd_row_workspace_bytes: bad argument");
  HeadPlan pl;
  if (!plan_heads(H, F, true, true, &pl)) plan_heads(H, 1, false, true, &pl);
  const int chunk = pick_chunk(nnz);
  *bytes = (size_t)num_chunks_for(nnz, chunk) * 2 * 4 * 8 * sizeof(float) + 256;
  return GNN_OK;
}

extern "C" int gnn_gat_bwd_col_workspace_bytes(int64_t nnz, int H, int F, size_t* bytes) {
  if (!bytes || nnz < 0 || H <= 0 || F <= 0) return bad("gnn_gat_bwd_col_workspace_bytes: bad argument");
  HeadPlan pl, ps;
  size_t a = 0, b = 0;
  if (plan_heads(H, F, true, true, &pl)) a = wgather_scratch_floats(nnz, pl.HP, pl.slab);
  if (plan_heads(H, F, false, true, &ps)) b = wgather_scratch_floats(nnz, ps.HP, ps.slab);
  *bytes = (a > b ? a : b) * sizeof(float) + 256;
  return GNN_OK;
}

extern "C" int gnn_gat_bwd_row(const int* row_ptr, const int* col_ind, int64_t n_rows,
                               int64_t nnz, const float* edge_max, const float* edge_sum,
                               const float* in_feat, const float* attn_row,
                               const float* attn_col, const float* grad_out, int H, int F,
                               float negative_slope, float* grad_attn_row, float* rowpack,
                               void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  if (n_rows < 0 || nnz < 0 || H <= 0 || F <= 0) return bad("gnn_gat_bwd_row: negative size");
  if (n_rows > INT32_MAX - 1 || nnz > INT32_MAX - 4096) return bad("gnn_gat_bwd_row: size exceeds int32 indexing");
  if (n_rows == 0) return GNN_OK;
  if (!row_ptr || (!col_ind && nnz) || !edge_max || !edge_sum || !in_feat || !attn_row ||
      !attn_col || !grad_out || !grad_attn_row || !rowpack)
    return bad("gnn_gat_bwd_row: null pointer");
  const int64_t HF = (int64_t)H * F;
  const bool aligned = aligned16(in_feat) && aligned16(grad_out) && HF % 4 == 0;
  HeadPlan pl;
  if (!plan_heads(H, F, aligned, true, &pl)) {
    set_last_error("gnn_gat_bwd_row: per-head width beyond the largest tile");
    return GNN_ERR_UNSUPPORTED;
  }
  if (!pl.fused) {
    set_last_error("gnn_gat_bwd_row: H > 8 or H*F beyond the largest tile is not supported");
    return GNN_ERR_UNSUPPORTED;
  }
  size_t need = 0;
  gnn_gat_bwd_row_workspace_bytes(nnz, H, F, &need);
  if (nnz > 0 && (!workspace || workspace_bytes < need)) {
    set_last_error("gnn_gat_bwd_row: workspace too small");
    return GNN_ERR_WORKSPACE;
  }
  const int chunk = pick_chunk(nnz);
  GatBwdRowParams p;
  p.g = ChunkGeom{row_ptr, col_ind, (int)n_rows, (int)nnz, chunk, num_chunks_for(nnz, chunk)};
  p.gout = grad_out; p.ld_gout = HF;
  p.feat = in_feat; p.ld_feat = HF;
  p.attn_seg = attn_row; p.attn_idx = attn_col;
  p.seg_max = edge_max; p.seg_sum = edge_sum;
  p.ld_attn = H; p.slope = negative_slope;
  p.H = H; p.F = F; p.width = (int)HF;
  p.grad_attn_seg = grad_attn_row; p.rowpack = rowpack;
  p.scratch = (float*)align_up((uintptr_t)workspace, 256);
  bool ok = dispatch_tile(pl.HP, (int)HF, pl.vec, [&](auto hp, auto q, auto v) {
    launch_row<decltype(hp)::value, decltype(q)::value, decltype(v)::value>(p, stream);
  });
  if (!ok) {
    set_last_error("gnn_gat_bwd_row: no tile for this shape");
    return GNN_ERR_UNSUPPORTED;
  }
  return check_launch("gnn_gat_bwd_row");
}

extern "C" int gnn_gat_bwd_col(const int* col_ptr, const int* row_ind, int64_t n_cols,
                               int64_t nnz, const float* in_feat, const float* attn_col,
                               const float* rowpack, const float* grad_out, int H, int F,
                               float negative_slope, float* grad_feat, float* grad_attn_col,
                               void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  return gnn_gat_bwd_col_part(col_ptr, row_ind, n_cols, nnz, in_feat, attn_col, rowpack, grad_out, H,
                              F, negative_slope, grad_feat, grad_attn_col, 0, workspace,
                              workspace_bytes, stream);
}

extern "C" int gnn_gat_bwd_col_part(const int* col_ptr, const int* row_ind, int64_t n_cols,
                                    int64_t nnz, const float* in_feat, const float* attn_col,
                                    const float* rowpack, const float* grad_out, int H, int F,
                                    float negative_slope, float* grad_feat, float* grad_attn_col,
                                    int accumulate, void* workspace, size_t workspace_bytes,
                                    cudaStream_t stream) {
  return gnn_gat_bwd_col_edges(col_ptr, row_ind, n_cols, nnz, in_feat, attn_col, rowpack, grad_out, H, F,
                               negative_slope, grad_feat, grad_attn_col, nullptr, accumulate, workspace,
                               workspace_bytes, stream);
}

extern "C" int gnn_gat_bwd_col_edges(const int* col_ptr, const int* row_ind, int64_t n_cols,
                                     int64_t nnz, const float* in_feat, const float* attn_col,
                                     const float* rowpack, const float* grad_out, int H, int F,
                                     float negative_slope, float* grad_feat, float* grad_attn_col,
                                     float* edge_grad, int accumulate, void* workspace,
                                     size_t workspace_bytes, cudaStream_t stream) {
  if (edge_grad && !aligned16(edge_grad)) return bad("gnn_gat_bwd_col: edge_grad must be 16-byte aligned");
  if (n_cols < 0 || nnz < 0 || H <= 0 || F <= 0) return bad("gnn_gat_bwd_col: negative size");
  if (n_cols > INT32_MAX - 1 || nnz > INT32_MAX - 4096) return bad("gnn_gat_bwd_col: size exceeds int32 indexing");
  if (n_cols == 0) return GNN_OK;
  if (!col_ptr || (!row_ind && nnz) || !in_feat || !attn_col || !rowpack || !grad_out ||
      !grad_feat || !grad_attn_col)
    return bad("gnn_gat_bwd_col: null pointer");
  const int64_t HF = (int64_t)H * F;
  const bool aligned = aligned16(in_feat) && aligned16(grad_out) && aligned16(grad_feat) && HF % 4 == 0;
  HeadPlan pl;
  if (!plan_heads(H, F, aligned, true, &pl) || !pl.fused) {
    set_last_error("gnn_gat_bwd_col: H > 8 or H*F beyond the largest tile is not supported");
    return GNN_ERR_UNSUPPORTED;
  }
  size_t need = 0;
  gnn_gat_bwd_col_workspace_bytes(nnz, H, F, &need);
  if (nnz > 0 && (!workspace || workspace_bytes < need)) {
    set_last_error("gnn_gat_bwd_col: workspace too small");
    return GNN_ERR_WORKSPACE;
  }
  const int chunk = pick_chunk(nnz);
  GatBwdColParams p;
  p.g = ChunkGeom{col_ptr, row_ind, (int)n_cols, (int)nnz, chunk, num_chunks_for(nnz, chunk)};
  p.gout = grad_out; p.ld_gout = HF;
  p.feat = in_feat; p.ld_feat = HF;
  p.attn_seg = attn_col; p.rowpack = rowpack;
  p.ld_attn = H; p.slope = negative_slope;
  p.H = H; p.F = F; p.width = (int)HF;
  p.grad_feat = grad_feat; p.ld_gfeat = HF;
  p.grad_attn_seg = grad_attn_col;
  p.scratch = (float*)align_up((uintptr_t)workspace, 256);
  p.aux_off = round_up4((int)HF);
  p.slot_stride = p.aux_off + round_up4(2 * pl.HP);
  p.accumulate = accumulate ? 1 : 0;
  p.edge_grad = edge_grad;
  // the sub-warp kernel reads the per-row record {attn_row, max, 1/sum, S} as one 128-bit word
  const bool narrow = narrow_shape(pl, H, HF) && aligned16(rowpack);
  bool ok = dispatch_tile(pl.HP, (int)HF, pl.vec, [&](auto hp, auto q, auto v) {
    launch_col<decltype(hp)::value, decltype(q)::value, decltype(v)::value>(p, stream, narrow);
  });
  if (!ok) {
    set_last_error("gnn_gat_bwd_col: no tile for this shape");
    return GNN_ERR_UNSUPPORTED;
  }
  return check_launch("gnn_gat_bwd_col");
}

extern "C" int gnn_gat_bwd_workspace_bytes(int64_t n_rows, int64_t nnz, int H, int F, size_t* bytes) {
  if (!bytes || n_rows < 0) return bad("gnn_gat_bwd_workspace_bytes: bad argument");
  size_t a = 0, b = 0;
  int rc = gnn_gat_bwd_row_workspace_bytes(nnz, H, F, &a);
  if (rc) return rc;
  rc = gnn_gat_bwd_col_workspace_bytes(nnz, H, F, &b);
  if (rc) return rc;
  *bytes = align_up((size_t)n_rows * 4 * H * sizeof(float), 256) + (a > b ? a : b) + 256;
  return GNN_OK;
}

extern "C" int gnn_gat_bwd(const int* row_ptr, const int* col_ind, const int* col_ptr,
                           const int* row_ind, int64_t n, int64_t nnz, const float* edge_max,
                           const float* edge_sum, const float* in_feat, const float* attn_row,
                           const float* attn_col, const float* grad_out, int H, int F,
                           float negative_slope, float* grad_feat, float* grad_attn_row,
                           float* grad_attn_col, void* workspace, size_t workspace_bytes,
                           cudaStream_t stream) {
  size_t need = 0;
  int rc = gnn_gat_bwd_workspace_bytes(n, nnz, H, F, &need);
  if (rc) return rc;
  if (n == 0) return GNN_OK;
  if (!workspace || workspace_bytes < need) {
    set_last_error("gnn_gat_bwd: workspace too small");
    return GNN_ERR_WORKSPACE;
  }
  char* base = (char*)align_up((uintptr_t)workspace, 256);
  float* rowpack = (float*)base;
  const size_t pack_bytes = align_up((size_t)n * 4 * H * sizeof(float), 256);
  void* scratch = base + pack_bytes;
  const size_t scratch_bytes = workspace_bytes - (size_t)((char*)scratch - (char*)workspace);
  rc = gnn_gat_bwd_row(row_ptr, col_ind, n, nnz, edge_max, edge_sum, in_feat, attn_row,
                       attn_col, grad_out, H, F, negative_slope, grad_attn_row, rowpack,
                       scratch, scratch_bytes, stream);
  if (rc) return rc;
  return gnn_gat_bwd_col(col_ptr, row_ind, n, nnz, in_feat, attn_col, rowpack, grad_out, H, F,
                         negative_slope, grad_feat, grad_attn_col, scratch, scratch_bytes, stream);
}

// ---------------------------------------------------------------------------
// gnn_gat_fwd_static_scratch: gnn_gat_fwd for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc (or torch's allocator) at
// the point where they run a layer: an inference server that has handed all
// device memory to its own pool at start-up, a plugin that runs inside
// somebody else's memory plan, code on a latency-critical path where an
// allocation could synchronise the device.  For them the scratch that
// gnn_gat_fwd needs for rows split across edge chunks lives in a fixed array
// inside the library's device image instead of a caller-provided workspace.
//
//  * The array is GNN_STATIC_SCRATCH_BYTES (16 MiB) and every GPU that loads
//    the library holds it until the process exits.
//  * A problem whose gnn_gat_fwd_workspace_bytes() exceeds that size is refused
//    with GNN_ERR_LIMIT; nothing is launched.
//  * The first call on each device looks the array's device address up
//    (cudaGetSymbolAddress, with that device current) and remembers it; make
//    that first call before any stream capture begins.
//  * All calls share the one array and it keeps whatever the previous call left
//    in it.  Nothing in it has to start at zero: every slot a merge reads was
//    written earlier in the same call.  Two calls that overlap on the GPU
//    (different streams, or different host threads) race on it and give wrong
//    results; run them one after the other on one stream.
namespace {

static __device__ __align__(256) unsigned char g_static_scratch[GNN_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void* g_static_scratch_addr[kMaxDevices] = {nullptr};

// Device address of g_static_scratch on the current device.  In host code the
// symbol itself is only a handle, never a device pointer, hence the lookup.
int static_scratch_address(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    set_last_error("gnn_gat_fwd_static_scratch: cannot identify the current device");
    return GNN_ERR_CUDA;
  }
  if (g_static_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_last_error(cudaGetErrorString(e));
      return GNN_ERR_CUDA;
    }
    g_static_scratch_addr[dev] = p;
  }
  *out = g_static_scratch_addr[dev];
  return GNN_OK;
}

}  // namespace

extern "C" int gnn_gat_fwd_static_scratch(const int* row_ptr, const int* col_ind, int64_t n_rows,
                                          int64_t nnz, const float* attn_row,
                                          const float* attn_col, const float* in_feat, int H,
                                          int F, float negative_slope, float* out,
                                          float* edge_max, float* edge_sum, cudaStream_t stream) {
  size_t need = 0;
  int rc = gnn_gat_fwd_workspace_bytes(nnz, H, F, &need);
  if (rc) return rc;
  if (need > (size_t)GNN_STATIC_SCRATCH_BYTES) {
    set_last_error("gnn_gat_fwd_static_scratch: this problem needs more scratch than the 16 MiB "
                   "built into the library; use gnn_gat_fwd with a caller-provided workspace");
    return GNN_ERR_LIMIT;
  }
  void* scratch = nullptr;
  rc = static_scratch_address(&scratch);
  if (rc) return rc;
  return gnn_gat_fwd(row_ptr, col_ind, n_rows, nnz, attn_row, attn_col, in_feat, H, F,
                     negative_slope, out, edge_max, edge_sum, scratch,
                     (size_t)GNN_STATIC_SCRATCH_BYTES, stream);
}
