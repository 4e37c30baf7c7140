// gnn_gat_fwd_act: the fused GAT forward that also writes ELU(out).
//
// The benchmark models apply ELU to the output of every hidden GAT layer
// (script/train/train_gatconv_our.py:50-52 stores the activation the layer is meant to apply).
// As a framework op that is one more read and write of an N x H x F matrix per layer; here the
// warp that has just normalised a row stores the activated row next to it.  The pre-activation
// output is still written: the backward takes S = <grad, out> and ELU' from it.
#include "../../include/gnn_b200.h"
#include "wgather.cuh"

using namespace gnn;

namespace {
int bad(const char* msg) {
  set_last_error(msg);
  return GNN_ERR_INVALID_ARG;
}
size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
}  // namespace

extern "C" int gnn_gat_fwd_act(const int* row_ptr, const int* col_ind, int64_t n_rows, int64_t nnz,
                               const float* attn_row, const float* attn_col, const float* in_feat, int H,
                               int F, float negative_slope, float alpha, float* out, float* act_out,
                               float* edge_max, float* edge_sum, void* workspace, size_t workspace_bytes,
                               cudaStream_t stream) {
  if (n_rows < 0 || nnz < 0 || H <= 0 || F <= 0) return bad("gnn_gat_fwd_act: negative size");
  if (n_rows > INT32_MAX - 1 || nnz > INT32_MAX - 4096) return bad("gnn_gat_fwd_act: size exceeds int32 indexing");
  if (n_rows == 0) return GNN_OK;
  if (!row_ptr || (!col_ind && nnz) || !attn_row || !attn_col || !in_feat || !out || !act_out || !edge_max ||
      !edge_sum)
    return bad("gnn_gat_fwd_act: null pointer");
  const int64_t HF = (int64_t)H * F;
  const bool aligned = aligned16(in_feat) && aligned16(out) && aligned16(act_out) && HF % 4 == 0;
  HeadPlan pl;
  if (!plan_heads(H, F, aligned, false, &pl) || !pl.fused) {
    set_last_error("gnn_gat_fwd_act: H > 8 or H*F beyond the largest tile (512 floats aligned / 256); "
                   "use gnn_gat_fwd and activate separately");
    return GNN_ERR_UNSUPPORTED;
  }
  size_t need = 0;
  gnn_gat_fwd_workspace_bytes(nnz, H, F, &need);
  if (nnz > 0 && (!workspace || workspace_bytes < need)) {
    set_last_error("gnn_gat_fwd_act: workspace too small");
    return GNN_ERR_WORKSPACE;
  }
  const int chunk = pick_chunk(nnz);
  WGatherParams p;
  p.g = ChunkGeom{row_ptr, col_ind, (int)n_rows, (int)nnz, chunk, num_chunks_for(nnz, chunk)};
  p.feat = in_feat; p.ld_feat = HF;
  p.out = out; p.ld_out = HF;
  p.H = H; p.F = F; p.width = (int)HF;
  p.scratch = (float*)align_up((uintptr_t)workspace, 256);
  p.aux_off = round_up4((int)HF);
  p.slot_stride = p.aux_off + round_up4(2 * pl.HP);
  p.accumulate = 0;
  p.finalize = 1;
  bool ok = dispatch_tile(pl.HP, (int)HF, pl.vec, [&](auto hp, auto q, auto v) {
    constexpr int HP = decltype(hp)::value;
    GatSoftmaxEluPolicy<HP> pol;
    pol.attn_seg = attn_row; pol.attn_idx = attn_col; pol.ld_attn = H; pol.slope = negative_slope;
    pol.seg_max = edge_max; pol.seg_sum = edge_sum;
    pol.act = act_out; pol.alpha = alpha;
    launch_wgather<GatSoftmaxEluPolicy, HP, decltype(q)::value, decltype(v)::value>(p, pol, stream);
  });
  if (!ok) {
    set_last_error("gnn_gat_fwd_act: no tile for this shape");
    return GNN_ERR_UNSUPPORTED;
  }
  return check_launch("gnn_gat_fwd_act");
}
