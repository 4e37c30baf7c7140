// gnn_gat_fwd_bf16: the fused GAT forward with the gathered feature rows stored as bfloat16.
//
// An opt-in storage mode, outside the fp32 parity contract of the other entry points: the
// gathered operand is what the forward spends its memory traffic on (E x H x F of the
// 4 E (1 + H + H F) bytes per layer), so halving its element size nearly halves the kernel's
// bytes.  Scores, softmax, accumulation and outputs stay fp32; the result equals
// gnn_gat_fwd on the bfloat16-rounded features within fp32 rounding.  The reference has no
// reduced-precision path.
#include "../../include/gnn_b200.h"
#include "wgather.cuh"

using namespace gnn;

namespace {
int bad(const char* msg) {
  set_last_error(msg);
  return GNN_ERR_INVALID_ARG;
}
size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// in[i] (fp32) -> out[i] (bfloat16, round to nearest even); n a multiple of 8, both 16-byte aligned
__global__ void to_bf16_kernel(const float* __restrict__ in, int64_t n8, uint4* __restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const float4 a = __ldg(reinterpret_cast<const float4*>(in) + 2 * i);
  const float4 b = __ldg(reinterpret_cast<const float4*>(in) + 2 * i + 1);
  auto rn = [](float x) -> unsigned {
    const unsigned u = __float_as_uint(x);
    if ((u & 0x7f800000u) == 0x7f800000u) return u >> 16;  // inf / nan: truncate
    return (u + 0x7fffu + ((u >> 16) & 1u)) >> 16;
  };
  uint4 o;
  o.x = rn(a.x) | (rn(a.y) << 16);
  o.y = rn(a.z) | (rn(a.w) << 16);
  o.z = rn(b.x) | (rn(b.y) << 16);
  o.w = rn(b.z) | (rn(b.w) << 16);
  out[i] = o;
}

// The forward kernel for bfloat16 rows.  Same structure as wgather_kernel (one warp per edge
// chunk, online softmax per piece, rows of the next edges requested while the current ones are
// consumed), but the rows in flight are held as the 128-bit words that arrived and widened only
// when they are consumed: a row occupies half the registers of an fp32 row, so twice as many
// rows are in flight per warp.  (With the rows widened on arrival the kernel ran no faster than
// the fp32 one: what bounds the gather is the number of rows in flight times the memory latency,
// not the bytes.)
template <int HP, int Q>
__global__ void __launch_bounds__(kThreadsPerCta)
gat_fwd_bf16_kernel(WGatherParams p, GatSoftmaxPolicy<HP> pol) {
  using Tile = RowTileBf16<Q>;
  constexpr int VW = 8;
  constexpr int U = Q >= 2 ? 4 : 8;
  __shared__ int cs_all[kWarpsPerCta][32];
  __shared__ float ws_all[kWarpsPerCta][32 * HP];
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  const int chunk_id = blockIdx.x * kWarpsPerCta + wib;
  if (chunk_id >= p.g.num_chunks) return;
  int* cs = cs_all[wib];
  float* ws = ws_all[wib];
  Tile t;
  t.init(lane, p.width, p.F, p.H);
  const uint4* rows = reinterpret_cast<const uint4*>(p.feat);
  const size_t ld16 = (size_t)p.ld_feat / 4;  // 16-byte words per row

  for_each_piece(p.g, chunk_id, [&](int s, int a, int b, bool first, bool last) {
    float segw[HP], segm[HP], segs[HP];
#pragma unroll
    for (int h = 0; h < HP; ++h) {
      segw[h] = h < p.H ? __ldg(pol.attn_seg + (size_t)s * pol.ld_attn + h) : 0.f;
      segm[h] = kNegBig;
      segs[h] = 0.f;
    }
    for (int base = a; base < b; base += 32) {
      const int e = base + lane;
      if (e < b) {
        const float* ac = pol.attn_idx + (size_t)__ldg(p.g.idx + e) * pol.ld_attn;
#pragma unroll
        for (int h = 0; h < HP; ++h) {
          if (h < p.H) {
            const float x = leaky_relu(segw[h] + __ldg(ac + h), pol.slope);
            if (x > segm[h]) {
              segs[h] = segs[h] * expf(segm[h] - x) + 1.f;
              segm[h] = x;
            } else {
              segs[h] += expf(x - segm[h]);
            }
          }
        }
      }
    }
#pragma unroll
    for (int h = 0; h < HP; ++h) {
      const float m = warp_max(segm[h]);
      segs[h] = warp_sum(segs[h] * expf(segm[h] - m));
      segm[h] = m;
    }

    float acc[Q][VW];
    t.zero(acc);
    for (int base = a; base < b; base += 32) {
      const int e = base + lane;
      const bool ok = e < b;
      const int c = __ldg(p.g.idx + (ok ? e : a));
      const float* ac = pol.attn_idx + (size_t)c * pol.ld_attn;
      float w[HP];
#pragma unroll
      for (int h = 0; h < HP; ++h) {
        w[h] = 0.f;
        if (h < p.H) w[h] = expf(leaky_relu(segw[h] + __ldg(ac + h), pol.slope) - segm[h]);
      }
      __syncwarp();
      cs[lane] = c;
#pragma unroll
      for (int h = 0; h < HP; ++h) ws[lane * HP + h] = ok ? w[h] : 0.f;
      __syncwarp();
      const int nb = min(32, b - base);
      const int nbr = (nb + U - 1) / U * U;
      auto load_rows = [&](uint4 (&r)[U][Q], int jj) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const uint4* row = rows + (size_t)cs[jj + u] * ld16;
#pragma unroll
          for (int q = 0; q < Q; ++q) r[u][q] = t.valid[q] ? __ldg(row + lane + 32 * q) : make_uint4(0, 0, 0, 0);
        }
      };
      auto accumulate = [&](const uint4 (&r)[U][Q], int jj) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
          for (int q = 0; q < Q; ++q) {
            const float wq = ws[(jj + u) * HP + t.head[q]];
            const unsigned x[4] = {r[u][q].x, r[u][q].y, r[u][q].z, r[u][q].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              acc[q][2 * i] = fmaf(wq, __uint_as_float(x[i] << 16), acc[q][2 * i]);
              acc[q][2 * i + 1] = fmaf(wq, __uint_as_float(x[i] & 0xffff0000u), acc[q][2 * i + 1]);
            }
          }
        }
      };
      uint4 ra[U][Q], rb[U][Q];
      load_rows(ra, 0);
#pragma unroll 1
      for (int jj = 0; jj < nbr; jj += 2 * U) {
        const bool more = jj + U < nbr;
        if (more) load_rows(rb, jj + U);
        accumulate(ra, jj);
        if (more) {
          if (jj + 2 * U < nbr) load_rows(ra, jj + 2 * U);
          accumulate(rb, jj + U);
        }
      }
    }

    if (first && last) {
      finish_segment<GatSoftmaxPolicy, HP, Q, Tile>(p, pol, t, lane, s, acc, segm, segs);
    } else {
      float* slot = p.scratch + slot_index(chunk_id, first) * p.slot_stride;
      t.store(slot, lane, acc);
#pragma unroll
      for (int h = 0; h < HP; ++h) {
        if (lane == h) {
          slot[p.aux_off + h] = segm[h];
          slot[p.aux_off + HP + h] = segs[h];
        }
      }
    }
  });
}

}  // namespace

extern "C" int gnn_to_bf16(const float* in, int64_t n, void* out, cudaStream_t stream) {
  if (n < 0 || n % 8 != 0) return bad("gnn_to_bf16: the element count must be a non-negative multiple of 8");
  if (n == 0) return GNN_OK;
  if (!in || !out || !aligned16(in) || !aligned16(out)) return bad("gnn_to_bf16: pointers must be 16-byte aligned");
  to_bf16_kernel<<<(unsigned)((n / 8 + 255) / 256), 256, 0, stream>>>(in, n / 8, (uint4*)out);
  return check_launch("gnn_to_bf16");
}

extern "C" int gnn_gat_fwd_bf16(const int* row_ptr, const int* col_ind, int64_t n_rows, int64_t nnz,
                                const float* attn_row, const float* attn_col, const void* in_feat_bf16, int H,
                                int F, float negative_slope, float* out, float* edge_max, float* edge_sum,
                                void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  if (n_rows < 0 || nnz < 0 || H <= 0 || F <= 0) return bad("gnn_gat_fwd_bf16: negative size");
  if (n_rows > INT32_MAX - 1 || nnz > INT32_MAX - 4096) return bad("gnn_gat_fwd_bf16: size exceeds int32 indexing");
  if (n_rows == 0) return GNN_OK;
  if (!row_ptr || (!col_ind && nnz) || !attn_row || !attn_col || !in_feat_bf16 || !out || !edge_max || !edge_sum)
    return bad("gnn_gat_fwd_bf16: null pointer");
  const int64_t HF = (int64_t)H * F;
  if (H > 8 || HF > 512 || HF % 8 != 0 || !aligned16(in_feat_bf16) || !aligned16(out)) {
    set_last_error("gnn_gat_fwd_bf16: needs H <= 8, H*F <= 512 and a multiple of 8, 16-byte aligned rows");
    return GNN_ERR_UNSUPPORTED;
  }
  size_t need = 0;
  gnn_gat_fwd_workspace_bytes(nnz, H, F, &need);
  if (nnz > 0 && (!workspace || workspace_bytes < need)) {
    set_last_error("gnn_gat_fwd_bf16: workspace too small");
    return GNN_ERR_WORKSPACE;
  }
  const int chunk = pick_chunk(nnz);
  const int HPv = next_pow2(H);
  WGatherParams p;
  p.g = ChunkGeom{row_ptr, col_ind, (int)n_rows, (int)nnz, chunk, num_chunks_for(nnz, chunk)};
  p.feat = reinterpret_cast<const float*>(in_feat_bf16);
  p.ld_feat = HF / 2;  // a bfloat16 row of HF elements is HF / 2 four-byte units
  p.out = out; p.ld_out = HF;
  p.H = H; p.F = F; p.width = (int)HF;
  p.scratch = (float*)align_up((uintptr_t)workspace, 256);
  p.aux_off = round_up4((int)HF);
  p.slot_stride = p.aux_off + round_up4(2 * HPv);
  p.accumulate = 0;
  p.finalize = 1;
  auto run = [&](auto hp, auto q) {
    constexpr int HP = decltype(hp)::value;
    constexpr int Q = decltype(q)::value;
    GatSoftmaxPolicy<HP> pol;
    pol.attn_seg = attn_row; pol.attn_idx = attn_col; pol.ld_attn = H; pol.slope = negative_slope;
    pol.seg_max = edge_max; pol.seg_sum = edge_sum;
    if (p.g.num_chunks > 0) {
      const int blocks = (p.g.num_chunks + kWarpsPerCta - 1) / kWarpsPerCta;
      gat_fwd_bf16_kernel<HP, Q><<<blocks, kThreadsPerCta, 0, stream>>>(p, pol);
    }
    launch_wgather_fixup<GatSoftmaxPolicy, HP, Q, true, RowTileBf16<Q>>(p, pol, stream);
  };
  using std::integral_constant;
  auto by_q = [&](auto hp) {
    if (HF <= 256) run(hp, integral_constant<int, 1>{});
    else run(hp, integral_constant<int, 2>{});
  };
  switch (HPv) {
    case 1: by_q(integral_constant<int, 1>{}); break;
    case 2: by_q(integral_constant<int, 2>{}); break;
    case 4: by_q(integral_constant<int, 4>{}); break;
    default: by_q(integral_constant<int, 8>{}); break;
  }
  return check_launch("gnn_gat_fwd_bf16");
}
