// Fused GAT backward, recompute flavour.  Two edge-balanced passes replace the
// reference's three kernels and its E x H temporary
// (src/fused_gat/fused_gat_SM.cu:560-607 mhspmm_backward_kernel, :656-732
// mhsddmm, :734-801 fused_backward_kernel):
//
//  row pass (CSR, segments = destination rows r, gathers h[c]):
//     g_j  = <G[r,h,:], h[c_j,h,:]>            per edge and head
//     a_j  = exp(LeakyReLU(attn_row[r]+attn_col[c_j]) - max[r]) / sum[r]
//     S    = sum_j a_j g_j
//     grad_attn_row[r,h] = sum_j a_j d_j g_j - S * sum_j a_j d_j,
//                          d_j = slope if the activated logit is < 0 else 1
//     rowpack[r] = {attn_row[r,:], max[r,:], 1/sum[r,:], S[:]}
//  col pass (CSC, segments = source columns c, gathers G[r]):
//     grad_feat[c,h,:]   = sum_r a(r,c) G[r,h,:]
//     grad_attn_col[c,h] = sum_r a(r,c) (<G[r,h,:], h[c,h,:]> - S[r,h]) d(r,c)
//
// Both passes are deterministic (no atomics): split segments are merged in
// chunk order by one warp.
//
// A caller that kept the forward output does not need the row pass: S[r] is then
// <G[r], out[r]> (node-wise, gat_bwd_edges.cu), the column pass runs with EDGES and stores
// a(r,c) d(r,c) (<G[r],h[c]> - S[r]) for every edge, and grad_attn_row is the per-row sum of
// those E x H values -- one gather of feature rows per edge instead of two.
#pragma once
#include "wgather.cuh"

namespace gnn {

struct GatBwdRowParams {
  ChunkGeom g;            // CSR: ptr = row_ptr, idx = col_ind
  const float* gout;      // [nseg] rows of grad_out, segment indexed
  int64_t ld_gout;
  const float* feat;      // gathered h rows, indexed by col_ind
  int64_t ld_feat;
  const float* attn_seg;  // attn_row [nseg][ld_attn]
  const float* attn_idx;  // attn_col [*][ld_attn]
  const float* seg_max;   // [nseg][ld_attn]
  const float* seg_sum;
  int ld_attn;
  float slope;
  int H, F, width;
  float* grad_attn_seg;   // [nseg][ld_attn]
  float* rowpack;         // [nseg][4*H]
  float* scratch;         // 2 * num_chunks slots of 4*HP floats
};

// HPS (heads per slot): when F * HPS equals the 128 floats one tile slot spans (128-bit
// accesses), slot q of a lane lies in head q*HPS + lane_head with lane_head = 4*lane/F
// fixed per lane, so the per-head bookkeeping needs HPS selects and no runtime indexing
// of register arrays.  HPS = 0 is the general mapping.
template <int HP, int Q, bool VEC, int HPS = 0>
__global__ void __launch_bounds__(kThreadsPerCta, 2)
gat_bwd_row_kernel(GatBwdRowParams p) {
  static_assert(HPS == 0 || Q * HPS <= HP, "slot-aligned heads need Q * HPS <= HP");
  constexpr int VW = VEC ? 4 : 1;
  constexpr int U0 = Unroll<Q, VEC>::U;
  constexpr int U = (U0 * HP > 32) ? 32 / HP : U0;
  constexpr int V = U * HP;
  constexpr int VA = 4 * HP;  // A1, A2, A3 and one padding group
  __shared__ int cs_all[kWarpsPerCta][32];
  __shared__ float gs_all[kWarpsPerCta][32 * HP];

  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  const int chunk_id = blockIdx.x * kWarpsPerCta + wib;
  if (chunk_id >= p.g.num_chunks) return;
  int* cs = cs_all[wib];
  float* gs = gs_all[wib];
  RowTile<Q, VEC> t;
  t.init(lane, p.width, p.F, p.H);
  const int lane_head = HPS > 1 ? (lane * VW) / p.F : 0;

  for_each_piece(p.g, chunk_id, [&](int s, int a, int b, bool first, bool last) {
    float gq[Q][VW];
    t.load(p.gout + (size_t)s * p.ld_gout, lane, gq);
    float ar[HP], mm[HP], is[HP];
#pragma unroll
    for (int h = 0; h < HP; ++h) {
      ar[h] = 0.f; mm[h] = 0.f; is[h] = 0.f;
      if (h < p.H) {
        ar[h] = __ldg(p.attn_seg + (size_t)s * p.ld_attn + h);
        mm[h] = __ldg(p.seg_max + (size_t)s * p.ld_attn + h);
        is[h] = 1.f / __ldg(p.seg_sum + (size_t)s * p.ld_attn + h);
      }
    }
    float A[VA];
#pragma unroll
    for (int i = 0; i < VA; ++i) A[i] = 0.f;

    for (int base = a; base < b; base += 32) {
      const int e = base + lane;
      const bool ok = e < b;
      const int c = __ldg(p.g.idx + (ok ? e : a));
      float al[HP], dd[HP];
      const float* ac = p.attn_idx + (size_t)c * p.ld_attn;
#pragma unroll
      for (int h = 0; h < HP; ++h) {
        al[h] = 0.f; dd[h] = 1.f;
        if (h < p.H) {
          const float x = leaky_relu(ar[h] + __ldg(ac + h), p.slope);
          al[h] = ok ? expf(x - mm[h]) * is[h] : 0.f;
          dd[h] = x < 0.f ? p.slope : 1.f;
        }
      }
      __syncwarp();
      cs[lane] = c;
      __syncwarp();
      const int nb = min(32, b - base);
      const int nbr = (nb + U - 1) / U * U;
      // Software pipeline: the rows of the next U edges are requested before the dot
      // products of the current U edges are reduced, so the shuffle chain of one group
      // overlaps the gather latency of the next.
      auto load_rows = [&](float (&v)[U][Q][VW], int jj) {
#pragma unroll
        for (int u = 0; u < U; ++u)
          t.load(p.feat + (size_t)cs[jj + u] * p.ld_feat, lane, v[u]);
      };
      auto process = [&](float (&v)[U][Q][VW], int jj) {
        float pv[V];
#pragma unroll
        for (int i = 0; i < V; ++i) pv[i] = 0.f;
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
          for (int q = 0; q < Q; ++q) {
            float d = 0.f;
#pragma unroll
            for (int i = 0; i < VW; ++i) d = fmaf(gq[q][i], v[u][q][i], d);
            if constexpr (HPS > 0) {
#pragma unroll
              for (int k = 0; k < HPS; ++k) pv[u * HP + q * HPS + k] = (lane_head == k) ? d : 0.f;
            } else {
#pragma unroll
              for (int h = 0; h < HP; ++h)
                if (t.head[q] == h) pv[u * HP + h] += d;
            }
          }
        }
        warp_multi_sum<V>(pv, lane);
        if ((lane & (32 / V - 1)) == 0) gs[jj * HP + lane / (32 / V)] = pv[0];
      };
      float va[U][Q][VW], vb[U][Q][VW];
      load_rows(va, 0);
#pragma unroll 1
      for (int jj = 0; jj < nbr; jj += 2 * U) {
        const bool more = jj + U < nbr;
        if (more) load_rows(vb, jj + U);
        process(va, jj);
        if (more) {
          if (jj + 2 * U < nbr) load_rows(va, jj + 2 * U);
          process(vb, jj + U);
        }
      }
      __syncwarp();
      if (ok) {
#pragma unroll
        for (int h = 0; h < HP; ++h) {
          const float gd = gs[lane * HP + h];
          A[h] = fmaf(al[h], gd, A[h]);
          A[HP + h] = fmaf(al[h] * dd[h], gd, A[HP + h]);
          A[2 * HP + h] = fmaf(al[h], dd[h], A[2 * HP + h]);
        }
      }
    }
    warp_multi_sum<VA>(A, lane);
    // value index v = k*HP + h sits on lanes [v*32/VA, (v+1)*32/VA)
    constexpr int LPV = 32 / VA >= 1 ? 32 / VA : 1;
    if (first && last) {
      const int h = lane < HP ? lane : 0;
      const float a1 = __shfl_sync(kFull, A[0], (0 * HP + h) * LPV);
      const float a2 = __shfl_sync(kFull, A[0], (1 * HP + h) * LPV);
      const float a3 = __shfl_sync(kFull, A[0], (2 * HP + h) * LPV);
      if (lane < p.H) {
        p.grad_attn_seg[(size_t)s * p.ld_attn + lane] = a2 - a1 * a3;
        float* rp = p.rowpack + (size_t)s * 4 * p.H;
        rp[lane] = __ldg(p.attn_seg + (size_t)s * p.ld_attn + lane);
        rp[p.H + lane] = __ldg(p.seg_max + (size_t)s * p.ld_attn + lane);
        rp[2 * p.H + lane] = 1.f / __ldg(p.seg_sum + (size_t)s * p.ld_attn + lane);
        rp[3 * p.H + lane] = a1;
      }
    } else {
      float* slot = p.scratch + slot_index(chunk_id, first) * VA;
      if ((lane & (LPV - 1)) == 0) slot[lane / LPV] = A[0];
    }
  });
}

template <int HP>
__global__ void __launch_bounds__(kThreadsPerCta)
gat_bwd_row_fixup_kernel(GatBwdRowParams p, int boundary_blocks) {
  constexpr int VA = 4 * HP;
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  if ((int)blockIdx.x < boundary_blocks) {
    const int bnd = 1 + blockIdx.x * kWarpsPerCta + wib;
    if (bnd >= p.g.num_chunks) return;
    const int x = bnd * p.g.chunk;
    const int s = find_seg(p.g.ptr, p.g.nseg, x);
    const int beg = __ldg(p.g.ptr + s);
    if (!(beg < x && beg >= x - p.g.chunk)) return;
    const int end = __ldg(p.g.ptr + s + 1);
    const int c0 = bnd - 1;
    const int c1 = (end - 1) / p.g.chunk;
    float tot = 0.f;  // lane v < VA sums value v over the pieces
    for (int c = c0; c <= c1; ++c) {
      const float* slot = p.scratch + slot_index(c, c == c0) * VA;
      if (lane < VA) tot += slot[lane];
    }
    const int h = lane < HP ? lane : 0;
    const float a1 = __shfl_sync(kFull, tot, 0 * HP + h);
    const float a2 = __shfl_sync(kFull, tot, 1 * HP + h);
    const float a3 = __shfl_sync(kFull, tot, 2 * HP + h);
    if (lane < p.H) {
      p.grad_attn_seg[(size_t)s * p.ld_attn + lane] = a2 - a1 * a3;
      float* rp = p.rowpack + (size_t)s * 4 * p.H;
      rp[lane] = __ldg(p.attn_seg + (size_t)s * p.ld_attn + lane);
      rp[p.H + lane] = __ldg(p.seg_max + (size_t)s * p.ld_attn + lane);
      rp[2 * p.H + lane] = 1.f / __ldg(p.seg_sum + (size_t)s * p.ld_attn + lane);
      rp[3 * p.H + lane] = a1;
    }
  } else {
    const int s = ((int)blockIdx.x - boundary_blocks) * kThreadsPerCta + threadIdx.x;
    if (s < p.g.nseg && __ldg(p.g.ptr + s) == __ldg(p.g.ptr + s + 1)) {
      for (int h = 0; h < p.H; ++h) {
        p.grad_attn_seg[(size_t)s * p.ld_attn + h] = 0.f;
        float* rp = p.rowpack + (size_t)s * 4 * p.H;
        rp[h] = __ldg(p.attn_seg + (size_t)s * p.ld_attn + h);
        rp[p.H + h] = kNegBig;
        rp[2 * p.H + h] = 0.f;
        rp[3 * p.H + h] = 0.f;
      }
    }
  }
}

struct GatBwdColParams {
  ChunkGeom g;             // CSC: ptr = col_ptr, idx = row_ind
  const float* gout;       // gathered grad_out rows, indexed by row_ind
  int64_t ld_gout;
  const float* feat;       // [nseg] rows of h, segment indexed
  int64_t ld_feat;
  const float* attn_seg;   // attn_col [nseg][ld_attn]
  const float* rowpack;    // [*][4*H], indexed by row_ind
  int ld_attn;
  float slope;
  int H, F, width;
  float* grad_feat;        // [nseg] rows
  int64_t ld_gfeat;
  float* grad_attn_seg;    // grad_attn_col [nseg][ld_attn]
  float* scratch;          // 2 * num_chunks slots of slot_stride floats
  int slot_stride;
  int aux_off;
  int accumulate = 0;      // 1: add to the grad_feat / grad_attn_col left by earlier launches
  float* edge_grad = nullptr;  // [nnz][H], position order of this CSC: gradient of every edge logit
};

// ACC is p.accumulate as a compile-time constant: the plain launch keeps the exact code of
// a kernel without the read-modify-write epilogue (the run-time branch alone changed the
// register allocation of the gather loop and halved its throughput for F = 64).
// EDGES: also store the gradient of every edge logit, a(r,c) d(r,c) (<G[r],h[c]> - S[r]),
// from which the caller sums grad_attn_row without a second gather pass.
template <int Q, bool VEC>
constexpr bool kColPipelined = VEC && Q <= 2;  // 128-bit tiles of at most 8 registers per lane and row

// (Two CTAs per SM are requested only for the pipelined narrow tiles; the widest tile gets
// there by itself, and with the explicit limit its gather loop is scheduled into spills.)
// RING: the gathered rows travel through the per-lane cp.async ring described in common.cuh.
template <int HP, int Q, bool VEC, int HPS = 0, bool ACC = false, bool EDGES = false, bool RING = false>
__global__ void __launch_bounds__(kThreadsPerCta, (kColPipelined<Q, VEC> || RING) ? 2 : 0)
gat_bwd_col_kernel(GatBwdColParams p) {
  static_assert(!RING || VEC, "the ring moves 16-byte units");
  extern __shared__ __align__(16) unsigned char col_ring_smem[];
  static_assert(HPS == 0 || Q * HPS <= HP, "slot-aligned heads need Q * HPS <= HP");
  constexpr int VW = VEC ? 4 : 1;
  constexpr int U0 = Unroll<Q, VEC>::U;
  constexpr int U = (U0 * HP > 32) ? 32 / HP : U0;
  constexpr int V = U * HP;
  constexpr bool PIPE = kColPipelined<Q, VEC> && U == Unroll<Q, VEC>::U;  // both row buffers fit beside the accumulators
  __shared__ int cs_all[kWarpsPerCta][32];
  __shared__ float ws_all[kWarpsPerCta][32 * HP];
  __shared__ float gs_all[kWarpsPerCta][32 * HP];

  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  const int chunk_id = blockIdx.x * kWarpsPerCta + wib;
  if (chunk_id >= p.g.num_chunks) return;
  int* cs = cs_all[wib];
  float* ws = ws_all[wib];
  float* gs = gs_all[wib];
  RowTile<Q, VEC> t;
  t.init(lane, p.width, p.F, p.H);
  const int lane_head = HPS > 1 ? (lane * VW) / p.F : 0;

  for_each_piece(p.g, chunk_id, [&](int s, int a, int b, bool first, bool last) {
    float fq[Q][VW];
    t.load(p.feat + (size_t)s * p.ld_feat, lane, fq);
    float ac[HP];
#pragma unroll
    for (int h = 0; h < HP; ++h)
      ac[h] = h < p.H ? __ldg(p.attn_seg + (size_t)s * p.ld_attn + h) : 0.f;
    float B[HP];
#pragma unroll
    for (int h = 0; h < HP; ++h) B[h] = 0.f;
    float acc[Q][VW];
    t.zero(acc);

    for (int base = a; base < b; base += 32) {
      const int e = base + lane;
      const bool ok = e < b;
      const int r = __ldg(p.g.idx + (ok ? e : a));
      const float* rp = p.rowpack + (size_t)r * 4 * p.H;
      float al[HP], dd[HP], sr[HP];
#pragma unroll
      for (int h = 0; h < HP; ++h) {
        al[h] = 0.f; dd[h] = 1.f; sr[h] = 0.f;
        if (h < p.H) {
          const float x = leaky_relu(__ldg(rp + h) + ac[h], p.slope);
          al[h] = ok ? expf(x - __ldg(rp + p.H + h)) * __ldg(rp + 2 * p.H + h) : 0.f;
          dd[h] = x < 0.f ? p.slope : 1.f;
          sr[h] = __ldg(rp + 3 * p.H + h);
        }
      }
      __syncwarp();
      cs[lane] = r;
#pragma unroll
      for (int h = 0; h < HP; ++h) ws[lane * HP + h] = al[h];
      __syncwarp();
      const int nb = min(32, b - base);
      const int nbr = (nb + U - 1) / U * U;
      if constexpr (PIPE) {
        // Two register buffers: the rows of the next U edges are requested before the
        // current U are consumed (narrow tiles leave the registers for it; without it the
        // throughput of this loop depended on what else the kernel variant contained).
        auto load_rows = [&](float (&v)[U][Q][VW], int jj) {
#pragma unroll
          for (int u = 0; u < U; ++u)
            t.load(p.gout + (size_t)cs[jj + u] * p.ld_gout, lane, v[u]);
        };
        auto process = [&](float (&v)[U][Q][VW], int jj) {
          float pv[V];
#pragma unroll
          for (int i = 0; i < V; ++i) pv[i] = 0.f;
#pragma unroll
          for (int u = 0; u < U; ++u) {
#pragma unroll
            for (int q = 0; q < Q; ++q) {
              const float wq = ws[(jj + u) * HP + (HPS > 0 ? q * HPS + lane_head : t.head[q])];
              float d = 0.f;
#pragma unroll
              for (int i = 0; i < VW; ++i) {
                acc[q][i] = fmaf(wq, v[u][q][i], acc[q][i]);
                d = fmaf(fq[q][i], v[u][q][i], d);
              }
              if constexpr (HPS > 0) {
#pragma unroll
                for (int k = 0; k < HPS; ++k) pv[u * HP + q * HPS + k] = (lane_head == k) ? d : 0.f;
              } else {
#pragma unroll
                for (int h = 0; h < HP; ++h)
                  if (t.head[q] == h) pv[u * HP + h] += d;
              }
            }
          }
          warp_multi_sum<V>(pv, lane);
          if ((lane & (32 / V - 1)) == 0) gs[jj * HP + lane / (32 / V)] = pv[0];
        };
        float va[U][Q][VW], vb[U][Q][VW];
        load_rows(va, 0);
#pragma unroll 1
        for (int jj = 0; jj < nbr; jj += 2 * U) {
          const bool more = jj + U < nbr;
          if (more) load_rows(vb, jj + U);
          process(va, jj);
          if (more) {
            if (jj + 2 * U < nbr) load_rows(va, jj + 2 * U);
            process(vb, jj + U);
          }
        }
      } else if constexpr (RING) {
        constexpr int G = kGatherRingRows / U;  // groups of U rows the ring holds
        static_assert(G >= 2 && G * U == kGatherRingRows, "ring rows must be a multiple of the group");
        float4* const ring = reinterpret_cast<float4*>(col_ring_smem) + (size_t)wib * (kGatherRingRows * Q * 32) + lane;
        auto issue = [&](int g) {  // rows [g*U, g*U + U) of this batch into ring slot g % G
          if (g * U < nbr) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const float4* row = reinterpret_cast<const float4*>(p.gout + (size_t)cs[g * U + u] * p.ld_gout) + lane;
              float4* dst = ring + ((g % G) * U + u) * (Q * 32);
#pragma unroll
              for (int q = 0; q < Q; ++q)
                if (t.valid[q]) cp_async_16(dst + q * 32, row + q * 32);
            }
          }
          cp_async_commit();  // (an empty group keeps the count of pending groups uniform)
        };
#pragma unroll
        for (int g = 0; g < G - 1; ++g) issue(g);
#pragma unroll 1
        for (int g = 0; g * U < nbr; ++g) {
          issue(g + G - 1);       // its slot was consumed in the previous iteration
          cp_async_wait<G - 1>();  // all but the newest G-1 groups have landed: group g is there
          const int jj = g * U;
          float v[U][Q][VW];
#pragma unroll
          for (int u = 0; u < U; ++u) {
#pragma unroll
            for (int q = 0; q < Q; ++q) {
              float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
              if (t.valid[q]) x = ring[((g % G) * U + u) * (Q * 32) + q * 32];
              v[u][q][0] = x.x; v[u][q][1] = x.y; v[u][q][2] = x.z; v[u][q][3] = x.w;
            }
          }
          float pv[V];
#pragma unroll
          for (int i = 0; i < V; ++i) pv[i] = 0.f;
#pragma unroll
          for (int u = 0; u < U; ++u) {
#pragma unroll
            for (int q = 0; q < Q; ++q) {
              const float wq = ws[(jj + u) * HP + (HPS > 0 ? q * HPS + lane_head : t.head[q])];
              float d = 0.f;
#pragma unroll
              for (int i = 0; i < VW; ++i) {
                acc[q][i] = fmaf(wq, v[u][q][i], acc[q][i]);
                d = fmaf(fq[q][i], v[u][q][i], d);
              }
              if constexpr (HPS > 0) {
#pragma unroll
                for (int k = 0; k < HPS; ++k) pv[u * HP + q * HPS + k] = (lane_head == k) ? d : 0.f;
              } else {
#pragma unroll
                for (int h = 0; h < HP; ++h)
                  if (t.head[q] == h) pv[u * HP + h] += d;
              }
            }
          }
          warp_multi_sum<V>(pv, lane);
          if ((lane & (32 / V - 1)) == 0) gs[jj * HP + lane / (32 / V)] = pv[0];
        }
        cp_async_wait<0>();  // only empty groups can be pending here
      } else
      // (the wide tiles keep the plain loop, written out: their register allocation is at
      // the two-CTA limit and changes with the form of this loop)
#pragma unroll 1
      for (int jj = 0; jj < nbr; jj += U) {
        float v[U][Q][VW];
#pragma unroll
        for (int u = 0; u < U; ++u)
          t.load(p.gout + (size_t)cs[jj + u] * p.ld_gout, lane, v[u]);
        float pv[V];
#pragma unroll
        for (int i = 0; i < V; ++i) pv[i] = 0.f;
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
          for (int q = 0; q < Q; ++q) {
            const float wq = ws[(jj + u) * HP + (HPS > 0 ? q * HPS + lane_head : t.head[q])];
            float d = 0.f;
#pragma unroll
            for (int i = 0; i < VW; ++i) {
              acc[q][i] = fmaf(wq, v[u][q][i], acc[q][i]);
              d = fmaf(fq[q][i], v[u][q][i], d);
            }
            if constexpr (HPS > 0) {
#pragma unroll
              for (int k = 0; k < HPS; ++k) pv[u * HP + q * HPS + k] = (lane_head == k) ? d : 0.f;
            } else {
#pragma unroll
              for (int h = 0; h < HP; ++h)
                if (t.head[q] == h) pv[u * HP + h] += d;
            }
          }
        }
        warp_multi_sum<V>(pv, lane);
        if ((lane & (32 / V - 1)) == 0) gs[jj * HP + lane / (32 / V)] = pv[0];
      }
      __syncwarp();
      if (ok) {
#pragma unroll
        for (int h = 0; h < HP; ++h) {
          const float gd = gs[lane * HP + h];
          B[h] = fmaf(al[h] * dd[h], gd - sr[h], B[h]);
        }
        if constexpr (EDGES) {
          float ge[HP];
#pragma unroll
          for (int h = 0; h < HP; ++h) ge[h] = al[h] * dd[h] * (gs[lane * HP + h] - sr[h]);
          float* eg = p.edge_grad + (size_t)e * p.H;
          if (HP == 4 && p.H == 4) {
            *reinterpret_cast<float4*>(eg) = make_float4(ge[0], ge[1], ge[2], ge[3]);
          } else {
#pragma unroll
            for (int h = 0; h < HP; ++h)
              if (h < p.H) eg[h] = ge[h];
          }
        }
      }
    }
    warp_multi_sum<HP>(B, lane);  // head h on lanes [h*32/HP, (h+1)*32/HP)
    constexpr int LPH = 32 / HP;
    if (first && last) {
      float* grow = p.grad_feat + (size_t)s * p.ld_gfeat;
      if constexpr (ACC) {
        float old[Q][VW];
        t.load_rw(grow, lane, old);
#pragma unroll
        for (int q = 0; q < Q; ++q)
#pragma unroll
          for (int i = 0; i < VW; ++i) acc[q][i] += old[q][i];
      }
      t.store(grow, lane, acc);
      if ((lane & (LPH - 1)) == 0 && lane / LPH < p.H) {
        float* ga = p.grad_attn_seg + (size_t)s * p.ld_attn + lane / LPH;
        if constexpr (ACC) *ga += B[0]; else *ga = B[0];
      }
    } else {
      float* slot = p.scratch + slot_index(chunk_id, first) * p.slot_stride;
      t.store(slot, lane, acc);
      if ((lane & (LPH - 1)) == 0) slot[p.aux_off + lane / LPH] = B[0];
    }
  });
}

template <int HP, int Q, bool VEC>
__global__ void __launch_bounds__(kThreadsPerCta)
gat_bwd_col_fixup_kernel(GatBwdColParams p, int boundary_blocks) {
  constexpr int VW = VEC ? 4 : 1;
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  RowTile<Q, VEC> t;
  t.init(lane, p.width, p.F, p.H);
  if ((int)blockIdx.x < boundary_blocks) {
    const int bnd = 1 + blockIdx.x * kWarpsPerCta + wib;
    if (bnd >= p.g.num_chunks) return;
    const int x = bnd * p.g.chunk;
    const int s = find_seg(p.g.ptr, p.g.nseg, x);
    const int beg = __ldg(p.g.ptr + s);
    if (!(beg < x && beg >= x - p.g.chunk)) return;
    const int end = __ldg(p.g.ptr + s + 1);
    const int c0 = bnd - 1;
    const int c1 = (end - 1) / p.g.chunk;
    float acc[Q][VW];
    t.zero(acc);
    float bt = 0.f;
    for (int c = c0; c <= c1; ++c) {
      const float* slot = p.scratch + slot_index(c, c == c0) * p.slot_stride;
      float v[Q][VW];
      t.load(slot, lane, v);
#pragma unroll
      for (int q = 0; q < Q; ++q)
#pragma unroll
        for (int i = 0; i < VW; ++i) acc[q][i] += v[q][i];
      if (lane < HP) bt += slot[p.aux_off + lane];
    }
    float* grow = p.grad_feat + (size_t)s * p.ld_gfeat;
    if (p.accumulate) {
      float old[Q][VW];
      t.load_rw(grow, lane, old);
#pragma unroll
      for (int q = 0; q < Q; ++q)
#pragma unroll
        for (int i = 0; i < VW; ++i) acc[q][i] += old[q][i];
    }
    t.store(grow, lane, acc);
    if (lane < p.H) {
      float* ga = p.grad_attn_seg + (size_t)s * p.ld_attn + lane;
      *ga = p.accumulate ? *ga + bt : bt;
    }
  } else {
    if (p.accumulate) return;  // segments without edges in this launch keep what they have
    const int s = ((int)blockIdx.x - boundary_blocks) * kThreadsPerCta + threadIdx.x;
    bool empty = false;
    if (s < p.g.nseg) empty = __ldg(p.g.ptr + s) == __ldg(p.g.ptr + s + 1);
    unsigned mask = __ballot_sync(kFull, empty);
    float z[Q][VW];
    t.zero(z);
    while (mask) {
      const int src = __ffs(mask) - 1;
      mask &= mask - 1;
      const int se = s - lane + src;
      t.store(p.grad_feat + (size_t)se * p.ld_gfeat, lane, z);
      if (lane < p.H) p.grad_attn_seg[(size_t)se * p.ld_attn + lane] = 0.f;
    }
  }
}

}  // namespace gnn
