// Fused GAT forward and backward column pass for one head with a narrow feature row (at most 64
// floats: the 1 x 47 / 1 x 41 / 1 x 7 output layers and their 16-byte-pitch forms 1 x 48 / 44 / 8).
// Same mathematics, chunk traversal, scratch slots and merge kernels as the general kernels
// (wgather.cuh, gat_bwd.cuh); what differs is the tiling of the warp:
//
//   general tile : 32 lanes share one gathered row (lane l owns floats l, l+32, ...).  With 47
//                  floats half of the second load is idle and every edge costs its own
//                  address arithmetic, weight fetch and (backward) 5-step warp reduction.
//   here         : the warp is cut into R = 32/LPR sub-warps of LPR lanes; sub-warp g works
//                  on edge j*R + g.  One warp instruction therefore serves R edges, the per-edge
//                  dot product of the backward is a log2(LPR)-step reduction that R edges
//                  share, and R*U rows are in flight per warp.  A lane owns floats i, i+LPR, ...
//                  (rows that rule out 128-bit accesses: 188 / 164 / 28 bytes) or, for rows of
//                  whole 16-byte units, the four consecutive floats 4i .. 4i+3.
//
// Measured on a 1 M-node / 42 M-edge R-MAT graph, 1 x 47: forward 1.90 -> 1.55 ms, column pass
// with edge gradients about 3.9 -> 2.27 ms.  What bounds the scalar form is the first-level cache's
// line look-ups (a 188-byte row starts anywhere in a 128-byte line, every 64-byte piece of it
// costs one or two look-ups, and the 4-byte gather of the source's score another): holding all
// 32 rows of a batch in flight with fewer resident warps was measured slower.  On a 2.45 M-node /
// 125 M-edge graph, 1 x 48 against 1 x 47: forward 4.65 -> 4.30 ms, column pass 7.04 -> 5.27 ms
// (with its rows in the shared-memory ring below; the same ring made the forward slower).
//
// Replaces, for these shapes, fused_forward_kernel_small_f_sm and
// mhspmm_backward_kernel_small_f + mhsddmm + fused_backward_kernel
// (src/fused_gat/fused_gat_SM.cu:380-489, :609-654, :656-801).
#pragma once
#include "gat_bwd.cuh"

namespace gnn {

// VEC (rows of a multiple of 4 floats, 16-byte aligned): lane i owns the four consecutive floats
// 4i .. 4i+3 (Q == 4) and moves them with one 128-bit access; otherwise it owns floats
// i, i+LPR, ... and moves them one by one.
template <int LPR, int Q, bool VEC = false>
struct SubTile {
  static_assert(!VEC || Q == 4, "a 128-bit unit is four floats");
  static constexpr int R = 32 / LPR;
  int sub;       // lane inside the sub-warp
  int grp;       // sub-warp index
  bool valid[Q];
  __device__ __forceinline__ int elem(int q) const { return VEC ? sub * 4 + q : sub + LPR * q; }
  __device__ __forceinline__ void init(int lane, int width) {
    sub = lane & (LPR - 1);
    grp = lane / LPR;
#pragma unroll
    for (int q = 0; q < Q; ++q) valid[q] = elem(q) < width;
  }
  __device__ __forceinline__ void load(const float* __restrict__ row, float (&v)[Q]) const {
    if constexpr (VEC) {
      float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
      if (valid[0]) x = __ldg(reinterpret_cast<const float4*>(row) + sub);
      v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
    } else {
#pragma unroll
      for (int q = 0; q < Q; ++q) v[q] = valid[q] ? __ldg(row + sub + LPR * q) : 0.f;
    }
  }
  // the same with an ordinary load, for rows this kernel also writes
  __device__ __forceinline__ void load_rw(const float* row, float (&v)[Q]) const {
    if constexpr (VEC) {
      float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
      if (valid[0]) x = *(reinterpret_cast<const float4*>(row) + sub);
      v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
    } else {
#pragma unroll
      for (int q = 0; q < Q; ++q) v[q] = valid[q] ? row[sub + LPR * q] : 0.f;
    }
  }
  // Sum over the R sub-warps; every sub-warp ends with the total.
  __device__ __forceinline__ void reduce_groups(float (&v)[Q]) const {
#pragma unroll
    for (int s = LPR; s < 32; s <<= 1)
#pragma unroll
      for (int q = 0; q < Q; ++q) v[q] += __shfl_xor_sync(kFull, v[q], s);
  }
  // Sum over the lanes of one sub-warp (all R sub-warps at once).
  __device__ __forceinline__ float reduce_lanes(float d) const {
#pragma unroll
    for (int s = LPR / 2; s > 0; s >>= 1) d += __shfl_xor_sync(kFull, d, s);
    return d;
  }
  // Element k of a row lives at row[k]: the scratch slots and outputs keep the plain layout,
  // so the merge kernels of the general tile read them unchanged.
  __device__ __forceinline__ void store(float* row, const float (&v)[Q]) const {
    if (grp == 0) {
      if constexpr (VEC) {
        if (valid[0]) reinterpret_cast<float4*>(row)[sub] = make_float4(v[0], v[1], v[2], v[3]);
      } else {
#pragma unroll
        for (int q = 0; q < Q; ++q)
          if (valid[q]) row[sub + LPR * q] = v[q];
      }
    }
  }
};

// Rows in flight per sub-warp before the first FMA consumes them.
template <int Q>
struct NarrowUnroll { static constexpr int U = Q >= 3 ? 4 : 8; };

// ---- forward ------------------------------------------------------------------------------
// p.H == 1, p.width <= LPR * Q.  Writes out / seg_max / seg_sum (or scratch slots for the
// pieces of split rows) exactly like wgather_kernel<GatSoftmaxPolicy, 1, ., false>.
template <int LPR, int Q, bool VEC = false>
__global__ void __launch_bounds__(kThreadsPerCta)
gat_fwd_narrow_kernel(WGatherParams p, GatSoftmaxPolicy<1> pol) {
  using Tile = SubTile<LPR, Q, VEC>;
  constexpr int R = Tile::R;
  constexpr int U = NarrowUnroll<Q>::U;
  __shared__ int cs_all[kWarpsPerCta][32];
  __shared__ float ws_all[kWarpsPerCta][32];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int chunk_id = blockIdx.x * kWarpsPerCta + wib;
  if (chunk_id >= p.g.num_chunks) return;
  int* cs = cs_all[wib];
  float* ws = ws_all[wib];
  Tile t;
  t.init(lane, p.width);

  for_each_piece(p.g, chunk_id, [&](int s, int a, int b, bool first, bool last) {
    const float segw = __ldg(pol.attn_seg + (size_t)s * pol.ld_attn);
    float m = kNegBig, ssum = 0.f;
    for (int base = a; base < b; base += 32) {
      const int e = base + lane;
      if (e < b) {
        const float x = leaky_relu(segw + __ldg(pol.attn_idx + (size_t)__ldg(p.g.idx + e) * pol.ld_attn), pol.slope);
        if (x > m) {
          ssum = ssum * expf(m - x) + 1.f;
          m = x;
        } else {
          ssum += expf(x - m);
        }
      }
    }
    {
      const float mm = warp_max(m);
      ssum = warp_sum(ssum * expf(m - mm));
      m = mm;
    }

    float acc[Q];
#pragma unroll
    for (int q = 0; q < Q; ++q) acc[q] = 0.f;
    for (int base = a; base < b; base += 32) {
      const int e = base + lane;
      const bool ok = e < b;
      const int c = __ldg(p.g.idx + (ok ? e : a));
      const float w = ok ? expf(leaky_relu(segw + __ldg(pol.attn_idx + (size_t)c * pol.ld_attn), pol.slope) - m) : 0.f;
      __syncwarp();
      cs[lane] = c;
      ws[lane] = w;
      __syncwarp();
      const int nb = min(32, b - base);
#pragma unroll 1
      for (int jj = 0; jj < nb; jj += R * U) {
        float v[U][Q];
        float wv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int j = jj + u * R + t.grp;  // < 32 always: R * U divides 32
          wv[u] = ws[j];                     // 0 past the end of the batch
          t.load(p.feat + (size_t)cs[j] * p.ld_feat, v[u]);
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
          for (int q = 0; q < Q; ++q) acc[q] = fmaf(wv[u], v[u][q], acc[q]);
      }
    }
    t.reduce_groups(acc);

    if (first && last) {
      float* orow = p.out + (size_t)s * p.ld_out;
      if (p.accumulate) {
        const float mo = pol.seg_max[(size_t)s * pol.ld_attn];
        const float so = pol.seg_sum[(size_t)s * pol.ld_attn];
        const float M = fmaxf(mo, m);
        const float fo = expf(mo - M), fn = expf(m - M);
        ssum = so * fo + ssum * fn;
        m = M;
        float old[Q];
        t.load_rw(orow, old);
#pragma unroll
        for (int q = 0; q < Q; ++q) acc[q] = fmaf(old[q], fo, acc[q] * fn);
      }
      if (p.finalize) {
        const float inv = 1.f / ssum;
#pragma unroll
        for (int q = 0; q < Q; ++q) acc[q] *= inv;
      }
      if (lane == 0) {
        pol.seg_max[(size_t)s * pol.ld_attn] = m;
        pol.seg_sum[(size_t)s * pol.ld_attn] = ssum;
      }
      t.store(orow, acc);
    } else {
      float* slot = p.scratch + slot_index(chunk_id, first) * p.slot_stride;
      t.store(slot, acc);
      if (lane == 0) {
        slot[p.aux_off] = m;
        slot[p.aux_off + 1] = ssum;
      }
    }
  });
}

// ---- backward column pass -------------------------------------------------------------------
// p.H == 1, p.width <= LPR * Q; same outputs and scratch layout as
// gat_bwd_col_kernel<1, ., false, 0, ACC, EDGES>.
// RING (VEC only): the lane's 16-byte unit of each gathered row goes through a ring of
// kNarrowRingSlots slots per lane in shared memory (cp.async, groups of two rows), as in the wide
// tile: rows stay in flight while earlier ones are reduced.
constexpr int kNarrowRingSlots = 8;
constexpr size_t kNarrowRingBytes = (size_t)kWarpsPerCta * kNarrowRingSlots * 32 * sizeof(float4);

template <int LPR, int Q, bool ACC, bool EDGES, bool VEC = false, bool RING = false>
__global__ void __launch_bounds__(kThreadsPerCta)
gat_bwd_col_narrow_kernel(GatBwdColParams p) {
  static_assert(!RING || VEC, "the ring moves 16-byte units");
  using Tile = SubTile<LPR, Q, VEC>;
  constexpr int R = Tile::R;
  constexpr int U = RING ? 2 : NarrowUnroll<Q>::U;
  extern __shared__ __align__(16) unsigned char narrow_ring_smem[];
  __shared__ int cs_all[kWarpsPerCta][32];
  __shared__ float ws_all[kWarpsPerCta][32];
  __shared__ float gs_all[kWarpsPerCta][32];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int chunk_id = blockIdx.x * kWarpsPerCta + wib;
  if (chunk_id >= p.g.num_chunks) return;
  int* cs = cs_all[wib];
  float* ws = ws_all[wib];
  float* gs = gs_all[wib];
  Tile t;
  t.init(lane, p.width);

  for_each_piece(p.g, chunk_id, [&](int s, int a, int b, bool first, bool last) {
    float fq[Q];
    t.load(p.feat + (size_t)s * p.ld_feat, fq);
    const float ac = __ldg(p.attn_seg + (size_t)s * p.ld_attn);
    float B = 0.f;
    float acc[Q];
#pragma unroll
    for (int q = 0; q < Q; ++q) acc[q] = 0.f;

    for (int base = a; base < b; base += 32) {
      const int e = base + lane;
      const bool ok = e < b;
      const int r = __ldg(p.g.idx + (ok ? e : a));
      const float4 rp = __ldg(reinterpret_cast<const float4*>(p.rowpack) + r);  // {attn_row, max, 1/sum, S}
      const float x = leaky_relu(rp.x + ac, p.slope);
      const float al = ok ? expf(x - rp.y) * rp.z : 0.f;
      const float dd = x < 0.f ? p.slope : 1.f;
      __syncwarp();
      cs[lane] = r;
      ws[lane] = al;
      __syncwarp();
      const int nb = min(32, b - base);
      [[maybe_unused]] float4* const ring =
          reinterpret_cast<float4*>(narrow_ring_smem) + (size_t)wib * (kNarrowRingSlots * 32) + lane;
      constexpr int G = kNarrowRingSlots / U;           // groups of U rows per lane the ring holds
      [[maybe_unused]] auto issue = [&](int g) {        // rows jj = g*R*U of this batch, this sub-warp's share
        const int jj = g * R * U;
        if (jj < nb) {
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int j = jj + u * R + t.grp;
            if (t.valid[0])
              cp_async_16(ring + ((g % G) * U + u) * 32,
                          reinterpret_cast<const float4*>(p.gout + (size_t)cs[j] * p.ld_gout) + t.sub);
          }
        }
        cp_async_commit();
      };
      if constexpr (RING) {
#pragma unroll
        for (int g = 0; g < G - 1; ++g) issue(g);
      }
#pragma unroll 1
      for (int jj = 0; jj < nb; jj += R * U) {
        float v[U][Q];
        float wv[U];
        if constexpr (RING) {
          const int g = jj / (R * U);
          issue(g + G - 1);
          cp_async_wait<G - 1>();
#pragma unroll
          for (int u = 0; u < U; ++u) {
            wv[u] = ws[jj + u * R + t.grp];
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t.valid[0]) x = ring[((g % G) * U + u) * 32];
            v[u][0] = x.x; v[u][1] = x.y; v[u][2] = x.z; v[u][3] = x.w;
          }
        } else {
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int j = jj + u * R + t.grp;
            wv[u] = ws[j];
            t.load(p.gout + (size_t)cs[j] * p.ld_gout, v[u]);
          }
        }
        float d[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          d[u] = 0.f;
#pragma unroll
          for (int q = 0; q < Q; ++q) {
            acc[q] = fmaf(wv[u], v[u][q], acc[q]);
            d[u] = fmaf(fq[q], v[u][q], d[u]);
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) d[u] = t.reduce_lanes(d[u]);
        if (t.sub == 0) {
#pragma unroll
          for (int u = 0; u < U; ++u) gs[jj + u * R + t.grp] = d[u];
        }
      }
      if constexpr (RING) cp_async_wait<0>();  // only empty groups can be pending
      __syncwarp();
      if (ok) {
        const float ge = al * dd * (gs[lane] - rp.w);
        B += ge;
        if constexpr (EDGES) p.edge_grad[e] = ge;
      }
    }
    t.reduce_groups(acc);
    B = warp_sum(B);
    if (first && last) {
      float* grow = p.grad_feat + (size_t)s * p.ld_gfeat;
      if constexpr (ACC) {
        float old[Q];
        t.load_rw(grow, old);
#pragma unroll
        for (int q = 0; q < Q; ++q) acc[q] += old[q];
      }
      t.store(grow, acc);
      if (lane == 0) {
        float* ga = p.grad_attn_seg + (size_t)s * p.ld_attn;
        if constexpr (ACC) *ga += B; else *ga = B;
      }
    } else {
      float* slot = p.scratch + slot_index(chunk_id, first) * p.slot_stride;
      t.store(slot, acc);
      if (lane == 0) slot[p.aux_off] = B;
    }
  });
}

}  // namespace gnn
