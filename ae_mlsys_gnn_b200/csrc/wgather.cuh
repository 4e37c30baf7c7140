// Weighted gather-reduce over the segments of a CSR/CSC array:
//   out[s, :] = sum_{e in segment s} w(s, e, idx[e])[head(:)] * feat[idx[e], :]
// with the per-edge, per-head weight w supplied by a policy (GAT attention
// softmax, stored edge values, constant one, Gaussian mixture kernel).
//
// One warp owns one chunk of consecutive edges (see for_each_piece); the lanes
// tile the feature row, so every gathered row is read with whole-warp 128-bit
// loads.  U rows are in flight per lane before the first FMA consumes them.
#pragma once
#include <type_traits>
#include "common.cuh"

namespace gnn {

template <int HP>
__device__ __forceinline__ float pick(const float (&a)[HP], int i) {
  float r = a[0];
#pragma unroll
  for (int h = 1; h < HP; ++h)
    if (i == h) r = a[h];
  return r;
}

template <int Q, bool VEC>
struct Unroll {
  static constexpr int R = Q * (VEC ? 4 : 1);
  static constexpr int U = R >= 16 ? 2 : (R >= 8 ? 4 : 8);
};

// Tile whose gathered rows are bfloat16 (an opt-in storage format of the gathered operand: half
// the bytes per edge, fp32 arithmetic): lane l owns elements (l + 32 q) * 8 + i, i < 8, read as
// one 128-bit word of 8 bfloat16 and widened; rows this kernel writes (outputs, scratch slots)
// stay fp32.  `row` pointers of gathered rows are typed float* but point at bfloat16 data: their
// leading dimension is given in units of 4 bytes.
template <int Q>
struct RowTileBf16 {
  static constexpr int VW = 8;
  bool valid[Q];
  int head[Q];
  __device__ __forceinline__ void init(int lane, int width, int F, int H) {
#pragma unroll
    for (int q = 0; q < Q; ++q) {
      const int e0 = (lane + 32 * q) * VW;
      valid[q] = e0 < width;
      const int h = e0 / F;
      head[q] = h < H ? h : H - 1;
    }
  }
  __device__ __forceinline__ void zero(float (&v)[Q][VW]) const {
#pragma unroll
    for (int q = 0; q < Q; ++q)
#pragma unroll
      for (int i = 0; i < VW; ++i) v[q][i] = 0.f;
  }
  __device__ __forceinline__ void load(const float* __restrict__ row, int lane, float (&v)[Q][VW]) const {
#pragma unroll
    for (int q = 0; q < Q; ++q) {
      if (valid[q]) {
        const uint4 t = __ldg(reinterpret_cast<const uint4*>(row) + lane + 32 * q);
        const unsigned w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {  // a bfloat16 is the upper half of the fp32 with the same value
          v[q][2 * i] = __uint_as_float(w[i] << 16);
          v[q][2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
      } else {
#pragma unroll
        for (int i = 0; i < VW; ++i) v[q][i] = 0.f;
      }
    }
  }
  __device__ __forceinline__ void load_rw(const float* row, int lane, float (&v)[Q][VW]) const {
#pragma unroll
    for (int q = 0; q < Q; ++q) {
      if (valid[q]) {
        const float4 a = *(reinterpret_cast<const float4*>(row) + (lane + 32 * q) * 2);
        const float4 b = *(reinterpret_cast<const float4*>(row) + (lane + 32 * q) * 2 + 1);
        v[q][0] = a.x; v[q][1] = a.y; v[q][2] = a.z; v[q][3] = a.w;
        v[q][4] = b.x; v[q][5] = b.y; v[q][6] = b.z; v[q][7] = b.w;
      } else {
#pragma unroll
        for (int i = 0; i < VW; ++i) v[q][i] = 0.f;
      }
    }
  }
  __device__ __forceinline__ void store(float* __restrict__ row, int lane, const float (&v)[Q][VW]) const {
#pragma unroll
    for (int q = 0; q < Q; ++q) {
      if (valid[q]) {
        float4* d = reinterpret_cast<float4*>(row) + (lane + 32 * q) * 2;
        d[0] = make_float4(v[q][0], v[q][1], v[q][2], v[q][3]);
        d[1] = make_float4(v[q][4], v[q][5], v[q][6], v[q][7]);
      }
    }
  }
};

struct WGatherParams {
  ChunkGeom g;
  const float* feat;   // gathered rows, indexed by idx[e]
  int64_t ld_feat;     // floats between consecutive rows of feat
  float* out;          // [nseg] rows, indexed by segment
  int64_t ld_out;
  int H;               // heads present (<= HP)
  int F;               // floats per head
  int width;           // H * F, floats handled per row
  float* scratch;      // 2 * num_chunks slots of slot_stride floats
  int slot_stride;     // round_up(width, 4) + aux floats, multiple of 4
  int aux_off;         // round_up(width, 4)
  // Several launches may build one result, each over the edges of one column block of
  // the graph (so that a block can be processed as soon as its rows have arrived):
  //   accumulate = 1 : `out` (and the softmax state seg_max / seg_sum) already hold the
  //                    partial result of earlier launches and are merged with this one;
  //   finalize   = 0 : leave the softmax result un-normalised for a later launch.
  // A single launch over the whole graph uses accumulate = 0, finalize = 1.
  int accumulate = 0;
  int finalize = 1;
};

// ----- weight policies ------------------------------------------------------

// GAT: w = exp(LeakyReLU(attn_seg[s,h] + attn_idx[c,h]) - max_s), normalised by
// the segment sum at the end (src/fused_gat/fused_gat_SM.cu:210-284).
template <int HP>
struct GatSoftmaxPolicy {
  static constexpr bool kSoftmax = true;
  static constexpr bool kElu = false;
  const float* attn_seg;  // [nseg][ld_attn]
  const float* attn_idx;  // [*][ld_attn]
  int ld_attn;
  float slope;
  float* seg_max;         // [nseg][ld_attn]
  float* seg_sum;
};

// The same, and next to out[s] the activated row act[s] = ELU(out[s]) is stored: the
// activation a model applies to the layer's output (script/train/train_gatconv_our.py:50-52)
// costs no pass of its own.  The backward needs both: out for the softmax identity and for
// ELU', act as the next layer's input.
template <int HP>
struct GatSoftmaxEluPolicy : GatSoftmaxPolicy<HP> {
  static constexpr bool kElu = true;
  float* act;    // [nseg] rows, leading dimension as `out`
  float alpha;
};

// Stored edge values att[e*ld + h] (nullptr: weight one).  When perm is given
// the value of edge e is att[perm[e]*ld + h].
template <int HP>
struct EdgeValuePolicy {
  static constexpr bool kSoftmax = false;
  static constexpr bool kElu = false;
  const float* att;
  const int* perm;
  int ld_att;
};

// Gaussian mixture weight, head h == mixture kernel k:
//   w = exp(-0.5 * sum_d ((pseudo[pe,d] - mu[k,d]) * inv_sigma[k,d])^2)
// (src/fused_gmmconv/gmmconv.cu:58-68), pe = perm ? perm[e] : e.
template <int HP>
struct GaussPolicy {
  static constexpr bool kSoftmax = false;
  static constexpr bool kElu = false;
  const float* pseudo;  // [E][D]
  const float* mu;      // [K][D]
  const float* inv_sigma;
  const int* perm;
  int D;
};

template <int HP>
__device__ __forceinline__ void edge_weights(const EdgeValuePolicy<HP>& pol,
                                             int H, int e, float (&w)[HP]) {
  if (pol.att == nullptr) {
#pragma unroll
    for (int h = 0; h < HP; ++h) w[h] = h < H ? 1.f : 0.f;
    return;
  }
  const size_t pe = pol.perm ? (size_t)__ldg(pol.perm + e) : (size_t)e;
#pragma unroll
  for (int h = 0; h < HP; ++h)
    w[h] = h < H ? __ldg(pol.att + pe * pol.ld_att + h) : 0.f;
}

template <int HP>
__device__ __forceinline__ void edge_weights(const GaussPolicy<HP>& pol, int H,
                                             int e, float (&w)[HP]) {
  const size_t pe = pol.perm ? (size_t)__ldg(pol.perm + e) : (size_t)e;
  float acc[HP];
#pragma unroll
  for (int h = 0; h < HP; ++h) acc[h] = 0.f;
  for (int d = 0; d < pol.D; ++d) {
    const float pd = __ldg(pol.pseudo + pe * pol.D + d);
#pragma unroll
    for (int h = 0; h < HP; ++h) {
      if (h < H) {
        float t = (pd - __ldg(pol.mu + h * pol.D + d)) *
                  __ldg(pol.inv_sigma + h * pol.D + d);
        acc[h] = fmaf(t, t, acc[h]);
      }
    }
  }
#pragma unroll
  for (int h = 0; h < HP; ++h) w[h] = h < H ? expf(-0.5f * acc[h]) : 0.f;
}

// Final step for one segment whose edges (of this launch) have all been reduced into
// acc (softmax: un-normalised, relative to maximum m, with exp-sum ssum): merge with the
// state left by earlier launches, normalise if asked to, store.
template <template <int> class Policy, int HP, int Q, class Tile>
__device__ __forceinline__ void finish_segment(const WGatherParams& p, const Policy<HP>& pol,
                                               const Tile& t, int lane, int s,
                                               float (&acc)[Q][Tile::VW], float (&m)[HP],
                                               float (&ssum)[HP]) {
  constexpr int VW = Tile::VW;
  float* orow = p.out + (size_t)s * p.ld_out;
  if constexpr (Policy<HP>::kSoftmax) {
    if (p.accumulate) {
      float fo[HP], fn[HP];
#pragma unroll
      for (int h = 0; h < HP; ++h) {
        fo[h] = 0.f; fn[h] = 1.f;
        if (h < p.H) {
          const float mo = pol.seg_max[(size_t)s * pol.ld_attn + h];
          const float so = pol.seg_sum[(size_t)s * pol.ld_attn + h];
          const float M = fmaxf(mo, m[h]);
          fo[h] = expf(mo - M);
          fn[h] = expf(m[h] - M);
          ssum[h] = so * fo[h] + ssum[h] * fn[h];
          m[h] = M;
        }
      }
      float old[Q][VW];
      t.load_rw(orow, lane, old);
#pragma unroll
      for (int q = 0; q < Q; ++q) {
        const float a = pick<HP>(fo, t.head[q]), b = pick<HP>(fn, t.head[q]);
#pragma unroll
        for (int i = 0; i < VW; ++i) acc[q][i] = fmaf(old[q][i], a, acc[q][i] * b);
      }
    }
    if (p.finalize) {
      float inv[HP];
#pragma unroll
      for (int h = 0; h < HP; ++h) inv[h] = 1.f / ssum[h];
#pragma unroll
      for (int q = 0; q < Q; ++q) {
        const float iv = pick<HP>(inv, t.head[q]);
#pragma unroll
        for (int i = 0; i < VW; ++i) acc[q][i] *= iv;
      }
    }
#pragma unroll
    for (int h = 0; h < HP; ++h) {
      if (lane == h && h < p.H) {
        pol.seg_max[(size_t)s * pol.ld_attn + h] = m[h];
        pol.seg_sum[(size_t)s * pol.ld_attn + h] = ssum[h];
      }
    }
  } else {
    if (p.accumulate) {
      float old[Q][VW];
      t.load_rw(orow, lane, old);
#pragma unroll
      for (int q = 0; q < Q; ++q)
#pragma unroll
        for (int i = 0; i < VW; ++i) acc[q][i] += old[q][i];
    }
  }
  t.store(orow, lane, acc);
  if constexpr (Policy<HP>::kElu) {
#pragma unroll
    for (int q = 0; q < Q; ++q)
#pragma unroll
      for (int i = 0; i < VW; ++i)  // exp2-based exponential: absolute error below 1e-6, a few instructions per element
        acc[q][i] = acc[q][i] > 0.f ? acc[q][i] : pol.alpha * (__expf(acc[q][i]) - 1.f);
    t.store(pol.act + (size_t)s * p.ld_out, lane, acc);
  }
}

// ----- main kernel ----------------------------------------------------------

template <template <int> class Policy, int HP, int Q, bool VEC, class Tile = RowTile<Q, VEC>>
__global__ void __launch_bounds__(kThreadsPerCta)
wgather_kernel(WGatherParams p, Policy<HP> pol) {
  constexpr int VW = Tile::VW;
  constexpr int U = Q * VW >= 16 ? 2 : (Q * VW >= 8 ? 4 : 8);
  constexpr bool SOFTMAX = Policy<HP>::kSoftmax;
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

  for_each_piece(p.g, chunk_id, [&](int s, int a, int b, bool first, bool last) {
    float segw[HP];   // GAT: attn_seg[s,h]
    float segm[HP];   // GAT: piece maximum
    float segs[HP];   // GAT: piece sum of exp
#pragma unroll
    for (int h = 0; h < HP; ++h) { segw[h] = 0.f; segm[h] = 0.f; segs[h] = 1.f; }

    if constexpr (SOFTMAX) {
      const auto& gp = pol;
#pragma unroll
      for (int h = 0; h < HP; ++h) {
        segw[h] = h < p.H ? __ldg(gp.attn_seg + (size_t)s * gp.ld_attn + h) : 0.f;
        segm[h] = kNegBig;
        segs[h] = 0.f;
      }
      for (int base = a; base < b; base += 32) {
        const int e = base + lane;
        if (e < b) {
          const int c = __ldg(p.g.idx + e);
          const float* ac = gp.attn_idx + (size_t)c * gp.ld_attn;
#pragma unroll
          for (int h = 0; h < HP; ++h) {
            if (h < p.H) {
              const float x = leaky_relu(segw[h] + __ldg(ac + h), gp.slope);
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
    }

    float acc[Q][VW];
    t.zero(acc);
    for (int base = a; base < b; base += 32) {
      const int e = base + lane;
      const bool ok = e < b;
      const int ee = ok ? e : a;
      const int c = __ldg(p.g.idx + ee);
      float w[HP];
      if constexpr (SOFTMAX) {
        const float* ac = pol.attn_idx + (size_t)c * pol.ld_attn;
#pragma unroll
        for (int h = 0; h < HP; ++h) {
          w[h] = 0.f;
          if (h < p.H)
            w[h] = expf(leaky_relu(segw[h] + __ldg(ac + h), pol.slope) - segm[h]);
        }
      } else {
        edge_weights<HP>(pol, p.H, ee, w);
      }
      __syncwarp();
      cs[lane] = c;
#pragma unroll
      for (int h = 0; h < HP; ++h) ws[lane * HP + h] = ok ? w[h] : 0.f;
      __syncwarp();
      const int nb = min(32, b - base);
      const int nbr = (nb + U - 1) / U * U;
      // Software pipeline: the next U rows are requested before the current U rows are
      // accumulated, so a warp always has gathers in flight.
      auto load_rows = [&](float (&v)[U][Q][VW], int jj) {
#pragma unroll
        for (int u = 0; u < U; ++u)
          t.load(p.feat + (size_t)cs[jj + u] * p.ld_feat, lane, v[u]);
      };
      auto accumulate = [&](float (&v)[U][Q][VW], int jj) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
          for (int q = 0; q < Q; ++q) {
            const float wq = ws[(jj + u) * HP + t.head[q]];
#pragma unroll
            for (int i = 0; i < VW; ++i) acc[q][i] = fmaf(wq, v[u][q][i], acc[q][i]);
          }
        }
      };
      float va[U][Q][VW], vb[U][Q][VW];
      load_rows(va, 0);
#pragma unroll 1
      for (int jj = 0; jj < nbr; jj += 2 * U) {
        const bool more = jj + U < nbr;
        if (more) load_rows(vb, jj + U);
        accumulate(va, jj);
        if (more) {
          if (jj + 2 * U < nbr) load_rows(va, jj + 2 * U);
          accumulate(vb, jj + U);
        }
      }
    }

    if (first && last) {
      finish_segment<Policy, HP, Q, Tile>(p, pol, t, lane, s, acc, segm, segs);
    } else {
      float* slot = p.scratch + slot_index(chunk_id, first) * p.slot_stride;
      t.store(slot, lane, acc);
      if constexpr (SOFTMAX) {
#pragma unroll
        for (int h = 0; h < HP; ++h) {
          if (lane == h) {
            slot[p.aux_off + h] = segm[h];
            slot[p.aux_off + HP + h] = segs[h];
          }
        }
      }
    }
  });
}

// ----- merge of split segments + defaults for empty segments -----------------
//
// Blocks [0, boundary_blocks) : one warp per chunk boundary; the warp whose
//   boundary is the first one inside a segment merges all pieces of that
//   segment in chunk order.
// Blocks [boundary_blocks, ...) : one thread per segment, empty segments get
//   zeros (and, for the softmax policy, max = -1e38 and sum = 0 like the
//   reference's empty rows).
template <template <int> class Policy, int HP, int Q, bool VEC, class Tile = RowTile<Q, VEC>>
__global__ void __launch_bounds__(kThreadsPerCta)
wgather_fixup_kernel(WGatherParams p, Policy<HP> pol, int boundary_blocks) {
  constexpr int VW = Tile::VW;
  constexpr bool SOFTMAX = Policy<HP>::kSoftmax;
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  Tile t;
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
    float m[HP], ssum[HP];
#pragma unroll
    for (int h = 0; h < HP; ++h) { m[h] = kNegBig; ssum[h] = 0.f; }
    if constexpr (SOFTMAX) {
      for (int c = c0; c <= c1; ++c) {
        const float* slot = p.scratch + slot_index(c, c == c0) * p.slot_stride;
#pragma unroll
        for (int h = 0; h < HP; ++h) m[h] = fmaxf(m[h], slot[p.aux_off + h]);
      }
    }
    float acc[Q][VW];
    t.zero(acc);
    for (int c = c0; c <= c1; ++c) {
      const float* slot = p.scratch + slot_index(c, c == c0) * p.slot_stride;
      float v[Q][VW];
      t.load_rw(slot, lane, v);  // slots hold fp32 whatever the gathered rows are
      if constexpr (SOFTMAX) {
        float sc[HP];
#pragma unroll
        for (int h = 0; h < HP; ++h) {
          sc[h] = expf(slot[p.aux_off + h] - m[h]);
          ssum[h] = fmaf(slot[p.aux_off + HP + h], sc[h], ssum[h]);
        }
#pragma unroll
        for (int q = 0; q < Q; ++q) {
          const float f = pick<HP>(sc, t.head[q]);
#pragma unroll
          for (int i = 0; i < VW; ++i) acc[q][i] = fmaf(f, v[q][i], acc[q][i]);
        }
      } else {
#pragma unroll
        for (int q = 0; q < Q; ++q)
#pragma unroll
          for (int i = 0; i < VW; ++i) acc[q][i] += v[q][i];
      }
    }
    finish_segment<Policy, HP, Q, Tile>(p, pol, t, lane, s, acc, m, ssum);
  } else {
    const int s = ((int)blockIdx.x - boundary_blocks) * kThreadsPerCta + threadIdx.x;
    bool empty = false;
    if (s < p.g.nseg) empty = __ldg(p.g.ptr + s) == __ldg(p.g.ptr + s + 1);
    // Segments without edges in this launch: the first launch gives them their defaults;
    // a later, finalising launch normalises what earlier launches accumulated.
    if (p.accumulate && !(SOFTMAX && p.finalize)) return;
    unsigned mask = __ballot_sync(kFull, empty);
    float z[Q][VW];
    t.zero(z);
    while (mask) {
      const int src = __ffs(mask) - 1;
      mask &= mask - 1;
      const int se = s - lane + src;
      if (!p.accumulate) {
        t.store(p.out + (size_t)se * p.ld_out, lane, z);
        if constexpr (Policy<HP>::kElu) t.store(pol.act + (size_t)se * p.ld_out, lane, z);
        if constexpr (SOFTMAX) {
          if (lane < p.H) {
            pol.seg_max[(size_t)se * pol.ld_attn + lane] = kNegBig;
            pol.seg_sum[(size_t)se * pol.ld_attn + lane] = 0.f;
          }
        }
      } else {
        if constexpr (SOFTMAX) {
          float inv[HP];
#pragma unroll
          for (int h = 0; h < HP; ++h) {
            const float sv = h < p.H ? pol.seg_sum[(size_t)se * pol.ld_attn + h] : 0.f;
            inv[h] = sv > 0.f ? 1.f / sv : 0.f;
          }
          float v[Q][VW];
          t.load_rw(p.out + (size_t)se * p.ld_out, lane, v);
#pragma unroll
          for (int q = 0; q < Q; ++q) {
            const float iv = pick<HP>(inv, t.head[q]);
#pragma unroll
            for (int i = 0; i < VW; ++i) v[q][i] *= iv;
          }
          t.store(p.out + (size_t)se * p.ld_out, lane, v);
        }
      }
    }
  }
}

// ----- host-side launch helpers ----------------------------------------------

inline int round_up4(int x) { return (x + 3) / 4 * 4; }

// Floats of scratch one weighted-gather launch needs for (nnz, H, width).
inline size_t wgather_scratch_floats(int64_t nnz, int HP, int width) {
  const int chunk = pick_chunk(nnz);
  const int nc = num_chunks_for(nnz, chunk);
  return (size_t)nc * 2 * (size_t)(round_up4(width) + round_up4(2 * HP));
}

inline int next_pow2(int h) {
  int p = 1;
  while (p < h) p <<= 1;
  return p;
}

// Calls fn(integral_constant<HP>, integral_constant<Q>, bool_constant<VEC>) for
// the smallest instantiated tile that covers `width` floats; false if none.
template <class Fn>
inline bool dispatch_tile(int HP, int width, bool vec, Fn&& fn) {
#define GNN_TILE(hp, q, v)                                            \
  fn(std::integral_constant<int, hp>{}, std::integral_constant<int, q>{}, \
     std::bool_constant<v>{});                                        \
  return true;
#define GNN_TILE_Q(hp)                                     \
  if (vec) {                                               \
    if (width <= 128) { GNN_TILE(hp, 1, true) }            \
    if (width <= 256) { GNN_TILE(hp, 2, true) }            \
    if (width <= 512) { GNN_TILE(hp, 4, true) }            \
  } else {                                                 \
    if (width <= 32) { GNN_TILE(hp, 1, false) }            \
    if (width <= 64) { GNN_TILE(hp, 2, false) }            \
    if (width <= 128) { GNN_TILE(hp, 4, false) }           \
    if (width <= 256) { GNN_TILE(hp, 8, false) }           \
  }                                                        \
  return false;
  switch (HP) {
    case 1: GNN_TILE_Q(1)
    case 2: GNN_TILE_Q(2)
    case 4: GNN_TILE_Q(4)
    case 8: GNN_TILE_Q(8)
    default: return false;
  }
#undef GNN_TILE_Q
#undef GNN_TILE
}

inline int max_tile_width(bool vec) { return vec ? 512 : 256; }

// How (H, F) maps onto the instantiated tiles.
struct HeadPlan {
  bool fused;   // all heads in one launch
  bool vec;     // 128-bit row accesses
  int HP;       // padded head count of the launch
  int slab;     // columns per launch in the per-head fallback
};

inline bool plan_heads(int H, int F, bool aligned, bool need_full_head, HeadPlan* pl) {
  const bool vec = aligned && (F % 4 == 0);
  const int cap = max_tile_width(vec);
  if (H <= 8 && (int64_t)H * F <= cap) {
    pl->fused = true; pl->vec = vec; pl->HP = next_pow2(H); pl->slab = H * F;
    return true;
  }
  if (need_full_head && F > cap) return false;
  pl->fused = false; pl->vec = vec; pl->HP = 1; pl->slab = F < cap ? F : cap;
  return true;
}

// The merge of split segments and the defaults of empty segments (second launch of every
// weighted gather).
template <template <int> class Policy, int HP, int Q, bool VEC, class Tile = RowTile<Q, VEC>>
inline void launch_wgather_fixup(const WGatherParams& p, const Policy<HP>& pol, cudaStream_t stream) {
  const int nbound = p.g.num_chunks > 1 ? p.g.num_chunks - 1 : 0;
  const int bblocks = (nbound + kWarpsPerCta - 1) / kWarpsPerCta;
  const int sblocks = (p.g.nseg + kThreadsPerCta - 1) / kThreadsPerCta;
  if (bblocks + sblocks > 0)
    wgather_fixup_kernel<Policy, HP, Q, VEC, Tile>
        <<<bblocks + sblocks, kThreadsPerCta, 0, stream>>>(p, pol, bblocks);
}

template <template <int> class Policy, int HP, int Q, bool VEC, class Tile = RowTile<Q, VEC>>
inline void launch_wgather(const WGatherParams& p, const Policy<HP>& pol,
                           cudaStream_t stream) {
  if (p.g.num_chunks > 0) {
    const int blocks = (p.g.num_chunks + kWarpsPerCta - 1) / kWarpsPerCta;
    wgather_kernel<Policy, HP, Q, VEC, Tile><<<blocks, kThreadsPerCta, 0, stream>>>(p, pol);
  }
  launch_wgather_fixup<Policy, HP, Q, VEC, Tile>(p, pol, stream);
}

}  // namespace gnn
