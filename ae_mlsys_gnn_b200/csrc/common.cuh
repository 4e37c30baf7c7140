// Shared device helpers for the sm_100a sparse kernels: error codes, warp
// reductions, the edge-chunk traversal of a CSR/CSC segment array, and the
// per-lane tiling of a dense feature row.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "../../include/gnn_b200.h"

namespace gnn {

constexpr int kWarpsPerCta = 8;
constexpr int kThreadsPerCta = kWarpsPerCta * 32;
constexpr unsigned kFull = 0xffffffffu;
// Row maximum used for a segment without edges; the reference starts its
// running maximum at the same value (src/fused_gat/fused_gat_SM.cu:213).
constexpr float kNegBig = -1e38f;

void set_last_error(const char* msg);
int check_launch(const char* what);

__device__ __forceinline__ float leaky_relu(float x, float slope) {
  return x > 0.f ? x : x * slope;
}

// Last segment s in [0, nseg) with ptr[s] <= x.  For 0 <= x < ptr[nseg] this is
// the non-empty segment that contains position x.
__device__ __forceinline__ int find_seg(const int* __restrict__ ptr, int nseg,
                                        int x) {
  int lo = 0, hi = nseg;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (__ldg(ptr + mid) <= x)
      lo = mid;
    else
      hi = mid;
  }
  return lo;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(kFull, v, s);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v = fmaxf(v, __shfl_xor_sync(kFull, v, s));
  return v;
}

// Sums V (a power of two, <= 32) per-lane values across the warp with
// V-1 + log2(32/V) shuffles.  On return x[0] of lane L holds the total of value
// index L >> log2(32/V), i.e. value v is replicated on lanes [v*32/V,(v+1)*32/V).
template <int V>
__device__ __forceinline__ void warp_multi_sum(float (&x)[V], int lane) {
  static_assert(V >= 1 && V <= 32 && (V & (V - 1)) == 0, "V must be 2^k <= 32");
  int s = 16;
#pragma unroll
  for (int n = V; n > 1; n >>= 1) {
    const bool up = (lane & s) != 0;
#pragma unroll
    for (int i = 0; i < n / 2; ++i) {
      float keep = up ? x[i + n / 2] : x[i];
      float send = up ? x[i] : x[i + n / 2];
      x[i] = keep + __shfl_xor_sync(kFull, send, s);
    }
    s >>= 1;
  }
#pragma unroll
  for (; s > 0; s >>= 1) x[0] += __shfl_xor_sync(kFull, x[0], s);
}

// ---------------------------------------------------------------------------
// Per-lane tiling of one dense row of `width` floats.  Lane l owns elements
// (l + 32 q) * VW + i for q < Q, i < VW, where VW = 4 for 128-bit accesses
// (width % 4 == 0, 16-byte aligned rows) and VW = 1 otherwise.  Every load of a
// warp therefore covers one contiguous 512-byte (or 128-byte) span.
template <int Q, bool VEC>
struct RowTile {
  static constexpr int VW = VEC ? 4 : 1;
  bool valid[Q];
  int head[Q];  // head (sub-row of length F) that slot q of this lane lies in

  __device__ __forceinline__ void init(int lane, int width, int F, int H) {
#pragma unroll
    for (int q = 0; q < Q; ++q) {
      int e0 = (lane + 32 * q) * VW;
      valid[q] = e0 < width;
      int h = e0 / F;
      head[q] = h < H ? h : H - 1;
    }
  }
  __device__ __forceinline__ void zero(float (&v)[Q][VW]) const {
#pragma unroll
    for (int q = 0; q < Q; ++q)
#pragma unroll
      for (int i = 0; i < VW; ++i) v[q][i] = 0.f;
  }
  __device__ __forceinline__ void load(const float* __restrict__ row, int lane,
                                       float (&v)[Q][VW]) const {
#pragma unroll
    for (int q = 0; q < Q; ++q) {
      if (valid[q]) {
        if constexpr (VEC) {
          float4 t = __ldg(reinterpret_cast<const float4*>(row) + lane + 32 * q);
          v[q][0] = t.x; v[q][1] = t.y; v[q][2] = t.z; v[q][3] = t.w;
        } else {
          v[q][0] = __ldg(row + lane + 32 * q);
        }
      } else {
#pragma unroll
        for (int i = 0; i < VW; ++i) v[q][i] = 0.f;
      }
    }
  }
  // Same as load, with ordinary (coherent) loads: for rows this kernel also writes.
  __device__ __forceinline__ void load_rw(const float* row, int lane, float (&v)[Q][VW]) const {
#pragma unroll
    for (int q = 0; q < Q; ++q) {
      if (valid[q]) {
        if constexpr (VEC) {
          float4 t = *(reinterpret_cast<const float4*>(row) + lane + 32 * q);
          v[q][0] = t.x; v[q][1] = t.y; v[q][2] = t.z; v[q][3] = t.w;
        } else {
          v[q][0] = row[lane + 32 * q];
        }
      } else {
#pragma unroll
        for (int i = 0; i < VW; ++i) v[q][i] = 0.f;
      }
    }
  }
  __device__ __forceinline__ void store(float* __restrict__ row, int lane,
                                        const float (&v)[Q][VW]) const {
#pragma unroll
    for (int q = 0; q < Q; ++q) {
      if (valid[q]) {
        if constexpr (VEC) {
          reinterpret_cast<float4*>(row)[lane + 32 * q] =
              make_float4(v[q][0], v[q][1], v[q][2], v[q][3]);
        } else {
          row[lane + 32 * q] = v[q][0];
        }
      }
    }
  }
};

// ---------------------------------------------------------------------------
// Ring of gathered rows in shared memory (wide 128-bit tiles).  Every lane copies the 16-byte
// units of a row that it will read itself with cp.async (groups of U rows, kGatherRingRows rows
// per warp), so rows stay in flight while earlier ones are consumed, waiting costs one
// cp.async.wait_group, and no lane ever reads another lane's copy: no barrier of any kind.
// A loop that holds a row in registers from request to use is limited to the rows its
// registers can hold, and has none in flight while it computes.
constexpr int kGatherRingRows = 6;
template <int Q>
constexpr size_t gather_ring_bytes() { return (size_t)kWarpsPerCta * kGatherRingRows * Q * 32 * sizeof(float4); }

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// ---------------------------------------------------------------------------
// Edge-chunk traversal.  The nnz positions of a segment array (CSR rows or CSC
// columns) are cut into chunks of `chunk` consecutive positions, one warp per
// chunk, so every warp moves the same number of gathered rows whatever the
// degree distribution.  A segment that crosses a chunk boundary is processed
// as several pieces; the pieces are merged afterwards by one warp per segment
// in chunk order, so results do not depend on scheduling.
struct ChunkGeom {
  const int* ptr;   // [nseg + 1]
  const int* idx;   // [nnz]
  int nseg;
  int nnz;
  int chunk;        // positions per warp, multiple of 32
  int num_chunks;   // ceil(nnz / chunk)
};

// Partial results of split segments live in two slots per chunk: slot 0 holds
// the piece that continues a segment begun in an earlier chunk, slot 1 the
// piece of a segment that begins in this chunk and runs past its end.
__device__ __forceinline__ size_t slot_index(int chunk_id, bool first_piece) {
  return (size_t)chunk_id * 2 + (first_piece ? 1 : 0);
}

// Empty segments walked one by one before the traversal searches for the end of the run.
constexpr int kEmptyRunWalk = 8;

template <class Body>
__device__ __forceinline__ void for_each_piece(const ChunkGeom& g, int chunk_id,
                                               Body&& body) {
  const int lo = chunk_id * g.chunk;
  const int hi = min(lo + g.chunk, g.nnz);
  int s = find_seg(g.ptr, g.nseg, lo);
  int beg = __ldg(g.ptr + s);
  int empties = 0;
  while (s < g.nseg && beg < hi) {
    const int end = __ldg(g.ptr + s + 1);
    if (end == beg) {
      // a segment without positions; after a few in a row, jump over the rest of the run
      // (one warp would otherwise walk a run of hundreds of thousands one by one)
      if (++empties > kEmptyRunWalk) {
        s = find_seg(g.ptr, g.nseg, beg);
        empties = 0;
      } else {
        ++s;
      }
      continue;
    }
    empties = 0;
    const int a = max(beg, lo);
    const int b = min(end, hi);
    if (b > a) body(s, a, b, /*first=*/beg >= lo, /*last=*/end <= hi);
    beg = end;
    ++s;
  }
}

// Chunk length forced by gnn_debug_set_chunk (0: none).  A test hook: it lets small graphs
// run the chunk lengths that only graphs of 10^8 edges pick by themselves.
extern int g_chunk_override;

// Host-side choice of the chunk length: aim at ~8 resident waves of warps on
// 148 SMs, never below one 32-edge batch nor above 4096 positions.
inline int pick_chunk(int64_t nnz) {
  if (g_chunk_override > 0) return g_chunk_override;
  const int64_t target_warps = 148LL * 64 * 4;
  int64_t c = (nnz + target_warps - 1) / target_warps;
  c = (c + 31) / 32 * 32;
  if (c < 32) c = 32;
  if (c > 4096) c = 4096;
  return (int)c;
}
inline int num_chunks_for(int64_t nnz, int chunk) {
  return (int)((nnz + chunk - 1) / chunk);
}
inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace gnn
