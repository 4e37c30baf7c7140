// Dense projection GEMM on the 5th-generation tensor cores with fp32-level accuracy.
//
//   C[M,N] = A[M,K] * op(B),   A, B, C fp32 row-major
//
// tcgen05 has no fp32 MMA; a single kind::tf32 product (10-bit mantissa) cannot meet
// the rel 1e-4 / abs 1e-5 parity bound against an fp32 GEMM for K up to 512.  Each
// operand is therefore split into a TF32-exact high part and the fp32 remainder,
//     a = a_hi + a_lo,  a_hi = tf32_rn(a),  a_lo = a - a_hi   (exact in fp32)
// and the product is accumulated in fp32 in tensor memory as
//     a_lo*b_hi + a_hi*b_lo + a_hi*b_hi            (error-compensated "3xTF32").
// Replaces the cuBLAS SGEMM behind torch.matmul(feat, W) / nn.Linear of the layers
// (layers/gatconv_layer.py:50, layers/edgeconv_layer.py:37-38, layers/gmmconv_layer.py:68).
//
// Kernel: one CTA per 128 x 128 output tile, 6 warps:
//   warp 0      : TMA producer  (cp.async.bulk.tensor 2-D, SWIZZLE_128B, no multicast)
//   warp 1      : TMEM allocation + single-thread tcgen05.mma issue, tcgen05.commit
//   warps 2..5  : epilogue, tcgen05.ld of the accumulator and global stores
// K is consumed in blocks of 32 floats (one 128-byte swizzle atom per row); a stage
// holds the hi and lo tiles of A and B (4 x 16 KB); 3 stages.  Out-of-range rows /
// columns / K are zero-filled by TMA and masked in the epilogue.
//
// Every mbarrier wait is bounded: on expiry the kernel raises a status word, drains
// (bounded) what it has in flight, frees its tensor memory and returns.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include "../../include/gnn_b200.h"
#include "common.cuh"

using namespace gnn;

namespace {

constexpr int BM = 128, BN = 128, BK = 32;
constexpr int kStages = 3;
constexpr int kTileBytes = BM * BK * 4;                 // 16 KB, same for A and B tiles
constexpr int kStageBytes = 4 * kTileBytes;             // A_hi, A_lo, B_hi, B_lo
constexpr int kGemmThreads = 192;
constexpr int kTmemCols = 128;
constexpr uint32_t kSpinLimit = 1u << 22;
constexpr size_t kSmemBytes = (size_t)kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait on a phase parity; false when the limit expired.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}

// Same for an operand stored K-blocked, [K/32][rows][32]: one tile is 16 KB contiguous in
// global memory whatever the length of the reduction axis.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte rows and the
// 128-byte swizzle: 8-row groups are 1024 bytes apart (SBO), LBO unused (1),
// descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;            // leading byte offset (ignored for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset
  d |= (uint64_t)1 << 46;            // version
  d |= (uint64_t)2 << 61;            // SWIZZLE_128B
  return d;
}

// Instruction descriptor: D = F32 (bits 4-5 = 1), A = B = TF32 (format 2 at bits 7-9 and
// 10-12), both K-major, N/8 at bits 17-22, M/16 at bits 24-28.
constexpr uint32_t kIdesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) |
                            ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(kIdesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

struct GemmParams {
  int M, N, K;
  float* C;
  int64_t ldc;
  int* status;           // set to 1 by a CTA whose bounded wait expired
  int kb_per_split;      // K blocks handled by one blockIdx.z (split-K); >= all of them when grid.z == 1
  int64_t split_stride;  // floats between the partial outputs of consecutive splits
  int blocked;           // operands are K-blocked (3-D tensor maps)
};

__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
                   const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo,
                   GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // swizzle atoms need 1024-byte alignment
  const uint32_t bars = base + kStages * kStageBytes;
  // barrier layout: full[kStages], empty[kStages], tmem_full, then the TMEM base address word
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (kStages + s); };
  const uint32_t tmem_full_bar = bars + 8u * (2 * kStages);
  const uint32_t tmem_slot = bars + 8u * (2 * kStages + 1);
  uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  const int total_kb = (p.K + BK - 1) / BK;
  const int kb_begin = blockIdx.z * p.kb_per_split;
  const int num_kb = max(0, min(p.kb_per_split, total_kb - kb_begin));
  float* const Cout = p.C + (size_t)blockIdx.z * p.split_stride;
  __shared__ int s_failed;

  if (threadIdx.x == 0) {
    s_failed = 0;
    for (int s = 0; s < kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    mbar_init(tmem_full_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_acc = *tmem_slot_ptr;

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % kStages;
        if (kb >= kStages && !mbar_wait(empty_bar(s), ((kb / kStages) - 1) & 1)) { s_failed = 1; break; }
        const uint32_t st = base + s * kStageBytes;
        mbar_expect_tx(full_bar(s), kStageBytes);
        if (p.blocked) {
          const int kblk = kb_begin + kb;
          tma_load_3d(st + 0 * kTileBytes, &map_a_hi, 0, m0, kblk, full_bar(s));
          tma_load_3d(st + 1 * kTileBytes, &map_a_lo, 0, m0, kblk, full_bar(s));
          tma_load_3d(st + 2 * kTileBytes, &map_b_hi, 0, n0, kblk, full_bar(s));
          tma_load_3d(st + 3 * kTileBytes, &map_b_lo, 0, n0, kblk, full_bar(s));
        } else {
          const int kc = (kb_begin + kb) * BK;
          tma_load_2d(st + 0 * kTileBytes, &map_a_hi, kc, m0, full_bar(s));
          tma_load_2d(st + 1 * kTileBytes, &map_a_lo, kc, m0, full_bar(s));
          tma_load_2d(st + 2 * kTileBytes, &map_b_hi, kc, n0, full_bar(s));
          tma_load_2d(st + 3 * kTileBytes, &map_b_lo, kc, n0, full_bar(s));
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % kStages;
        if (!mbar_wait(full_bar(s), (kb / kStages) & 1)) { s_failed = 1; ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t st = base + s * kStageBytes;
        const uint64_t a_hi = make_desc(st), a_lo = make_desc(st + kTileBytes);
        const uint64_t b_hi = make_desc(st + 2 * kTileBytes), b_lo = make_desc(st + 3 * kTileBytes);
#pragma unroll
        for (int k = 0; k < BK / 8; ++k) {
          const uint64_t adv = (uint64_t)(k * 32 >> 4);  // 8 tf32 = 32 bytes along K inside the atom
          umma_tf32(tmem_acc, a_lo + adv, b_hi + adv, (kb | k) != 0);
          umma_tf32(tmem_acc, a_hi + adv, b_lo + adv, 1);
          umma_tf32(tmem_acc, a_hi + adv, b_hi + adv, 1);
        }
        umma_commit(empty_bar(s));  // the stage is free once these MMAs have read it
      }
      umma_commit(tmem_full_bar);   // accumulator complete (or whatever was issued)
    }
  } else {
    // epilogue: warp w may touch TMEM lanes [32*(w%4), 32*(w%4)+32)
    const int lg = warp & 3;
    const bool ready = mbar_wait(tmem_full_bar, 0);
    if (!ready) s_failed = 1;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ready && !s_failed) {
      const int row = m0 + lg * 32 + lane;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        const uint32_t taddr = tmem_acc + ((uint32_t)(lg * 32) << 16) + (uint32_t)(c * 32);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
              "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
              "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
            : "r"(taddr) : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (num_kb == 0) {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;  // an empty split contributes nothing
        }
        if (row < p.M) {
          float* crow = Cout + (size_t)row * p.ldc + n0 + c * 32;
          const int ncols = min(32, p.N - (n0 + c * 32));
          if (ncols == 32 && ((uintptr_t)crow & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<float4*>(crow + j) =
                  make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                              __uint_as_float(r[j + 3]));
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < ncols) crow[j] = __uint_as_float(r[j]);
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (s_failed) {
    // something expired: give the copies this CTA may still have in flight a bounded
    // time to land before its shared memory is released
    if (threadIdx.x == 0) {
      *p.status = 1;
      for (int s = 0; s < kStages; ++s) { mbar_wait(full_bar(s), 0); mbar_wait(full_bar(s), 1); }
    }
    __syncthreads();
  }
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(kTmemCols) : "memory");
  }
}

// hi = tf32_rn(x) (low 13 mantissa bits zero), lo = x - hi.
__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo) {
  uint32_t h;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
  hi = __uint_as_float(h);
  lo = x - hi;
}

__global__ void split_kernel(const float* __restrict__ x, int64_t n, float* __restrict__ hi,
                             float* __restrict__ lo) {
  const int64_t i4 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i4 + 3 < n && (((uintptr_t)x | (uintptr_t)hi | (uintptr_t)lo) & 15) == 0) {
    const float4 v = *reinterpret_cast<const float4*>(x + i4);
    float4 h, l;
    split_tf32(v.x, h.x, l.x); split_tf32(v.y, h.y, l.y);
    split_tf32(v.z, h.z, l.z); split_tf32(v.w, h.w, l.w);
    *reinterpret_cast<float4*>(hi + i4) = h;
    *reinterpret_cast<float4*>(lo + i4) = l;
  } else {
    for (int64_t i = i4; i < n && i < i4 + 4; ++i) split_tf32(x[i], hi[i], lo[i]);
  }
}

// B given as K x N row-major -> hi/lo as N x K with leading dimension ld >= K (K contiguous).
// blockIdx.x walks K (which may be millions of rows), blockIdx.y walks N.
__global__ void split_transpose_kernel(const float* __restrict__ b, int64_t K, int N, int64_t ld,
                                       float* __restrict__ hi, float* __restrict__ lo) {
  __shared__ float tile[32][33];
  const int64_t k0 = (int64_t)blockIdx.x * 32;
  const int n0 = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int64_t k = k0 + r;
    const int n = n0 + threadIdx.x;
    tile[r][threadIdx.x] = (k < K && n < N) ? b[(size_t)k * N + n] : 0.f;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int n = n0 + r;
    const int64_t k = k0 + threadIdx.x;
    if (n < N && k < K) split_tf32(tile[threadIdx.x][r], hi[(size_t)n * ld + k], lo[(size_t)n * ld + k]);
  }
}

// b given as K x N row-major -> hi/lo K-blocked: [ceil(K/32)][N][32] (positions past K zero).
__global__ void split_transpose_blocked_kernel(const float* __restrict__ b, int64_t K, int N,
                                               float* __restrict__ hi, float* __restrict__ lo) {
  __shared__ float tile[32][33];
  const int64_t k0 = (int64_t)blockIdx.x * 32;
  const int n0 = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int64_t k = k0 + r;
    const int n = n0 + threadIdx.x;
    tile[r][threadIdx.x] = (k < K && n < N) ? b[(size_t)k * N + n] : 0.f;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int n = n0 + r;
    if (n < N) {
      const size_t o = ((size_t)blockIdx.x * N + n) * 32 + threadIdx.x;
      split_tf32(tile[threadIdx.x][r], hi[o], lo[o]);
    }
  }
}

// out[i] = sum over splits of partial[z][i], in split order (deterministic).
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, int splits, int64_t count,
                                     float* __restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  float s = 0.f;
  for (int z = 0; z < splits; ++z) s += partial[(size_t)z * count + i];
  out[i] = s;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// 2-D map over a row-major [rows, cols] fp32 matrix, box = 32 columns x 128 rows.
bool make_map(CUtensorMap* m, const float* ptr, int64_t rows, int64_t cols, int64_t ld = 0) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  if (ld == 0) ld = cols;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)BM};
  cuuint32_t estr[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)ptr, dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 3-D map over a K-blocked operand [kblocks][rows][32]: box = 32 x 128 rows x 1 block.
bool make_map_blocked(CUtensorMap* m, const float* ptr, int64_t rows, int64_t kblocks) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {32, (cuuint64_t)rows, (cuuint64_t)kblocks};
  cuuint64_t strides[2] = {32 * 4, (cuuint64_t)rows * 32 * 4};
  cuuint32_t box[3] = {(cuuint32_t)BK, (cuuint32_t)BM, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)ptr, dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

int bad(const char* m) {
  set_last_error(m);
  return GNN_ERR_INVALID_ARG;
}

}  // namespace

extern "C" int gnn_gemm_tf32x3_supported(int64_t M, int64_t N, int64_t K) {
  return M > 0 && N > 0 && K > 0 && K % 4 == 0 && M < (1LL << 31) && N < (1LL << 31) && K < (1LL << 31);
}

extern "C" int gnn_gemm_tf32x3_workspace_bytes(int64_t M, int64_t N, int64_t K, size_t* bytes) {
  if (!bytes || M < 0 || N < 0 || K < 0) return bad("gnn_gemm_tf32x3_workspace_bytes: bad argument");
  *bytes = 2 * align_up((size_t)M * K * 4, 256) + 2 * align_up((size_t)N * K * 4, 256) + 512;
  return GNN_OK;
}

extern "C" int gnn_gemm_tf32x3(const float* A, const float* B, int b_is_n_by_k, float* C, int64_t M,
                               int64_t N, int64_t K, void* workspace, size_t workspace_bytes,
                               int* status, cudaStream_t stream) {
  if (M < 0 || N < 0 || K < 0) return bad("gnn_gemm_tf32x3: negative size");
  if (M == 0 || N == 0) return GNN_OK;
  if (!A || !B || !C || !status) return bad("gnn_gemm_tf32x3: null pointer");
  if (!gnn_gemm_tf32x3_supported(M, N, K) || ((uintptr_t)A & 15)) {
    set_last_error("gnn_gemm_tf32x3: K must be a multiple of 4 and A 16-byte aligned");
    return GNN_ERR_UNSUPPORTED;
  }
  size_t need = 0;
  gnn_gemm_tf32x3_workspace_bytes(M, N, K, &need);
  if (!workspace || workspace_bytes < need) {
    set_last_error("gnn_gemm_tf32x3: workspace too small");
    return GNN_ERR_WORKSPACE;
  }
  char* w = (char*)align_up((uintptr_t)workspace, 256);
  const size_t ab = align_up((size_t)M * K * 4, 256), bb = align_up((size_t)N * K * 4, 256);
  float* a_hi = (float*)w;
  float* a_lo = (float*)(w + ab);
  float* b_hi = (float*)(w + 2 * ab);
  float* b_lo = (float*)(w + 2 * ab + bb);

  const int64_t na = M * K;
  split_kernel<<<(unsigned)((na / 4 + 256) / 256), 256, 0, stream>>>(A, na, a_hi, a_lo);
  if (b_is_n_by_k) {
    const int64_t nb = N * K;
    split_kernel<<<(unsigned)((nb / 4 + 256) / 256), 256, 0, stream>>>(B, nb, b_hi, b_lo);
  } else {
    dim3 grid((unsigned)((K + 31) / 32), (unsigned)((N + 31) / 32));
    split_transpose_kernel<<<grid, dim3(32, 8), 0, stream>>>(B, K, (int)N, K, b_hi, b_lo);
  }
  CUtensorMap ma_hi, ma_lo, mb_hi, mb_lo;
  if (!make_map(&ma_hi, a_hi, M, K) || !make_map(&ma_lo, a_lo, M, K) || !make_map(&mb_hi, b_hi, N, K) ||
      !make_map(&mb_lo, b_lo, N, K)) {
    set_last_error("gnn_gemm_tf32x3: cuTensorMapEncodeTiled failed");
    return GNN_ERR_CUDA;
  }
  if (cudaFuncSetAttribute(gemm_tf32x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes) !=
      cudaSuccess) {
    set_last_error("gnn_gemm_tf32x3: cannot reserve dynamic shared memory");
    return GNN_ERR_CUDA;
  }
  GemmParams p{(int)M, (int)N, (int)K, C, N, status, (int)((K + BK - 1) / BK), 0, 0};
  dim3 grid((unsigned)((M + BM - 1) / BM), (unsigned)((N + BN - 1) / BN));
  gemm_tf32x3_kernel<<<grid, kGemmThreads, kSmemBytes, stream>>>(ma_hi, ma_lo, mb_hi, mb_lo, p);
  return check_launch("gnn_gemm_tf32x3");
}

// ---- C[K1,N1] = A^T * B with A [M,K1], B [M,N1]: the weight gradient X^T * dH -------------
// Both operands are transposed (and split) into [K1, M] / [N1, M] so that the reduction
// dimension M is contiguous, then the same kernel runs with the M axis cut into `splits`
// ranges (split-K) whose partial tiles are summed in order.

namespace {
int tn_splits(int64_t K1, int64_t N1, int64_t M) {
  const int64_t tiles = ((K1 + BM - 1) / BM) * ((N1 + BN - 1) / BN);
  int64_t s = (2 * 148 + tiles - 1) / tiles;
  const int64_t total_kb = (M + BK - 1) / BK;
  if (s > total_kb) s = total_kb;
  if (s < 1) s = 1;
  return (int)s;
}
}  // namespace

extern "C" int gnn_gemm_tf32x3_tn_workspace_bytes(int64_t M, int64_t K1, int64_t N1, size_t* bytes) {
  if (!bytes || M < 0 || K1 < 0 || N1 < 0) return bad("gnn_gemm_tf32x3_tn_workspace_bytes: bad argument");
  const int64_t ld = (M + 31) / 32 * 32;  // K-blocked storage: whole blocks of 32
  *bytes = 2 * align_up((size_t)K1 * ld * 4, 256) + 2 * align_up((size_t)N1 * ld * 4, 256) +
           align_up((size_t)tn_splits(K1, N1, M) * K1 * N1 * 4, 256) + 512;
  return GNN_OK;
}

extern "C" int gnn_gemm_tf32x3_tn(const float* A, const float* B, float* C, int64_t M, int64_t K1,
                                  int64_t N1, void* workspace, size_t workspace_bytes, int* status,
                                  cudaStream_t stream) {
  if (M < 0 || K1 < 0 || N1 < 0) return bad("gnn_gemm_tf32x3_tn: negative size");
  if (K1 == 0 || N1 == 0) return GNN_OK;
  if (!C || !status || (M && (!A || !B))) return bad("gnn_gemm_tf32x3_tn: null pointer");
  if (M >= (1LL << 31) || K1 >= (1LL << 31) || N1 >= (1LL << 31)) return bad("gnn_gemm_tf32x3_tn: size exceeds int32");
  size_t need = 0;
  gnn_gemm_tf32x3_tn_workspace_bytes(M, K1, N1, &need);
  if (!workspace || workspace_bytes < need) {
    set_last_error("gnn_gemm_tf32x3_tn: workspace too small");
    return GNN_ERR_WORKSPACE;
  }
  if (M == 0) {
    cudaMemsetAsync(C, 0, (size_t)K1 * N1 * 4, stream);
    return check_launch("gnn_gemm_tf32x3_tn");
  }
  const int64_t ld = (M + 31) / 32 * 32;
  const int64_t kblocks = ld / 32;
  char* w = (char*)align_up((uintptr_t)workspace, 256);
  const size_t ab = align_up((size_t)K1 * ld * 4, 256), bb = align_up((size_t)N1 * ld * 4, 256);
  float* a_hi = (float*)w;
  float* a_lo = (float*)(w + ab);
  float* b_hi = (float*)(w + 2 * ab);
  float* b_lo = (float*)(w + 2 * ab + bb);
  float* partial = (float*)(w + 2 * ab + 2 * bb);
  {
    dim3 ga((unsigned)((M + 31) / 32), (unsigned)((K1 + 31) / 32));
    split_transpose_blocked_kernel<<<ga, dim3(32, 8), 0, stream>>>(A, M, (int)K1, a_hi, a_lo);
    dim3 gb((unsigned)((M + 31) / 32), (unsigned)((N1 + 31) / 32));
    split_transpose_blocked_kernel<<<gb, dim3(32, 8), 0, stream>>>(B, M, (int)N1, b_hi, b_lo);
  }
  CUtensorMap ma_hi, ma_lo, mb_hi, mb_lo;
  if (!make_map_blocked(&ma_hi, a_hi, K1, kblocks) || !make_map_blocked(&ma_lo, a_lo, K1, kblocks) ||
      !make_map_blocked(&mb_hi, b_hi, N1, kblocks) || !make_map_blocked(&mb_lo, b_lo, N1, kblocks)) {
    set_last_error("gnn_gemm_tf32x3_tn: cuTensorMapEncodeTiled failed");
    return GNN_ERR_CUDA;
  }
  if (cudaFuncSetAttribute(gemm_tf32x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes) !=
      cudaSuccess) {
    set_last_error("gnn_gemm_tf32x3_tn: cannot reserve dynamic shared memory");
    return GNN_ERR_CUDA;
  }
  const int splits = tn_splits(K1, N1, M);
  const int total_kb = (int)((M + BK - 1) / BK);
  const int per = (total_kb + splits - 1) / splits;
  GemmParams p{(int)K1, (int)N1, (int)M, partial, N1, status, per, K1 * N1, 1};
  dim3 grid((unsigned)((K1 + BM - 1) / BM), (unsigned)((N1 + BN - 1) / BN), (unsigned)splits);
  gemm_tf32x3_kernel<<<grid, kGemmThreads, kSmemBytes, stream>>>(ma_hi, ma_lo, mb_hi, mb_lo, p);
  const int64_t count = K1 * N1;
  splitk_reduce_kernel<<<(unsigned)((count + 255) / 256), 256, 0, stream>>>(partial, splits, count, C);
  return check_launch("gnn_gemm_tf32x3_tn");
}
