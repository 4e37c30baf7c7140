// Dense projection GEMMs of the layers on the 5th-generation tensor cores with fp32-level
// accuracy: C entry points and the small pre-pass kernels.  The GEMM kernel itself is the
// persistent tcgen05 kernel of gemm_persistent.cu.
//
//   gnn_gemm_tf32x3     C[M,N] = A[M,K] * op(B)          projection and its input gradient
//   gnn_gemm_tf32x3_tn  C[K1,N1] = A[M,K1]^T * B[M,N1]   weight gradient
//
// tcgen05 has no fp32 MMA; a single kind::tf32 product (10-bit mantissa) cannot meet the
// rel 1e-4 / abs 1e-5 parity bound against an fp32 GEMM for K up to 512.  Each operand is
// therefore split into a TF32-exact high part and the fp32 remainder, a = a_hi + a_lo, and
// the product is accumulated in fp32 in tensor memory as
//     a_lo*b_hi + a_hi*b_lo + a_hi*b_hi            (error-compensated "3xTF32").
// Replaces the cuBLAS SGEMM behind torch.matmul(feat, W) / nn.Linear of the layers
// (layers/gatconv_layer.py:50, layers/edgeconv_layer.py:37-38, layers/gmmconv_layer.py:68)
// and behind their autograd.
//
// The node-sized operands (A; both operands of the weight gradient) are read where they
// lie and split inside the GEMM kernel.  Only the weights (a few hundred KB) are split, and
// transposed when given K x N, by a pre-pass; so is an operand of the weight gradient whose
// rows TMA cannot address (row length not a multiple of 4 floats).
#include <cuda_runtime.h>
#include <stdint.h>
#include "../../include/gnn_b200.h"
#include "common.cuh"
#include "gemm_persistent.cuh"

using namespace gnn;

namespace {

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

// b given as K x N row-major -> hi/lo as N x K with leading dimension ld >= K (K contiguous).
// blockIdx.x walks K, blockIdx.y walks N.
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
// K may be millions of rows: one tile is then 16 KB contiguous whatever K is.
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

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

int bad(const char* m) {
  set_last_error(m);
  return GNN_ERR_INVALID_ARG;
}

// Ranges of the reduction axis for the weight gradient: enough (output tile, range) pairs
// for four per SM of a 148-SM part, so that the persistent CTAs finish together.
int tn_splits(int64_t K1, int64_t N1, int64_t M) {
  const int64_t tiles = ((K1 + 127) / 128) * ((N1 + 127) / 128);
  int64_t s = (4 * 148) / tiles;
  const int64_t total_kb = (M + 31) / 32;
  if (s > total_kb) s = total_kb;
  if (s < 1) s = 1;
  return (int)s;
}

// Bytes of the transposed hi + lo copies of a weight-gradient operand with `cols` columns
// (0 when TMA can read its rows directly).
size_t tn_prepass_bytes(int64_t M, int64_t cols) {
  if (cols % 4 == 0) return 0;
  const int64_t ld = (M + 31) / 32 * 32;
  return 2 * align_up((size_t)cols * ld * 4, 256);
}

}  // namespace

extern "C" int gnn_gemm_tf32x3_supported(int64_t M, int64_t N, int64_t K) {
  return M > 0 && N > 0 && K > 0 && K % 4 == 0 && M < (1LL << 31) && N < (1LL << 31) && K < (1LL << 31);
}

extern "C" int gnn_gemm_tf32x3_workspace_bytes(int64_t M, int64_t N, int64_t K, size_t* bytes) {
  if (!bytes || M < 0 || N < 0 || K < 0) return bad("gnn_gemm_tf32x3_workspace_bytes: bad argument");
  *bytes = 2 * align_up((size_t)N * K * 4, 256) + 512;  // hi and lo of the weights
  return GNN_OK;
}

extern "C" int gnn_gemm_tf32x3(const float* A, const float* B, int b_is_n_by_k, float* C, int64_t M,
                               int64_t N, int64_t K, void* workspace, size_t workspace_bytes,
                               int* status, cudaStream_t stream) {
  return gnn_gemm_tf32x3_scores(A, B, b_is_n_by_k, C, M, N, K, nullptr, nullptr, 0, 0, nullptr, nullptr,
                                workspace, workspace_bytes, status, stream);
}

extern "C" int gnn_gemm_tf32x3_scores_supported(int heads, int head_w) {
  return heads >= 1 && head_w >= 1 && gemm_scores_ok(heads, head_w);
}

extern "C" int gnn_gemm_tf32x3_scores(const float* A, const float* B, int b_is_n_by_k, float* C, int64_t M,
                                      int64_t N, int64_t K, const float* attn_l, const float* attn_r, int heads,
                                      int head_w, float* score_l, float* score_r, void* workspace,
                                      size_t workspace_bytes, int* status, cudaStream_t stream) {
  const bool with_scores = attn_l || attn_r || score_l || score_r;
  if (with_scores) {
    if (!attn_l || !attn_r || !score_l || !score_r) return bad("gnn_gemm_tf32x3_scores: null pointer");
    if (heads < 1 || head_w < 1 || (int64_t)heads * head_w != N) return bad("gnn_gemm_tf32x3_scores: heads * head_w must equal N");
    if (!gemm_scores_ok(heads, head_w) || !aligned16(attn_l) || !aligned16(attn_r)) {
      set_last_error("gnn_gemm_tf32x3_scores: head width must be 32, 64 or 128 (or one head of at most 128) "
                     "and the attention vectors 16-byte aligned");
      return GNN_ERR_UNSUPPORTED;
    }
  }
  if (M < 0 || N < 0 || K < 0) return bad("gnn_gemm_tf32x3: negative size");
  if (M == 0 || N == 0) return GNN_OK;
  if (!A || !B || !C || !status) return bad("gnn_gemm_tf32x3: null pointer");
  if (!gnn_gemm_tf32x3_supported(M, N, K) || !tma_rows_ok(A, K)) {
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
  const size_t bb = align_up((size_t)N * K * 4, 256);
  float* b_hi = (float*)w;
  float* b_lo = (float*)(w + bb);
  if (b_is_n_by_k) {
    const int64_t nb = N * K;
    split_kernel<<<(unsigned)((nb / 4 + 256) / 256), 256, 0, stream>>>(B, nb, b_hi, b_lo);
  } else {
    dim3 grid((unsigned)((K + 31) / 32), (unsigned)((N + 31) / 32));
    split_transpose_kernel<<<grid, dim3(32, 8), 0, stream>>>(B, K, (int)N, K, b_hi, b_lo);
  }
  const GemmOperand oa{kKMajorRaw, A, nullptr, M};
  const GemmOperand ob{kKMajorSplit, b_hi, b_lo, N};
  const GemmScores sc{attn_l, attn_r, score_l, score_r, heads, head_w};
  const int rc = launch_gemm_persistent(oa, ob, K, C, N, 1, 0, status, stream, with_scores ? &sc : nullptr);
  if (rc != GNN_OK) return rc;
  return check_launch("gnn_gemm_tf32x3");
}

extern "C" int gnn_gemm_tf32x3_tn_workspace_bytes(int64_t M, int64_t K1, int64_t N1, size_t* bytes) {
  if (!bytes || M < 0 || K1 < 0 || N1 < 0) return bad("gnn_gemm_tf32x3_tn_workspace_bytes: bad argument");
  *bytes = tn_prepass_bytes(M, K1) + tn_prepass_bytes(M, N1) +
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
  if ((K1 % 4 == 0 && !tma_rows_ok(A, K1)) || (N1 % 4 == 0 && !tma_rows_ok(B, N1))) {
    set_last_error("gnn_gemm_tf32x3_tn: operands must be 16-byte aligned");
    return GNN_ERR_UNSUPPORTED;
  }
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
  char* w = (char*)align_up((uintptr_t)workspace, 256);
  const size_t ab = tn_prepass_bytes(M, K1), bb = tn_prepass_bytes(M, N1);
  float* partial = (float*)(w + ab + bb);
  // operands whose rows TMA can read are used where they lie (MN-major tiles, split in
  // shared memory); the others get the transposing pre-pass
  GemmOperand oa{kMnMajorRaw, A, nullptr, K1}, ob{kMnMajorRaw, B, nullptr, N1};
  if (ab) {
    float* hi = (float*)w;
    float* lo = (float*)(w + ab / 2);
    dim3 ga((unsigned)((M + 31) / 32), (unsigned)((K1 + 31) / 32));
    split_transpose_blocked_kernel<<<ga, dim3(32, 8), 0, stream>>>(A, M, (int)K1, hi, lo);
    oa = GemmOperand{kKMajorSplitBlocked, hi, lo, K1};
  }
  if (bb) {
    float* hi = (float*)(w + ab);
    float* lo = (float*)(w + ab + bb / 2);
    dim3 gb((unsigned)((M + 31) / 32), (unsigned)((N1 + 31) / 32));
    split_transpose_blocked_kernel<<<gb, dim3(32, 8), 0, stream>>>(B, M, (int)N1, hi, lo);
    ob = GemmOperand{kKMajorSplitBlocked, hi, lo, N1};
  }
  const int splits = tn_splits(K1, N1, M);
  const int rc = launch_gemm_persistent(oa, ob, M, partial, N1, splits, K1 * N1, status, stream);
  if (rc != GNN_OK) return rc;
  const int64_t count = K1 * N1;
  splitk_reduce_kernel<<<(unsigned)((count + 255) / 256), 256, 0, stream>>>(partial, splits, count, C);
  return check_launch("gnn_gemm_tf32x3_tn");
}
