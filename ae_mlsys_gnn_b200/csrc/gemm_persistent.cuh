// Host-side interface of the persistent 3xTF32 tcgen05 GEMM (gemm_persistent.cu), used by
// the C entry points in gemm_tf32x3.cu.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace gnn {

// How one operand of the product reaches the kernel.
enum OperandMode : int {
  // fp32 matrix [rows][K], K contiguous; the kernel splits it into hi/lo in shared memory
  kKMajorRaw = 0,
  // hi and lo given separately, each [rows][K] (prepared by a pre-pass; for small operands)
  kKMajorSplit = 1,
  // hi and lo given separately, K-blocked [ceil(K/32)][rows][32]
  kKMajorSplitBlocked = 2,
  // fp32 matrix [K][rows], rows contiguous (the reduction axis is the slow one); split in the kernel
  kMnMajorRaw = 3,
};

struct GemmOperand {
  OperandMode mode;
  const float* p0;  // raw matrix, or hi
  const float* p1;  // lo (split modes)
  int64_t rows;     // extent along the output dimension (M for A, N for B)
};

// Attention scores formed in the epilogue (splits == 1): C rows are `heads` heads of `head_w` floats.
struct GemmScores {
  const float* attn_l;  // [heads][head_w]
  const float* attn_r;
  float* score_l;       // [M][heads]
  float* score_r;
  int heads, head_w;
};

// Shapes for which the epilogue can form the scores: every head inside one 128-column tile and
// starting on a 32-column chunk.
inline bool gemm_scores_ok(int heads, int head_w) {
  return (heads == 1 && head_w <= 128) || head_w == 32 || head_w == 64 || head_w == 128;
}

// C[z][M][N] (z < splits) = sum over the z-th range of K blocks of A * B^T.
// Returns 0, or a negative GNN_ERR_* after set_last_error.
int launch_gemm_persistent(const GemmOperand& a, const GemmOperand& b, int64_t K, float* C, int64_t ldc,
                           int splits, int64_t split_stride, int* status, cudaStream_t stream,
                           const GemmScores* scores = nullptr);

// Whether an operand with `cols` contiguous floats per row and base pointer p can be read by TMA.
inline bool tma_rows_ok(const void* p, int64_t cols) {
  return (reinterpret_cast<uintptr_t>(p) & 15) == 0 && cols % 4 == 0;
}

}  // namespace gnn
