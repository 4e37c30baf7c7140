/*
 * gnn_b200 — C ABI of the sm_100a fused GNN sparse kernels.
 *
 * One shared library (libgnn_b200.so) replaces the per-operator pybind11 modules
 * that the reference JIT-builds from src/ at import time
 * (operators/fused_gat.py:9-25, operators/fused_edgeconv.py:9-13,
 * operators/fused_gmmconv.py:10-39, ...).  Conventions:
 *
 *  - every pointer is a device pointer on the current CUDA device unless stated;
 *  - indices are int32, values fp32, all arrays dense and contiguous, row-major;
 *  - "CSR" is the in-edge CSR of the reference: segment = destination node,
 *    idx = source node.  A segment array (ptr[n_seg+1], idx[nnz]) may equally be
 *    a CSC (segment = source, idx = destination) or one rank's row block of a
 *    partitioned graph: arrays described as "segment indexed" have n_seg rows,
 *    arrays described as "gathered" are indexed by the values stored in idx;
 *  - the caller owns every buffer, outputs and workspace included.  The byte
 *    size of a workspace comes from the matching *_workspace_bytes function;
 *    a workspace is scratch: its contents are undefined before and after a call;
 *  - every function only enqueues work on `stream` and returns 0, or a negative
 *    GNN_ERR_* code with a message available from gnn_last_error_string().  No
 *    function aborts, allocates device memory or synchronises (the reference
 *    asserts / exit()s: src/fused_gat/fused_gat_SM.cpp:22-36,
 *    src/util/computeUtil.h:14-22);
 *  - outputs are deterministic (bit-identical from run to run) except where a
 *    function says it uses atomics.
 */
#ifndef GNN_B200_H_
#define GNN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GNN_B200_ABI_VERSION 1

#define GNN_OK 0
#define GNN_ERR_INVALID_ARG (-1)
#define GNN_ERR_CUDA (-2)
#define GNN_ERR_WORKSPACE (-3)
#define GNN_ERR_UNSUPPORTED (-4)
#define GNN_ERR_LIMIT (-5)

#ifndef __CUDA_RUNTIME_H__
typedef struct CUstream_st* cudaStream_t;
#endif

/* Message of the last error returned on the calling thread. */
const char* gnn_last_error_string(void);
int gnn_abi_version(void);

/* Test hook, no counterpart in the reference.  Every edge-balanced kernel cuts the nnz
 * positions of its segment array into chunks of `chunk` consecutive positions, one warp
 * each; the length is chosen from nnz (32 below ~1.2 M edges, up to 4096 at 10^8).  This
 * call forces it for all later calls of the process (chunk = 0 restores the automatic
 * choice), so that a test can run the long-chunk code paths on a graph small enough for
 * a CPU oracle.  A multiple of 32 in [32, 4096].  Workspace sizes follow the forced
 * length: query *_workspace_bytes after setting it.  Not thread-safe against running calls. */
int gnn_debug_set_chunk(int chunk);

/* ---- csr2csc -----------------------------------------------------------------
 * Replaces transpose.csr2csc (src/csr2csc/csr2csc.cu:7-43, bound in
 * src/csr2csc/csr2csc.cc) and the host SciPy transpose of the training scripts
 * (script/train/train_gatconv_our.py:107-121).  Stable counting order: inside a
 * column the CSR order is kept, so row ids ascend.  permute[i] is the CSR
 * position of the i-th CSC edge, as int32 (the reference carries it as float32).
 * The matrix may be rectangular (n_rows x n_cols). */
int gnn_csr2csc_workspace_bytes(int64_t nnz, size_t* bytes);
int gnn_csr2csc(const int* row_ptr, const int* col_ind, int64_t n_rows, int64_t n_cols,
                int64_t nnz, int* col_ptr /*[n_cols+1]*/, int* row_ind /*[nnz]*/,
                int* permute /*[nnz]*/, void* workspace, size_t workspace_bytes,
                cudaStream_t stream);

/* ---- fused GAT, recompute flavour ------------------------------------------------
 * gnn_gat_fwd replaces fused_gat_SM.gat_forward
 * (src/fused_gat/fused_gat_SM.cpp:14-38, src/fused_gat/fused_gat_SM.cu:514-558):
 *   e = LeakyReLU(attn_row[r,h] + attn_col[c,h]); m = max e; s = sum exp(e - m)
 *   out[r,h,:] = sum_c exp(e - m)/s * in_feat[c,h,:]; edge_max = m; edge_sum = s
 * A row without edges gets out = 0, edge_max = -1e38, edge_sum = 0.
 * attn_row/out/edge_max/edge_sum are segment indexed [n_rows]; attn_col/in_feat
 * are gathered. */
int gnn_gat_fwd_workspace_bytes(int64_t nnz, int H, int F, size_t* bytes);
int gnn_gat_fwd(const int* row_ptr, const int* col_ind, int64_t n_rows, int64_t nnz,
                const float* attn_row /*[n_rows,H]*/, const float* attn_col /*[*,H]*/,
                const float* in_feat /*[*,H,F]*/, int H, int F, float negative_slope,
                float* out /*[n_rows,H,F]*/, float* edge_max /*[n_rows,H]*/,
                float* edge_sum /*[n_rows,H]*/, void* workspace, size_t workspace_bytes,
                cudaStream_t stream);

/* gnn_gat_fwd over ONE column block of the graph: the CSR given holds only the edges whose
 * sources lie in that block, and several calls build one result, so that a block can be
 * aggregated as soon as its source rows have arrived from the other GPUs.  accumulate = 0
 * on the first block, 1 afterwards (out, edge_max, edge_sum then carry the running,
 * un-normalised state); finalize = 1 on the last block only.  accumulate = 0, finalize = 1
 * is gnn_gat_fwd.  No counterpart in the reference (single GPU). */
int gnn_gat_fwd_part(const int* row_ptr, const int* col_ind, int64_t n_rows, int64_t nnz,
                     const float* attn_row, const float* attn_col, const float* in_feat, int H,
                     int F, float negative_slope, float* out, float* edge_max, float* edge_sum,
                     int accumulate, int finalize, void* workspace, size_t workspace_bytes,
                     cudaStream_t stream);

/* gnn_gat_fwd for callers that cannot allocate device memory when they run a layer (a
 * server whose memory pool took the whole GPU at start-up, a plugin inside another
 * program's memory plan, a latency-critical path).  Has no counterpart in the
 * reference.  Same arguments and results as gnn_gat_fwd, minus the workspace: the
 * scratch is a GNN_STATIC_SCRATCH_BYTES array in the library's device image, held by
 * every GPU that loads the library until the process exits.  Problems whose
 * gnn_gat_fwd_workspace_bytes() is larger are refused with GNN_ERR_LIMIT.  The first
 * call on a device resolves the array's address; make it before any stream capture.
 * All calls share the array (contents of the previous call remain, none of it needs
 * to be zero), so calls that overlap on the GPU race: issue them back to back on one
 * stream. */
#define GNN_STATIC_SCRATCH_BYTES (16 << 20)
int gnn_gat_fwd_static_scratch(const int* row_ptr, const int* col_ind, int64_t n_rows, int64_t nnz,
                               const float* attn_row, const float* attn_col, const float* in_feat,
                               int H, int F, float negative_slope, float* out, float* edge_max,
                               float* edge_sum, cudaStream_t stream);

/* gnn_gat_bwd replaces fused_gat_SM.gat_backward
 * (src/fused_gat/fused_gat_SM.cpp:55-118, src/fused_gat/fused_gat_SM.cu:831-893)
 * on a square graph given as CSR and CSC.  No E x H temporary, no atomics.
 * Requires H <= 8 and H*F <= 512 (16-byte aligned rows, F % 4 == 0) or 256. */
int gnn_gat_bwd_workspace_bytes(int64_t n_rows, int64_t nnz, int H, int F, size_t* bytes);
int gnn_gat_bwd(const int* row_ptr, const int* col_ind, const int* col_ptr, const int* row_ind,
                int64_t n, int64_t nnz, const float* edge_max, const float* edge_sum,
                const float* in_feat, const float* attn_row, const float* attn_col,
                const float* grad_out, int H, int F, float negative_slope,
                float* grad_feat /*[n,H,F]*/, float* grad_attn_row /*[n,H]*/,
                float* grad_attn_col /*[n,H]*/, void* workspace, size_t workspace_bytes,
                cudaStream_t stream);

/* The two passes of gnn_gat_bwd, exposed so that a partitioned graph can
 * exchange rowpack and grad_out between them.  No counterpart in the reference,
 * which is single-GPU.
 *  row pass: CSR row block; edge_max/edge_sum/attn_row/grad_out segment indexed,
 *            in_feat/attn_col gathered.  Writes grad_attn_row [n_rows,H] and
 *            rowpack [n_rows,4,H] = {attn_row, edge_max, 1/edge_sum, S}.
 *  col pass: CSC column block; in_feat/attn_col segment indexed, rowpack/grad_out
 *            gathered.  Writes grad_feat [n_cols,H,F], grad_attn_col [n_cols,H]. */
int gnn_gat_bwd_row_workspace_bytes(int64_t nnz, int H, int F, size_t* bytes);
int gnn_gat_bwd_row(const int* row_ptr, const int* col_ind, int64_t n_rows, int64_t nnz,
                    const float* edge_max, const float* edge_sum, const float* in_feat,
                    const float* attn_row, const float* attn_col, const float* grad_out,
                    int H, int F, float negative_slope, float* grad_attn_row, float* rowpack,
                    void* workspace, size_t workspace_bytes, cudaStream_t stream);
int gnn_gat_bwd_col_workspace_bytes(int64_t nnz, int H, int F, size_t* bytes);
int gnn_gat_bwd_col(const int* col_ptr, const int* row_ind, int64_t n_cols, int64_t nnz,
                    const float* in_feat, const float* attn_col, const float* rowpack,
                    const float* grad_out, int H, int F, float negative_slope,
                    float* grad_feat, float* grad_attn_col, void* workspace,
                    size_t workspace_bytes, cudaStream_t stream);

/* Attention scores of a GAT layer in one pass over the projected features, and their
 * backward fused with the accumulation into grad_feat.  Replaces the framework kernels
 * behind layers/gatconv_layer.py:52-53 (attn_row = (attn_l*h).sum(-1), attn_col =
 * (attn_r*h).sum(-1)) and autograd's backward of those lines:
 *   fwd: attn_row[n,h] = <attn_l[h,:], feat[n,h,:]>, attn_col[n,h] = <attn_r[h,:], feat[n,h,:]>
 *   bwd: grad_feat[n,h,:] += grad_attn_row[n,h]*attn_l[h,:] + grad_attn_col[n,h]*attn_r[h,:]  (in place)
 *        grad_attn_l[h,:] = sum_n grad_attn_row[n,h]*feat[n,h,:], grad_attn_r likewise.
 * Requires H <= 8 and H*F <= 512 (aligned) / 256. */
int gnn_gat_scores_fwd(const float* feat /*[n,H,F]*/, const float* attn_l /*[H,F]*/,
                       const float* attn_r /*[H,F]*/, int64_t n, int H, int F,
                       float* attn_row /*[n,H]*/, float* attn_col /*[n,H]*/, cudaStream_t stream);
int gnn_gat_scores_bwd_workspace_bytes(int64_t n, int H, int F, size_t* bytes);
int gnn_gat_scores_bwd(const float* feat, const float* attn_l, const float* attn_r,
                       const float* grad_attn_row, const float* grad_attn_col, int64_t n, int H,
                       int F, float* grad_feat /*[n,H,F], updated in place*/,
                       float* grad_attn_l /*[H,F]*/, float* grad_attn_r /*[H,F]*/, void* workspace,
                       size_t workspace_bytes, cudaStream_t stream);

/* Column pass over ONE row block of the graph (CSC restricted to destinations of that
 * block); accumulate = 1 adds to the grad_feat / grad_attn_col of earlier calls. */
int gnn_gat_bwd_col_part(const int* col_ptr, const int* row_ind, int64_t n_cols, int64_t nnz,
                         const float* in_feat, const float* attn_col, const float* rowpack,
                         const float* grad_out, int H, int F, float negative_slope,
                         float* grad_feat, float* grad_attn_col, int accumulate, void* workspace,
                         size_t workspace_bytes, cudaStream_t stream);

/* gnn_gat_bwd_col_part that also stores the gradient of every edge logit:
 * edge_grad[p*H + h] for the p-th position of this CSC (16-byte aligned; NULL = do not
 * store).  With gnn_gat_bwd_pack before and gnn_gat_bwd_row_sum after, this is the whole
 * backward of fused_gat_SM.gat_backward (src/fused_gat/fused_gat_SM.cu:865-893) with one
 * gather pass instead of two, for callers that kept the forward output. */
int gnn_gat_bwd_col_edges(const int* col_ptr, const int* row_ind, int64_t n_cols, int64_t nnz,
                          const float* in_feat, const float* attn_col, const float* rowpack,
                          const float* grad_out, int H, int F, float negative_slope,
                          float* grad_feat, float* grad_attn_col, float* edge_grad, int accumulate,
                          void* workspace, size_t workspace_bytes, cudaStream_t stream);

/* rowpack[r] = {attn_row[r,:], edge_max[r,:], 1/edge_sum[r,:], S[r,:]} (4*H floats per row)
 * with S[r,h] = <grad_out[r,h,:], out[r,h,:]>, `out` being the forward output of
 * gnn_gat_fwd for the same inputs: the per-row record the column pass reads, without the
 * row pass over the edges. */
int gnn_gat_bwd_pack(int64_t n_rows, const float* out, const float* grad_out, const float* attn_row,
                     const float* edge_max, const float* edge_sum, int H, int F, float* rowpack,
                     cudaStream_t stream);

/* gnn_gat_bwd_pack for a layer whose output went through ELU (alpha) before the loss:
 * grad_act is the gradient with respect to elu(out); the kernel writes
 * grad_pre = grad_act * (out > 0 ? 1 : alpha*exp(out)) (the grad_out the column pass takes)
 * and uses it for S.  Replaces the framework's elu-backward pass over the same matrices
 * (the reference applies its activations in the model, script/train/train_gatconv_our.py:47-53). */
int gnn_gat_bwd_pack_elu(int64_t n_rows, const float* out, const float* grad_act, const float* attn_row,
                         const float* edge_max, const float* edge_sum, int H, int F, float alpha,
                         float* grad_pre, float* rowpack, cudaStream_t stream);

/* grad_attn_row[r,h] = sum over the CSR edges e of row r of edge_grad[csr_pos[e]*H + h];
 * csr_pos[e] is the position of CSR edge e in the CSC whose column pass filled edge_grad
 * (the inverse of the permutation gnn_csr2csc returns).  Deterministic. */
int gnn_gat_bwd_row_sum_workspace_bytes(int64_t nnz, int H, size_t* bytes);
int gnn_gat_bwd_row_sum(const int* row_ptr, const int* csr_pos, int64_t n_rows, int64_t nnz,
                        const float* edge_grad, int H, float* grad_attn_row, void* workspace,
                        size_t workspace_bytes, cudaStream_t stream);

/* inv[perm[i]] = i for a permutation of 0..n-1 (e.g. gnn_csr2csc's permute -> csr_pos). */
int gnn_invert_permutation(const int* perm, int64_t n, int* inv, cudaStream_t stream);

/* Per-edge activated logits and normalised attention (E x H each), the tensors the
 * stash / fusescatter variants keep: fused_gat_stash.gat_forward and
 * fused_gat.gat_forward (src/fused_gat/fused_gat_stash.cu:193-288,
 * src/fused_gat/fused_gat.cu:235-300). */
int gnn_gat_edge_alpha(const int* row_ptr, const int* col_ind, int64_t n_rows, int64_t nnz,
                       const float* attn_row, const float* attn_col, const float* edge_max,
                       const float* edge_sum, int H, float negative_slope,
                       float* edge_relu /*[nnz,H]*/, float* edge_alpha /*[nnz,H]*/,
                       cudaStream_t stream);

/* ---- fused EdgeConv ----------------------------------------------------------------
 * Replaces fused_edgeconv.edgeconv_forward / edgeconv_backward
 * (src/fused_edgeconv/fused_edgeconv.cpp:10-57, fused_edgeconv.cu:148-200).
 *   out[i,f] = max_j (h_dst[i,f] + h_src[src_ind[i*k+j],f]),  max_idx = winning id
 * with the reference's tie rule, so max_idx is bit-exact; it is int32 here (the
 * reference stores it in a float32 tensor).  The backward zero-fills grad_src and
 * scatters with fp32 atomics (sum order not fixed). */
int gnn_edgeconv_fwd(int k, const int* src_ind /*[n*k]*/, const float* h_src /*[*,F]*/,
                     const float* h_dst /*[n,F]*/, int64_t n, int F, float* out /*[n,F]*/,
                     int* max_idx /*[n,F]*/, cudaStream_t stream);
int gnn_edgeconv_bwd(const float* grad_out /*[n,F]*/, const int* max_idx /*[n,F]*/, int64_t n,
                     int64_t n_src, int F, float* grad_src /*[n_src,F]*/, cudaStream_t stream);

/* The same pair with the LeakyReLU(slope > 0) the DGCNN model applies to every EdgeConv
 * output (script/train/train_edgeconv_our.py:44-52) folded in, saving one read and one
 * write of [n,F] in each direction: the forward stores leaky(max) (max_idx unchanged, the
 * activation being monotone), the backward applies LeakyReLU' by the sign of `out`, writes
 * the result as grad_dst (the gradient of h_dst) and scatters it into grad_src. */
int gnn_edgeconv_fwd_act(int k, const int* src_ind, const float* h_src, const float* h_dst,
                         int64_t n, int F, float slope, float* out, int* max_idx,
                         cudaStream_t stream);
int gnn_edgeconv_bwd_act(const float* grad_out /*[n,F]*/, const float* out /*[n,F]*/, float slope,
                         const int* max_idx, int64_t n, int64_t n_src, int F,
                         float* grad_src /*[n_src,F]*/, float* grad_dst /*[n,F]*/,
                         cudaStream_t stream);

/* ---- fused GMMConv ------------------------------------------------------------------
 * gnn_gmm_fwd replaces gmm.gmmconv (src/fused_gmmconv/gmmconv.cc,
 * gmmconv.cu:48-80,201-219):
 *   w[e,k] = exp(-0.5 sum_d ((pseudo[pe,d]-mu[k,d]) inv_sigma[k,d])^2)
 *   out[s,k,:] = sum_e w[e,k] node_feat[idx[e],k,:]
 * pe = perm ? perm[e] : e, so the transposed pass of the backward needs no
 * separate mhtranspose of pseudo (operators/fused_gmmconv.py:54-56).
 * Requires K <= 8 and K*F <= 512 (aligned) / 256. */
int gnn_gmm_fwd_workspace_bytes(int64_t nnz, int K, int F, size_t* bytes);
int gnn_gmm_fwd(const int* ptr, const int* idx, int64_t n_seg, int64_t nnz,
                const float* node_feat /*[*,K,F]*/, const float* pseudo /*[nnz,D]*/,
                const int* perm /*[nnz] or NULL*/, const float* mu /*[K,D]*/,
                const float* inv_sigma /*[K,D]*/, int K, int D, int F,
                float* out /*[n_seg,K,F]*/, void* workspace, size_t workspace_bytes,
                cudaStream_t stream);
/* The tail of the GMMConv layer as one pass (layers/gmmconv_layer.py:69-75, where it is a
 * framework sum over the kernel axis plus up to two additions):
 *   out[n,f] = sum_k x[n,k,f] + residual[n,f] + bias[f]      (residual, bias: NULL = absent)
 * and its backward for x, grad_x[n,k,:] = grad_out[n,:] (the gradients of residual and bias
 * are grad_out itself and its column sum, left to the caller). */
int gnn_gmm_sum_fwd(const float* x /*[n,K,F]*/, const float* residual /*[n,F] or NULL*/,
                    const float* bias /*[F] or NULL*/, int64_t n, int K, int F,
                    float* out /*[n,F]*/, cudaStream_t stream);
int gnn_gmm_sum_bwd(const float* grad_out /*[n,F]*/, int64_t n, int K, int F,
                    float* grad_x /*[n,K,F]*/, cudaStream_t stream);
/* gmm.Gaussian (gmmconv.cu:34-46,186-199). */
int gnn_gaussian_fwd(const float* pseudo, const float* mu, const float* inv_sigma, int64_t E,
                     int K, int D, float* out /*[E,K]*/, cudaStream_t stream);
/* gmm.GaussianBp (gmmconv.cu:154-184,265-285) with the analytic gradients; D <= 8. */
int gnn_gaussian_bwd_workspace_bytes(int64_t E, int K, int D, size_t* bytes);
int gnn_gaussian_bwd(const float* pseudo, const float* mu, const float* inv_sigma,
                     const float* grad_w /*[E,K]*/, int64_t E, int K, int D,
                     float* grad_pseudo /*[E,D]*/, float* grad_mu /*[K,D]*/,
                     float* grad_inv_sigma /*[K,D]*/, void* workspace, size_t workspace_bytes,
                     cudaStream_t stream);

/* ---- dense projection on the tensor cores ---------------------------------------------------
 * C[M,N] = A[M,K] * op(B) in fp32-level accuracy on tcgen05 (error-compensated 3xTF32,
 * fp32 accumulation in tensor memory, TMA operand loads).  Replaces the cuBLAS SGEMM behind
 * torch.matmul(feat, W) / nn.Linear in the layers (layers/gatconv_layer.py:50,
 * layers/edgeconv_layer.py:37-38, layers/gmmconv_layer.py:68).  B is K x N row-major
 * (b_is_n_by_k = 0) or N x K row-major (b_is_n_by_k = 1, the nn.Linear weight layout).
 * Requires K % 4 == 0 and 16-byte aligned A.  `status` is a device int the caller zeroes;
 * a CTA whose bounded barrier wait expires sets it to 1 (results are then invalid). */
int gnn_gemm_tf32x3_supported(int64_t M, int64_t N, int64_t K);
int gnn_gemm_tf32x3_workspace_bytes(int64_t M, int64_t N, int64_t K, size_t* bytes);
int gnn_gemm_tf32x3(const float* A, const float* B, int b_is_n_by_k, float* C, int64_t M, int64_t N,
                    int64_t K, void* workspace, size_t workspace_bytes, int* status,
                    cudaStream_t stream);

/* gnn_gemm_tf32x3 for the projection of a GAT layer: C rows are `heads` heads of `head_w` floats
 * (heads * head_w == N), and the per-node attention scores of layers/gatconv_layer.py:52-53,
 *   score_l[m, h] = <C[m, h, :], attn_l[h, :]>,   score_r[m, h] = <C[m, h, :], attn_r[h, :]>,
 * are formed in the GEMM's epilogue by the thread that stores the row: no pass over C afterwards.
 * head_w must be 32, 64 or 128, or heads == 1 with N <= 128 (gnn_gemm_tf32x3_scores_supported). */
int gnn_gemm_tf32x3_scores_supported(int heads, int head_w);
int gnn_gemm_tf32x3_scores(const float* A, const float* B, int b_is_n_by_k, float* C, int64_t M, int64_t N,
                           int64_t K, const float* attn_l /*[heads,head_w]*/, const float* attn_r, int heads,
                           int head_w, float* score_l /*[M,heads]*/, float* score_r, void* workspace,
                           size_t workspace_bytes, int* status, cudaStream_t stream);

/* C[K1,N1] = A^T * B with A [M,K1], B [M,N1] (the weight gradient X^T * dH of a projection;
 * autograd's MmBackward in the reference, a cuBLAS SGEMM).  Same 3xTF32 tcgen05 kernel, the
 * reduction axis M cut into ranges whose partial tiles are summed in a fixed order. */
int gnn_gemm_tf32x3_tn_workspace_bytes(int64_t M, int64_t K1, int64_t N1, size_t* bytes);
int gnn_gemm_tf32x3_tn(const float* A, const float* B, float* C, int64_t M, int64_t K1, int64_t N1,
                       void* workspace, size_t workspace_bytes, int* status, cudaStream_t stream);

/* ---- unfused operators that share the API ------------------------------------------------
 * gnn_mhspmm: mhspmm.mhspmm (src/spmm/mhspmm.cu:4-66) and, with H = 1, the
 * single-head csr_spmm / csr_spmm_no_edge_value that operators/spmm.py:35-41
 * expects (att == NULL: unit weights).  perm (optional) reads att[perm[e]]. */
int gnn_mhspmm_workspace_bytes(int64_t nnz, int H, int F, size_t* bytes);
int gnn_mhspmm(const int* ptr, const int* idx, int64_t n_seg, int64_t nnz,
               const float* att /*[nnz,H] or NULL*/, const int* perm /*[nnz] or NULL*/,
               const float* feat /*[*,H,F]*/, int H, int F, float* out /*[n_seg,H,F]*/,
               void* workspace, size_t workspace_bytes, cudaStream_t stream);
/* mhsddmm.mhsddmm (src/sddmm/mhsddmm.cu:5-99) and, with H = 1, sddmm.csr_sddmm
 * (src/sddmm/sddmm.cu:361-404): out[e,h] = <A[seg(e),h,:], B[idx[e],h,:]>. */
int gnn_mhsddmm(const int* ptr, const int* idx, int64_t n_seg, int64_t nnz,
                const float* A /*[n_seg,H,F]*/, const float* B /*[*,H,F]*/, int H, int F,
                float* out /*[nnz,H]*/, cudaStream_t stream);
/* sddmm.coo_sddmm (src/sddmm/sddmm.cpp:12-27). */
int gnn_sddmm_coo(const int* row_ind, const int* col_ind, int64_t nnz, const float* A,
                  const float* B, int F, float* out /*[nnz]*/, cudaStream_t stream);
/* mhtranspose.mhtranspose (src/csr2csc/mhtranspose.cu:6-47): out[i,:] = vals[permute[i],:]. */
int gnn_mhtranspose(const int* permute, const float* vals /*[E,H]*/, int64_t E, int H,
                    float* out /*[E,H]*/, cudaStream_t stream);
/* u_add_v.u_add_v_forward / u_add_v_backward (src/u_add_v/u_add_v.cu:4-90).  The
 * backward zero-fills both outputs and accumulates with fp32 atomics. */
int gnn_u_add_v_fwd(const int* row_ptr, const int* col_ind, int64_t n_rows, int64_t nnz,
                    const float* row_val /*[n_rows,F]*/, const float* col_val /*[*,F]*/, int F,
                    float* out /*[nnz,F]*/, cudaStream_t stream);
int gnn_u_add_v_bwd(const int* row_ptr, const int* col_ind, int64_t n_rows, int64_t n_cols,
                    int64_t nnz, const float* grad_out /*[nnz,F]*/, int F,
                    float* grad_row /*[n_rows,F]*/, float* grad_col /*[n_cols,F]*/,
                    cudaStream_t stream);
/* edge_softmax.edge_softmax / edge_softmax_backward (src/edge_softmax/edge_softmax.cu:7-128). */
int gnn_edge_softmax_fwd(const int* row_ptr, int64_t n_rows, int64_t nnz, const float* in /*[nnz,H]*/,
                         int H, float* out /*[nnz,H]*/, cudaStream_t stream);
int gnn_edge_softmax_bwd(const int* row_ptr, int64_t n_rows, int64_t nnz, const float* y,
                         const float* grad_y, int H, float* grad_x, cudaStream_t stream);

/* gnn_gat_fwd with the model's activation on the layer output folded in: act_out = ELU(out)
 * (alpha as in torch.nn.functional.elu) is stored next to out by the warp that normalises the
 * row.  The reference's models apply the activation as a separate framework op after the layer
 * (script/train/train_gatconv_our.py:50-52).  Same arguments and workspace as gnn_gat_fwd;
 * H <= 8 and H*F within one tile (512 floats, 256 if rows are not 16-byte aligned). */
int gnn_gat_fwd_act(const int* row_ptr, const int* col_ind, int64_t n_rows, int64_t nnz,
                    const float* attn_row, const float* attn_col, const float* in_feat, int H, int F,
                    float negative_slope, float alpha, float* out /*[n_rows,H,F]*/,
                    float* act_out /*[n_rows,H,F]*/, float* edge_max, float* edge_sum, void* workspace,
                    size_t workspace_bytes, cudaStream_t stream);

/* ---- opt-in: gathered operand stored as bfloat16 (no counterpart in the reference) -----------
 * gnn_gat_fwd_bf16 is gnn_gat_fwd with in_feat given as bfloat16 [*,H,F] (half the gather traffic);
 * scores, softmax, accumulation and outputs are fp32.  Outside the fp32 parity contract of the
 * other entry points: the result equals gnn_gat_fwd on the bfloat16-rounded features.
 * H <= 8, H*F <= 512 and a multiple of 8, 16-byte aligned.  Workspace as gnn_gat_fwd.
 * gnn_to_bf16 converts n fp32 values (n % 8 == 0) with round-to-nearest-even. */
int gnn_to_bf16(const float* in, int64_t n, void* out_bf16, cudaStream_t stream);
int gnn_gat_fwd_bf16(const int* row_ptr, const int* col_ind, int64_t n_rows, int64_t nnz,
                     const float* attn_row, const float* attn_col, const void* in_feat_bf16, int H, int F,
                     float negative_slope, float* out, float* edge_max, float* edge_sum, void* workspace,
                     size_t workspace_bytes, cudaStream_t stream);

/* ---- graph construction ------------------------------------------------------------------
 * gnn_coo_to_csr replaces the host-side preprocessing of the reference's scripts
 * (script/train/train_gatconv_our.py:82-95: dgl.remove_self_loop / add_self_loop, then
 * scipy.sparse.csr_matrix((ones, (row, col))) -> indptr, indices; train_gmmconv_our.py:80-93).
 * dst/src [n_pairs] are the endpoints of directed edges src -> dst.  Output: the in-edge CSR
 * sorted by (dst, src) with duplicate pairs removed; with self_loops != 0 pairs with
 * dst == src are dropped and one (i, i) per node is added.  Pairs with an endpoint outside
 * [0, n_nodes) are dropped.  col_ind must hold n_pairs + (self_loops ? n_nodes : 0) entries;
 * the number actually written goes to *nnz_out (device memory, int64).  Integer work: the
 * result equals SciPy's bit for bit. */
int gnn_coo_to_csr_workspace_bytes(int64_t n_pairs, int64_t n_nodes, size_t* bytes);
int gnn_coo_to_csr(const int* dst, const int* src, int64_t n_pairs, int64_t n_nodes, int self_loops,
                   int* row_ptr /*[n_nodes+1]*/, int* col_ind, long long* nnz_out, void* workspace,
                   size_t workspace_bytes, cudaStream_t stream);

/* Row-block partition bookkeeping (no counterpart in the reference: single GPU).
 * gnn_edge_balanced_bounds: bounds[g] (device, parts+1 entries) = first row whose first edge is
 * at or after g * nnz / parts.
 * gnn_halo_needs: positions [world*n_nodes + 1] = exclusive scan of the flags "an edge of a row of
 * block q has id v outside block q", laid out [q][v] (bounds: device array of world+1 rows).
 * gnn_compact_flagged: out[positions[i]] = i % period for every i in [0, n) whose flag is set,
 * i.e. the sorted id lists of all blocks one after the other.
 * gnn_halo_remap: ext[e] = idx[e] - lo for ids inside [lo, hi), else (hi - lo) + rank of the id
 * among the flagged ids of this block (positions_of_rank = positions + rank * n_nodes). */
int gnn_edge_balanced_bounds(const int* row_ptr, int64_t n_rows, int parts, int* bounds, cudaStream_t stream);
int gnn_halo_needs_workspace_bytes(int64_t n_nodes, int world, size_t* bytes);
int gnn_halo_needs(const int* ptr, const int* idx, int64_t n_nodes, int64_t nnz, const int* bounds, int world,
                   unsigned* positions, void* workspace, size_t workspace_bytes, cudaStream_t stream);
int gnn_compact_flagged(const unsigned* positions, int64_t n, int64_t period, int* out, cudaStream_t stream);
int gnn_halo_remap(const int* idx, int64_t nnz, int lo, int hi, const unsigned* positions_of_rank, int* ext,
                   cudaStream_t stream);

/* ---- k-nearest-neighbour graph of point clouds ----------------------------------------
 * The graph EdgeConv runs on: the reference builds it with DGL's KNNGraph(k) in front of
 * every layer (script/train/train_edgeconv_our.py:20,52).  points [n_clouds, n_points,
 * n_coords] float32; src_ind[(b*P + i)*k + j] = b*P + index of the j-th nearest point of
 * cloud b to its point i (the layout gnn_edgeconv_fwd reads).  Squared Euclidean distance
 * in float64, coordinates summed in ascending order without fused multiply-add; neighbours
 * ordered by (distance, index), so a point is its own first neighbour.  Nothing of size
 * n_points x n_points is stored.  k <= 64, k <= n_points. */
int gnn_knn_graph(const float* points, int64_t n_clouds, int64_t n_points, int n_coords, int k,
                  int* src_ind /*[n_clouds*n_points*k]*/, cudaStream_t stream);

/* ---- halo exchange over peer-mapped memory (no counterpart in the reference: single GPU) --
 * gnn_peer_alloc: device memory other processes of the node can map; writes its IPC handle
 * (GNN_PEER_HANDLE_BYTES bytes, host memory).  gnn_peer_open maps the allocation behind a
 * handle received from another process (enabling peer access on first use) and returns the
 * address it has in THIS process.  These four calls are for set-up: unlike the rest of the
 * library they allocate / map device memory and may synchronise.
 *
 * gnn_halo_push: for i in [send_off[q], send_off[q+1]) stores row send_idx[i] of x
 * (row_floats floats per row) to dst[q] + (i - send_off[q]) * row_floats, and rows
 * [0, n_own) of x to own_dst (NULL: skip).  send_off [world+1] and dst [world] are HOST
 * arrays; dst[q] is a device address in a peer's allocation (from gnn_peer_open), already
 * advanced to where this rank's rows go.  Ordinary stores, no atomics.  The stores are
 * visible to the peer once the kernel has completed: order that against the consumer with
 * a collective or an event on `stream`. */
#define GNN_MAX_PEERS 8
#define GNN_PEER_HANDLE_BYTES 64
int gnn_peer_alloc(size_t bytes, void** ptr, unsigned char* handle);
int gnn_peer_free(void* ptr);
int gnn_peer_open(const unsigned char* handle, void** ptr);
int gnn_peer_close(void* ptr);
int gnn_halo_push(const float* x, int64_t row_floats, const int* send_idx, const int64_t* send_off,
                  float* const* dst, int world, float* own_dst, int64_t n_own, cudaStream_t stream);
/* The same with an explicit range per rank, for pushing part of a send list (the rows a
 * producer has finished so far): rank q gets rows send_idx[send_beg[q] .. send_beg[q] +
 * send_cnt[q]) at dst[q] + j * row_floats, j counting from 0 inside the range.  send_beg,
 * send_cnt and dst are HOST arrays of `world` entries. */
int gnn_halo_push_ranges(const float* x, int64_t row_floats, const int* send_idx,
                         const int64_t* send_beg, const int64_t* send_cnt, float* const* dst,
                         int world, float* own_dst, int64_t n_own, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* GNN_B200_H_ */
