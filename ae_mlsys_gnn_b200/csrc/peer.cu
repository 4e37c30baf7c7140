// Halo exchange of a row-block partition over peer-mapped memory (NVLink / NVSwitch).
//
// The reference is single-GPU; nothing here has a counterpart in it.  In the partitioned GAT
// every rank needs, per layer and direction, the rows of other ranks' per-node tensors that
// its block of the graph references (its halo).  A collective library moves them as
// "gather the rows into a send buffer, all-to-all, done"; here the owner of the rows stores
// them straight into the halo region of the receiver's buffer:
//
//   gnn_halo_push    one kernel: for every row of the send list, read it from the local tensor
//                    and write it with ordinary 128-bit stores through the receiver's mapped
//                    pointer, at the position the receiver's remapped graph expects; the
//                    rank's own rows are copied into the front of its own buffer by the same
//                    launch.  Plain peer stores only: no TMA, no multicast.
//   gnn_peer_alloc / gnn_peer_open / gnn_peer_close / gnn_peer_free
//                    device allocations that other processes of the node can map
//                    (cudaIpcGetMemHandle / cudaIpcOpenMemHandle).  Set-up time only: these
//                    are the only functions of the library that allocate device memory.
//
// Completion is the caller's business: stores of a kernel are visible to the peer once the
// kernel has completed, so the caller orders "all ranks' push kernels are complete" before
// the consumer with a collective on the same stream (a one-element all-reduce).
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "../../include/gnn_b200.h"
#include "common.cuh"

using namespace gnn;

namespace {

constexpr int kMaxPeers = GNN_MAX_PEERS;

int bad(const char* m) {
  set_last_error(m);
  return GNN_ERR_INVALID_ARG;
}

int cuda_fail(const char* what, cudaError_t e) {
  char buf[256];
  snprintf(buf, sizeof(buf), "%s: %s", what, cudaGetErrorString(e));
  set_last_error(buf);
  return GNN_ERR_CUDA;
}

struct PushParams {
  const float* x;           // [*, row_floats] local per-node tensor
  const int* send_idx;      // local row ids, grouped by destination rank
  int64_t send_beg[kMaxPeers];  // rank q's rows are send_idx[send_beg[q] .. send_beg[q] + send_cnt[q])
  int64_t send_cnt[kMaxPeers];
  float* dst[kMaxPeers];    // receiver q's buffer, already advanced to where this rank's rows go
  float* own_dst;           // this rank's own buffer (rows 0..n_own-1), may be null
  int64_t n_own;
  int64_t row_floats;
  int world;
  int n_groups;             // destination ranks with rows to receive
  int group[kMaxPeers];     // their ranks
  int64_t group_max;        // rows of the largest group
};

// LPR lanes per row (a power of two, 32 for rows of 32 units or more; a unit is 16 bytes with
// VEC, else one float), so a warp moves 32 / LPR rows at a time and consecutive lanes write
// consecutive units: 512 contiguous bytes of the destination per warp instruction for wide rows.
// The rows are visited in slots that cycle through the destination ranks (slot s: rank
// group[s % n_groups], its row s / n_groups), so at every moment a sender's stores are spread
// over all its receivers and no receiver has all the senders of the node storing into it at
// once; a slot past the end of a shorter group is skipped.  The rank's own rows follow.
// The per-rank tables are copied to shared memory first: indexing kernel parameters with a
// run-time index would send every access through local memory.
template <bool VEC>
__global__ void __launch_bounds__(256)
halo_push_kernel(PushParams p, int lpr) {
  __shared__ int64_t s_beg[kMaxPeers], s_cnt[kMaxPeers];
  __shared__ float* s_dst[kMaxPeers];
  __shared__ int s_group[kMaxPeers];
  if (threadIdx.x < kMaxPeers) {
    s_beg[threadIdx.x] = p.send_beg[threadIdx.x];
    s_cnt[threadIdx.x] = p.send_cnt[threadIdx.x];
    s_dst[threadIdx.x] = p.dst[threadIdx.x];
    s_group[threadIdx.x] = p.group[threadIdx.x];
  }
  __syncthreads();
  const int upr = (int)(VEC ? p.row_floats / 4 : p.row_floats);  // units per row
  const int rpw = 32 / lpr;                                       // rows per warp and step
  const int lane = threadIdx.x & 31;
  const int sub = lane / lpr, off = lane % lpr;
  const int64_t n_slots = p.group_max * p.n_groups;
  const int64_t total = n_slots + p.n_own;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t base = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * rpw; base < total;
       base += warps * rpw) {
    const int64_t slot = base + sub;
    if (slot >= total) continue;
    const float* src;
    float* dst;
    if (slot < n_slots) {
      const int64_t i = slot / p.n_groups;
      const int q = s_group[(int)(slot - i * p.n_groups)];
      if (i >= s_cnt[q]) continue;
      src = p.x + (size_t)__ldg(p.send_idx + s_beg[q] + i) * p.row_floats;
      dst = s_dst[q] + (size_t)i * p.row_floats;
    } else {
      const int64_t r = slot - n_slots;
      src = p.x + (size_t)r * p.row_floats;
      dst = p.own_dst + (size_t)r * p.row_floats;
    }
    if (VEC) {
      const float4* s4 = reinterpret_cast<const float4*>(src);
      float4* d4 = reinterpret_cast<float4*>(dst);
      // up to four units per lane requested before the first is stored
      int u = off;
      for (; u + 3 * lpr < upr; u += 4 * lpr) {
        const float4 a = __ldg(s4 + u), b = __ldg(s4 + u + lpr), c = __ldg(s4 + u + 2 * lpr), d = __ldg(s4 + u + 3 * lpr);
        d4[u] = a; d4[u + lpr] = b; d4[u + 2 * lpr] = c; d4[u + 3 * lpr] = d;
      }
      for (; u < upr; u += lpr) d4[u] = __ldg(s4 + u);
    } else {
      for (int u = off; u < upr; u += lpr) dst[u] = __ldg(src + u);
    }
  }
}

}  // namespace

extern "C" int gnn_peer_alloc(size_t bytes, void** ptr, unsigned char* handle /*[GNN_PEER_HANDLE_BYTES]*/) {
  if (!ptr || !handle || bytes == 0) return bad("gnn_peer_alloc: bad argument");
  static_assert(sizeof(cudaIpcMemHandle_t) <= GNN_PEER_HANDLE_BYTES, "handle size");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return cuda_fail("gnn_peer_alloc: cudaMalloc", e);
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return cuda_fail("gnn_peer_alloc: cudaIpcGetMemHandle", e);
  }
  memset(handle, 0, GNN_PEER_HANDLE_BYTES);
  memcpy(handle, &h, sizeof(h));
  *ptr = p;
  return GNN_OK;
}

extern "C" int gnn_peer_free(void* ptr) {
  if (!ptr) return GNN_OK;
  cudaError_t e = cudaFree(ptr);
  return e == cudaSuccess ? GNN_OK : cuda_fail("gnn_peer_free", e);
}

extern "C" int gnn_peer_open(const unsigned char* handle, void** ptr) {
  if (!handle || !ptr) return bad("gnn_peer_open: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return cuda_fail("gnn_peer_open: cudaIpcOpenMemHandle", e);
  *ptr = p;
  return GNN_OK;
}

extern "C" int gnn_peer_close(void* ptr) {
  if (!ptr) return GNN_OK;
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  return e == cudaSuccess ? GNN_OK : cuda_fail("gnn_peer_close", e);
}

extern "C" int gnn_halo_push_ranges(const float* x, int64_t row_floats, const int* send_idx,
                                    const int64_t* send_beg, const int64_t* send_cnt, float* const* dst,
                                    int world, float* own_dst, int64_t n_own, cudaStream_t stream) {
  if (world < 1 || world > kMaxPeers) return bad("gnn_halo_push: world must be in [1, GNN_MAX_PEERS]");
  if (row_floats <= 0 || n_own < 0 || !send_beg || !send_cnt || !dst) return bad("gnn_halo_push: bad argument");
  PushParams p;
  p.x = x; p.send_idx = send_idx; p.own_dst = own_dst; p.n_own = own_dst ? n_own : 0;
  p.row_floats = row_floats; p.world = world;
  bool vec = row_floats % 4 == 0 && aligned16(x) && (!own_dst || aligned16(own_dst));
  p.n_groups = 0;
  p.group_max = 0;
  int64_t n_send = 0;
  for (int q = 0; q < kMaxPeers; ++q) {
    p.group[q] = 0;
    p.dst[q] = q < world ? dst[q] : nullptr;
    p.send_beg[q] = q < world ? send_beg[q] : 0;
    p.send_cnt[q] = q < world ? send_cnt[q] : 0;
    if (q >= world) continue;
    const int64_t cnt = send_cnt[q];
    if (cnt < 0 || send_beg[q] < 0) return bad("gnn_halo_push: negative range");
    if (cnt == 0) continue;
    if (!dst[q]) return bad("gnn_halo_push: rows for a rank without a destination pointer");
    if (!aligned16(dst[q])) vec = false;
    p.group[p.n_groups++] = q;
    if (cnt > p.group_max) p.group_max = cnt;
    n_send += cnt;
  }
  if (n_send > 0 && (!send_idx || !x)) return bad("gnn_halo_push: null pointer");
  if (p.n_own > 0 && !x) return bad("gnn_halo_push: null pointer");
  if (p.n_groups == 0) p.n_groups = 1;  // no rows to send: zero slots, the divisor stays valid
  const int64_t slots = p.group_max * p.n_groups + p.n_own;
  if (slots == 0) return GNN_OK;
  const int64_t upr = vec ? row_floats / 4 : row_floats;
  int lpr = 1;
  while (lpr < 32 && lpr < upr) lpr <<= 1;
  const int64_t warps = (slots + 32 / lpr - 1) / (32 / lpr);
  int64_t blocks = (warps + 7) / 8;
  // grid-stride beyond a few waves (GNN_B200_PUSH_BLOCKS_PER_SM, 1..32: measured at 2, 4 and 32
  // blocks per SM the transfer time does not depend on it)
  static const int per_sm = [] {
    const char* e = getenv("GNN_B200_PUSH_BLOCKS_PER_SM");
    const int v = e ? atoi(e) : 32;
    return v < 1 ? 1 : (v > 32 ? 32 : v);
  }();
  const int64_t cap = 148LL * per_sm;
  if (blocks > cap) blocks = cap;
  if (vec) halo_push_kernel<true><<<(unsigned)blocks, 256, 0, stream>>>(p, lpr);
  else halo_push_kernel<false><<<(unsigned)blocks, 256, 0, stream>>>(p, lpr);
  return check_launch("gnn_halo_push");
}

extern "C" int gnn_halo_push(const float* x, int64_t row_floats, const int* send_idx, const int64_t* send_off,
                             float* const* dst, int world, float* own_dst, int64_t n_own, cudaStream_t stream) {
  if (world < 1 || world > kMaxPeers) return bad("gnn_halo_push: world must be in [1, GNN_MAX_PEERS]");
  if (!send_off) return bad("gnn_halo_push: bad argument");
  int64_t beg[kMaxPeers], cnt[kMaxPeers];
  for (int q = 0; q < world; ++q) {
    beg[q] = send_off[q];
    cnt[q] = send_off[q + 1] - send_off[q];
    if (cnt[q] < 0) return bad("gnn_halo_push: send_off must ascend");
  }
  return gnn_halo_push_ranges(x, row_floats, send_idx, beg, cnt, dst, world, own_dst, n_own, stream);
}
