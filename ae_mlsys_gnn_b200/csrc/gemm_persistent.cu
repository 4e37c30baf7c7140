// Persistent, warp-specialised 3xTF32 GEMM on the 5th-generation tensor cores.
//
//   C[z] = A * B^T over the z-th range of the reduction axis,   fp32 in, fp32 out
//
// with the error-compensated product  a_lo*b_hi + a_hi*b_lo + a_hi*b_hi  accumulated in
// fp32 in tensor memory.  For an operand split in the kernel a_hi is the fp32 value as it
// lies in shared memory (kind::tf32 reads the upper 19 bits, i.e. truncates) and
// a_lo = a - trunc_tf32(a), which is exact in fp32; pre-split operands use
// a_hi = tf32_rn(a), a_lo = a - a_hi.
//
// One CTA per SM walks over the output tiles (128 x 128, the column tile fastest so that
// the CTAs working at the same time share their A rows through L2).  10 warps:
//   warp 0      TMA producer: one stage = one block of 32 along the reduction axis
//   warp 1      tensor-memory allocation and single-thread tcgen05.mma issue
//   warps 2-5   operand conversion: write the lo part of the fp32 tile that TMA delivered
//               into a second buffer -- elementwise, so the swizzle that TMA applied stays
//               what the MMA descriptors expect
//   warps 6-9   epilogue: tcgen05.ld of a finished accumulator and global stores
// The accumulator is double buffered (2 x 128 tensor-memory columns): the epilogue of one
// tile overlaps the main loop of the next.  The large operand is therefore read from HBM
// once, as fp32, with no pre-pass.
//
// Operands whose reduction axis is the slow one in memory (the weight gradient X^T * dH,
// both operands [nodes][features]) are loaded as MN-major tiles: four 32 x 32 boxes per
// 128 rows with the 32-byte-atom variant of the 128-byte swizzle, and descriptors with the
// MN-major bit set -- no transposed copies.
//
// Every mbarrier wait is bounded in time: on expiry the CTA raises a shared flag that ends
// all its loops, sets the status word, gives its copies in flight a bounded time to land,
// frees its tensor memory and returns.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include "../../include/gnn_b200.h"
#include "common.cuh"
#include "gemm_persistent.cuh"

namespace gnn {
namespace {

constexpr int BM = 128, BK = 32;
constexpr int kTileBytes = BM * BK * 4;      // 16 KB: one 128-row operand tile (raw/hi or lo)
constexpr int kConvThreads = 128;
constexpr int kThreads = 32 * 10;
constexpr int kAccBufs = 2;
constexpr int kMaxStages = 3;
constexpr int kNumBars = 3 * kMaxStages + 2 * kAccBufs;
// Epilogue staging: a 32 x 32 fp32 block per epilogue warp (4 KB), through which the rows a
// thread holds are turned into stores that cover whole 128-byte lines.
constexpr int kEpiStageBytes = 4 * 32 * 32 * 4;
constexpr int kEpiStageOffset = (8 * kNumBars + 16 + 127) / 128 * 128;  // after the barriers and the TMEM slot, 128-byte aligned

// Geometry of one instantiation.  BN = 128: three stages, 256 tensor-memory columns, any operand
// mode.  BN = 256 (B given as split hi/lo, K-major: the projection weights): the B tile is
// 256 rows, two stages of 96 KB, all 512 tensor-memory columns; per multiply-add it reads 2/3 of
// the shared-memory bytes of the 128-wide tile, which is what bounds this kernel.
template <int BN>
struct Geom {
  static constexpr int kStages = BN == 128 ? 3 : 2;
  static constexpr int kBTileBytes = BN * BK * 4;
  static constexpr int kStageBytes = 2 * kTileBytes + 2 * kBTileBytes;  // A0, A1, B0, B1
  static constexpr int kTmemCols = kAccBufs * BN;
  static constexpr size_t kSmemBytes =
      (size_t)kStages * kStageBytes + 1024 /*alignment slack*/ + kEpiStageOffset + kEpiStageBytes;
};
// The tensor core adds into its fp32 accumulator with truncation: a chain of n MMAs comes
// out low by about n * 2^-26 of its value (measured: -4e-4 after 25,000 MMAs).  After this
// many K blocks (12 MMAs each) the accumulator is therefore drained and the running sum
// continues in the registers of the epilogue threads with round-to-nearest adds.
constexpr int kChainKb = 16;
constexpr long long kWaitCycles = 4000000000LL;   // about two seconds
constexpr long long kDrainCycles = 200000000LL;   // about a tenth of a second

struct Params {
  int M, N;                 // output rows, columns
  int total_kb;             // blocks of 32 along the reduction axis
  int kb_per_split;         // blocks handled by one split
  int tiles_m, tiles_n, num_tiles;  // num_tiles = tiles_m * tiles_n * splits
  float* C;
  int64_t ldc;
  int64_t split_stride;     // floats between the outputs of consecutive splits
  int* status;
  int a_mode, b_mode;       // OperandMode
  int chain_kb;             // K blocks accumulated in tensor memory before the sum moves to registers
  // Optional epilogue of the GAT projection: the output row is H heads of head_w floats, and
  //   score_l[row, h] = <C[row, h, :], attn_l[h, :]>,  score_r[row, h] = <C[row, h, :], attn_r[h, :]>
  // (layers/gatconv_layer.py:52-53) are formed by the thread that holds the row, while it stores it.
  // Requires every head to lie inside one column tile and to start on a 32-column chunk:
  // head_w in {32, 64, 128}, or one head with N <= 128.  nullptr: off.
  const float* attn_l;
  const float* attn_r;
  float* score_l;
  float* score_r;
  int heads, head_w;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Waits for the phase of the given parity; gives up (false) when another role of the CTA
// has failed (failed != nullptr and set) or when the time limit has passed.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* failed,
                                          long long limit = kWaitCycles) {
  const long long t0 = clock64();
  for (uint32_t i = 0;; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
    if ((i & 15) == 15) {
      if (failed && *failed) return false;
      if (clock64() - t0 > limit) return false;
    }
  }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}

// Shared-memory matrix descriptors (version 1).
//   K-major tile [128 rows][32 floats], TMA SWIZZLE_128B, layout type 2: rows are 128 bytes,
//   8-row groups 1024 bytes apart (stride offset); the leading offset is not used.  A K
//   slice of 8 is 32 bytes further.
//   MN-major tile [4 groups][32 reduction rows][32 floats], TMA SWIZZLE_128B_ATOM_32B,
//   layout type 1 (128-byte swizzle on 32-byte units; 32-bit MN-major data reads as zeros
//   with layout type 2): a group of 32 output rows is one 4 KB box (leading offset 4096);
//   inside it the swizzle pattern repeats every 4 reduction rows, and a K slice of 8 is two
//   such 512-byte atoms (stride offset 512).  The next K slice is 1024 bytes further.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                              uint32_t layout_type) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)layout_type << 61;
  return d;
}
__device__ __forceinline__ uint64_t operand_desc(uint32_t saddr, bool mn_major) {
  return mn_major ? make_desc(saddr, 4096, 512, 1) : make_desc(saddr, 16, 1024, 2);
}

// Instruction descriptor: D = F32 (1 at bits 4-5), A = B = TF32 (2 at bits 7-9, 10-12),
// bit 15 / 16 = A / B is MN-major, N/8 at bits 17-22, M/16 at bits 24-28.
__device__ __forceinline__ uint32_t make_idesc(int n_mma, bool a_mn, bool b_mn) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) |
         ((uint32_t)(n_mma >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool is_raw(int mode) { return mode == kKMajorRaw || mode == kMnMajorRaw; }
__device__ __forceinline__ uint32_t operand_tx_bytes(int mode, int tile_bytes) {
  return is_raw(mode) ? tile_bytes : 2 * tile_bytes;
}

// Issues the copies of one operand for one stage.  r0: first output row of the tile;
// kblk: index of the block of 32 along the reduction axis; tile_bytes: bytes of one tile of
// this operand (the second copy of a split operand follows the first).
__device__ __forceinline__ void load_operand(int mode, uint32_t x0, const CUtensorMap* m0, const CUtensorMap* m1,
                                             int r0, int kblk, uint32_t bar, int tile_bytes = kTileBytes) {
  if (mode == kKMajorRaw) {
    tma_load_2d(x0, m0, kblk * BK, r0, bar);
  } else if (mode == kKMajorSplit) {
    tma_load_2d(x0, m0, kblk * BK, r0, bar);
    tma_load_2d(x0 + tile_bytes, m1, kblk * BK, r0, bar);
  } else if (mode == kKMajorSplitBlocked) {
    tma_load_3d(x0, m0, 0, r0, kblk, bar);
    tma_load_3d(x0 + tile_bytes, m1, 0, r0, kblk, bar);
  } else {
#pragma unroll
    for (int g = 0; g < BM / 32; ++g) tma_load_2d(x0 + g * 4096, m0, r0 + 32 * g, kblk * BK, bar);
  }
}

// lo = x - trunc_tf32(x) into the second buffer; the first keeps the fp32 values, of which
// the tensor core reads the upper 19 bits.  128 threads, 16 KB.
__device__ __forceinline__ void convert_tile(const uint8_t* x0, uint8_t* x1, int tid) {
  float4 v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = *reinterpret_cast<const float4*>(x0 + (i * kConvThreads + tid) * 16);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float4 l;
    l.x = v[i].x - __uint_as_float(__float_as_uint(v[i].x) & 0xFFFFE000u);
    l.y = v[i].y - __uint_as_float(__float_as_uint(v[i].y) & 0xFFFFE000u);
    l.z = v[i].z - __uint_as_float(__float_as_uint(v[i].z) & 0xFFFFE000u);
    l.w = v[i].w - __uint_as_float(__float_as_uint(v[i].w) & 0xFFFFE000u);
    *reinterpret_cast<float4*>(x1 + (i * kConvThreads + tid) * 16) = l;
  }
}

struct TileCoord {
  int m0, n0, kb_begin, num_kb, z;
  int chains;  // accumulator chains of at most chain_kb K blocks (1 for an empty range)
};
template <int BN>
__device__ __forceinline__ TileCoord decode_tile(const Params& p, int tile) {
  TileCoord t;
  const int nt = tile % p.tiles_n;
  const int rest = tile / p.tiles_n;
  const int mt = rest % p.tiles_m;
  t.z = rest / p.tiles_m;
  t.m0 = mt * BM;
  t.n0 = nt * BN;
  t.kb_begin = t.z * p.kb_per_split;
  t.num_kb = max(0, min(p.kb_per_split, p.total_kb - t.kb_begin));
  t.chains = max(1, (t.num_kb + p.chain_kb - 1) / p.chain_kb);
  return t;
}

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_persistent_kernel(const __grid_constant__ CUtensorMap map_a0, const __grid_constant__ CUtensorMap map_a1,
                       const __grid_constant__ CUtensorMap map_b0, const __grid_constant__ CUtensorMap map_b1,
                       Params p) {
  constexpr int kStages = Geom<BN>::kStages;
  constexpr int kStageBytes = Geom<BN>::kStageBytes;
  constexpr int kBTileBytes = Geom<BN>::kBTileBytes;
  constexpr int kTmemCols = Geom<BN>::kTmemCols;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;  // swizzle atoms need 1024-byte alignment
  uint8_t* const base_ptr = smem_raw + (base - raw_addr);
  const uint32_t bars = base + kStages * kStageBytes;
  auto full_bar = [&](int s) { return bars + 8u * s; };                       // TMA -> converters
  auto conv_bar = [&](int s) { return bars + 8u * (kStages + s); };           // converters -> MMA
  auto empty_bar = [&](int s) { return bars + 8u * (2 * kStages + s); };      // MMA -> TMA
  auto acc_full_bar = [&](int b) { return bars + 8u * (3 * kMaxStages + b); };   // MMA -> epilogue
  auto acc_empty_bar = [&](int b) { return bars + 8u * (3 * kMaxStages + kAccBufs + b); };  // epilogue -> MMA
  const uint32_t tmem_slot = bars + 8u * kNumBars;
  uint32_t* const tmem_slot_ptr = reinterpret_cast<uint32_t*>(base_ptr + kStages * kStageBytes + 8 * kNumBars);
  float4* const epi_stage = reinterpret_cast<float4*>(base_ptr + kStages * kStageBytes + kEpiStageOffset);

  __shared__ volatile int s_failed;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    s_failed = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(conv_bar(s), kConvThreads);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < kAccBufs; ++b) {
      mbar_init(acc_full_bar(b), 1);
      mbar_init(acc_empty_bar(b), 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      const uint32_t tx = operand_tx_bytes(p.a_mode, kTileBytes) + operand_tx_bytes(p.b_mode, kBTileBytes);
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < p.num_tiles && !s_failed; tile += gridDim.x) {
        const TileCoord t = decode_tile<BN>(p, tile);
        for (int kb = 0; kb < t.num_kb; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t round = it / kStages;
          if (round > 0 && !mbar_wait(empty_bar(s), (round - 1) & 1, &s_failed)) { s_failed = 1; break; }
          const uint32_t st = base + s * kStageBytes;
          mbar_expect_tx(full_bar(s), tx);
          load_operand(p.a_mode, st, &map_a0, &map_a1, t.m0, t.kb_begin + kb, full_bar(s));
          load_operand(p.b_mode, st + 2 * kTileBytes, &map_b0, &map_b1, t.n0, t.kb_begin + kb, full_bar(s),
                       kBTileBytes);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issue
    if (lane == 0) {
      const bool a_mn = p.a_mode == kMnMajorRaw, b_mn = p.b_mode == kMnMajorRaw;
      const uint64_t a_step = a_mn ? (1024 >> 4) : (32 >> 4);  // descriptor advance per K slice of 8
      const uint64_t b_step = b_mn ? (1024 >> 4) : (32 >> 4);
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.num_tiles && ok && !s_failed; tile += gridDim.x) {
        const TileCoord t = decode_tile<BN>(p, tile);
        int n_mma = min(BN, p.N - t.n0);
        n_mma = (n_mma + 15) & ~15;
        const uint32_t idesc = make_idesc(n_mma, a_mn, b_mn);
        for (int c = 0; c < t.chains && ok; ++c, ++tcount) {
          const int buf = tcount & 1;
          const uint32_t use = tcount >> 1;
          // a fresh barrier lets the wait for parity 1 through: the first use of a buffer does not block
          if (!mbar_wait(acc_empty_bar(buf), (use & 1) ^ 1, &s_failed)) { s_failed = 1; ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t tmem_acc = tmem_base + (uint32_t)(buf * BN);
          const int kb0 = c * p.chain_kb, kb1 = min(t.num_kb, kb0 + p.chain_kb);
          for (int kb = kb0; kb < kb1; ++kb, ++it) {
            const int s = it % kStages;
            if (!mbar_wait(conv_bar(s), (it / kStages) & 1, &s_failed)) { s_failed = 1; ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t st = base + s * kStageBytes;
            const uint64_t a_hi = operand_desc(st, a_mn);
            const uint64_t a_lo = operand_desc(st + kTileBytes, a_mn);
            const uint64_t b_hi = operand_desc(st + 2 * kTileBytes, b_mn);
            const uint64_t b_lo = operand_desc(st + 2 * kTileBytes + kBTileBytes, b_mn);
#pragma unroll
            for (int k = 0; k < BK / 8; ++k) {
              const uint64_t da = a_step * k, db = b_step * k;
              umma_tf32(tmem_acc, a_lo + da, b_hi + db, idesc, (kb > kb0) || (k != 0));
              umma_tf32(tmem_acc, a_hi + da, b_lo + db, idesc, 1);
              umma_tf32(tmem_acc, a_hi + da, b_hi + db, idesc, 1);
            }
            umma_commit(empty_bar(s));  // the stage is free once these MMAs have read it
          }
          if (ok) umma_commit(acc_full_bar(buf));  // this chain's accumulator is complete
        }
      }
    }
  } else if (warp < 6) {
    // ---------------------------------------------------------------- operand conversion
    const int tid = threadIdx.x - 64;
    const bool conv_a = is_raw(p.a_mode), conv_b = is_raw(p.b_mode);
    uint32_t it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.num_tiles && ok && !s_failed; tile += gridDim.x) {
      const TileCoord t = decode_tile<BN>(p, tile);
      for (int kb = 0; kb < t.num_kb; ++kb, ++it) {
        const int s = it % kStages;
        if (!mbar_wait(full_bar(s), (it / kStages) & 1, &s_failed)) { s_failed = 1; ok = false; break; }
        uint8_t* st = base_ptr + s * kStageBytes;
        if (conv_a) convert_tile(st, st + kTileBytes, tid);
        if constexpr (BN == 128) {  // the 256-wide tile takes B already split
          if (conv_b) convert_tile(st + 2 * kTileBytes, st + 3 * kTileBytes, tid);
        }
        // the tensor core reads shared memory through the async proxy
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive(conv_bar(s));
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int lg = warp & 3;  // this warp may touch tensor-memory lanes [32*lg, 32*lg + 32)
    uint32_t tcount = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.num_tiles && ok && !s_failed; tile += gridDim.x) {
      const TileCoord t = decode_tile<BN>(p, tile);
      const int row = t.m0 + lg * 32 + lane;
      float* const Cout = p.C + (size_t)t.z * p.split_stride;
      // running fp32 sum of this thread's output row when the tile has several chains (the
      // 256-wide tile is only launched for reductions that fit one chain)
      float sum[BN == 128 ? BN : 1];
      float dl = 0.f, dr = 0.f;  // running dot products of the current head with attn_l / attn_r
      for (int ch = 0; ch < t.chains; ++ch, ++tcount) {
        const int buf = tcount & 1;
        if (!mbar_wait(acc_full_bar(buf), (tcount >> 1) & 1, &s_failed)) { s_failed = 1; ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const bool last = ch == t.chains - 1;
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          const int col0 = t.n0 + c * 32;
          if (col0 >= p.N) break;
          uint32_t r[32];
          const uint32_t taddr = tmem_base + ((uint32_t)(lg * 32) << 16) + (uint32_t)(buf * BN + c * 32);
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
          if (t.num_kb == 0) {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0u;  // an empty range contributes nothing
          }
          if constexpr (BN == 128) {
            if (t.chains > 1) {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const float v = __uint_as_float(r[j]);
                sum[c * 32 + j] = ch == 0 ? v : sum[c * 32 + j] + v;
                r[j] = __float_as_uint(sum[c * 32 + j]);
              }
            }
          }
          if (last && p.score_l != nullptr) {
            const int ncols = min(32, p.N - col0);
            if (ncols == 32) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                const float4 al = __ldg(reinterpret_cast<const float4*>(p.attn_l + col0 + j));
                const float4 ar = __ldg(reinterpret_cast<const float4*>(p.attn_r + col0 + j));
                dl = fmaf(__uint_as_float(r[j]), al.x, dl); dr = fmaf(__uint_as_float(r[j]), ar.x, dr);
                dl = fmaf(__uint_as_float(r[j + 1]), al.y, dl); dr = fmaf(__uint_as_float(r[j + 1]), ar.y, dr);
                dl = fmaf(__uint_as_float(r[j + 2]), al.z, dl); dr = fmaf(__uint_as_float(r[j + 2]), ar.z, dr);
                dl = fmaf(__uint_as_float(r[j + 3]), al.w, dl); dr = fmaf(__uint_as_float(r[j + 3]), ar.w, dr);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (j < ncols) {
                  dl = fmaf(__uint_as_float(r[j]), __ldg(p.attn_l + col0 + j), dl);
                  dr = fmaf(__uint_as_float(r[j]), __ldg(p.attn_r + col0 + j), dr);
                }
            }
            const int end = col0 + ncols;  // a head ends with this chunk?
            if (end % p.head_w == 0 || end == p.N) {
              if (row < p.M) {
                const int head = (end - 1) / p.head_w;
                p.score_l[(size_t)row * p.heads + head] = dl;
                p.score_r[(size_t)row * p.heads + head] = dr;
              }
              dl = dr = 0.f;
            }
          }
          // A thread holds 32 consecutive floats of ONE row, so storing them directly makes every
          // warp instruction touch 32 different lines, 16 bytes each.  Full chunks of aligned
          // outputs go through the warp's staging block instead (written row-wise with the
          // 16-byte units of row r rotated by r mod 8, read back four rows at a time, both
          // conflict-free): every store instruction then covers four whole 128-byte lines.
          const bool staged = last && p.N - col0 >= 32 && (p.ldc & 3) == 0 && ((uintptr_t)Cout & 15) == 0;  // warp-uniform
          if (staged) {
            float4* const stg = epi_stage + lg * 256;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              stg[lane * 8 + (j ^ (lane & 7))] =
                  make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                              __uint_as_float(r[4 * j + 3]));
            __syncwarp();
            const int u = lane & 7;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rr = i * 4 + (lane >> 3);
              const float4 v = stg[rr * 8 + (u ^ (rr & 7))];
              const int grow = t.m0 + lg * 32 + rr;
              if (grow < p.M) *reinterpret_cast<float4*>(Cout + (size_t)grow * p.ldc + col0 + u * 4) = v;
            }
            __syncwarp();  // the block is rewritten by the next chunk
          } else if (last && row < p.M) {
            float* crow = Cout + (size_t)row * p.ldc + col0;
            const int ncols = min(32, p.N - col0);
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
        // the buffer may be overwritten once all four epilogue warps have read it
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty_bar(buf));
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (s_failed) {
    // something expired: give the copies this CTA may still have in flight a bounded time
    // to land before its shared memory is released
    if (threadIdx.x == 0) {
      *p.status = 1;
      for (int s = 0; s < kStages; ++s) {
        mbar_wait(full_bar(s), 0, nullptr, kDrainCycles);
        mbar_wait(full_bar(s), 1, nullptr, kDrainCycles);
      }
    }
    __syncthreads();
  }
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

}  // namespace
}  // namespace gnn

// ------------------------------------------------------------------------------------------
// host side

namespace gnn {
namespace {

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

// 2-D map over a row-major fp32 matrix [outer][inner], 128-byte swizzle, zero fill outside.
bool encode_2d(CUtensorMap* m, const float* ptr, int64_t outer, int64_t inner, int box_inner, int box_outer,
               CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)inner * 4};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)ptr, dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 3-D map over a K-blocked operand [kblocks][rows][32]: box = 32 x 128 rows x 1 block.
bool encode_blocked(CUtensorMap* m, const float* ptr, int64_t rows, int64_t kblocks) {
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

// box_rows: output rows of this operand per tile (128, or 256 for the wide B tile)
bool encode_operand(const GemmOperand& o, int64_t K, CUtensorMap* m0, CUtensorMap* m1, int box_rows = BM) {
  const int64_t kblocks = (K + BK - 1) / BK;
  switch (o.mode) {
    case kKMajorRaw:
      *m1 = CUtensorMap{};
      return encode_2d(m0, o.p0, o.rows, K, BK, box_rows);
    case kKMajorSplit:
      return encode_2d(m0, o.p0, o.rows, K, BK, box_rows) && encode_2d(m1, o.p1, o.rows, K, BK, box_rows);
    case kKMajorSplitBlocked:
      return encode_blocked(m0, o.p0, o.rows, kblocks) && encode_blocked(m1, o.p1, o.rows, kblocks);
    case kMnMajorRaw:
      *m1 = CUtensorMap{};
      return encode_2d(m0, o.p0, K, o.rows, 32, BK, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
  }
  return false;
}

template <int BN>
int launch_instance(const CUtensorMap& ma0, const CUtensorMap& ma1, const CUtensorMap& mb0, const CUtensorMap& mb1,
                    Params p, int64_t b_rows, int splits, cudaStream_t stream) {
  static bool attr_set = false;  // per process and instantiation; the attribute is per device
  static int attr_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set || attr_dev != dev) {
    if (cudaFuncSetAttribute(gemm_persistent_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)Geom<BN>::kSmemBytes) != cudaSuccess) {
      set_last_error("gnn_gemm_tf32x3: cannot reserve dynamic shared memory");
      return GNN_ERR_CUDA;
    }
    attr_set = true;
    attr_dev = dev;
  }
  int sms = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 148;
  p.tiles_n = (int)((b_rows + BN - 1) / BN);
  const int64_t tiles = (int64_t)p.tiles_m * p.tiles_n * splits;
  if (tiles > INT32_MAX) {
    set_last_error("gnn_gemm_tf32x3: too many output tiles");
    return GNN_ERR_INVALID_ARG;
  }
  p.num_tiles = (int)tiles;
  const int grid = (int)(tiles < sms ? tiles : sms);
  gemm_persistent_kernel<BN><<<grid, kThreads, Geom<BN>::kSmemBytes, stream>>>(ma0, ma1, mb0, mb1, p);
  return GNN_OK;
}

}  // namespace

int launch_gemm_persistent(const GemmOperand& a, const GemmOperand& b, int64_t K, float* C, int64_t ldc,
                           int splits, int64_t split_stride, int* status, cudaStream_t stream,
                           const GemmScores* scores) {
  Params p;
  p.M = (int)a.rows;
  p.N = (int)b.rows;
  p.total_kb = (int)((K + BK - 1) / BK);
  p.kb_per_split = (p.total_kb + splits - 1) / splits;
  p.tiles_m = (int)((a.rows + BM - 1) / BM);
  p.tiles_n = 0;
  p.num_tiles = 0;
  p.C = C;
  p.ldc = ldc;
  p.split_stride = split_stride;
  p.status = status;
  p.a_mode = a.mode;
  p.b_mode = b.mode;
  p.chain_kb = kChainKb;
  p.attn_l = p.attn_r = nullptr;
  p.score_l = p.score_r = nullptr;
  p.heads = 1;
  p.head_w = (int)b.rows;
  if (scores) {
    p.attn_l = scores->attn_l; p.attn_r = scores->attn_r;
    p.score_l = scores->score_l; p.score_r = scores->score_r;
    p.heads = scores->heads; p.head_w = scores->head_w;
  }
  // the 256-wide column tile: weights given split and K-major, a reduction that fits one
  // accumulator chain, at least 256 output columns (GNN_B200_GEMM_BN=128 keeps the narrow tile)
  static const bool wide_ok = [] {
    const char* e = getenv("GNN_B200_GEMM_BN");
    return !(e && e[0] == '1' && e[1] == '2' && e[2] == '8');
  }();
  const bool wide = wide_ok && b.mode == kKMajorSplit && a.mode == kKMajorRaw && splits == 1 && b.rows >= 256 &&
                    p.total_kb <= kChainKb;
  CUtensorMap ma0, ma1, mb0, mb1;
  if (!encode_operand(a, K, &ma0, &ma1) || !encode_operand(b, K, &mb0, &mb1, wide ? 256 : BM)) {
    set_last_error("gnn_gemm_tf32x3: cuTensorMapEncodeTiled failed");
    return GNN_ERR_CUDA;
  }
  return wide ? launch_instance<256>(ma0, ma1, mb0, mb1, p, b.rows, splits, stream)
              : launch_instance<128>(ma0, ma1, mb0, mb1, p, b.rows, splits, stream);
}

}  // namespace gnn
