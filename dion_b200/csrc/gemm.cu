// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   warp 0      : TMA producer (one elected lane) - 128B-swizzled tiles of A and B
//   warp 1      : TMEM allocator + tcgen05.mma issuer (one elected lane)
//   warps 2..9  : epilogue - tcgen05.ld of the fp32 accumulator, fused
//                 alpha/beta/activation, bf16 or fp32 stores (optionally transposed
//                 mirror, bf16 shadow copy, or fp32 atomic accumulation for split-K)
//
//   warps 10-11 : all-gather variant only (GemmArgs::Gather) - copy the row blocks of A that
//                 other GPUs produced out of their symmetric-memory slots while the tiles
//                 of the rows already in place are being multiplied
//
// The accumulator is double buffered in TMEM (2 x BLOCK_N columns) so the epilogue
// of tile i overlaps the main loop of tile i+1.  Operands may be bf16 (kind::f16)
// or fp32 read as tf32 (kind::tf32); each operand may be K-major or MN-major, which
// covers A*B, A*B^T, A^T*B and A^T*B^T on row-major storage without copies.
//
// This replaces the cuBLAS bmm / addmm / baddbmm calls of the reference optimizers
// (dion/dion.py:801,839,1494-1530; dion/muon.py:620-647;
// dion/newton_schulz_triton.py:58-258,363-369) and the Linear layers of the model.
#include "gemm.h"

#include <cuda.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <memory>
#include <mutex>
#include <string>

#include "umma.cuh"

namespace dion {

namespace {

constexpr int kBlockM = 128;
constexpr int kNumEpilogueWarps = 8;  // two per TMEM lane quadrant, each takes half of the tile's columns
constexpr int kNumThreads = 64 + 32 * kNumEpilogueWarps;
constexpr int kNumGatherThreads = 64;  // two more warps in the all-gather variant (register budget of 384 threads)
constexpr int kGatherUnitBytes = 64 * 1024;  // what one CTA's copier warps move at a time
constexpr int kNumSplitThreads = 128;  // four converter warps in the variant that splits fp32 operands in shared memory

// Operand A gathered from the ranks of a group while the product runs (GemmArgs::Gather).
struct GatherParams {
  int world, rank, channel;
  int rows;        // rows per source rank
  int chunk_rows;  // rows per readiness counter: a multiple of the tile height that divides `rows`
  int m_rot;       // m-tile the schedule starts with (this rank's first tile)
  unsigned epoch;
  long long row_bytes;
  long long flag_off, slot_off;
  const char* in;
  char* out;
  int units_per_chunk;  // ceil(chunk bytes / kGatherUnitBytes)
  void* peers[kGatherMaxPeers];
  unsigned* next_unit;  // work counter of the copier warps
  unsigned* staged;     // units of this rank's own rows that reached the staging slot
  unsigned* ready;      // per chunk: units in place; a chunk is complete at units_per_chunk
  unsigned long long budget_ns;
};

struct KernelParams {
  int M, N, K, batch, split_k;
  int tiles_m, tiles_n, tiles_per_batch, total_tiles;
  int kblocks_total, kblocks_per_split;
  int kblocks_seg;  // k-blocks per operand segment: kblocks_total for a plain product, a third of it for hi / lo operands
  float alpha, beta;
  const void* C;
  int c_is_bf16;
  long long ldc, c_batch_stride;
  const void* const* c_ptrs;
  const float* c_col_scale;
  void* D;
  int d_is_bf16;
  long long ldd, d_batch_stride;
  void* const* d_ptrs;
  int d_dup;  // destinations per batch element in d_ptrs (>= 1)
  void* D2;
  long long ldd2, d2_batch_stride;
  void* const* d2_ptrs;
  int epilogue, act, symmetric;
  int scatter_mode, scatter_block, scatter_dests;  // D tiles go to per-destination buffers (peer memory)
  void* const* scatter_ptrs;
  int vec_c, vec_d, vec_d2;  // 16-byte vector access allowed
  int stage;                 // turn epilogue accesses through shared memory (coalesced)
  int* status;
  GatherParams g;            // used by the kGather instantiations only
};

// kPair: two CTAs of a cluster work on one 256 x kBlockN tile (tcgen05 cta_group::2).  Each CTA
// loads its own 128 rows of A and half of the tile's B rows, so every byte of B is fetched from
// L2 once per 256 output rows instead of once per 128.
// kSplit: fp32 operands are split into tf32 hi / lo halves inside the kernel (see the converter warps).
template <bool kTf32, int kAMajor, int kBMajor, int kBlockN, bool kPair = false, bool kSplit = false>
struct Cfg {
  static_assert(!kSplit || (kTf32 && !kPair && kBlockN <= 128), "in-kernel splitting: fp32 operands, unpaired tiles of up to 128 columns");
  static constexpr int ES = kTf32 ? 4 : 2;
  static constexpr int BK = 128 / ES;      // K elements per stage (one 128B swizzle span)
  static constexpr int CH = 128 / ES;      // M/N elements per 128B chunk (MN-major tiles)
  static constexpr int UMMA_K = 32 / ES;   // K per tcgen05.mma
  static constexpr int KSTEPS = BK / UMMA_K;
  static constexpr int A_BYTES = kBlockM * 128;
  static constexpr int TILE_M = kPair ? 2 * kBlockM : kBlockM;
  static constexpr int B_ROWS = kPair ? kBlockN / 2 : kBlockN;  // B rows (N) held by one CTA
  static constexpr int B_BYTES = B_ROWS * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TX_BYTES = kPair ? 2 * STAGE_BYTES : STAGE_BYTES;  // what one full barrier phase receives
  // kSplit keeps the lo halves of a stage right behind its hi halves (same layout, LO_OFFSET further on)
  static constexpr int STAGE_STRIDE = kSplit ? 2 * STAGE_BYTES : STAGE_BYTES;
  static constexpr int LO_OFFSET = STAGE_BYTES;
  static constexpr int STAGES = 196608 / STAGE_STRIDE;  // 4 / 6 / 8 stages in 192 KB (3 / 4 when splitting)
  // Two accumulator buffers (the epilogue of one tile overlaps the main loop of the next).  fp32 operands
  // on tiles up to 128 columns get a second accumulator per buffer, for the small cross terms of a
  // hi / lo product: added into the large accumulator one by one they would lose their low bits at
  // every step, summed on their own and added once in the epilogue they do not.
  static constexpr bool CROSS_ACC = kTf32 && !kPair && kBlockN <= 128;
  static constexpr int ACC_STRIDE = CROSS_ACC ? 2 * kBlockN : kBlockN;
  static constexpr int TMEM_COLS = (2 * ACC_STRIDE <= 32) ? 32 : 2 * ACC_STRIDE;  // power of two
  static constexpr int SMEM_BYTES = STAGES * STAGE_STRIDE + 1024 /*align*/ + 256 /*barriers*/ + 8 * 32 * 128 /*epilogue staging*/;
  // descriptor strides
  static constexpr uint32_t A_LBO = (kAMajor == kMajorK) ? 16u : (uint32_t)BK * 128u;
  static constexpr uint32_t B_LBO = (kBMajor == kMajorK) ? 16u : (uint32_t)BK * 128u;
  static constexpr uint32_t A_KSTEP = (kAMajor == kMajorK) ? 32u : (uint32_t)UMMA_K * 128u;
  static constexpr uint32_t B_KSTEP = (kBMajor == kMajorK) ? 32u : (uint32_t)UMMA_K * 128u;
  // MN-major fp32 tiles use the 32-byte-atom swizzle: 4 K-rows (512 B) per atom
  static constexpr bool A_ATOM32 = kTf32 && kAMajor == kMajorMN;
  static constexpr bool B_ATOM32 = kTf32 && kBMajor == kMajorMN;
  static constexpr uint32_t A_SBO = A_ATOM32 ? 512u : 1024u;
  static constexpr uint32_t B_SBO = B_ATOM32 ? 512u : 1024u;
  static constexpr uint32_t A_LAYOUT = A_ATOM32 ? kLayoutSw128Atom32 : kLayoutSw128;
  static constexpr uint32_t B_LAYOUT = B_ATOM32 ? kLayoutSw128Atom32 : kLayoutSw128;
};

struct TileCoord {
  int batch, split, m_blk, n_blk;
};

template <bool kGather = false>
__device__ __forceinline__ TileCoord decode_tile(const KernelParams& p, int tile) {
  TileCoord t;
  const int per_bs = p.tiles_per_batch;
  const int bs = tile / per_bs;
  int r = tile - bs * per_bs;
  t.batch = bs / p.split_k;
  t.split = bs - t.batch * p.split_k;
  if (p.symmetric) {
    // r enumerates pairs (i <= j) row by row: row i has (tiles_n - i) entries.
    int i = 0;
    int row_len = p.tiles_n;
    while (r >= row_len) {
      r -= row_len;
      ++i;
      --row_len;
    }
    t.m_blk = i;
    t.n_blk = i + r;
  } else {
    // n fastest, so that CTAs running together share the same rows of A through L2
    t.m_blk = r / p.tiles_n;
    t.n_blk = r - t.m_blk * p.tiles_n;
    if constexpr (kGather) {
      // start with the rows this rank produced itself; the other ranks' rows follow in ring order,
      // which is also the order in which they are fetched
      t.m_blk += p.g.m_rot;
      if (t.m_blk >= p.tiles_m) t.m_blk -= p.tiles_m;
    }
  }
  return t;
}

__device__ __forceinline__ float apply_act(float x, int act) {
  if (act == kActRelu2) {
    const float r = fmaxf(x, 0.f);
    return r * r;
  }
  return x;
}

// 32 consecutive columns of one row, bf16 destination
__device__ __forceinline__ void store_chunk_bf16(__nv_bfloat16* dp, const float (&v)[32], bool vec, int ncols) {
  if (vec) {
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
      uint4 q;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
      for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(v[i + 2 * j], v[i + 2 * j + 1]);
      *reinterpret_cast<uint4*>(dp + i) = q;
    }
  } else {
    for (int i = 0; i < 32; ++i)
      if (i < ncols) dp[i] = __float2bfloat16(v[i]);
  }
}

// 32 consecutive columns of one row of C (bf16 or fp32) as floats; missing columns read as 0
__device__ __forceinline__ void load_chunk(const char* base, bool is_bf16, long long elem, float (&c)[32], bool vec,
                                           int ncols) {
  if (is_bf16) {
    const __nv_bfloat16* cp = reinterpret_cast<const __nv_bfloat16*>(base) + elem;
    if (vec) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        const uint4 q = *reinterpret_cast<const uint4*>(cp + i);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h[j]);
          c[i + 2 * j] = f.x;
          c[i + 2 * j + 1] = f.y;
        }
      }
    } else {
      for (int i = 0; i < 32; ++i) c[i] = i < ncols ? __bfloat162float(cp[i]) : 0.f;
    }
  } else {
    const float* cp = reinterpret_cast<const float*>(base) + elem;
    if (vec) {
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        const float4 q = *reinterpret_cast<const float4*>(cp + i);
        c[i] = q.x;
        c[i + 1] = q.y;
        c[i + 2] = q.z;
        c[i + 3] = q.w;
      }
    } else {
      for (int i = 0; i < 32; ++i) c[i] = i < ncols ? cp[i] : 0.f;
    }
  }
}

// One special-function instruction instead of the IEEE-rounded sequence of sqrtf(): the operand is a bf16 value and the
// result scales a gradient that is rounded to bf16 again, 2^-22 of relative error is far below either.
__device__ __forceinline__ float sqrt_approx(float x) {
  float y;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---- epilogue staging: one warp turns a 32-row block through shared memory.  A buffer holds 32
// rows of 128 bytes; the 16-byte segment index is XOR-ed with the row so that both the
// row-per-lane side and the segment-per-lane side are free of bank conflicts.
constexpr int kStageBytes = 32 * 128;

__device__ __forceinline__ uint32_t stage_off(int row, int seg) { return row * 128 + ((seg ^ (row & 7)) << 4); }

// lane's own row, 32 bf16 values into segments [seg0, seg0 + 4)
__device__ __forceinline__ void stage_put_bf16(uint8_t* st, int lane, int seg0, const float (&v)[32]) {
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    uint4 q;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(v[8 * s + 2 * j], v[8 * s + 2 * j + 1]);
    *reinterpret_cast<uint4*>(st + stage_off(lane, seg0 + s)) = q;
  }
}
// lane's own row, 32 fp32 values into segments [0, 8)
__device__ __forceinline__ void stage_put_f32(uint8_t* st, int lane, const float (&v)[32]) {
#pragma unroll
  for (int s = 0; s < 8; ++s)
    *reinterpret_cast<float4*>(st + stage_off(lane, s)) = make_float4(v[4 * s], v[4 * s + 1], v[4 * s + 2], v[4 * s + 3]);
}
// lane's own row back as floats: 4 segments of bf16 or 8 segments of fp32
__device__ __forceinline__ void stage_get(const uint8_t* st, int lane, bool is_bf16, float (&c)[32]) {
  if (is_bf16) {
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const uint4 q = *reinterpret_cast<const uint4*>(st + stage_off(lane, s));
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        c[8 * s + 2 * j] = f.x;
        c[8 * s + 2 * j + 1] = f.y;
      }
    }
  } else {
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      const float4 q = *reinterpret_cast<const float4*>(st + stage_off(lane, s));
      c[4 * s] = q.x;
      c[4 * s + 1] = q.y;
      c[4 * s + 2] = q.z;
      c[4 * s + 3] = q.w;
    }
  }
}
// Buffer -> global: `nseg` (4 or 8) lanes cover one row, 32 / nseg rows per instruction.
// row_ptr(grow) is the address of the first staged byte of global row `grow`.
template <int NSEG, typename RowPtr>
__device__ __forceinline__ void stage_flush(const uint8_t* st, int lane, int row_first, int M, RowPtr row_ptr) {
  constexpr int SHIFT = NSEG == 8 ? 3 : 2;
  const int seg = lane & (NSEG - 1);
  const int rsub = lane >> SHIFT;
  uint4 q[NSEG];
#pragma unroll
  for (int i = 0; i < NSEG; ++i) q[i] = *reinterpret_cast<const uint4*>(st + stage_off(i * (32 >> SHIFT) + rsub, seg));
#pragma unroll
  for (int i = 0; i < NSEG; ++i) {
    const int r = i * (32 >> SHIFT) + rsub;
    if (row_first + r < M) *reinterpret_cast<uint4*>(row_ptr(row_first + r) + seg * 16) = q[i];
  }
}
// global -> buffer, same lane mapping; rows past M read as zero
template <int NSEG, typename RowPtr>
__device__ __forceinline__ void stage_fetch(uint8_t* st, int lane, int row_first, int M, RowPtr row_ptr) {
  constexpr int SHIFT = NSEG == 8 ? 3 : 2;
  const int seg = lane & (NSEG - 1);
  const int rsub = lane >> SHIFT;
  uint4 q[NSEG];
#pragma unroll
  for (int i = 0; i < NSEG; ++i) {
    const int r = i * (32 >> SHIFT) + rsub;
    q[i] = make_uint4(0u, 0u, 0u, 0u);
    if (row_first + r < M) q[i] = *reinterpret_cast<const uint4*>(row_ptr(row_first + r) + seg * 16);
  }
#pragma unroll
  for (int i = 0; i < NSEG; ++i) *reinterpret_cast<uint4*>(st + stage_off(i * (32 >> SHIFT) + rsub, seg)) = q[i];
}

__device__ __forceinline__ unsigned ld_acquire_gpu_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys_u32(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// orders plain stores / loads of this thread with accesses made through TMA
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// mbarrier wait with a caller-chosen budget (the all-gather variant may wait for another GPU)
__device__ __forceinline__ bool mbar_wait_for(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                              unsigned long long budget_ns) {
  const unsigned long long t0 = global_timer_ns();
#pragma unroll 1
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 128; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (*abort_flag != 0) return false;
    if (global_timer_ns() - t0 > budget_ns) return false;
  }
}

// kSplit (fp32 operands, 3xTF32 accuracy without hi / lo copies in global memory): four more warps
// take every stage that TMA delivered, clear the low 13 mantissa bits of each fp32 value in place (hi)
// and write the remainders (lo) LO_OFFSET further on, same layout - an element-wise pass that does not
// need to know the swizzle.  The MMA warp then issues hi*hi into the main accumulator and lo*hi, hi*lo
// into the cross-term accumulator for every K-step.  Operand bytes cross L2 once instead of three times.
template <bool kTf32, int kAMajor, int kBMajor, int kBlockN, bool kPair, bool kGather = false, bool kSplit = false>
__global__ void __launch_bounds__(kNumThreads + (kGather ? kNumGatherThreads : 0) + (kSplit ? kNumSplitThreads : 0), 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const __grid_constant__ CUtensorMap tmap_a_lo, const __grid_constant__ CUtensorMap tmap_b_lo,
            const KernelParams p) {
  static_assert(!(kSplit && kGather), "the converter warps and the copier warps use the same warp slots");
  using C = Cfg<kTf32, kAMajor, kBMajor, kBlockN, kPair, kSplit>;
  extern __shared__ uint8_t smem_raw[];
  // 128B swizzle atoms need 1024-byte aligned tiles.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* bar_area = smem + C::STAGES * C::STAGE_STRIDE;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_area);
  uint64_t* empty_bar = full_bar + C::STAGES;
  uint64_t* tmem_full = empty_bar + C::STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint64_t* conv_bar = tmem_empty + 2;  // kSplit: stage has been split (one arrival per converter warp)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(conv_bar + (kSplit ? C::STAGES : 0));
  static_assert((2 * C::STAGES + 4 + (kSplit ? C::STAGES : 0)) * 8 + 16 <= 256, "barrier area");
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* gather_word = abort_flag + 1;  // broadcast slot of the copier warps
  uint8_t* stage_area = bar_area + 256;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // CTA pair: rank 0 leads (issues the MMAs, owns the full / tmem_empty barriers in use)
  uint32_t cta_rank = 0;
  if constexpr (kPair) cta_rank = cluster_ctarank();
  const int worker = kPair ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int num_workers = kPair ? (int)(gridDim.x >> 1) : (int)gridDim.x;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if constexpr (kTf32) {
      if (p.kblocks_seg < p.kblocks_total) {
        tma_prefetch_desc(&tmap_a_lo);
        tma_prefetch_desc(&tmap_b_lo);
      }
    }
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
      if constexpr (kSplit) mbar_init(&conv_bar[s], kNumSplitThreads / 32);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], kPair ? 2 * kNumEpilogueWarps : kNumEpilogueWarps);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    if constexpr (kPair) {
      tmem_alloc_pair(tmem_slot, C::TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, C::TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (kPair) cluster_sync_all();  // both CTAs' barriers and TMEM exist before either is used
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // debug build: the allocation lies inside the 512 columns of tensor memory
  if (threadIdx.x == 0) (void)DION_DBG_OK((tmem_base & 0xffffu) + C::TMEM_COLS <= 512u, p.status);

  const int kb_per_split = p.kblocks_per_split;
  // every wait inside the pipeline; the all-gather variant allows for the time another GPU may take
  auto wait = [&](uint64_t* bar, uint32_t parity) -> bool {
    if constexpr (kGather) return mbar_wait_for(bar, parity, abort_flag, kWaitBudgetNs + p.g.budget_ns);
    else return mbar_wait(bar, parity, abort_flag);
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      [[maybe_unused]] int ready_chunk = -1;
      for (int tile = worker; tile < p.total_tiles && ok; tile += num_workers) {
        const TileCoord t = decode_tile<kGather>(p, tile);
        const int m0 = t.m_blk * C::TILE_M + (int)cta_rank * kBlockM;
        const int n0 = t.n_blk * kBlockN + (int)cta_rank * (kPair ? C::B_ROWS : 0);
        const int kb0 = t.split * kb_per_split;
        const int kb1 = min(kb0 + kb_per_split, p.kblocks_total);
        if constexpr (kGather) {
          // the rows of this tile are in place once every unit of their chunk has been counted
          const int chunk = m0 / p.g.chunk_rows;
          if (chunk != ready_chunk) {
            const unsigned long long t0 = global_timer_ns();
            while (ld_acquire_gpu_u32(p.g.ready + chunk) < (unsigned)p.g.units_per_chunk) {
              if (*abort_flag != 0 || global_timer_ns() - t0 > kWaitBudgetNs + p.g.budget_ns) {
                ok = false;
                break;
              }
            }
            if (!ok) {
              *abort_flag = 1;
              if (p.status) atomicCAS(p.status, 0, kStatusPeerTimeout);
              break;
            }
            fence_proxy_async_all();
            ready_chunk = chunk;
          }
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!wait(&empty_bar[stage], phase ^ 1u)) {
            ok = false;
            *abort_flag = 1;
            if (p.status) atomicCAS(p.status, 0, kStatusProducerTimeout);
            break;
          }
          // the leader's full barrier collects the bytes of both CTAs
          if (cta_rank == 0) mbar_arrive_expect_tx(&full_bar[stage], C::TX_BYTES);
          const uint32_t bar = kPair ? mapa_shared(smem_u32(&full_bar[stage]), 0) : smem_u32(&full_bar[stage]);
          auto load = [&](void* dst, const CUtensorMap* map, int c0, int c1) {
            if constexpr (kPair) tma_load_3d_pair(dst, map, bar, c0, c1, t.batch);
            else tma_load_3d(dst, map, &full_bar[stage], c0, c1, t.batch);
          };
          uint8_t* sa = smem + stage * C::STAGE_STRIDE;
          uint8_t* sb = sa + C::A_BYTES;
          // hi / lo operands: the K range is walked three times, as A B, A_lo B and A B_lo
          const CUtensorMap* map_a = &tmap_a;
          const CUtensorMap* map_b = &tmap_b;
          int kk = kb;
          if constexpr (kTf32) {
            if (kb >= p.kblocks_seg) {
              const int seg = kb / p.kblocks_seg;
              kk = kb - seg * p.kblocks_seg;
              if (seg == 1) map_a = &tmap_a_lo;
              else map_b = &tmap_b_lo;
            }
          }
          const int k0 = kk * C::BK;
          if constexpr (kAMajor == kMajorK) {
            load(sa, map_a, k0, m0);
          } else {
#pragma unroll
            for (int c = 0; c < kBlockM / C::CH; ++c) load(sa + c * (C::BK * 128), map_a, m0 + c * C::CH, k0);
          }
          if constexpr (kBMajor == kMajorK) {
            load(sb, map_b, k0, n0);
          } else {
#pragma unroll
            for (int c = 0; c < C::B_ROWS / C::CH; ++c) load(sb + c * (C::BK * 128), map_b, n0 + c * C::CH, k0);
          }
          if (++stage == C::STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && cta_rank == 0) {
      constexpr uint32_t idesc = make_instr_desc(kTf32 ? 2 : 1, kAMajor, kBMajor, C::TILE_M, kBlockN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = worker; tile < p.total_tiles && ok; tile += num_workers, ++it) {
        const TileCoord t = decode_tile<kGather>(p, tile);
        const int kb0 = t.split * kb_per_split;
        const int kb1 = min(kb0 + kb_per_split, p.kblocks_total);
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!wait(&tmem_empty[acc], acc_phase ^ 1u)) {
          ok = false;
          *abort_flag = 1;
          if (p.status) atomicCAS(p.status, 0, kStatusMmaTimeout);
          break;
        }
        tc_fence_after();
        const uint32_t d_main = tmem_base + acc * C::ACC_STRIDE;
        for (int kb = kb0; kb < kb1; ++kb) {
          // hi / lo operands: the first K-segment (hi * hi) goes to the main accumulator, the two cross
          // segments to the second one, which starts from zero at the first of them
          uint32_t d_tmem = d_main;
          bool fresh = kb == kb0;
          if constexpr (C::CROSS_ACC) {
            if (kb >= p.kblocks_seg) {
              d_tmem = d_main + kBlockN;
              fresh = kb == p.kblocks_seg;
            }
          }
          // the operands of a stage are ready when TMA delivered them - or, when they are split in
          // shared memory, when the converter warps are through with the stage
          if (!wait(kSplit ? &conv_bar[stage] : &full_bar[stage], phase)) {
            ok = false;
            *abort_flag = 1;
            if (p.status) atomicCAS(p.status, 0, kStatusMmaTimeout);
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * C::STAGE_STRIDE);
          const uint32_t sb = sa + C::A_BYTES;
#pragma unroll
          for (int j = 0; j < C::KSTEPS; ++j) {
            const uint64_t da = make_smem_desc(sa + j * C::A_KSTEP, C::A_LBO, C::A_SBO, C::A_LAYOUT);
            const uint64_t db = make_smem_desc(sb + j * C::B_KSTEP, C::B_LBO, C::B_SBO, C::B_LAYOUT);
            if constexpr (kSplit) {
              const uint64_t da_lo = make_smem_desc(sa + C::LO_OFFSET + j * C::A_KSTEP, C::A_LBO, C::A_SBO, C::A_LAYOUT);
              const uint64_t db_lo = make_smem_desc(sb + C::LO_OFFSET + j * C::B_KSTEP, C::B_LBO, C::B_SBO, C::B_LAYOUT);
              const uint32_t first = (!fresh || j > 0) ? 1u : 0u;
              umma_ss<true>(d_main, da, db, idesc, first);                 // hi * hi
              umma_ss<true>(d_main + kBlockN, da_lo, db, idesc, first);    // lo * hi
              umma_ss<true>(d_main + kBlockN, da, db_lo, idesc, 1u);       // hi * lo
            } else if constexpr (kPair) {
              umma_ss_pair<kTf32>(d_tmem, da, db, idesc, (!fresh || j > 0) ? 1u : 0u);
            } else {
              umma_ss<kTf32>(d_tmem, da, db, idesc, (!fresh || j > 0) ? 1u : 0u);
            }
          }
          // frees the smem stage (of both CTAs) once these MMAs retire
          if constexpr (kPair) umma_commit_pair(&empty_bar[stage], 3);
          else umma_commit(&empty_bar[stage]);
          if (++stage == C::STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) {
          if constexpr (kPair) umma_commit_pair(&tmem_full[acc], 3);
          else umma_commit(&tmem_full[acc]);
        }
      }
    }
  } else if (kSplit && warp >= 2 + kNumEpilogueWarps) {
    // ------------------------------------------------------------------ converter: fp32 stage -> tf32 hi / lo
    const int ct = (int)threadIdx.x - kNumThreads;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = worker; tile < p.total_tiles && ok; tile += num_workers) {
      const TileCoord t = decode_tile<false>(p, tile);
      const int kb0 = t.split * kb_per_split;
      const int kb1 = min(kb0 + kb_per_split, p.kblocks_total);
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!wait(&full_bar[stage], phase)) {
          ok = false;
          *abort_flag = 1;
          if (p.status) atomicCAS(p.status, 0, kStatusProducerTimeout);
          break;
        }
        uint8_t* hi = smem + stage * C::STAGE_STRIDE;
#pragma unroll 4
        for (int off = ct * 16; off < C::STAGE_BYTES; off += kNumSplitThreads * 16) {
          const float4 q = *reinterpret_cast<const float4*>(hi + off);
          float4 h, l;
          h.x = __int_as_float(__float_as_int(q.x) & 0xffffe000);
          h.y = __int_as_float(__float_as_int(q.y) & 0xffffe000);
          h.z = __int_as_float(__float_as_int(q.z) & 0xffffe000);
          h.w = __int_as_float(__float_as_int(q.w) & 0xffffe000);
          l.x = q.x - h.x;
          l.y = q.y - h.y;
          l.z = q.z - h.z;
          l.w = q.w - h.w;
          *reinterpret_cast<float4*>(hi + off) = h;
          *reinterpret_cast<float4*>(hi + C::LO_OFFSET + off) = l;
        }
        // these stores are read by the tensor core (async proxy)
        fence_proxy_async_all();
        __syncwarp();
        if (lane == 0) mbar_arrive(&conv_bar[stage]);
        if (++stage == C::STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (kGather && warp >= 2 + kNumEpilogueWarps) {
    // ------------------------------------------------------------------ all-gather of operand A
    // The copy is cut into units of kGatherUnitBytes, numbered in the order in which the tiles need
    // them (this rank's rows, then the next ranks' in ring order).  The 64 copier threads of a CTA
    // take the next unit from a global counter, so the copy advances with whatever CTAs are running
    // and no CTA ever waits for another one of this launch.
    const GatherParams& g = p.g;
    const int ct = (int)threadIdx.x - kNumThreads;
    const long long chunk_bytes = (long long)g.chunk_rows * g.row_bytes;
    const int chunks_per_rank = g.rows / g.chunk_rows;
    const int units_per_chunk = g.units_per_chunk;
    const int units_per_rank = chunks_per_rank * units_per_chunk;
    const int total_units = units_per_rank * g.world;
    auto copier_sync = [] { asm volatile("bar.sync 1, %0;" ::"n"(kNumGatherThreads) : "memory"); };
    int waited_for = g.rank;  // ranks up to this one (in ring order) have announced their rows
    for (;;) {
      if (ct == 0) *gather_word = (int)atomicAdd(g.next_unit, 1u);
      copier_sync();
      const int unit = *gather_word;
      copier_sync();  // everybody has read the word before it is written again
      if (unit >= total_units) break;
      const int ring = unit / units_per_rank;
      const int in_rank = unit - ring * units_per_rank;
      const int c = in_rank / units_per_chunk;
      const int u = in_rank - c * units_per_chunk;
      const int src_rank = (g.rank + ring) % g.world;
      if (src_rank != waited_for && ring > 0) {
        if (ct == 0) {
          const unsigned* f = reinterpret_cast<const unsigned*>(reinterpret_cast<const char*>(g.peers[g.rank]) +
                                                                g.flag_off) + g.channel * kGatherMaxPeers + src_rank;
          const unsigned long long t0 = global_timer_ns();
          int arrived = 1;
          while ((int)(ld_acquire_sys_u32(f) - g.epoch) < 0) {
            if (*abort_flag != 0 || global_timer_ns() - t0 > g.budget_ns) {
              arrived = 0;
              break;
            }
          }
          if (!arrived) {
            *abort_flag = 1;
            if (p.status) atomicCAS(p.status, 0, kStatusPeerTimeout);
          }
          *gather_word = arrived;
        }
        copier_sync();
        const bool arrived = *gather_word != 0;
        copier_sync();
        if (!arrived) break;
        waited_for = src_rank;
      }
      // bytes [lo, hi) of chunk c of src_rank's rows
      const long long lo = (long long)u * kGatherUnitBytes;
      const long long hi = min(lo + (long long)kGatherUnitBytes, chunk_bytes);
      const long long off = (long long)c * chunk_bytes;
      const long long nvec = (hi - lo) / 16;
      const uint4* src;
      uint4* dst;
      uint4* dst2 = nullptr;
      char* block = g.out + (long long)src_rank * g.rows * g.row_bytes;
      if (ring == 0) {
        // this rank's rows: into the staging slot the peers read, and into its own block of A
        src = reinterpret_cast<const uint4*>(g.in + off + lo);
        dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(g.peers[g.rank]) + g.slot_off + off + lo);
        if (block != g.in) dst2 = reinterpret_cast<uint4*>(block + off + lo);
      } else {
        src = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(g.peers[src_rank]) + g.slot_off + off + lo);
        dst = reinterpret_cast<uint4*>(block + off + lo);
      }
      // eight independent 16-byte loads in flight per thread (the sources are mostly peer memory)
      for (long long v = ct; v < nvec; v += 8 * kNumGatherThreads) {
        uint4 q[8];
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (v + k * kNumGatherThreads < nvec) q[k] = src[v + k * kNumGatherThreads];
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (v + k * kNumGatherThreads < nvec) {
            dst[v + k * kNumGatherThreads] = q[k];
            if (dst2 != nullptr) dst2[v + k * kNumGatherThreads] = q[k];
          }
      }
      // the unit is visible to every CTA's TMA loads (and, for this rank's rows, to the peers)
      // before it is counted
      if (ring == 0) __threadfence_system();
      else __threadfence();
      fence_proxy_async_all();
      copier_sync();
      if (ct == 0) {
        atomicAdd(g.ready + src_rank * chunks_per_rank + c, 1u);
        if (ring == 0) {
          // whoever stages the last unit of this rank's rows tells every peer that the slot is complete
          const unsigned prev = atomicAdd(g.staged, 1u);
          if (prev == (unsigned)units_per_rank - 1) {
            __threadfence_system();
            for (int q = 0; q < g.world; ++q) {
              unsigned* f = reinterpret_cast<unsigned*>(reinterpret_cast<char*>(g.peers[q]) + g.flag_off);
              st_release_sys_u32(f + g.channel * kGatherMaxPeers + g.rank, g.epoch);
            }
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    int it = 0;
    bool ok = true;
    for (int tile = worker; tile < p.total_tiles && ok; tile += num_workers, ++it) {
      const TileCoord t = decode_tile<kGather>(p, tile);
      const int m0 = t.m_blk * C::TILE_M + (int)cta_rank * kBlockM;
      const int n0 = t.n_blk * kBlockN;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      const int kb0 = t.split * kb_per_split;
      const bool has_work = kb0 < p.kblocks_total;
      const int row = m0 + quad * 32 + lane;
      // debug build: the tile lies inside the problem and the output base is 16-byte aligned where vector stores go
      const bool row_ok = row < p.M && DION_DBG_OK(t.batch < p.batch && m0 < p.M + C::TILE_M && n0 < p.N, p.status);
      const char* c_base = nullptr;
      char* d_base;
      char* d2_base = nullptr;
      if (p.C || p.c_ptrs)
        c_base = p.c_ptrs ? reinterpret_cast<const char*>(p.c_ptrs[t.batch])
                          : reinterpret_cast<const char*>(p.C) +
                                (long long)t.batch * p.c_batch_stride * (p.c_is_bf16 ? 2 : 4);
      d_base = p.d_ptrs ? reinterpret_cast<char*>(p.d_ptrs[(long long)t.batch * p.d_dup])
                        : reinterpret_cast<char*>(p.D) +
                              (long long)t.batch * p.d_batch_stride * (p.d_is_bf16 ? 2 : 4);
      const int ndup = p.d_ptrs ? p.d_dup : 1;
      if (p.D2 || p.d2_ptrs)
        d2_base = p.d2_ptrs ? reinterpret_cast<char*>(p.d2_ptrs[t.batch])
                            : reinterpret_cast<char*>(p.D2) + (long long)t.batch * p.d2_batch_stride * 2;
      const bool mirror = p.symmetric && (t.m_blk != t.n_blk);

      // After tcgen05.ld every lane holds one row of the tile, so a direct access would touch 32
      // different lines per instruction.  Tiles that are full width and 16-byte aligned are turned
      // through this warp's staging buffer instead, so that consecutive lanes move consecutive
      // bytes (C on its way in, D and the second output D2 on their way out, one after the other).
      uint8_t* st = stage_area + (warp - 2) * kStageBytes;
      const int row_first = m0 + quad * 32;
      const bool full_tile = n0 + kBlockN <= p.N;
      const bool atomic = p.epilogue == kEpiAtomicAdd;
      const bool use_c = c_base != nullptr && !atomic &&
                         (p.beta != 0.f || p.act == kActMulRelu2Grad || p.act == kActMulRelu2GradSq);
      const bool stage_c = p.stage && use_c && full_tile && p.vec_c;
      const bool stage_d = p.stage && !atomic && full_tile && p.vec_d;
      const bool stage_d2 = p.stage && d2_base != nullptr && full_tile && p.vec_d2;
      const int es_c = p.c_is_bf16 ? 2 : 4;
      const int es_d = p.d_is_bf16 ? 2 : 4;

      // address of element (grow, col) of D with the scatter modes applied
      auto d_addr = [&](int grow, int col) -> char* {
        char* base = d_base;
        long long r = grow;
        int cc = col;
        if (p.scatter_mode == 1) {
          int k = grow / p.scatter_block;
          if (!DION_DBG_OK(k < p.scatter_dests, p.status)) k = p.scatter_dests - 1;
          base = reinterpret_cast<char*>(p.scatter_ptrs[(long long)t.batch * p.scatter_dests + k]);
          r = grow - (long long)k * p.scatter_block;
        } else if (p.scatter_mode == 2) {
          int k = col / p.scatter_block;
          if (!DION_DBG_OK(k < p.scatter_dests, p.status)) k = p.scatter_dests - 1;
          base = reinterpret_cast<char*>(p.scatter_ptrs[(long long)t.batch * p.scatter_dests + k]);
          cc = col - k * p.scatter_block;
        }
        return base + (r * p.ldd + cc) * es_d;
      };

      constexpr int kChunksPerWarp = kBlockN / 32 / (kNumEpilogueWarps / 4);
      const int c_first = ((warp - 2) >> 2) * kChunksPerWarp;

      // A staged bf16 C operand is fetched one chunk ahead: the loads of the first chunk go out before this
      // warp waits for the accumulator, those of chunk c + 1 while chunk c is converted and stored, so that
      // their latency does not add to every chunk (with 8 epilogue warps per CTA nothing else hides it).
      // Same lane mapping as stage_fetch<4>: 4 lanes per row, 8 rows per instruction.
      const bool prefetch_c = !kSplit && stage_c && p.c_is_bf16;  // the splitting variants have no registers to spare
      uint4 cq[4];
      auto c_prefetch = [&](int chunk) {
        const char* cp = c_base + ((long long)(row_first + (lane >> 2)) * p.ldc + n0 + chunk * 32) * 2 + (lane & 3) * 16;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          cq[i] = make_uint4(0u, 0u, 0u, 0u);
          if (row_first + i * 8 + (lane >> 2) < p.M) cq[i] = *reinterpret_cast<const uint4*>(cp + (long long)i * 8 * p.ldc * 2);
        }
      };
      if (prefetch_c) c_prefetch(c_first);

      if (!wait(&tmem_full[acc], acc_phase)) {
        ok = false;
        *abort_flag = 1;
        if (p.status) atomicCAS(p.status, 0, kStatusEpilogueTimeout);
        break;
      }
      tc_fence_after();

#pragma unroll 1
      for (int c = c_first; c < c_first + kChunksPerWarp; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;  // warp-uniform
        float v[32];
        const uint32_t taddr = tmem_base + acc * C::ACC_STRIDE + c * 32 + ((uint32_t)(quad * 32) << 16);
        tmem_ld_32x32(taddr, v);
        tmem_ld_wait();
        if constexpr (C::CROSS_ACC) {
          if (kSplit || p.kblocks_total > p.kblocks_seg) {  // hi / lo operands: add the cross terms, summed on their own
            float x[32];
            tmem_ld_32x32(taddr + kBlockN, x);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] += x[i];
          }
        }
        if (!has_work) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0.f;
        }
        if (p.alpha != 1.f) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] *= p.alpha;
        }

        const bool full_cols = col0 + 32 <= p.N;
        const int ncols = p.N - col0;  // valid columns of this chunk when it is the ragged last one

        // second output (bf16): staged or direct
        auto emit_d2 = [&]() {
          if (stage_d2) {
            stage_put_bf16(st, lane, 0, v);
            __syncwarp();
            stage_flush<4>(st, lane, row_first, p.M,
                           [&](int grow) { return d2_base + ((long long)grow * p.ldd2 + col0) * 2; });
            __syncwarp();
          } else if (row_ok) {
            store_chunk_bf16(reinterpret_cast<__nv_bfloat16*>(d2_base) + (long long)row * p.ldd2 + col0, v,
                             full_cols && p.vec_d2, ncols);
          }
        };

        bool d2_done = false;
        if (p.act == kActRelu2SavePre) {
          // D2 keeps the pre-activation (what the backward pass needs), D gets relu(x)^2
          if (d2_base != nullptr) emit_d2();
          d2_done = true;
        }
        if (p.act == kActRelu2 || p.act == kActRelu2SavePre) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = apply_act(v[i], kActRelu2);
        }
        if (atomic) {
          if (row_ok) {
            float* dp = reinterpret_cast<float*>(d_base) + (long long)row * p.ldd + col0;
            if (full_cols && p.vec_d) {
#pragma unroll
              for (int i = 0; i < 32; i += 4)
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dp + i),
                             "f"(v[i]), "f"(v[i + 1]), "f"(v[i + 2]), "f"(v[i + 3])
                             : "memory");
            } else {
              for (int i = 0; i < 32; ++i)
                if (col0 + i < p.N) atomicAdd(dp + i, v[i]);
            }
          }
        } else {
          // C operand: added (beta * C) or, for the ReLU^2 backward, multiplied in as 2 * relu(C)
          if (use_c) {
            float cv[32];
            if (prefetch_c) {
#pragma unroll
              for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(st + stage_off(i * 8 + (lane >> 2), lane & 3)) = cq[i];
              __syncwarp();
              stage_get(st, lane, true, cv);
              __syncwarp();
              if (c + 1 < c_first + kChunksPerWarp) c_prefetch(c + 1);  // a full tile: every chunk is in range
            } else if (stage_c) {
              auto c_row = [&](int grow) { return c_base + ((long long)grow * p.ldc + col0) * es_c; };
              if (p.c_is_bf16) stage_fetch<4>(st, lane, row_first, p.M, c_row);
              else stage_fetch<8>(st, lane, row_first, p.M, c_row);
              __syncwarp();
              stage_get(st, lane, p.c_is_bf16 != 0, cv);
              __syncwarp();
            } else if (row_ok) {
              load_chunk(c_base, p.c_is_bf16 != 0, (long long)row * p.ldc + col0, cv, full_cols && p.vec_c, ncols);
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) cv[i] = 0.f;
            }
            if (p.act == kActMulRelu2Grad) {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] *= 2.f * fmaxf(cv[i], 0.f);
            } else if (p.act == kActMulRelu2GradSq) {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] *= 2.f * sqrt_approx(fmaxf(cv[i], 0.f));
            } else if (p.c_col_scale != nullptr) {
              // every lane reads the same 32 factors (a broadcast load per factor)
              const float* cs = p.c_col_scale + (long long)t.batch * p.N + col0;
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] += p.beta * cv[i] * (col0 + i < p.N ? cs[i] : 0.f);
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] += p.beta * cv[i];
            }
          }
          if (stage_d) {
            auto d_row = [&](int grow) { return d_addr(grow, col0); };
            if (p.d_is_bf16) stage_put_bf16(st, lane, 0, v);
            else stage_put_f32(st, lane, v);
            __syncwarp();
            // the staged block goes to every destination of this batch element (d_addr reads d_base)
            for (int dup = 0; dup < ndup; ++dup) {
              if (dup > 0) d_base = reinterpret_cast<char*>(p.d_ptrs[(long long)t.batch * p.d_dup + dup]);
              if (p.d_is_bf16) stage_flush<4>(st, lane, row_first, p.M, d_row);
              else stage_flush<8>(st, lane, row_first, p.M, d_row);
            }
            __syncwarp();
          } else if (row_ok) {
            for (int dup = 0; dup < ndup; ++dup) {
              if (dup > 0) d_base = reinterpret_cast<char*>(p.d_ptrs[(long long)t.batch * p.d_dup + dup]);
              char* dptr = d_addr(row, col0);
              if (p.d_is_bf16) {
                store_chunk_bf16(reinterpret_cast<__nv_bfloat16*>(dptr), v, full_cols && p.vec_d, ncols);
              } else {
                float* dp = reinterpret_cast<float*>(dptr);
                if (full_cols && p.vec_d) {
#pragma unroll
                  for (int i = 0; i < 32; i += 4)
                    *reinterpret_cast<float4*>(dp + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                } else {
                  for (int i = 0; i < 32; ++i)
                    if (col0 + i < p.N) dp[i] = v[i];
                }
              }
            }
          }
          // later chunks of this tile start from the first destination again
          if (ndup > 1) d_base = reinterpret_cast<char*>(p.d_ptrs[(long long)t.batch * p.d_dup]);
          if (d2_base != nullptr && !d2_done) emit_d2();
          if (mirror && p.vec_d && full_cols && row_first + 32 <= p.M) {
            // Transposed copy of an off-diagonal tile, D[col, row], turned through the staging buffer:
            // every lane parks its row as a column, then the warp writes the 32 transposed rows with
            // 16-byte stores (4 instructions for bf16, 8 for fp32) instead of 32 narrow ones.
            if (p.d_is_bf16) {
              __nv_bfloat16* tb = reinterpret_cast<__nv_bfloat16*>(st);
#pragma unroll
              for (int i = 0; i < 32; ++i) tb[i * 32 + lane] = __float2bfloat16(v[i]);
              __syncwarp();
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const int cc = (lane >> 2) + 8 * k, seg = lane & 3;
                const uint4 q = *reinterpret_cast<const uint4*>(st + cc * 64 + seg * 16);
                *reinterpret_cast<uint4*>(d_base + ((long long)(col0 + cc) * p.ldd + row_first + seg * 8) * 2) = q;
              }
            } else {
              float* tf = reinterpret_cast<float*>(st);
#pragma unroll
              for (int i = 0; i < 32; ++i) tf[i * 32 + lane] = v[i];
              __syncwarp();
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                const int cc = (lane >> 3) + 4 * k, seg = lane & 7;
                const uint4 q = *reinterpret_cast<const uint4*>(st + cc * 128 + seg * 16);
                *reinterpret_cast<uint4*>(d_base + ((long long)(col0 + cc) * p.ldd + row_first + seg * 4) * 4) = q;
              }
            }
            __syncwarp();
          } else if (mirror && row_ok) {
            // ragged or unaligned tiles: D[col, row] element by element; lanes hold
            // consecutive rows, so each store instruction is contiguous across the warp
            if (p.d_is_bf16) {
              __nv_bfloat16* dt = reinterpret_cast<__nv_bfloat16*>(d_base);
              for (int i = 0; i < 32; ++i)
                if (col0 + i < p.N) dt[(long long)(col0 + i) * p.ldd + row] = __float2bfloat16(v[i]);
            } else {
              float* dt = reinterpret_cast<float*>(d_base);
              for (int i = 0; i < 32; ++i)
                if (col0 + i < p.N) dt[(long long)(col0 + i) * p.ldd + row] = v[i];
            }
          }
        }
      }
      // hand the accumulator buffer back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (cta_rank == 0) mbar_arrive(&tmem_empty[acc]);
        else mbar_arrive_cluster(mapa_shared(smem_u32(&tmem_empty[acc]), 0));
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    // a wait gave up: let copies that are still in flight land before the CTA retires
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  // a CTA of a pair must outlive its peer's last access to its shared memory, barriers and TMEM
  if constexpr (kPair) cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    if constexpr (kPair) tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
    else tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------- host side

thread_local std::string g_last_error;

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

EncodeFn get_encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(sym);
  });
  return fn;
}

struct TmapKey {
  const void* base;
  uint64_t inner, rows, batch, pitch, bstride;
  uint32_t box_inner, box_rows;
  int32_t dtype, atom32;
};
struct TmapSlot {
  CUtensorMap map;
  TmapKey key;
  bool valid;
};
constexpr size_t kTmapSlots = 2048;  // power of two; a GPT-160M step uses about 600 distinct maps

bool tmap_cache_enabled() {  // DION_B200_TMAP_CACHE=0 encodes every map afresh
  static const bool on = [] {
    const char* e = getenv("DION_B200_TMAP_CACHE");
    return !(e && e[0] == '0');
  }();
  return on;
}

// Tensor map over a row-major [batch][rows][inner] array with a [1][box_rows][box_inner] box.
bool make_tmap(CUtensorMap* map, const void* base, int dtype, uint64_t inner, uint64_t rows, uint64_t batch,
               uint64_t row_pitch_elems, uint64_t batch_stride_elems, uint32_t box_inner, uint32_t box_rows,
               bool atom32) {
  EncodeFn fn = get_encode_fn();
  if (!fn) {
    g_last_error = "cuTensorMapEncodeTiled is not available from this driver";
    return false;
  }
  const uint64_t es = dtype == kBF16 ? 2 : 4;
  cuuint64_t dims[3] = {inner, rows, batch};
  uint64_t bstride = batch_stride_elems * es;
  if (batch <= 1 || bstride == 0) bstride = rows * row_pitch_elems * es;
  cuuint64_t strides[2] = {row_pitch_elems * es, bstride};
  cuuint32_t box[3] = {box_inner, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (strides[0] & 15) || (strides[1] & 15)) {
    g_last_error = "GEMM operand must be 16-byte aligned with pitches that are multiples of 16 bytes";
    return false;
  }
  // A tensor map depends only on the address and the geometry, never on what the memory holds, and a training
  // step asks for the same few hundred maps again and again: keep them in a direct-mapped per-thread table.
  TmapSlot* slot = nullptr;
  if (tmap_cache_enabled()) {
    TmapKey key;
    memset(&key, 0, sizeof(key));
    key.base = base;
    key.inner = inner; key.rows = rows; key.batch = batch;
    key.pitch = strides[0]; key.bstride = strides[1];
    key.box_inner = box_inner; key.box_rows = box_rows;
    key.dtype = dtype; key.atom32 = atom32 ? 1 : 0;
    uint64_t h = 1469598103934665603ull;
    const unsigned char* kb = reinterpret_cast<const unsigned char*>(&key);
    for (size_t i = 0; i < sizeof(key); ++i) h = (h ^ kb[i]) * 1099511628211ull;
    static thread_local std::unique_ptr<TmapSlot[]> table(new TmapSlot[kTmapSlots]());  // freed with the thread
    slot = &table[(h ^ (h >> 29)) & (kTmapSlots - 1)];
    if (slot->valid && memcmp(&slot->key, &key, sizeof(key)) == 0) {
      memcpy(map, &slot->map, sizeof(CUtensorMap));
      return true;
    }
    slot->valid = false;
    slot->key = key;
  }
  CUresult r = fn(map, dtype == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[160];
    snprintf(buf, sizeof(buf), "cuTensorMapEncodeTiled failed with code %d", (int)r);
    g_last_error = buf;
    return false;
  }
  if (slot) {
    memcpy(&slot->map, map, sizeof(CUtensorMap));
    slot->valid = true;
  }
  return true;
}

int num_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

template <bool kTf32, int kAMajor, int kBMajor, int kBlockN, bool kPair = false, bool kGather = false, bool kSplit = false>
cudaError_t launch_cfg(const GemmArgs& a, const KernelParams& kp, cudaStream_t stream) {
  using C = Cfg<kTf32, kAMajor, kBMajor, kBlockN, kPair, kSplit>;
  CUtensorMap ta, tb, ta_lo, tb_lo;
  const int dt = kTf32 ? kF32 : kBF16;
  auto map_a = [&](CUtensorMap* m, const void* base) {
    if (kAMajor == kMajorK) return make_tmap(m, base, dt, a.K, a.M, a.batch, a.lda, a.a_batch_stride, C::BK, kBlockM, false);
    return make_tmap(m, base, dt, a.M, a.K, a.batch, a.lda, a.a_batch_stride, C::CH, C::BK, C::A_ATOM32);
  };
  auto map_b = [&](CUtensorMap* m, const void* base) {
    if (kBMajor == kMajorK) return make_tmap(m, base, dt, a.K, a.N, a.batch, a.ldb, a.b_batch_stride, C::BK, C::B_ROWS, false);
    return make_tmap(m, base, dt, a.N, a.K, a.batch, a.ldb, a.b_batch_stride, C::CH, C::BK, C::B_ATOM32);
  };
  if (!map_a(&ta, a.A) || !map_b(&tb, a.B)) return cudaErrorInvalidValue;
  if (a.A_lo != nullptr) {
    if (!map_a(&ta_lo, a.A_lo) || !map_b(&tb_lo, a.B_lo)) return cudaErrorInvalidValue;
  } else {
    ta_lo = ta;  // never read
    tb_lo = tb;
  }

  auto kernel = gemm_kernel<kTf32, kAMajor, kBMajor, kBlockN, kPair, kGather, kSplit>;
  constexpr int kThreads = kNumThreads + (kGather ? kNumGatherThreads : 0) + (kSplit ? kNumSplitThreads : 0);
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  int grid = a.max_ctas > 0 ? a.max_ctas : num_sms();
  if constexpr (kPair) {
    grid /= 2;  // clusters of two CTAs, one tile per cluster at a time
    if (grid > kp.total_tiles) grid = kp.total_tiles;
    if (grid < 1) grid = 1;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(2 * grid, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, ta, tb, ta_lo, tb_lo, kp);
  } else {
    if (grid > kp.total_tiles) grid = kp.total_tiles;
    kernel<<<grid, kThreads, C::SMEM_BYTES, stream>>>(ta, tb, ta_lo, tb_lo, kp);
    return cudaGetLastError();
  }
}

template <bool kTf32, int kAMajor, int kBMajor>
cudaError_t launch_bn(const GemmArgs& a, const KernelParams& kp, int bn, bool pair, cudaStream_t s) {
  if (pair) return launch_cfg<kTf32, kAMajor, kBMajor, 256, true>(a, kp, s);
  switch (bn) {
    case 64: return launch_cfg<kTf32, kAMajor, kBMajor, 64>(a, kp, s);
    case 128: return launch_cfg<kTf32, kAMajor, kBMajor, 128>(a, kp, s);
    default: return launch_cfg<kTf32, kAMajor, kBMajor, 256>(a, kp, s);
  }
}

// fp32 operands split in shared memory: 64- and 128-column tiles
template <int kAMajor, int kBMajor>
cudaError_t launch_split_bn(const GemmArgs& a, const KernelParams& kp, int bn, cudaStream_t s) {
  if (bn == 64) return launch_cfg<true, kAMajor, kBMajor, 64, false, false, true>(a, kp, s);
  return launch_cfg<true, kAMajor, kBMajor, 128, false, false, true>(a, kp, s);
}

cudaError_t launch_split(const GemmArgs& a, const KernelParams& kp, int bn, cudaStream_t s) {
  if (a.a_major == kMajorK) {
    if (a.b_major == kMajorK) return launch_split_bn<kMajorK, kMajorK>(a, kp, bn, s);
    return launch_split_bn<kMajorK, kMajorMN>(a, kp, bn, s);
  }
  if (a.b_major == kMajorK) return launch_split_bn<kMajorMN, kMajorK>(a, kp, bn, s);
  return launch_split_bn<kMajorMN, kMajorMN>(a, kp, bn, s);
}

template <bool kTf32>
cudaError_t launch_major(const GemmArgs& a, const KernelParams& kp, int bn, bool pair, cudaStream_t s) {
  if (a.a_major == kMajorK) {
    if (a.b_major == kMajorK) return launch_bn<kTf32, kMajorK, kMajorK>(a, kp, bn, pair, s);
    return launch_bn<kTf32, kMajorK, kMajorMN>(a, kp, bn, pair, s);
  }
  if (a.b_major == kMajorK) return launch_bn<kTf32, kMajorMN, kMajorK>(a, kp, bn, pair, s);
  return launch_bn<kTf32, kMajorMN, kMajorMN>(a, kp, bn, pair, s);
}

struct Tiling {
  int bn;
  bool pair;
  int tile_m;
};

// Tile width, CTA pairing and tile height for a problem (the heuristics of gemm_launch).
Tiling choose_tiling(const GemmArgs& a) {
  int bn = a.block_n;
  // symmetric products with long K and enough 256 x 256 tiles on and above the diagonal run on CTA pairs
  // as well (half the B traffic per CTA, wide MMAs); short K is bound by the epilogue, where 128-wide
  // tiles spread the mirrored stores over more CTAs
  bool sym_pair = false;
  if (a.symmetric) {
    const long long tn = (a.N + 255) / 256;
    const long long t = tn * (tn + 1) / 2 * a.batch;
    static const int sym_pair_env = [] {
      const char* e = getenv("DION_B200_GEMM_SYM_PAIR");
      return (e && e[0] == '0') ? 0 : 1;
    }();
    sym_pair = sym_pair_env && a.pair >= 0 && a.split_k == 1 && a.K >= 1024 && a.N >= 512 && t >= num_sms() / 2 / 2 &&
               a.A_lo == nullptr && !a.split3;
    bn = sym_pair ? 256 : 128;
  } else if (bn != 64 && bn != 128 && bn != 256) {
    // widest tile that still gives every SM work; narrow N picks a narrow tile
    const long long tm = (a.M + kBlockM - 1) / kBlockM;
    const long long sms = num_sms();
    bn = 256;
    if (a.N <= 64) {
      bn = 64;
    } else if (a.N <= 128) {
      bn = 128;
    } else {
      const long long t256 = tm * ((a.N + 255) / 256) * a.batch * a.split_k;
      if (t256 < sms) bn = 128;
      if ((a.N % 256) != 0 && (a.N % 256) <= 128 && a.N < 1024) bn = 128;
    }
  }

  // CTA pairs (256-row tiles, half the B traffic per CTA) for GEMMs with enough 256 x 256 tiles to
  // keep every pair busy; DION_B200_GEMM_PAIR=0 turns them off, a.pair = 1 / -1 forces / forbids.
  static const int pair_env = [] {
    const char* e = getenv("DION_B200_GEMM_PAIR");
    return (e && e[0] == '0') ? 0 : 1;
  }();
  bool pair = false;
  if (a.pair > 0 && !a.symmetric) bn = 256;
  if (!a.symmetric && bn == 256 && a.pair >= 0 && (pair_env || a.pair > 0)) {
    const long long t = (long long)((a.M + 255) / 256) * ((a.N + 255) / 256) * a.batch * a.split_k;
    // short-K tiles are bound by the epilogue, which a pair does not speed up
    pair = a.pair > 0 || (t >= 2 * (num_sms() / 2) && a.K / a.split_k >= 1024);
  }

  if (sym_pair) pair = true;
  if (a.A_lo != nullptr || a.split3) {  // the cross-term accumulator exists on unpaired tiles of up to 128 columns
    pair = false;
    if (bn > 128) bn = 128;
  }
  if (a.gather.world > 0 && bn == 64) bn = 128;  // the all-gather variant is built for 128- and 256-wide tiles
  Tiling t;
  t.bn = bn;
  t.pair = pair;
  t.tile_m = pair ? 2 * kBlockM : kBlockM;
  return t;
}

// Parameters of the all-gather variant for a problem and its tiling; false if the shapes do not fit.
bool plan_gather(const GemmArgs& a, const Tiling& tl, GatherParams* g) {
  const GemmArgs::Gather& ga = a.gather;
  const bool tf32 = a.ab_dtype == kF32;
  const bool shapes_ok = !tf32 && a.a_major == kMajorK && a.b_major == kMajorK && a.batch == 1 && a.split_k == 1 &&
                         !a.symmetric && a.lda == a.K && ga.world <= kGatherMaxPeers && ga.rank >= 0 &&
                         ga.rank < ga.world && ga.rows > 0 && (long long)ga.rows * ga.world == a.M &&
                         ga.rows % tl.tile_m == 0 && (a.K * 2) % 16 == 0;
  if (!shapes_ok) return false;
  memset(g, 0, sizeof(*g));
  g->world = ga.world;
  g->rank = ga.rank;
  g->channel = ga.channel;
  g->rows = ga.rows;
  int per_chunk = 8;  // tiles per readiness counter: few counters, but work can start early
  while (per_chunk > 1 && (ga.rows % (tl.tile_m * per_chunk) != 0 || ga.rows / (tl.tile_m * per_chunk) < 4)) per_chunk /= 2;
  g->chunk_rows = tl.tile_m * per_chunk;
  g->m_rot = ga.rank * (ga.rows / tl.tile_m);
  g->epoch = ga.epoch;
  g->row_bytes = (long long)a.K * 2;
  g->flag_off = ga.flag_off;
  g->slot_off = ga.slot_off;
  g->in = reinterpret_cast<const char*>(ga.in);
  g->out = reinterpret_cast<char*>(const_cast<void*>(a.A));
  g->units_per_chunk = (int)(((long long)g->chunk_rows * g->row_bytes + kGatherUnitBytes - 1) / kGatherUnitBytes);
  for (int i = 0; i < kGatherMaxPeers; ++i) g->peers[i] = ga.peers[i];
  g->next_unit = ga.counters;
  g->staged = ga.counters ? ga.counters + 1 : nullptr;
  g->ready = ga.counters ? ga.counters + 2 : nullptr;
  g->budget_ns = (unsigned long long)(ga.budget_ns > 0 ? ga.budget_ns : (long long)kWaitBudgetNs);
  return true;
}

bool aligned16(const void* p, long long ld, int es) {
  return (reinterpret_cast<uintptr_t>(p) & 15) == 0 && ((ld * es) & 15) == 0;
}

}  // namespace

const char* gemm_last_error() { return g_last_error.c_str(); }

bool gemm_gather_plan(const GemmArgs& a, int (&out)[8]) {
  const Tiling tl = choose_tiling(a);
  GatherParams g;
  if (!plan_gather(a, tl, &g)) return false;
  out[0] = tl.tile_m;
  out[1] = tl.bn;
  out[2] = tl.pair ? 1 : 0;
  out[3] = g.chunk_rows;
  out[4] = g.units_per_chunk;
  out[5] = g.m_rot;
  out[6] = (a.M + tl.tile_m - 1) / tl.tile_m;
  out[7] = (a.N + tl.bn - 1) / tl.bn;
  return true;
}

cudaError_t gemm_launch(const GemmArgs& a, cudaStream_t stream) {
  g_last_error.clear();
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || a.batch <= 0 || a.split_k <= 0) {
    g_last_error = "GEMM sizes must be positive";
    return cudaErrorInvalidValue;
  }
  if (a.split_k > 1 && a.epilogue != kEpiAtomicAdd) {
    g_last_error = "split_k > 1 needs the atomic-add epilogue";
    return cudaErrorInvalidValue;
  }
  if (a.epilogue == kEpiAtomicAdd && a.d_dtype != kF32) {
    g_last_error = "the atomic-add epilogue needs an fp32 output";
    return cudaErrorInvalidValue;
  }
  if (a.split3 && (a.ab_dtype != kF32 || a.A_lo != nullptr || a.split_k != 1 || a.gather.world > 0)) {
    g_last_error = "in-kernel splitting: fp32 operands without separate low halves, no split-K";
    return cudaErrorInvalidValue;
  }
  if ((a.A_lo != nullptr) != (a.B_lo != nullptr) ||
      (a.A_lo != nullptr && (a.ab_dtype != kF32 || a.split_k != 1 || a.gather.world > 0))) {
    g_last_error = "hi / lo operands: both low halves, fp32 operands, no split-K";
    return cudaErrorInvalidValue;
  }
  if (a.symmetric && a.M != a.N) {
    g_last_error = "symmetric mode needs M == N";
    return cudaErrorInvalidValue;
  }
  if (!a.D && !a.d_ptrs && !a.scatter_ptrs) {
    g_last_error = "GEMM output missing";
    return cudaErrorInvalidValue;
  }
  if (a.d_dup > 1 && (!a.d_ptrs || a.symmetric || a.scatter_mode != 0 || a.epilogue != kEpiStore)) {
    g_last_error = "several destinations per batch element need d_ptrs and a plain store epilogue";
    return cudaErrorInvalidValue;
  }
  if (a.scatter_mode != 0) {
    if (!a.scatter_ptrs || a.scatter_block <= 0 || a.scatter_dests <= 0 || a.symmetric ||
        a.epilogue != kEpiStore || (a.scatter_mode == 2 && a.scatter_block % 32 != 0) ||
        (long long)a.scatter_block * a.scatter_dests < (a.scatter_mode == 1 ? a.M : a.N)) {
      g_last_error = "invalid scatter epilogue (mode 2 needs a block that is a multiple of 32 columns)";
      return cudaErrorInvalidValue;
    }
  }
  const bool tf32 = a.ab_dtype == kF32;
  const int es = tf32 ? 4 : 2;
  const int bk = 128 / es;

  const Tiling tiling = choose_tiling(a);
  const int bn = tiling.bn;
  const bool pair = tiling.pair;
  const int tile_m = tiling.tile_m;

  KernelParams kp;
  memset(&kp, 0, sizeof(kp));
  kp.M = a.M;
  kp.N = a.N;
  kp.K = a.K;
  kp.batch = a.batch;
  kp.split_k = a.split_k;
  kp.tiles_m = (a.M + tile_m - 1) / tile_m;
  kp.tiles_n = (a.N + bn - 1) / bn;
  kp.tiles_per_batch = a.symmetric ? kp.tiles_n * (kp.tiles_n + 1) / 2 : kp.tiles_m * kp.tiles_n;
  const long long total = (long long)kp.tiles_per_batch * a.batch * a.split_k;
  if (total > 0x7fffffffLL) {
    g_last_error = "too many tiles";
    return cudaErrorInvalidValue;
  }
  kp.total_tiles = (int)total;
  kp.kblocks_seg = (a.K + bk - 1) / bk;
  kp.kblocks_total = a.A_lo != nullptr ? 3 * kp.kblocks_seg : kp.kblocks_seg;
  kp.kblocks_per_split = (kp.kblocks_total + a.split_k - 1) / a.split_k;
  kp.alpha = a.alpha;
  kp.beta = a.beta;
  kp.C = a.C;
  kp.c_is_bf16 = a.c_dtype == kBF16;
  kp.ldc = a.ldc;
  kp.c_batch_stride = a.c_batch_stride;
  kp.c_ptrs = a.c_ptrs;
  kp.c_col_scale = a.c_col_scale;
  kp.D = a.D;
  kp.d_is_bf16 = a.d_dtype == kBF16;
  kp.ldd = a.ldd;
  kp.d_batch_stride = a.d_batch_stride;
  kp.d_ptrs = a.d_ptrs;
  kp.d_dup = a.d_dup > 0 ? a.d_dup : 1;
  kp.D2 = a.D2;
  kp.ldd2 = a.ldd2;
  kp.d2_batch_stride = a.d2_batch_stride;
  kp.d2_ptrs = a.d2_ptrs;
  kp.epilogue = a.epilogue;
  kp.act = a.act;
  kp.symmetric = a.symmetric;
  kp.scatter_mode = a.scatter_mode;
  kp.scatter_block = a.scatter_block;
  kp.scatter_dests = a.scatter_dests;
  kp.scatter_ptrs = a.scatter_ptrs;
  kp.status = a.status;
  // Vector access needs aligned bases and pitches; per-batch pointer arrays are
  // required to satisfy this by contract (checked by the Python wrapper).
  const int ces = kp.c_is_bf16 ? 2 : 4, des = kp.d_is_bf16 ? 2 : 4;
  kp.vec_c = (a.c_ptrs || aligned16(a.C, a.ldc, ces)) && ((a.c_batch_stride * ces) % 16 == 0);
  kp.vec_d = (a.d_ptrs || aligned16(a.D, a.ldd, des)) && ((a.d_batch_stride * des) % 16 == 0);
  if (a.scatter_mode != 0) kp.vec_d = ((a.ldd * des) % 16 == 0);  // block bases are 16-byte aligned by contract
  kp.vec_d2 = (a.d2_ptrs || aligned16(a.D2, a.ldd2, 2)) && ((a.d2_batch_stride * 2) % 16 == 0);
  {
    static const int stage_env = [] {
      const char* e = getenv("DION_B200_GEMM_STAGE");
      return (e && e[0] == '0') ? 0 : 1;
    }();
    kp.stage = stage_env;
  }

  if (a.gather.world > 0) {
    // operand A is gathered from the group inside the kernel
    const GemmArgs::Gather& ga = a.gather;
    if (!plan_gather(a, tiling, &kp.g) || !ga.in || !ga.counters || (reinterpret_cast<uintptr_t>(ga.in) & 15) != 0 ||
        (ga.slot_off & 15) != 0) {
      g_last_error = "all-gather variant: bf16 K-major operands, one batch, contiguous A of world * rows rows with "
                     "rows a multiple of the tile height";
      return cudaErrorInvalidValue;
    }
    const int words = 2 + a.M / kp.g.chunk_rows;
    if (words > ga.counter_words) {
      g_last_error = "all-gather variant: counter buffer too small";
      return cudaErrorInvalidValue;
    }
    cudaError_t e = cudaMemsetAsync(ga.counters, 0, sizeof(unsigned) * (size_t)words, stream);
    if (e != cudaSuccess) return e;
    if (pair) return launch_cfg<false, kMajorK, kMajorK, 256, true, true>(a, kp, stream);
    if (bn == 128) return launch_cfg<false, kMajorK, kMajorK, 128, false, true>(a, kp, stream);
    return launch_cfg<false, kMajorK, kMajorK, 256, false, true>(a, kp, stream);
  }
  if (a.split3) return launch_split(a, kp, bn, stream);
  return tf32 ? launch_major<true>(a, kp, bn, pair, stream) : launch_major<false>(a, kp, bn, pair, stream);
}

}  // namespace dion
