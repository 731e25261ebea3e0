// Causal flash attention for sm_100a: S = Q K^T and O += P V on tcgen05 tensor cores with the
// accumulators in tensor memory, operands staged by TMA, softmax in registers (one query row per
// thread, read from tensor memory with tcgen05.ld).  It stands in for the fused attention the
// reference gets from F.scaled_dot_product_attention (models/gpt_model.py:90-92).
//
// Forward, one CTA per (128 query rows, batch, head); two CTAs share an SM so that one CTA's
// softmax overlaps the other's MMAs:
//   warp 0      TMA: Q once, then K_j and V_j (two stages each) for every 64-row kv tile
//   warp 1      MMA issue: S_j = Q K_j^T into one of two S buffers, O (+)= P_j V_j
//   warps 2-5   softmax: running max / sum in the log2 domain, P_j as bf16 back into tensor memory
//               over S_j (the second MMA reads its A operand from there), lazy rescaling of O (only
//               when the running max grew by more than 2^8), final O / l and the log-sum-exp
// Layouts: q [B*T, H*D], k / v [B*T, Hkv*D], out [B*T, H*D] (bf16, row-major), lse [B, H, T] fp32.
// Every mbarrier wait is bounded; a wait that gives up sets the status word and the CTA drains.
#include <cuda.h>
#include <cuda_bf16.h>
#include <math.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "gemm.h"
#include "kernels.h"
#include "umma.cuh"

namespace dion {

namespace {

constexpr int kAttnThreads = 192;
constexpr int kBM = 128;  // query rows per CTA
constexpr int kBN = 64;   // kv rows per iteration
constexpr float kRescaleThreshold = 8.f;  // log2 units

template <int D>
struct AttnCfg {
  static constexpr int PANELS = D / 64;             // 128-byte panels along the head dimension
  static constexpr int Q_BYTES = kBM * D * 2;
  static constexpr int K_BYTES = kBN * D * 2;
  static constexpr int V_BYTES = kBN * D * 2;
  // two CTAs per SM: 2 * (SMEM + 1 KB reserved) must fit in 228 KB; the 896 bytes of slack cover the
  // alignment of the (128-byte aligned) dynamic shared memory base to 1024
  static constexpr int SMEM = Q_BYTES + 2 * K_BYTES + 2 * V_BYTES + 128 + 896;
  static constexpr int S_COLS = kBN;                // fp32 columns of one S buffer
  static constexpr int O_COL = 2 * kBN;             // O starts after the two S buffers
  static constexpr int TMEM_COLS = 256;             // 2 * 64 + D <= 256
};

struct AttnParams {
  __nv_bfloat16* out;
  float* lse;
  int T, H, Hkv;
  float scale_log2;  // softmax scale * log2(e)
  int* status;
};

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const float (&v)[32]) {
  const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// The MMA-issuing thread is on the critical path of every kv iteration (tiles are small, so one
// tcgen05.mma runs for only 30-70 cycles); descriptors are therefore kept as two 32-bit halves and
// stepped with a single integer add: the start-address field (bits [0,14), units of 16 bytes) never
// carries because shared-memory offsets stay below 256 KB.
struct DescHalves {
  uint32_t lo, hi;
};
__device__ __forceinline__ DescHalves desc_halves(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  const uint64_t d = make_smem_desc(smem_addr, lbo_bytes, sbo_bytes);
  return DescHalves{(uint32_t)d, (uint32_t)(d >> 32)};
}
// D[tmem] (+)= A[smem] * B[smem], bf16, descriptors given as halves plus byte offsets
__device__ __forceinline__ void umma_ss_h(uint32_t tmem_d, DescHalves a, uint32_t a_off, DescHalves b, uint32_t b_off,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}" ::"r"(tmem_d),
      "r"(a.lo + (a_off >> 4)), "r"(a.hi), "r"(b.lo + (b_off >> 4)), "r"(b.hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_ts_h(uint32_t tmem_d, uint32_t tmem_a, DescHalves b, uint32_t b_off,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "r"(b.lo + (b_off >> 4)), "r"(b.hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

// barrier of the two warps (64 threads) that share TMEM lane quadrant `quad`; immediate barrier
// numbers, so that the kernel reserves five named barriers instead of all sixteen
__device__ __forceinline__ void pair_barrier(int quad) {
  switch (quad) {
    case 0: asm volatile("bar.sync 1, 64;" ::: "memory"); break;
    case 1: asm volatile("bar.sync 2, 64;" ::: "memory"); break;
    case 2: asm volatile("bar.sync 3, 64;" ::: "memory"); break;
    default: asm volatile("bar.sync 4, 64;" ::: "memory"); break;
  }
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D>
__global__ void __launch_bounds__(kAttnThreads, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
  using C = AttnCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + C::Q_BYTES;          // two stages
  uint8_t* sV = sK + 2 * C::K_BYTES;      // two stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + 2 * C::V_BYTES);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // 2
  uint64_t* k_empty = bars + 3;     // 2
  uint64_t* v_full = bars + 5;      // 2
  uint64_t* v_empty = bars + 7;     // 2   PV_j retired: V stage j & 1 and the P buffer free, O stable
  uint64_t* s_full = bars + 9;      // 2
  uint64_t* p_full = bars + 11;     // 2
  // (bars + 13 unused)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // heavy (late) query tiles first, so that the tail of the grid is made of short CTAs
  const int q_tile = (int)gridDim.x - 1 - (int)blockIdx.x;
  const int bh = blockIdx.y;
  const int b = bh / p.H, h = bh - b * p.H;
  const int hk = h / (p.H / p.Hkv);
  const int q_row0 = b * p.T + q_tile * kBM;      // row in the [B*T, .] matrices
  const int n_tiles = min((q_tile * kBM + kBM + kBN - 1) / kBN, (p.T + kBN - 1) / kBN);  // causal

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 4);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, C::Q_BYTES);
#pragma unroll
      for (int c = 0; c < C::PANELS; ++c) tma_load_2d(sQ + c * (kBM * 128), &tmap_q, q_full, h * D + c * 64, q_row0);
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j & 1;
        const int kv_row = b * p.T + j * kBN;
        if (!mbar_wait(&k_empty[s], ((j >> 1) & 1) ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        mbar_arrive_expect_tx(&k_full[s], C::K_BYTES);
#pragma unroll
        for (int c = 0; c < C::PANELS; ++c)
          tma_load_2d(sK + s * C::K_BYTES + c * (kBN * 128), &tmap_k, &k_full[s], hk * D + c * 64, kv_row);
        if (!mbar_wait(&v_empty[s], ((j >> 1) & 1) ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        mbar_arrive_expect_tx(&v_full[s], C::V_BYTES);
#pragma unroll
        for (int c = 0; c < C::PANELS; ++c)
          tma_load_2d(sV + s * C::V_BYTES + c * (kBN * 128), &tmap_v, &v_full[s], hk * D + c * 64, kv_row);
      }
      if (!ok) {
        *abort_flag = 1;
        if (p.status) atomicCAS(p.status, 0, kStatusProducerTimeout);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_instr_desc(1, kMajorK, kMajorK, kBM, kBN);
      constexpr uint32_t idesc_pv = make_instr_desc(1, kMajorK, kMajorMN, kBM, D);
      const DescHalves dq_ = desc_halves(smem_u32(sQ), 16, 1024);
      const DescHalves dk0 = desc_halves(smem_u32(sK), 16, 1024), dk1 = desc_halves(smem_u32(sK + C::K_BYTES), 16, 1024);
      const DescHalves dv0 = desc_halves(smem_u32(sV), kBN * 128, 1024),
                       dv1 = desc_halves(smem_u32(sV + C::V_BYTES), kBN * 128, 1024);
      bool ok = mbar_wait(q_full, 0, abort_flag);
      // S_j and P_j share tensor-memory columns (P_j overwrites the first half of S_j), and the
      // tensor core executes this thread's MMAs in issue order, so S_{j+2} = Q K_{j+2}^T, issued after
      // P_j V_j, cannot overtake it; the softmax has finished reading S_j once p_full[j & 1] completed.
      auto issue_qk = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(&k_full[s], (j >> 1) & 1, abort_flag)) return false;
        tc_fence_after();
        const DescHalves dk_s = s ? dk1 : dk0;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off_a = (kk >> 2) * (kBM * 128) + (kk & 3) * 32;
          const uint32_t off_b = (kk >> 2) * (kBN * 128) + (kk & 3) * 32;
          umma_ss_h(tmem_base + s * C::S_COLS, dq_, off_a, dk_s, off_b, idesc_qk, kk > 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[s]);
        umma_commit(&s_full[s]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      if (ok && n_tiles > 1) ok = issue_qk(1);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&v_full[s], (j >> 1) & 1, abort_flag) || !mbar_wait(&p_full[s], (j >> 1) & 1, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const DescHalves dv_s = s ? dv1 : dv0;
#pragma unroll
        for (int kk = 0; kk < kBN / 16; ++kk) {
          // P from tensor memory: 16 bf16 of a row = 8 columns per step; V: MN-major, PANELS chunks of
          // 64 head columns, 16 kv rows per step
          umma_ts_h(tmem_base + C::O_COL, tmem_base + s * C::S_COLS + kk * 8, dv_s, kk * (16 * 128), idesc_pv,
                    (j > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&v_empty[s]);
        if (j + 2 < n_tiles) ok = issue_qk(j + 2);
      }
      if (!ok) {
        *abort_flag = 1;
        if (p.status) atomicCAS(p.status, 0, kStatusMmaTimeout);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax / epilogue
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    const int q_pos = q_tile * kBM + row_in_tile;            // position in the sequence
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
    float m_used = -INFINITY;  // reference max of the exponentials accumulated so far (log2 domain)
    float l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j & 1;
      if (!mbar_wait(&s_full[s], (j >> 1) & 1, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      float sc[kBN];
      {
        float(&lo)[32] = *reinterpret_cast<float(*)[32]>(&sc[0]);
        float(&hi)[32] = *reinterpret_cast<float(*)[32]>(&sc[32]);
        tmem_ld_32x32(lane_base + s * C::S_COLS, lo);
        tmem_ld_32x32(lane_base + s * C::S_COLS + 32, hi);
        tmem_ld_wait();
      }

      const int col0 = j * kBN;
      const bool diag = col0 + kBN - 1 > q_tile * kBM;  // some column of this tile may exceed some row
      if (diag) {
#pragma unroll
        for (int i = 0; i < kBN; ++i)
          if (col0 + i > q_pos) sc[i] = -INFINITY;
      }
      // row maximum of the raw scores (the scale is positive), four independent chains
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < kBN; i += 8) {
#pragma unroll
        for (int t = 0; t < 4; ++t) mx4[t] = fmaxf(mx4[t], fmaxf(sc[i + 2 * t], sc[i + 2 * t + 1]));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
      const float m_new = fmaxf(m_used, mx);
      const bool need = (j == 0) || (m_new - m_used > kRescaleThreshold);
      if (__any_sync(0xffffffffu, need)) {
        if (j > 0) {
          // O may only be touched between two PV products: P_{j-1} V_{j-1} must have retired, and
          // P_j V_j cannot start before this warp delivered P_j
          if (!mbar_wait(&v_empty[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag)) {
            ok = false;
            break;
          }
          const float alpha = (m_new == -INFINITY) ? 1.f : fast_exp2(m_used - m_new);
          l *= alpha;
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            float o[32];
            tmem_ld_32x32(lane_base + C::O_COL + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] *= alpha;
            tmem_st_32x32(lane_base + C::O_COL + c * 32, o);
          }
          tmem_st_wait();
          tc_fence_before();
        }
        m_used = m_new;
      }
      const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      // exponentials, packed to bf16 pairs and stored over the first half of this row of S_j
      float pk[32];
#pragma unroll
      for (int c = 0; c < kBN / 8; ++c) {
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float e0 = fast_exp2(fmaf(sc[8 * c + 2 * t], p.scale_log2, neg_m));
          const float e1 = fast_exp2(fmaf(sc[8 * c + 2 * t + 1], p.scale_log2, neg_m));
          const __nv_bfloat162 h2 = __floats2bfloat162_rn(e0, e1);
          pk[4 * c + t] = __uint_as_float(*reinterpret_cast<const uint32_t*>(&h2));
          sum4[t] += e0 + e1;
        }
      }
      tmem_st_32x32(lane_base + s * C::S_COLS, pk);
      const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      l += sum;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[s]);
    }
    // final: wait for the last PV, normalise, write out and the log-sum-exp
    if (ok && !mbar_wait(&v_empty[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1, abort_flag)) ok = false;
    if (ok) {
      tc_fence_after();
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      const bool row_ok = q_pos < p.T;
      __nv_bfloat16* orow = p.out + ((long long)(b * p.T + q_pos) * p.H + h) * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        float o[32];
        tmem_ld_32x32(lane_base + C::O_COL + c * 32, o);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 q;
            __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
            for (int t = 0; t < 4; ++t) hh[t] = __floats2bfloat162_rn(o[i + 2 * t] * inv_l, o[i + 2 * t + 1] * inv_l);
            *reinterpret_cast<uint4*>(orow + c * 32 + i) = q;
          }
        }
      }
      if (row_ok && p.lse)
        p.lse[((long long)b * p.H + h) * p.T + q_pos] = (l > 0.f) ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
    } else {
      *abort_flag = 1;
      if (p.status) atomicCAS(p.status, 0, kStatusEpilogueTimeout);
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
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ============================================================================================ backward
// dQ, dK, dV of causal attention from q, k, v, dO, the forward's log-sum-exp and
// delta_i = sum_d O_id dO_id (`attn_delta_kernel`).  With S = scale * Q K^T, P = exp(S - lse):
//   dV = P^T dO,  dP = dO V^T,  dS = P o (dP - delta) * scale,  dQ = dS K,  dK = dS^T Q.
// Two kernels, neither needs atomics:
//   attn_bwd_dq_kernel   one CTA per 128 query rows, loops over kv tiles (S, dP, dQ in tensor memory)
//   attn_bwd_dkv_kernel  one CTA per 128 kv rows, loops over query tiles and over the query heads
//                        that share the kv head (S^T, dP^T double buffered, dV, dK in tensor memory)
// P and dS are rebuilt in registers from S and dP and handed to the next MMA as bf16 through tensor
// memory, over the columns they were read from.

struct AttnBwdParams {
  __nv_bfloat16* dq;
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  const float* lse;
  const float* delta;
  int T, H, Hkv;
  float scale, scale_log2;
  int* status;
};

__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
  const __nv_bfloat162 h2 = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h2);
}

// untiled bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completing on `bar`
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// delta[b, h, t] = sum_d O[b, t, h, d] * dO[b, t, h, d]; D / 8 lanes per (b, t, h) row, 16 bytes per lane
template <int D>
__global__ void __launch_bounds__(256) attn_delta_kernel(const __nv_bfloat16* __restrict__ o,
                                                        const __nv_bfloat16* __restrict__ d_o,
                                                        float* __restrict__ delta, long long rows, int T, int H) {
  constexpr int LPR = D / 8;  // lanes per row: 16 (D = 128) or 8 (D = 64)
  const long long row = ((long long)blockIdx.x * 256 + threadIdx.x) / LPR;  // index into [B, T, H]
  const int sub = threadIdx.x % LPR;
  float s = 0.f;
  if (row < rows) {
    const uint4 a = *reinterpret_cast<const uint4*>(o + row * D + sub * 8);
    const uint4 g = *reinterpret_cast<const uint4*>(d_o + row * D + sub * 8);
    const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = __bfloat1622float2(ah[i]), y = __bfloat1622float2(gh[i]);
      s = fmaf(x.x, y.x, fmaf(x.y, y.y, s));
    }
  }
#pragma unroll
  for (int off = LPR / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (sub == 0 && row < rows) {
    const long long bt = row / H;
    const int h = (int)(row - bt * H);
    const long long b = bt / T;
    const int t = (int)(bt - b * T);
    delta[(b * H + h) * T + t] = s;
  }
}

template <int D>
struct BwdQCfg {
  static constexpr int PANELS = D / 64;
  static constexpr int Q_BYTES = kBM * D * 2;
  static constexpr int K_BYTES = kBN * D * 2;
  static constexpr int SMEM = 2 * Q_BYTES + 3 * K_BYTES + 128 + 896;  // Q, dO, K x 2, V
  static constexpr int S_COL = 0, DP_COL = kBN, DQ_COL = 2 * kBN;
  static constexpr int TMEM_COLS = 256;
};

template <int D>
__global__ void __launch_bounds__(kAttnThreads, 2)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                   const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                   const AttnBwdParams p) {
  using C = BwdQCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = sQ + C::Q_BYTES;
  uint8_t* sK = sDO + C::Q_BYTES;      // two stages
  uint8_t* sV = sK + 2 * C::K_BYTES;   // one stage
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + C::K_BYTES);
  uint64_t* q_full = bars;         // 1
  uint64_t* k_full = bars + 1;     // 2
  uint64_t* k_empty = bars + 3;    // 2
  uint64_t* v_full = bars + 5;     // 1
  uint64_t* v_empty = bars + 6;    // 1
  uint64_t* sdp_full = bars + 7;   // 1
  uint64_t* ds_full = bars + 8;    // 1 (four warps arrive)
  uint64_t* dq_full = bars + 9;    // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q_tile = (int)gridDim.x - 1 - (int)blockIdx.x;
  const int bh = blockIdx.y;
  const int b = bh / p.H, h = bh - b * p.H;
  const int hk = h / (p.H / p.Hkv);
  const int q_row0 = b * p.T + q_tile * kBM;
  const int n_tiles = min((q_tile * kBM + kBM + kBN - 1) / kBN, (p.T + kBN - 1) / kBN);

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_do);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
    }
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    mbar_init(sdp_full, 1);
    mbar_init(ds_full, 4);
    mbar_init(dq_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, 2 * C::Q_BYTES);
#pragma unroll
      for (int c = 0; c < C::PANELS; ++c) {
        tma_load_2d(sQ + c * (kBM * 128), &tmap_q, q_full, h * D + c * 64, q_row0);
        tma_load_2d(sDO + c * (kBM * 128), &tmap_do, q_full, h * D + c * 64, q_row0);
      }
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j & 1;
        const int kv_row = b * p.T + j * kBN;
        if (!mbar_wait(&k_empty[s], ((j >> 1) & 1) ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        mbar_arrive_expect_tx(&k_full[s], C::K_BYTES);
#pragma unroll
        for (int c = 0; c < C::PANELS; ++c)
          tma_load_2d(sK + s * C::K_BYTES + c * (kBN * 128), &tmap_k, &k_full[s], hk * D + c * 64, kv_row);
        if (!mbar_wait(v_empty, (j & 1) ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        mbar_arrive_expect_tx(v_full, C::K_BYTES);
#pragma unroll
        for (int c = 0; c < C::PANELS; ++c) tma_load_2d(sV + c * (kBN * 128), &tmap_v, v_full, hk * D + c * 64, kv_row);
      }
      if (!ok) {
        *abort_flag = 1;
        if (p.status) atomicCAS(p.status, 0, kStatusProducerTimeout);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_instr_desc(1, kMajorK, kMajorK, kBM, kBN);
      constexpr uint32_t idesc_dq = make_instr_desc(1, kMajorK, kMajorMN, kBM, D);
      const DescHalves dq_ = desc_halves(smem_u32(sQ), 16, 1024), ddo_ = desc_halves(smem_u32(sDO), 16, 1024);
      const DescHalves dk0 = desc_halves(smem_u32(sK), 16, 1024), dk1 = desc_halves(smem_u32(sK + C::K_BYTES), 16, 1024);
      const DescHalves dv_ = desc_halves(smem_u32(sV), 16, 1024);
      // K_j once more, read as [64 kv rows (K) x D (N)], MN-major, for dQ += dS K_j
      const DescHalves dkm0 = desc_halves(smem_u32(sK), kBN * 128, 1024),
                       dkm1 = desc_halves(smem_u32(sK + C::K_BYTES), kBN * 128, 1024);
      bool ok = mbar_wait(q_full, 0, abort_flag);
      // S_j = Q K_j^T and dP_j = dO V_j^T.  Both overwrite columns the previous dS lives in; they are
      // issued after dS_{j-1} K_{j-1}, which the tensor core therefore finishes first.
      auto issue_sdp = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(&k_full[s], (j >> 1) & 1, abort_flag) || !mbar_wait(v_full, j & 1, abort_flag)) return false;
        tc_fence_after();
        const DescHalves dk_s = s ? dk1 : dk0;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off_a = (kk >> 2) * (kBM * 128) + (kk & 3) * 32;
          const uint32_t off_b = (kk >> 2) * (kBN * 128) + (kk & 3) * 32;
          umma_ss_h(tmem_base + C::S_COL, dq_, off_a, dk_s, off_b, idesc_s, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off_a = (kk >> 2) * (kBM * 128) + (kk & 3) * 32;
          const uint32_t off_b = (kk >> 2) * (kBN * 128) + (kk & 3) * 32;
          umma_ss_h(tmem_base + C::DP_COL, ddo_, off_a, dv_, off_b, idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(v_empty);
        umma_commit(sdp_full);
        return true;
      };
      if (ok) ok = issue_sdp(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j & 1;
        if (!mbar_wait(ds_full, j & 1, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const DescHalves dkm_s = s ? dkm1 : dkm0;
#pragma unroll
        for (int kk = 0; kk < kBN / 16; ++kk)
          umma_ts_h(tmem_base + C::DQ_COL, tmem_base + C::S_COL + kk * 8, dkm_s, kk * (16 * 128), idesc_dq,
                    (j > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&k_empty[s]);
        if (j + 1 < n_tiles) ok = issue_sdp(j + 1);
      }
      if (ok) umma_commit(dq_full);
      else {
        *abort_flag = 1;
        if (p.status) atomicCAS(p.status, 0, kStatusMmaTimeout);
      }
    }
  } else {
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    const int q_pos = q_tile * kBM + row_in_tile;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
    const long long stat_idx = ((long long)b * p.H + h) * p.T + q_pos;
    const float neg_lse2 = -p.lse[stat_idx] * 1.4426950408889634f;
    const float dlt = p.delta[stat_idx];
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      if (!mbar_wait(sdp_full, j & 1, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int col0 = j * kBN;
      const bool diag = col0 + kBN - 1 > q_tile * kBM;
      float pk[32];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        float sc[32], dp[32];
        tmem_ld_32x32(lane_base + C::S_COL + half * 32, sc);
        tmem_ld_32x32(lane_base + C::DP_COL + half * 32, dp);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = fast_exp2(fmaf(sc[i], p.scale_log2, neg_lse2));
          float p1 = fast_exp2(fmaf(sc[i + 1], p.scale_log2, neg_lse2));
          if (diag) {
            if (col0 + half * 32 + i > q_pos) p0 = 0.f;
            if (col0 + half * 32 + i + 1 > q_pos) p1 = 0.f;
          }
          const float d0 = p0 * (dp[i] - dlt) * p.scale;
          const float d1 = p1 * (dp[i + 1] - dlt) * p.scale;
          pk[half * 16 + (i >> 1)] = __uint_as_float(pack_bf16x2(d0, d1));
        }
      }
      tmem_st_32x32(lane_base + C::S_COL, pk);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
    }
    if (ok && !mbar_wait(dq_full, 0, abort_flag)) ok = false;
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* orow = p.dq + ((long long)(b * p.T + q_pos) * p.H + h) * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        float o[32];
        tmem_ld_32x32(lane_base + C::DQ_COL + c * 32, o);
        tmem_ld_wait();
        if (q_pos < p.T) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 q;
            q.x = pack_bf16x2(o[i], o[i + 1]);
            q.y = pack_bf16x2(o[i + 2], o[i + 3]);
            q.z = pack_bf16x2(o[i + 4], o[i + 5]);
            q.w = pack_bf16x2(o[i + 6], o[i + 7]);
            *reinterpret_cast<uint4*>(orow + c * 32 + i) = q;
          }
        }
      }
    } else {
      *abort_flag = 1;
      if (p.status) atomicCAS(p.status, 0, kStatusEpilogueTimeout);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------- dK, dV
constexpr int kKvThreads = 64 + 32 * 8;  // TMA warp, MMA warp, eight softmax warps (two per lane quadrant)
constexpr int kBQ = 64;                  // query rows per iteration

template <int D>
struct BwdKvCfg {
  static constexpr int PANELS = D / 64;
  static constexpr int KV_BYTES = kBM * D * 2;         // K or V tile: 128 kv rows
  static constexpr int Q_BYTES = kBQ * D * 2;          // Q_i or dO_i tile: 64 query rows
  static constexpr int STAT_BYTES = kBQ * 4;           // lse_i or delta_i
  static constexpr int TILE_BYTES = 2 * Q_BYTES;                   // Q_i and dO_i of one stage
  static constexpr int STAGE_BYTES = TILE_BYTES + 2 * STAT_BYTES;  // what one stage's barrier receives
  static constexpr int STAGES = 3;                                  // query-side tiles in flight
  static constexpr int SMEM = 2 * KV_BYTES + STAGES * STAGE_BYTES + 256 + 1024;
  // D = 128: S^T / dP^T double buffered, one CTA per SM (512 columns).  D = 64: single buffers and
  // 256 columns, so that two CTAs share an SM and cover each other's prologue, epilogue and waits.
  static constexpr int NBUF = D == 128 ? 2 : 1;
  static constexpr int ST_COL = 0;                   // NBUF buffers of 64 columns
  static constexpr int DPT_COL = NBUF * kBQ;         // NBUF buffers of 64 columns
  static constexpr int DV_COL = 2 * NBUF * kBQ;
  static constexpr int DK_COL = DV_COL + D;
  static constexpr int TMEM_COLS = D == 128 ? 512 : 256;
  static constexpr int CTAS_PER_SM = D == 128 ? 1 : 2;
};

template <int D>
__global__ void __launch_bounds__(kKvThreads, BwdKvCfg<D>::CTAS_PER_SM)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                    const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                    const AttnBwdParams p) {
  using C = BwdKvCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + C::KV_BYTES;
  uint8_t* sStage = sV + C::KV_BYTES;           // per stage: Q_i, dO_i (1024-byte aligned tiles)
  uint8_t* sStat = sStage + C::STAGES * C::TILE_BYTES;  // per stage: lse_i, delta_i
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStat + C::STAGES * 2 * C::STAT_BYTES);
  uint64_t* kv_full = bars;          // 1
  uint64_t* qdo_full = bars + 1;     // 3
  uint64_t* qdo_empty = bars + 4;    // 3
  uint64_t* sdp_full = bars + 7;     // 2
  uint64_t* pds_full = bars + 9;     // 2 (eight warps arrive)
  uint64_t* acc_full = bars + 11;    // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kv_tile = blockIdx.x;                 // light (late) kv tiles last
  const int bhk = blockIdx.y;
  const int b = bhk / p.Hkv, hk = bhk - b * p.Hkv;
  const int group = p.H / p.Hkv;
  const int kv0 = kv_tile * kBM;
  const int i_first = kv0 / kBQ;                  // first query tile that sees this kv tile
  const int n_q = p.T / kBQ - i_first;            // query tiles per head
  const int n_it = n_q * group;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_do);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    mbar_init(kv_full, 1);
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&qdo_full[s], 1);
      mbar_init(&qdo_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sdp_full[s], 1);
      mbar_init(&pds_full[s], 8);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(kv_full, 2 * C::KV_BYTES);
#pragma unroll
      for (int c = 0; c < C::PANELS; ++c) {
        tma_load_2d(sK + c * (kBM * 128), &tmap_k, kv_full, hk * D + c * 64, b * p.T + kv0);
        tma_load_2d(sV + c * (kBM * 128), &tmap_v, kv_full, hk * D + c * 64, b * p.T + kv0);
      }
      bool ok = true;
      for (int it = 0; it < n_it && ok; ++it) {
        const int s = it % C::STAGES;
        const int g = it / n_q, i = i_first + (it - g * n_q);
        const int h = hk * group + g;
        if (!mbar_wait(&qdo_empty[s], ((it / C::STAGES) & 1) ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        uint8_t* st = sStage + s * C::TILE_BYTES;
        uint8_t* stat_s = sStat + s * 2 * C::STAT_BYTES;
        mbar_arrive_expect_tx(&qdo_full[s], C::STAGE_BYTES);
        const int row = b * p.T + i * kBQ;
#pragma unroll
        for (int c = 0; c < C::PANELS; ++c) {
          tma_load_2d(st + c * (kBQ * 128), &tmap_q, &qdo_full[s], h * D + c * 64, row);
          tma_load_2d(st + C::Q_BYTES + c * (kBQ * 128), &tmap_do, &qdo_full[s], h * D + c * 64, row);
        }
        const long long stat = ((long long)b * p.H + h) * p.T + i * kBQ;
        bulk_load_1d(stat_s, p.lse + stat, C::STAT_BYTES, &qdo_full[s]);
        bulk_load_1d(stat_s + C::STAT_BYTES, p.delta + stat, C::STAT_BYTES, &qdo_full[s]);
      }
      if (!ok) {
        *abort_flag = 1;
        if (p.status) atomicCAS(p.status, 0, kStatusProducerTimeout);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_instr_desc(1, kMajorK, kMajorK, kBM, kBQ);
      constexpr uint32_t idesc_acc = make_instr_desc(1, kMajorK, kMajorMN, kBM, D);
      const DescHalves dk_ = desc_halves(smem_u32(sK), 16, 1024), dv_ = desc_halves(smem_u32(sV), 16, 1024);
      // stage 0 of the query-side tiles, K-major (for S^T, dP^T) and MN-major (for dV, dK)
      const DescHalves dq_ = desc_halves(smem_u32(sStage), 16, 1024),
                       ddo_ = desc_halves(smem_u32(sStage + C::Q_BYTES), 16, 1024);
      const DescHalves dqm_ = desc_halves(smem_u32(sStage), kBQ * 128, 1024),
                       ddom_ = desc_halves(smem_u32(sStage + C::Q_BYTES), kBQ * 128, 1024);
      bool ok = mbar_wait(kv_full, 0, abort_flag);
      // S^T = K Q_i^T and dP^T = V dO_i^T into buffer it & 1
      auto issue_sdp = [&](int it) -> bool {
        const int s = it % C::NBUF, st = it % C::STAGES;
        if (!mbar_wait(&qdo_full[st], (it / C::STAGES) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t st_off = st * C::TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off_a = (kk >> 2) * (kBM * 128) + (kk & 3) * 32;
          const uint32_t off_b = (kk >> 2) * (kBQ * 128) + (kk & 3) * 32;
          umma_ss_h(tmem_base + C::ST_COL + s * kBQ, dk_, off_a, dq_, st_off + off_b, idesc_s, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off_a = (kk >> 2) * (kBM * 128) + (kk & 3) * 32;
          const uint32_t off_b = (kk >> 2) * (kBQ * 128) + (kk & 3) * 32;
          umma_ss_h(tmem_base + C::DPT_COL + s * kBQ, dv_, off_a, ddo_, st_off + off_b, idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&sdp_full[s]);
        return true;
      };
      if (ok) ok = issue_sdp(0);
      if (ok && C::NBUF > 1 && n_it > 1) ok = issue_sdp(1);
      for (int it = 0; it < n_it && ok; ++it) {
        const int s = it % C::NBUF;
        if (!mbar_wait(&pds_full[s], (it / C::NBUF) & 1, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const int st = it % C::STAGES;
        const uint32_t st_off = st * C::TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < kBQ / 16; ++kk) {
          // dV += P^T dO_i and dK += dS^T Q_i: A from tensor memory (bf16 pairs, 8 columns per step),
          // B = the query-side tile read as [64 rows (K) x D (N)], MN-major
          umma_ts_h(tmem_base + C::DV_COL, tmem_base + C::ST_COL + s * kBQ + kk * 8, ddom_, st_off + kk * (16 * 128),
                    idesc_acc, (it > 0 || kk > 0) ? 1u : 0u);
          umma_ts_h(tmem_base + C::DK_COL, tmem_base + C::DPT_COL + s * kBQ + kk * 8, dqm_, st_off + kk * (16 * 128),
                    idesc_acc, (it > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&qdo_empty[st]);
        if (it + C::NBUF < n_it) ok = issue_sdp(it + C::NBUF);
      }
      if (ok) umma_commit(acc_full);
      else {
        *abort_flag = 1;
        if (p.status) atomicCAS(p.status, 0, kStatusMmaTimeout);
      }
    }
  } else {
    // eight warps: quadrant = warp & 3 (kv rows), half = which 32 of the 64 query columns
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row_in_tile = quad * 32 + lane;
    const int kv_pos = kv0 + row_in_tile;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
    bool ok = true;
    // A failed wait clears `ok` but the loop keeps its shape: both warps of a quadrant must reach
    // the named barrier the same number of times.
    for (int it = 0; it < n_it; ++it) {
      const int s = it % C::NBUF;
      const int g = it / n_q, i = i_first + (it - g * n_q);
      if (ok && !mbar_wait(&sdp_full[s], (it / C::NBUF) & 1, abort_flag)) ok = false;
      tc_fence_after();
      const float* lse_s = reinterpret_cast<const float*>(sStat + (it % C::STAGES) * 2 * C::STAT_BYTES) + half * 32;
      const float* dlt_s = lse_s + kBQ;
      float sc[32], dp[32];
      if (ok) {
        tmem_ld_32x32(lane_base + C::ST_COL + s * kBQ + half * 32, sc);
        tmem_ld_32x32(lane_base + C::DPT_COL + s * kBQ + half * 32, dp);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c) sc[c] = dp[c] = 0.f;
      }
      const int qcol0 = i * kBQ + half * 32;           // sequence position of this thread's first column
      const bool diag = qcol0 < kv0 + kBM;             // some query of this block precedes some kv row
      uint32_t pp[16], dd[16];
#pragma unroll
      for (int c = 0; c < 32; c += 4) {
        const float4 l4 = *reinterpret_cast<const float4*>(lse_s + c);
        const float4 d4 = *reinterpret_cast<const float4*>(dlt_s + c);
        const float ls[4] = {l4.x, l4.y, l4.z, l4.w};
        const float dl[4] = {d4.x, d4.y, d4.z, d4.w};
        float pv[4], dv[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          float e = fast_exp2(fmaf(sc[c + t], p.scale_log2, -ls[t] * 1.4426950408889634f));
          if (diag && qcol0 + c + t < kv_pos) e = 0.f;
          pv[t] = e;
          dv[t] = e * (dp[c + t] - dl[t]) * p.scale;
        }
        pp[c >> 1] = pack_bf16x2(pv[0], pv[1]);
        pp[(c >> 1) + 1] = pack_bf16x2(pv[2], pv[3]);
        dd[c >> 1] = pack_bf16x2(dv[0], dv[1]);
        dd[(c >> 1) + 1] = pack_bf16x2(dv[2], dv[3]);
      }
      // both warps of a quadrant must have read S^T / dP^T before either overwrites its part: the
      // packed halves land in columns [0, 32) of the buffers, which the other warp may still be loading
      pair_barrier(quad);
      if (!__all_sync(0xffffffffu, ok)) {
        ok = false;
        continue;
      }
      tmem_st_32x16(lane_base + C::ST_COL + s * kBQ + half * 16, pp);
      tmem_st_32x16(lane_base + C::DPT_COL + s * kBQ + half * 16, dd);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&pds_full[s]);
    }
    if (ok && !mbar_wait(acc_full, 0, abort_flag)) ok = false;
    if (ok) {
      tc_fence_after();
      // warp `half` 0 writes dV, `half` 1 writes dK
      __nv_bfloat16* base = (half == 0 ? p.dv : p.dk) + ((long long)(b * p.T + kv_pos) * p.Hkv + hk) * D;
      const uint32_t col = half == 0 ? C::DV_COL : C::DK_COL;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        float o[32];
        tmem_ld_32x32(lane_base + col + c * 32, o);
        tmem_ld_wait();
        if (kv_pos < p.T) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 q;
            q.x = pack_bf16x2(o[i], o[i + 1]);
            q.y = pack_bf16x2(o[i + 2], o[i + 3]);
            q.z = pack_bf16x2(o[i + 4], o[i + 5]);
            q.w = pack_bf16x2(o[i + 6], o[i + 7]);
            *reinterpret_cast<uint4*>(base + c * 32 + i) = q;
          }
        }
      }
    } else {
      *abort_flag = 1;
      if (p.status) atomicCAS(p.status, 0, kStatusEpilogueTimeout);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn attn_encode_fn() {
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

// [rows, cols] bf16 row-major with pitch `ld` elements; box = 64 columns x box_rows rows, 128-byte swizzle
bool attn_tmap(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows, uint64_t ld, uint32_t box_rows) {
  EncodeFn fn = attn_encode_fn();
  if (!fn) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * 2) & 15)) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int D>
cudaError_t attn_fwd_launch_d(const void* q, const void* k, const void* v, void* out, float* lse, int B, int T, int H,
                              int Hkv, float scale, int* status, cudaStream_t stream) {
  using C = AttnCfg<D>;
  CUtensorMap tq, tk, tv;
  const uint64_t rows = (uint64_t)B * T;
  if (!attn_tmap(&tq, q, (uint64_t)H * D, rows, (uint64_t)H * D, kBM) ||
      !attn_tmap(&tk, k, (uint64_t)Hkv * D, rows, (uint64_t)Hkv * D, kBN) ||
      !attn_tmap(&tv, v, (uint64_t)Hkv * D, rows, (uint64_t)Hkv * D, kBN))
    return cudaErrorInvalidValue;
  auto kernel = attn_fwd_kernel<D>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  AttnParams p;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.T = T;
  p.H = H;
  p.Hkv = Hkv;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  dim3 grid((T + kBM - 1) / kBM, B * H);
  kernel<<<grid, kAttnThreads, C::SMEM, stream>>>(tq, tk, tv, p);
  return cudaGetLastError();
}

template <int D>
cudaError_t attn_bwd_launch_d(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                              const float* lse, float* delta, void* dq, void* dk, void* dv, int B, int T, int H,
                              int Hkv, float scale, int* status, cudaStream_t stream) {
  const uint64_t rows = (uint64_t)B * T;
  CUtensorMap q128, do128, k64, v64, q64, do64, k128, v128;
  const uint64_t wq = (uint64_t)H * D, wk = (uint64_t)Hkv * D;
  if (!attn_tmap(&q128, q, wq, rows, wq, kBM) || !attn_tmap(&do128, d_o, wq, rows, wq, kBM) ||
      !attn_tmap(&k64, k, wk, rows, wk, kBN) || !attn_tmap(&v64, v, wk, rows, wk, kBN) ||
      !attn_tmap(&q64, q, wq, rows, wq, kBQ) || !attn_tmap(&do64, d_o, wq, rows, wq, kBQ) ||
      !attn_tmap(&k128, k, wk, rows, wk, kBM) || !attn_tmap(&v128, v, wk, rows, wk, kBM))
    return cudaErrorInvalidValue;
  auto kq = attn_bwd_dq_kernel<D>;
  auto kkv = attn_bwd_dkv_kernel<D>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdQCfg<D>::SMEM);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(kkv, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdKvCfg<D>::SMEM);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  const long long nrows = (long long)B * T * H;
  attn_delta_kernel<D><<<(unsigned)((nrows * (D / 8) + 255) / 256), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(o), reinterpret_cast<const __nv_bfloat16*>(d_o), delta, nrows, T, H);
  AttnBwdParams p;
  p.dq = reinterpret_cast<__nv_bfloat16*>(dq);
  p.dk = reinterpret_cast<__nv_bfloat16*>(dk);
  p.dv = reinterpret_cast<__nv_bfloat16*>(dv);
  p.lse = lse;
  p.delta = delta;
  p.T = T;
  p.H = H;
  p.Hkv = Hkv;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  kkv<<<dim3(T / kBM, B * Hkv), kKvThreads, BwdKvCfg<D>::SMEM, stream>>>(q64, do64, k128, v128, p);
  kq<<<dim3(T / kBM, B * H), kAttnThreads, BwdQCfg<D>::SMEM, stream>>>(q128, do128, k64, v64, p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t attn_bwd_launch(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                            const float* lse, float* delta, void* dq, void* dk, void* dv, int B, int T, int H, int Hkv,
                            int D, float scale, int* status, cudaStream_t stream) {
  if (B <= 0 || T <= 0 || H <= 0 || Hkv <= 0 || H % Hkv != 0 || B * H > 65535 || T % kBM != 0)
    return cudaErrorInvalidValue;
  if (D == 128)
    return attn_bwd_launch_d<128>(q, k, v, o, d_o, lse, delta, dq, dk, dv, B, T, H, Hkv, scale, status, stream);
  if (D == 64)
    return attn_bwd_launch_d<64>(q, k, v, o, d_o, lse, delta, dq, dk, dv, B, T, H, Hkv, scale, status, stream);
  return cudaErrorInvalidValue;
}

cudaError_t attn_fwd_launch(const void* q, const void* k, const void* v, void* out, float* lse, int B, int T, int H,
                            int Hkv, int D, float scale, int* status, cudaStream_t stream) {
  if (B <= 0 || T <= 0 || H <= 0 || Hkv <= 0 || H % Hkv != 0 || B * H > 65535) return cudaErrorInvalidValue;
  // the TMA boxes of one sequence must not run into the next one: whole kv tiles per sequence
  if (T % kBM != 0) return cudaErrorInvalidValue;
  if (D == 128) return attn_fwd_launch_d<128>(q, k, v, out, lse, B, T, H, Hkv, scale, status, stream);
  if (D == 64) return attn_fwd_launch_d<64>(q, k, v, out, lse, B, T, H, Hkv, scale, status, stream);
  return cudaErrorInvalidValue;
}

}  // namespace dion
