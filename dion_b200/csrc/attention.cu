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

// D[tmem] (+)= A[tmem] * B[smem]: A (128 rows, one per lane, bf16 pairs along the columns) is read
// from tensor memory
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
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
      bool ok = mbar_wait(q_full, 0, abort_flag);
      // S_j and P_j share tensor-memory columns (P_j overwrites the first half of S_j), and the
      // tensor core executes this thread's MMAs in issue order, so S_{j+2} = Q K_{j+2}^T, issued after
      // P_j V_j, cannot overtake it; the softmax has finished reading S_j once p_full[j & 1] completed.
      auto issue_qk = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(&k_full[s], (j >> 1) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t a0 = smem_u32(sQ), b0 = smem_u32(sK + s * C::K_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off_a = (kk >> 2) * (kBM * 128) + (kk & 3) * 32;
          const uint32_t off_b = (kk >> 2) * (kBN * 128) + (kk & 3) * 32;
          umma_ss<false>(tmem_base + s * C::S_COLS, make_smem_desc(a0 + off_a, 16, 1024),
                         make_smem_desc(b0 + off_b, 16, 1024), idesc_qk, kk > 0 ? 1u : 0u);
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
        const uint32_t b0 = smem_u32(sV + s * C::V_BYTES);
#pragma unroll
        for (int kk = 0; kk < kBN / 16; ++kk) {
          // P from tensor memory: 16 bf16 of a row = 8 columns per step; V: MN-major, PANELS chunks of
          // 64 head columns, 16 kv rows per step
          umma_ts(tmem_base + C::O_COL, tmem_base + s * C::S_COLS + kk * 8,
                  make_smem_desc(b0 + kk * (16 * 128), kBN * 128, 1024), idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
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

}  // namespace

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
