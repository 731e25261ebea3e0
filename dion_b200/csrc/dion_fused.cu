// Kernels that fuse Dion's reductions over ranks with the arithmetic that follows them.
//
// The power-iteration products P = A Q and R = A^T P are partial sums when A is sharded (FSDP,
// tensor parallelism) or when the data-parallel replicas synchronise the low-rank factors instead of
// the gradients.  The reference reduces them with NCCL calls between its matmuls
// (dion/dion.py:801-844, 921-960, 1071-1110) and then runs a chain of small element-wise kernels
// (fix_all_zero_or_nan, local_column_sum_sq, column_normalize, update_Q_matrix_;
// dion/dion.py:1416-1491, 1533-1561).  Here the GEMM that produces a partial product stores its
// tiles straight into "slots" of the consuming ranks' symmetric memory while it is still
// multiplying (slot s of a buffer receives rank s's contribution), and the kernels below
//
//   1. announce "my contribution is complete" to the peers and wait (bounded) for theirs,
//   2. add the slots up in rank order - every rank that reads the same slots gets the same bits -,
//   3. and do the arithmetic of the next stage in the same pass:
//        slot_reduce : P (fp32) and its tf32 hi / lo halves for the 3xTF32 Gram product, optionally
//                      handing the sum on to the slots of a second group (hierarchical reduction)
//        r_post      : all-zero / NaN guard of R and P, R in the momentum dtype, column sums of
//                      squares and, when no further reduction is needed, the column-normalised new Q
//        q_norm      : the column normalisation alone (after the sums of squares were reduced)
//
// The slots a kernel reads are local memory (the peers pushed them), so these kernels run at HBM
// speed; only the flag words cross NVLink here.  Nothing in this file uses TMA.
#include <cuda_bf16.h>
#include <float.h>

#include "kernels.h"
#include "symm_flags.cuh"
#include "umma.cuh"

namespace dion {

namespace {

__device__ __forceinline__ float load_elem(const void* p, int type, long long i) {
  return type == kElemF32 ? reinterpret_cast<const float*>(p)[i]
                          : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ void store_elem(void* p, int type, long long i, float v) {
  if (type == kElemF32) reinterpret_cast<float*>(p)[i] = v;
  else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16(v);
}
// torch.nan_to_num: NaN -> 0, +-inf -> +-largest finite value
__device__ __forceinline__ float nan_to_num(float v) {
  if (v != v) return 0.f;
  if (v == INFINITY) return FLT_MAX;
  if (v == -INFINITY) return -FLT_MAX;
  return v;
}

// Announce (one CTA) and wait (every CTA) on `channel`; returns false when a peer did not arrive.
__device__ __forceinline__ bool exchange_ready(const SlotWait& w, int* status) {
  __shared__ int ok_flag;
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();
  if (w.world > 1 && threadIdx.x < 32) {
    if (blockIdx.x == 0 && blockIdx.y == 0) {
      __threadfence_system();
      signal_peers(w.peers, w.flag_off, w.channel, w.rank, w.world, w.epoch, threadIdx.x);
    }
    if (!wait_peers(w.peers, w.flag_off, w.channel, w.rank, w.world, w.epoch, threadIdx.x, w.budget_ns)) {
      ok_flag = 0;
      if (status) atomicCAS(status, 0, kStatusPeerTimeout);
    }
  }
  __syncthreads();
  return ok_flag != 0;
}

__global__ void __launch_bounds__(512) slot_reduce_kernel(const SlotReduceArgs a) {
  if (!exchange_ready(a.wait, a.status)) return;
  const long long nvec = a.numel >> 2;
  const long long stride = (long long)gridDim.x * blockDim.x;
  // The slots were written by other GPUs: plain (coherent) loads, never the read-only path.
  const float4* base = reinterpret_cast<const float4*>(a.slots);
  const long long sstride = a.slot_stride >> 2;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += stride) {
    float4 acc = base[v];
    for (int s = 1; s < a.nslots; ++s) {
      const float4 x = base[s * sstride + v];
      acc.x += x.x;
      acc.y += x.y;
      acc.z += x.z;
      acc.w += x.w;
    }
    acc.x *= a.scale;
    acc.y *= a.scale;
    acc.z *= a.scale;
    acc.w *= a.scale;
    if (a.out) reinterpret_cast<float4*>(a.out)[v] = acc;
    for (int d = 0; d < a.ndest; ++d) reinterpret_cast<float4*>(a.dest[d])[v] = acc;
    if (a.hi) {
      float4 h, l;
      h.x = __int_as_float(__float_as_int(acc.x) & 0xffffe000);
      h.y = __int_as_float(__float_as_int(acc.y) & 0xffffe000);
      h.z = __int_as_float(__float_as_int(acc.z) & 0xffffe000);
      h.w = __int_as_float(__float_as_int(acc.w) & 0xffffe000);
      l.x = acc.x - h.x;
      l.y = acc.y - h.y;
      l.z = acc.z - h.z;
      l.w = acc.w - h.w;
      reinterpret_cast<float4*>(a.hi)[v] = h;
      reinterpret_cast<float4*>(a.lo)[v] = l;
    }
  }
}

// One CTA per (32 columns, matrix); 8 row lanes x 32 column lanes.
__global__ void __launch_bounds__(256) r_post_kernel(const RPostArgs a) {
  if (!exchange_ready(a.wait, a.status)) return;
  __shared__ float red[8][33];
  __shared__ float tot[32];
  const int b = blockIdx.y;
  const int lane = threadIdx.x & 31;
  const int rlane = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + lane;
  const bool live = col < a.r;
  const bool nz = a.nonzero == nullptr || a.nonzero[b] != 0;
  const long long mat = (long long)b * a.n * a.r;

  // guarded R[b][i][col]: the rank-ordered sum of the slots, or the previous Q for an all-zero momentum
  auto guarded = [&](int i) -> float {
    if (!nz) return load_elem(a.Qm, a.q_type, (long long)b * a.q_bs + (long long)i * a.q_ld + col);
    const long long e = mat + (long long)i * a.r + col;
    float v = a.slots[e];
    for (int s = 1; s < a.nslots; ++s) v += a.slots[s * a.slot_stride + e];
    return nan_to_num(v * a.scale);
  };

  float s = 0.f;
  if (live) {
    for (int i = rlane; i < a.n; i += 8) {
      const float v = guarded(i);
      const long long e = mat + (long long)i * a.r + col;
      if (a.R32) a.R32[e] = v;
      if (a.Rm) store_elem(a.Rm, a.rm_type, e, v);
      s = fmaf(v, v, s);
    }
    // P[b][:, col]: zero for an all-zero momentum, NaN / inf replaced otherwise; written only where it changes
    if (a.P) {
      for (long long i = rlane; i < a.p_rows; i += 8) {
        const long long e = (long long)b * a.p_bs + i * a.p_ld + col;
        const float v = load_elem(a.P, a.p_type, e);
        const float w = nz ? nan_to_num(v) : 0.f;
        if (!(w == v)) store_elem(a.P, a.p_type, e, w);
      }
    }
  }
  red[rlane][lane] = s;
  __syncthreads();
  if (rlane == 0) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += red[k][lane];
    tot[lane] = t;
    if (live && a.ss) a.ss[(long long)b * a.r + col] = t;
  }
  if (!a.finish) return;
  __syncthreads();
  if (!live) return;
  // new Q: column-normalised R; a column that came out zero keeps the previous Q
  const float t = tot[lane];
  const float inv = 1.f / (sqrtf(t) + a.eps);
  const bool in_slice = col >= a.qs_col0 && col < a.qs_col0 + a.qs_cols;
  for (int i = rlane; i < a.n; i += 8) {
    const long long qe = (long long)b * a.q_bs + (long long)i * a.q_ld + col;
    const float q = t > 0.f ? guarded(i) * inv : load_elem(a.Qm, a.q_type, qe);
    if (a.Qn) store_elem(a.Qn, a.qn_type, mat + (long long)i * a.r + col, q);
    if (a.Qs && in_slice)
      store_elem(a.Qs, a.qs_type, ((long long)b * a.n + i) * a.qs_cols + (col - a.qs_col0), q);
  }
}

__global__ void __launch_bounds__(256) q_norm_kernel(const QNormArgs a) {
  const int b = blockIdx.y;
  const int lane = threadIdx.x & 31;
  const int rlane = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + lane;
  if (col >= a.r) return;
  const float t = a.ss[(long long)b * a.r + col];
  const float inv = 1.f / (sqrtf(t) + a.eps);
  const bool in_slice = col >= a.qs_col0 && col < a.qs_col0 + a.qs_cols;
  const long long mat = (long long)b * a.n * a.r;
  for (int i = rlane; i < a.n; i += 8) {
    const long long e = mat + (long long)i * a.r + col;
    const float q = t > 0.f ? a.R32[e] * inv
                            : load_elem(a.Qm, a.q_type, (long long)b * a.q_bs + (long long)i * a.q_ld + col);
    if (a.Qn) store_elem(a.Qn, a.qn_type, e, q);
    if (a.Qs && in_slice)
      store_elem(a.Qs, a.qs_type, ((long long)b * a.n + i) * a.qs_cols + (col - a.qs_col0), q);
  }
}

bool wait_ok(const SlotWait& w) {
  return w.world >= 0 && w.world <= kMaxPeers && (w.world <= 1 || (w.rank >= 0 && w.rank < w.world));
}

}  // namespace

cudaError_t slot_reduce_launch(const SlotReduceArgs& a, cudaStream_t s) {
  // a rank without data of its own still has to announce itself to the peers that wait for it
  if (a.numel == 0 && a.wait.world <= 1) return cudaSuccess;
  if (!wait_ok(a.wait) || a.nslots < 1 || a.ndest < 0 || a.ndest > kMaxPeers || (a.numel & 3) || (a.slot_stride & 3) ||
      (reinterpret_cast<uintptr_t>(a.slots) & 15) || (reinterpret_cast<uintptr_t>(a.out) & 15) ||
      (reinterpret_cast<uintptr_t>(a.hi) & 15) || (reinterpret_cast<uintptr_t>(a.lo) & 15) ||
      ((a.hi == nullptr) != (a.lo == nullptr)))
    return cudaErrorInvalidValue;
  for (int d = 0; d < a.ndest; ++d)
    if (a.dest[d] == nullptr || (reinterpret_cast<uintptr_t>(a.dest[d]) & 15)) return cudaErrorInvalidValue;
  const long long nvec = a.numel >> 2;
  long long grid = (nvec + 512 * 4 - 1) / (512 * 4);
  if (grid > 2 * 148) grid = 2 * 148;
  if (grid < 1) grid = 1;
  slot_reduce_kernel<<<(int)grid, 512, 0, s>>>(a);
  return cudaGetLastError();
}

cudaError_t r_post_launch(const RPostArgs& a, cudaStream_t s) {
  if (a.B == 0 || a.n == 0 || a.r == 0) return cudaSuccess;
  if (!wait_ok(a.wait) || a.nslots < 1 || a.B > 65535 || a.slots == nullptr || a.Qm == nullptr ||
      (a.finish && a.Qs != nullptr && (a.qs_cols <= 0 || a.qs_col0 < 0 || a.qs_col0 + a.qs_cols > a.r)))
    return cudaErrorInvalidValue;
  r_post_kernel<<<dim3((a.r + 31) / 32, a.B), 256, 0, s>>>(a);
  return cudaGetLastError();
}

cudaError_t q_norm_launch(const QNormArgs& a, cudaStream_t s) {
  if (a.B == 0 || a.n == 0 || a.r == 0) return cudaSuccess;
  if (a.B > 65535 || a.R32 == nullptr || a.ss == nullptr || a.Qm == nullptr ||
      (a.Qs != nullptr && (a.qs_cols <= 0 || a.qs_col0 < 0 || a.qs_col0 + a.qs_cols > a.r)))
    return cudaErrorInvalidValue;
  q_norm_kernel<<<dim3((a.r + 31) / 32, a.B), 256, 0, s>>>(a);
  return cudaGetLastError();
}

}  // namespace dion
