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
  if (threadIdx.x == 0) ok_flag = DION_DBG_OK(w.world <= kMaxPeers && (w.world <= 1 || (w.rank >= 0 && w.rank < w.world)) &&
                                                  w.channel >= 0 && w.channel * kMaxPeers + kMaxPeers <= 1024 / 2, status) ? 1 : 0;
  __syncthreads();
  if (ok_flag && w.world > 1 && threadIdx.x < 32) {
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
  // debug build: vector accesses need aligned slots and a slot stride that keeps the alignment
  if (!DION_DBG_OK((reinterpret_cast<uintptr_t>(a.slots) & 15) == 0 && (a.slot_stride & 3) == 0 && a.nslots >= 1 &&
                       a.ndest <= kMaxPeers, a.status))
    return;
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

// bf16 flavour of slot_reduce for activations (tensor-parallel row-parallel products): out = sum of the
// slots in slot order (fp32 accumulation) + optional residual, bf16 in and out, 16-byte accesses.
__global__ void __launch_bounds__(512) slot_reduce_bf16_kernel(const SlotReduceBf16Args a) {
  if (!exchange_ready(a.wait, a.status)) return;
  const long long nvec = a.numel >> 3;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const uint4* base = reinterpret_cast<const uint4*>(a.slots);
  const long long sstride = a.slot_stride >> 3;
  const uint4* res = reinterpret_cast<const uint4*>(a.residual);
  uint4* out = reinterpret_cast<uint4*>(a.out);
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += stride) {
    float acc[8];
    {
      const uint4 q = base[v];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] = f.x;
        acc[2 * j + 1] = f.y;
      }
    }
    for (int s = 1; s < a.nslots; ++s) {
      const uint4 q = base[s * sstride + v];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    if (res != nullptr) {
      const uint4 q = res[v];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    out[v] = o;
  }
}

// Four consecutive columns of one row as floats (fp32: one 16-byte access, bf16: one 8-byte access).
__device__ __forceinline__ float4 load_quad(const void* p, int type, long long i) {
  if (type == kElemF32) return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
  const uint2 q = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store_quad(void* p, int type, long long i, const float4& v) {
  if (type == kElemF32) {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + i) = v;
  } else {
    uint2 q;
    *reinterpret_cast<__nv_bfloat162*>(&q.x) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162*>(&q.y) = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p) + i) = q;
  }
}

// One CTA per (strip of kStrip columns, matrix): 8 warps take the rows in turn, a lane owns kV consecutive
// columns, so that a warp moves kStrip * 4 contiguous bytes of a row per access.  kV = 4 (strips of 128
// columns, 16-byte accesses) needs r, the pitches and the column offsets to be multiples of 4 and aligned
// bases; kV = 1 (strips of 32 columns) takes everything else.
template <int kV>
__global__ void __launch_bounds__(256) r_post_kernel(const RPostArgs a) {
  if (!exchange_ready(a.wait, a.status)) return;
  __shared__ float red[8][32 * kV + 1];
  __shared__ float tot[32 * kV];
  const int b = blockIdx.y;
  const int lane = threadIdx.x & 31;
  const int rlane = threadIdx.x >> 5;
  const int col = (blockIdx.x * 32 + lane) * kV;
  const bool live = col < a.r;  // kV = 4: r is a multiple of 4, so a live lane owns four valid columns
  const bool nz = a.nonzero == nullptr || a.nonzero[b] != 0;
  const long long mat = (long long)b * a.n * a.r;

  // guarded R[b][i][col ..]: the rank-ordered sum of the slots, or the previous Q for an all-zero momentum
  auto guarded = [&](int i, float (&v)[kV]) {
    if (!nz) {
      const long long qe = (long long)b * a.q_bs + (long long)i * a.q_ld + col;
      if constexpr (kV == 4) {
        const float4 q = load_quad(a.Qm, a.q_type, qe);
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
      } else {
        v[0] = load_elem(a.Qm, a.q_type, qe);
      }
      return;
    }
    const long long e = mat + (long long)i * a.r + col;
    if constexpr (kV == 4) {
      float4 s = *reinterpret_cast<const float4*>(a.slots + e);
      for (int k = 1; k < a.nslots; ++k) {
        const float4 x = *reinterpret_cast<const float4*>(a.slots + k * a.slot_stride + e);
        s.x += x.x; s.y += x.y; s.z += x.z; s.w += x.w;
      }
      v[0] = nan_to_num(s.x * a.scale); v[1] = nan_to_num(s.y * a.scale);
      v[2] = nan_to_num(s.z * a.scale); v[3] = nan_to_num(s.w * a.scale);
    } else {
      float s = a.slots[e];
      for (int k = 1; k < a.nslots; ++k) s += a.slots[k * a.slot_stride + e];
      v[0] = nan_to_num(s * a.scale);
    }
  };
  auto put = [&](void* p, int type, long long e, const float (&v)[kV]) {
    if constexpr (kV == 4) store_quad(p, type, e, make_float4(v[0], v[1], v[2], v[3]));
    else store_elem(p, type, e, v[0]);
  };

  float ss[kV];
#pragma unroll
  for (int k = 0; k < kV; ++k) ss[k] = 0.f;
  if (live) {
    for (int i = rlane; i < a.n; i += 8) {
      float v[kV];
      guarded(i, v);
      const long long e = mat + (long long)i * a.r + col;
      if (a.R32) put(a.R32, kElemF32, e, v);
      if (a.Rm) put(a.Rm, a.rm_type, e, v);
#pragma unroll
      for (int k = 0; k < kV; ++k) ss[k] = fmaf(v[k], v[k], ss[k]);
    }
    // P[b][:, col ..]: zero for an all-zero momentum, NaN / inf replaced otherwise; written only where it changes
    if (a.P) {
      for (long long i = rlane; i < a.p_rows; i += 8) {
        const long long e = (long long)b * a.p_bs + i * a.p_ld + col;
        float v[kV], w[kV];
        if constexpr (kV == 4) {
          const float4 q = load_quad(a.P, a.p_type, e);
          v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
        } else {
          v[0] = load_elem(a.P, a.p_type, e);
        }
        bool same = true;
#pragma unroll
        for (int k = 0; k < kV; ++k) {
          w[k] = nz ? nan_to_num(v[k]) : 0.f;
          same = same && (w[k] == v[k]);
        }
        if (!same) put(a.P, a.p_type, e, w);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < kV; ++k) red[rlane][lane * kV + k] = ss[k];
  __syncthreads();
  if (threadIdx.x < 32 * kV) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += red[k][threadIdx.x];
    tot[threadIdx.x] = t;
    const int c = blockIdx.x * 32 * kV + threadIdx.x;
    if (c < a.r && a.ss) a.ss[(long long)b * a.r + c] = t;
  }
  if (!a.finish) return;
  __syncthreads();
  if (!live) return;
  // new Q: column-normalised R; a column that came out zero keeps the previous Q
  float inv[kV];
  bool keep[kV];
#pragma unroll
  for (int k = 0; k < kV; ++k) {
    const float t = tot[lane * kV + k];
    keep[k] = !(t > 0.f);
    inv[k] = 1.f / (sqrtf(t) + a.eps);
  }
  // the Q state holds columns [qs_col0, qs_col0 + qs_cols); kV = 4: both are multiples of 4
  const bool in_slice = col >= a.qs_col0 && col < a.qs_col0 + a.qs_cols;
  for (int i = rlane; i < a.n; i += 8) {
    float q[kV];
    guarded(i, q);
    bool any_keep = false;
#pragma unroll
    for (int k = 0; k < kV; ++k) {
      q[k] *= inv[k];
      any_keep = any_keep || keep[k];
    }
    if (any_keep) {
      const long long qe = (long long)b * a.q_bs + (long long)i * a.q_ld + col;
#pragma unroll
      for (int k = 0; k < kV; ++k)
        if (keep[k]) q[k] = load_elem(a.Qm, a.q_type, qe + k);
    }
    if (a.Qn) put(a.Qn, a.qn_type, mat + (long long)i * a.r + col, q);
    if (a.Qs && in_slice) put(a.Qs, a.qs_type, ((long long)b * a.n + i) * a.qs_cols + (col - a.qs_col0), q);
  }
}

template <int kV>
__global__ void __launch_bounds__(256) q_norm_kernel(const QNormArgs a) {
  const int b = blockIdx.y;
  const int lane = threadIdx.x & 31;
  const int rlane = threadIdx.x >> 5;
  const int col = (blockIdx.x * 32 + lane) * kV;
  if (col >= a.r) return;
  float inv[kV];
  bool keep[kV], any_keep = false;
#pragma unroll
  for (int k = 0; k < kV; ++k) {
    const float t = a.ss[(long long)b * a.r + col + k];
    keep[k] = !(t > 0.f);
    any_keep = any_keep || keep[k];
    inv[k] = 1.f / (sqrtf(t) + a.eps);
  }
  const bool in_slice = col >= a.qs_col0 && col < a.qs_col0 + a.qs_cols;
  const long long mat = (long long)b * a.n * a.r;
  for (int i = rlane; i < a.n; i += 8) {
    const long long e = mat + (long long)i * a.r + col;
    float q[kV];
    if constexpr (kV == 4) {
      const float4 x = *reinterpret_cast<const float4*>(a.R32 + e);
      q[0] = x.x * inv[0]; q[1] = x.y * inv[1]; q[2] = x.z * inv[2]; q[3] = x.w * inv[3];
    } else {
      q[0] = a.R32[e] * inv[0];
    }
    if (any_keep) {
      const long long qe = (long long)b * a.q_bs + (long long)i * a.q_ld + col;
#pragma unroll
      for (int k = 0; k < kV; ++k)
        if (keep[k]) q[k] = load_elem(a.Qm, a.q_type, qe + k);
    }
    if constexpr (kV == 4) {
      const float4 v = make_float4(q[0], q[1], q[2], q[3]);
      if (a.Qn) store_quad(a.Qn, a.qn_type, e, v);
      if (a.Qs && in_slice) store_quad(a.Qs, a.qs_type, ((long long)b * a.n + i) * a.qs_cols + (col - a.qs_col0), v);
    } else {
      if (a.Qn) store_elem(a.Qn, a.qn_type, e, q[0]);
      if (a.Qs && in_slice) store_elem(a.Qs, a.qs_type, ((long long)b * a.n + i) * a.qs_cols + (col - a.qs_col0), q[0]);
    }
  }
}

// 16-byte (fp32) or 8-byte (bf16) accesses of four elements at element offsets that are multiples of 4
bool quad_ok(const void* p, int type, long long ld, long long bs) {
  if (p == nullptr) return true;
  const uintptr_t align = type == kElemF32 ? 15 : 7;
  return (reinterpret_cast<uintptr_t>(p) & align) == 0 && (ld & 3) == 0 && (bs & 3) == 0;
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

cudaError_t slot_reduce_bf16_launch(const SlotReduceBf16Args& a, cudaStream_t s) {
  if (a.numel == 0 && a.wait.world <= 1) return cudaSuccess;
  if (!wait_ok(a.wait) || a.nslots < 1 || (a.numel & 7) || (a.slot_stride & 7) || a.out == nullptr ||
      ((reinterpret_cast<uintptr_t>(a.slots) | reinterpret_cast<uintptr_t>(a.out) | reinterpret_cast<uintptr_t>(a.residual)) & 15))
    return cudaErrorInvalidValue;
  const long long nvec = a.numel >> 3;
  long long grid = (nvec + 512 * 4 - 1) / (512 * 4);
  if (grid > 2 * 148) grid = 2 * 148;
  if (grid < 1) grid = 1;
  slot_reduce_bf16_kernel<<<(int)grid, 512, 0, s>>>(a);
  return cudaGetLastError();
}

cudaError_t r_post_launch(const RPostArgs& a, cudaStream_t s) {
  if (a.B == 0 || a.n == 0 || a.r == 0) return cudaSuccess;
  if (!wait_ok(a.wait) || a.nslots < 1 || a.B > 65535 || a.slots == nullptr || a.Qm == nullptr ||
      (a.finish && a.Qs != nullptr && (a.qs_cols <= 0 || a.qs_col0 < 0 || a.qs_col0 + a.qs_cols > a.r)))
    return cudaErrorInvalidValue;
  const long long mat = (long long)a.n * a.r;
  const bool wide = (a.r & 3) == 0 && quad_ok(a.slots, kElemF32, a.r, a.slot_stride) && (mat & 3) == 0 &&
                    quad_ok(a.Qm, a.q_type, a.q_ld, a.q_bs) && quad_ok(a.P, a.p_type, a.p_ld, a.p_bs) &&
                    quad_ok(a.R32, kElemF32, a.r, mat) && quad_ok(a.Rm, a.rm_type, a.r, mat) &&
                    quad_ok(a.Qn, a.qn_type, a.r, mat) &&
                    (a.Qs == nullptr || (quad_ok(a.Qs, a.qs_type, a.qs_cols, (long long)a.n * a.qs_cols) && (a.qs_col0 & 3) == 0));
  if (wide) r_post_kernel<4><<<dim3((a.r + 127) / 128, a.B), 256, 0, s>>>(a);
  else r_post_kernel<1><<<dim3((a.r + 31) / 32, a.B), 256, 0, s>>>(a);
  return cudaGetLastError();
}

cudaError_t q_norm_launch(const QNormArgs& a, cudaStream_t s) {
  if (a.B == 0 || a.n == 0 || a.r == 0) return cudaSuccess;
  if (a.B > 65535 || a.R32 == nullptr || a.ss == nullptr || a.Qm == nullptr ||
      (a.Qs != nullptr && (a.qs_cols <= 0 || a.qs_col0 < 0 || a.qs_col0 + a.qs_cols > a.r)))
    return cudaErrorInvalidValue;
  const long long mat = (long long)a.n * a.r;
  const bool wide = (a.r & 3) == 0 && (mat & 3) == 0 && quad_ok(a.R32, kElemF32, a.r, mat) &&
                    quad_ok(a.Qn, a.qn_type, a.r, mat) &&
                    (a.Qs == nullptr || (quad_ok(a.Qs, a.qs_type, a.qs_cols, (long long)a.n * a.qs_cols) && (a.qs_col0 & 3) == 0));
  if (wide) q_norm_kernel<4><<<dim3((a.r + 127) / 128, a.B), 256, 0, s>>>(a);
  else q_norm_kernel<1><<<dim3((a.r + 31) / 32, a.B), 256, 0, s>>>(a);
  return cudaGetLastError();
}

}  // namespace dion
