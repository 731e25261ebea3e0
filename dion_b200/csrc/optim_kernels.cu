// Multi-tensor optimizer kernels: one launch updates a whole list of parameters.
// They replace the torch._foreach_* / Inductor-fused updates of the reference
// (dion/scalar_opts.py:89-187, dion/muon.py:525-573, dion/dion.py:794).
#include <cuda_bf16.h>

#include "kernels.h"

namespace dion {

namespace {

constexpr int kThreads = 256;
constexpr int kVecPerThread = 4;
constexpr int kBlockElems = kThreads * 4 * kVecPerThread;  // 4096 elements per block

__device__ __forceinline__ int find_tensor(const TensorListChunk& tl, int block) {
  int lo = 0, hi = tl.num_tensors - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (tl.block_start[mid] <= block) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__device__ __forceinline__ bool vec_ok(const void* p, int type) {
  return (reinterpret_cast<uintptr_t>(p) & (type == kElemF32 ? 15 : 7)) == 0;
}

__device__ __forceinline__ float4 load4(const void* p, int type, long long i) {
  if (type == kElemF32) return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
  const uint2 q = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(void* p, int type, long long i, float4 v) {
  if (type == kElemF32) {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + i) = v;
  } else {
    uint2 q;
    *reinterpret_cast<__nv_bfloat162*>(&q.x) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162*>(&q.y) = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p) + i) = q;
  }
}
__device__ __forceinline__ float load1(const void* p, int type, long long i) {
  return type == kElemF32 ? reinterpret_cast<const float*>(p)[i]
                          : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ void store1(void* p, int type, long long i, float v) {
  if (type == kElemF32) reinterpret_cast<float*>(p)[i] = v;
  else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16(v);
}

// Round a float through a storage type, so that math on a just-written state value
// sees what a reload from memory would see.
__device__ __forceinline__ float round_to(float v, int type) {
  return type == kElemF32 ? v : __bfloat162float(__float2bfloat16(v));
}

// Generic driver: Op::apply(float (&vals)[NL][4-or-1]) style is awkward in CUDA, so each
// kernel below spells its loop with this macro-free helper structure instead.
template <typename Body>
__device__ __forceinline__ void for_each_vec(long long n, long long base, bool vec, Body body) {
  if (vec) {
#pragma unroll
    for (int v = 0; v < kVecPerThread; ++v) {
      const long long i = base + ((long long)v * kThreads + threadIdx.x) * 4;
      if (i + 3 < n) {
        body(i, 4);
      } else {
        for (long long j = i; j < n; ++j) body(j, 1);
      }
    }
  } else {
    for (int v = 0; v < kVecPerThread * 4; ++v) {
      const long long i = base + (long long)v * kThreads + threadIdx.x;
      if (i < n) body(i, 1);
    }
  }
}

__device__ __forceinline__ float sgn(float x) { return (x > 0.f) ? 1.f : ((x < 0.f) ? -1.f : 0.f); }

__global__ void __launch_bounds__(kThreads) adamw_kernel(const __grid_constant__ TensorListChunk tl, int g_type,
                                                        int m_type, int v_type, int has_shadow, AdamWHyper h) {
  const int t = find_tensor(tl, blockIdx.x);
  const long long n = tl.numel[t];
  const long long base = (long long)(blockIdx.x - tl.block_start[t]) * kBlockElems;
  float* X = reinterpret_cast<float*>(tl.ptrs[0][t]);
  const void* G = tl.ptrs[1][t];
  void* M = tl.ptrs[2][t];
  void* V = tl.ptrs[3][t];
  void* S = has_shadow ? tl.ptrs[4][t] : nullptr;
  const bool vec = vec_ok(X, kElemF32) && vec_ok(G, g_type) && vec_ok(M, m_type) && vec_ok(V, v_type) &&
                   (!S || vec_ok(S, kElemBF16));
  const float decay = 1.f - h.lr * h.weight_decay;
  const float adj_lr = h.lr / h.bias_correction1;
  auto one = [&](float x, float g, float& m, float& v) {
    const float gm = round_to(g, m_type);  // gradient is cast to the state dtype first
    m = round_to(m + (1.f - h.beta1) * (gm - m), m_type);
    const float g2 = round_to(gm * gm, v_type);
    v = round_to(v + (1.f - h.beta2) * (g2 - v), v_type);
    const float denom = sqrtf(v) / h.bias_correction2_sqrt + h.eps;
    return x * decay - adj_lr * (m / denom);
  };
  for_each_vec(n, base, vec, [&](long long i, int w) {
    if (w == 4) {
      float4 x = *reinterpret_cast<float4*>(X + i);
      const float4 g = load4(G, g_type, i);
      float4 m = load4(M, m_type, i), v = load4(V, v_type, i);
      x.x = one(x.x, g.x, m.x, v.x);
      x.y = one(x.y, g.y, m.y, v.y);
      x.z = one(x.z, g.z, m.z, v.z);
      x.w = one(x.w, g.w, m.w, v.w);
      *reinterpret_cast<float4*>(X + i) = x;
      store4(M, m_type, i, m);
      store4(V, v_type, i, v);
      if (S) store4(S, kElemBF16, i, x);
    } else {
      float m = load1(M, m_type, i), v = load1(V, v_type, i);
      const float x = one(X[i], load1(G, g_type, i), m, v);
      X[i] = x;
      store1(M, m_type, i, m);
      store1(V, v_type, i, v);
      if (S) store1(S, kElemBF16, i, x);
    }
  });
}

__global__ void __launch_bounds__(kThreads) lion_kernel(const __grid_constant__ TensorListChunk tl, int g_type,
                                                       int m_type, int has_shadow, LionHyper h) {
  const int t = find_tensor(tl, blockIdx.x);
  const long long n = tl.numel[t];
  const long long base = (long long)(blockIdx.x - tl.block_start[t]) * kBlockElems;
  float* X = reinterpret_cast<float*>(tl.ptrs[0][t]);
  const void* G = tl.ptrs[1][t];
  void* M = tl.ptrs[2][t];
  void* S = has_shadow ? tl.ptrs[4][t] : nullptr;
  const bool vec = vec_ok(X, kElemF32) && vec_ok(G, g_type) && vec_ok(M, m_type) && (!S || vec_ok(S, kElemBF16));
  const float decay = 1.f - h.lr * h.weight_decay;
  auto one = [&](float x, float g, float& m) {
    const float gm = round_to(g, m_type);
    const float u = sgn(round_to(m + (1.f - h.beta1) * (gm - m), m_type));
    m = round_to(m + (1.f - h.beta2) * (gm - m), m_type);
    return x * decay - h.lr * u;
  };
  for_each_vec(n, base, vec, [&](long long i, int w) {
    if (w == 4) {
      float4 x = *reinterpret_cast<float4*>(X + i);
      const float4 g = load4(G, g_type, i);
      float4 m = load4(M, m_type, i);
      x.x = one(x.x, g.x, m.x);
      x.y = one(x.y, g.y, m.y);
      x.z = one(x.z, g.z, m.z);
      x.w = one(x.w, g.w, m.w);
      *reinterpret_cast<float4*>(X + i) = x;
      store4(M, m_type, i, m);
      if (S) store4(S, kElemBF16, i, x);
    } else {
      float m = load1(M, m_type, i);
      const float x = one(X[i], load1(G, g_type, i), m);
      X[i] = x;
      store1(M, m_type, i, m);
      if (S) store1(S, kElemBF16, i, x);
    }
  });
}

__device__ __forceinline__ float block_sum(float v) {
  __shared__ float red[kThreads / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = 0.f;
  if (threadIdx.x < kThreads / 32) r = red[threadIdx.x];
  if (threadIdx.x < 32) {
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  }
  return r;  // valid in thread 0
}

__global__ void __launch_bounds__(kThreads) muon_pre_kernel(const __grid_constant__ TensorListChunk tl, int g_type,
                                                           float mu, int nesterov, float* sumsq) {
  const int t = find_tensor(tl, blockIdx.x);
  const long long n = tl.numel[t];
  const long long base = (long long)(blockIdx.x - tl.block_start[t]) * kBlockElems;
  const void* G = tl.ptrs[0][t];
  float* M = reinterpret_cast<float*>(tl.ptrs[1][t]);
  void* U = tl.ptrs[2][t];
  const bool vec = vec_ok(G, g_type) && vec_ok(M, kElemF32) && vec_ok(U, kElemBF16);
  float acc = 0.f;
  auto one = [&](float g, float& m) {
    m = mu * m + g;
    const float u = nesterov ? (mu * m + g) : m;
    const float ub = __bfloat162float(__float2bfloat16(u));
    acc += ub * ub;
    return u;
  };
  for_each_vec(n, base, vec, [&](long long i, int w) {
    if (w == 4) {
      const float4 g = load4(G, g_type, i);
      float4 m = *reinterpret_cast<float4*>(M + i);
      float4 u;
      u.x = one(g.x, m.x);
      u.y = one(g.y, m.y);
      u.z = one(g.z, m.z);
      u.w = one(g.w, m.w);
      *reinterpret_cast<float4*>(M + i) = m;
      store4(U, kElemBF16, i, u);
    } else {
      float m = M[i];
      const float u = one(load1(G, g_type, i), m);
      M[i] = m;
      store1(U, kElemBF16, i, u);
    }
  });
  if (sumsq != nullptr) {
    const float s = block_sum(acc);
    if (threadIdx.x == 0) atomicAdd(sumsq + t, s);
  }
}

__global__ void __launch_bounds__(kThreads) muon_post_kernel(const __grid_constant__ TensorListChunk tl,
                                                            int has_shadow, float decay, float step) {
  const int t = find_tensor(tl, blockIdx.x);
  const long long n = tl.numel[t];
  const long long base = (long long)(blockIdx.x - tl.block_start[t]) * kBlockElems;
  float* X = reinterpret_cast<float*>(tl.ptrs[0][t]);
  const void* U = tl.ptrs[1][t];
  void* S = has_shadow ? tl.ptrs[4][t] : nullptr;
  const bool vec = vec_ok(X, kElemF32) && vec_ok(U, kElemBF16) && (!S || vec_ok(S, kElemBF16));
  for_each_vec(n, base, vec, [&](long long i, int w) {
    if (w == 4) {
      float4 x = *reinterpret_cast<float4*>(X + i);
      const float4 u = load4(U, kElemBF16, i);
      x.x = x.x * decay - step * u.x;
      x.y = x.y * decay - step * u.y;
      x.z = x.z * decay - step * u.z;
      x.w = x.w * decay - step * u.w;
      *reinterpret_cast<float4*>(X + i) = x;
      if (S) store4(S, kElemBF16, i, x);
    } else {
      const float x = X[i] * decay - step * load1(U, kElemBF16, i);
      X[i] = x;
      if (S) store1(S, kElemBF16, i, x);
    }
  });
}

__global__ void __launch_bounds__(kThreads) dion_accum_kernel(const __grid_constant__ TensorListChunk tl, int g_type,
                                                             int m_type, int* nonzero) {
  const int t = find_tensor(tl, blockIdx.x);
  const long long n = tl.numel[t];
  const long long base = (long long)(blockIdx.x - tl.block_start[t]) * kBlockElems;
  const void* G = tl.ptrs[0][t];
  void* M = tl.ptrs[1][t];
  const bool vec = vec_ok(G, g_type) && vec_ok(M, m_type);
  int nz = 0;
  for_each_vec(n, base, vec, [&](long long i, int w) {
    if (w == 4) {
      const float4 g = load4(G, g_type, i);
      float4 m = load4(M, m_type, i);
      m.x = round_to(m.x + g.x, m_type);
      m.y = round_to(m.y + g.y, m_type);
      m.z = round_to(m.z + g.z, m_type);
      m.w = round_to(m.w + g.w, m_type);
      nz |= (m.x != 0.f) | (m.y != 0.f) | (m.z != 0.f) | (m.w != 0.f);
      store4(M, m_type, i, m);
    } else {
      const float m = round_to(load1(M, m_type, i) + load1(G, g_type, i), m_type);
      nz |= (m != 0.f);
      store1(M, m_type, i, m);
    }
  });
  if (nonzero != nullptr) {
    nz = __syncthreads_or(nz);
    if (threadIdx.x == 0 && nz) atomicOr(nonzero + t, 1);
  }
}

__global__ void __launch_bounds__(kThreads) cast_kernel(const __grid_constant__ TensorListChunk tl, int src_type,
                                                       int dst_type) {
  const int t = find_tensor(tl, blockIdx.x);
  const long long n = tl.numel[t];
  const long long base = (long long)(blockIdx.x - tl.block_start[t]) * kBlockElems;
  const void* S = tl.ptrs[0][t];
  void* D = tl.ptrs[1][t];
  const bool vec = vec_ok(S, src_type) && vec_ok(D, dst_type);
  for_each_vec(n, base, vec, [&](long long i, int w) {
    if (w == 4) store4(D, dst_type, i, load4(S, src_type, i));
    else store1(D, dst_type, i, load1(S, src_type, i));
  });
}

// ---- Frobenius scaling in front of Newton-Schulz (X / (||X||_F + eps), dion/muon.py:628-631):
// partial sums of squares per chunk, then every block of the scaling pass adds the partials of its
// matrix in the same fixed order, so the result does not depend on how the blocks are scheduled.
constexpr int kFrobChunk = 16384;  // bf16 elements per block

__global__ void __launch_bounds__(kThreads) frob_partial_kernel(const __nv_bfloat16* __restrict__ x,
                                                               float* __restrict__ partial, long long per, int nchunk) {
  const long long b = blockIdx.y;
  const long long lo = (long long)blockIdx.x * kFrobChunk;
  const long long hi = min(per, lo + (long long)kFrobChunk);
  const __nv_bfloat16* xb = x + b * per;
  float acc = 0.f;
  if (((reinterpret_cast<uintptr_t>(xb) | (uintptr_t)(per * 2)) & 15) == 0) {
    for (long long i = lo + threadIdx.x * 8; i + 7 < hi; i += kThreads * 8) {
      const uint4 q = *reinterpret_cast<const uint4*>(xb + i);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc = fmaf(f.x, f.x, acc);
        acc = fmaf(f.y, f.y, acc);
      }
    }
    for (long long i = lo + ((hi - lo) & ~7LL) + threadIdx.x; i < hi; i += kThreads) {
      const float f = __bfloat162float(xb[i]);
      acc = fmaf(f, f, acc);
    }
  } else {
    for (long long i = lo + threadIdx.x; i < hi; i += kThreads) {
      const float f = __bfloat162float(xb[i]);
      acc = fmaf(f, f, acc);
    }
  }
  const float s = block_sum(acc);
  if (threadIdx.x == 0) partial[b * nchunk + blockIdx.x] = s;
}

__global__ void __launch_bounds__(kThreads) frob_scale_kernel(const __nv_bfloat16* __restrict__ x,
                                                             __nv_bfloat16* __restrict__ out,
                                                             const float* __restrict__ partial, int npart,
                                                             const float* __restrict__ sumsq, float eps, long long per) {
  __shared__ float scale_s;
  const long long b = blockIdx.y;
  float acc = 0.f;
  if (sumsq == nullptr)
    for (int i = threadIdx.x; i < npart; i += kThreads) acc += partial[b * npart + i];
  const float tot = block_sum(acc);
  if (threadIdx.x == 0) scale_s = 1.f / (sqrtf(sumsq != nullptr ? sumsq[b] : tot) + eps);
  __syncthreads();
  const float sc = scale_s;
  const long long lo = (long long)blockIdx.x * kFrobChunk;
  const long long hi = min(per, lo + (long long)kFrobChunk);
  const __nv_bfloat16* xb = x + b * per;
  __nv_bfloat16* ob = out + b * per;
  if (((reinterpret_cast<uintptr_t>(xb) | reinterpret_cast<uintptr_t>(ob) | (uintptr_t)(per * 2)) & 15) == 0) {
    for (long long i = lo + threadIdx.x * 8; i + 7 < hi; i += kThreads * 8) {
      uint4 q = *reinterpret_cast<const uint4*>(xb + i);
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        h[j] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
      }
      *reinterpret_cast<uint4*>(ob + i) = q;
    }
    for (long long i = lo + ((hi - lo) & ~7LL) + threadIdx.x; i < hi; i += kThreads)
      ob[i] = __float2bfloat16(__bfloat162float(xb[i]) * sc);
  } else {
    for (long long i = lo + threadIdx.x; i < hi; i += kThreads) ob[i] = __float2bfloat16(__bfloat162float(xb[i]) * sc);
  }
}

inline int total_blocks(const TensorListChunk& tl) { return tl.block_start[tl.num_tensors]; }

}  // namespace

int multi_tensor_block_elems() { return kBlockElems; }

int frob_chunks(long long per) { return (int)((per + kFrobChunk - 1) / kFrobChunk); }

cudaError_t frob_scale_launch(const void* x, void* out, float* partial, const float* sumsq, float eps, int batch,
                              long long per, cudaStream_t s) {
  if (batch == 0 || per == 0) return cudaSuccess;
  if (batch > 65535 || (sumsq == nullptr && partial == nullptr)) return cudaErrorInvalidValue;
  const int nchunk = frob_chunks(per);
  const dim3 grid(nchunk, batch);
  if (sumsq == nullptr) {
    frob_partial_kernel<<<grid, kThreads, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), partial, per, nchunk);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  frob_scale_kernel<<<grid, kThreads, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x),
                                              reinterpret_cast<__nv_bfloat16*>(out), partial, nchunk, sumsq, eps, per);
  return cudaGetLastError();
}

cudaError_t adamw_multi_launch(const TensorListChunk& tl, int g_type, int m_type, int v_type, bool has_shadow,
                               const AdamWHyper& h, cudaStream_t s) {
  if (total_blocks(tl) == 0) return cudaSuccess;
  adamw_kernel<<<total_blocks(tl), kThreads, 0, s>>>(tl, g_type, m_type, v_type, has_shadow ? 1 : 0, h);
  return cudaGetLastError();
}
cudaError_t lion_multi_launch(const TensorListChunk& tl, int g_type, int m_type, bool has_shadow,
                              const LionHyper& h, cudaStream_t s) {
  if (total_blocks(tl) == 0) return cudaSuccess;
  lion_kernel<<<total_blocks(tl), kThreads, 0, s>>>(tl, g_type, m_type, has_shadow ? 1 : 0, h);
  return cudaGetLastError();
}
cudaError_t muon_pre_multi_launch(const TensorListChunk& tl, int g_type, float mu, bool nesterov, float* sumsq,
                                  cudaStream_t s) {
  if (total_blocks(tl) == 0) return cudaSuccess;
  muon_pre_kernel<<<total_blocks(tl), kThreads, 0, s>>>(tl, g_type, mu, nesterov ? 1 : 0, sumsq);
  return cudaGetLastError();
}
cudaError_t muon_post_multi_launch(const TensorListChunk& tl, bool has_shadow, float decay, float step,
                                   cudaStream_t s) {
  if (total_blocks(tl) == 0) return cudaSuccess;
  muon_post_kernel<<<total_blocks(tl), kThreads, 0, s>>>(tl, has_shadow ? 1 : 0, decay, step);
  return cudaGetLastError();
}
cudaError_t dion_accum_multi_launch(const TensorListChunk& tl, int g_type, int m_type, int* nonzero,
                                    cudaStream_t s) {
  if (total_blocks(tl) == 0) return cudaSuccess;
  dion_accum_kernel<<<total_blocks(tl), kThreads, 0, s>>>(tl, g_type, m_type, nonzero);
  return cudaGetLastError();
}
cudaError_t cast_multi_launch(const TensorListChunk& tl, int src_type, int dst_type, cudaStream_t s) {
  if (total_blocks(tl) == 0) return cudaSuccess;
  cast_kernel<<<total_blocks(tl), kThreads, 0, s>>>(tl, src_type, dst_type);
  return cudaGetLastError();
}

}  // namespace dion
