// Bandwidth-bound kernels of the Llama-shaped decoder that the GPT model does not need: RMSNorm with a
// learnable gain (forward, and a backward that also produces the gain's gradient) and the SwiGLU gate
// silu(g) * u (forward and backward).  bf16 activations, fp32 math.  The reference has no Llama model;
// these stand where a compiled PyTorch model would get Inductor-generated kernels.
#include <cuda_bf16.h>

#include "kernels.h"

namespace dion {

namespace {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ void unpack8(const uint4& q, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 t = __bfloat1622float2(h[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 q;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
  for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
  return q;
}
// eight consecutive gains as floats (the gain vector is fp32 or bf16)
__device__ __forceinline__ void load_gain8(const void* g, int type, int col, float (&w)[8]) {
  if (type == kElemF32) {
    const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(g) + col);
    const float4 b = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(g) + col + 4);
    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
  } else {
    unpack8(*reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(g) + col), w);
  }
}

constexpr int kMaxVec = 16;  // 16 vectors of 8 elements per lane: rows of up to 4096 columns

// y = x * rsqrt(mean(x^2) + eps) * gain; one warp per row, the row stays in registers between the passes.
template <int kVec>
__global__ void __launch_bounds__(256) rmsnorm_gain_fwd_kernel(const bf16* __restrict__ x, const void* __restrict__ gain,
                                                              int gain_type, bf16* __restrict__ y,
                                                              float* __restrict__ rstd, long long rows, int dim,
                                                              float eps) {
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int nvec = dim >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * dim);
  uint4* yr = reinterpret_cast<uint4*>(y + row * dim);
  uint4 keep[kVec];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const int v = lane + i * 32;
    if (v < nvec) {
      keep[i] = xr[v];
      float f[8];
      unpack8(keep[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
    }
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / (float)dim + eps);
  if (lane == 0) rstd[row] = r;
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const int v = lane + i * 32;
    if (v < nvec) {
      float f[8], w[8];
      unpack8(keep[i], f);
      load_gain8(gain, gain_type, v * 8, w);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] *= r * w[j];
      yr[v] = pack8(f);
    }
  }
}

// dx = r * (dy * gain) - x * r^3 * mean(dy * gain * x);  dgain += dy * x * r, summed over rows.
// A block walks a contiguous range of rows; every warp adds the rows it handles into its own fp32 row of
// shared memory (no atomics, a fixed order), the block adds its eight rows and writes one partial vector:
// partial[block][dim].  The caller sums the partials - the result does not depend on scheduling.
template <int kVec>
__global__ void __launch_bounds__(256) rmsnorm_gain_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                                              const float* __restrict__ rstd,
                                                              const void* __restrict__ gain, int gain_type,
                                                              bf16* __restrict__ dx, float* __restrict__ partial,
                                                              long long rows, int dim, long long rows_per_block) {
  extern __shared__ float acc[];  // [8][dim]
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nvec = dim >> 3;
  float* mine = acc + (long long)warp * dim;
  for (int c = lane; c < dim; c += 32) mine[c] = 0.f;
  __syncwarp();
  const long long r0 = (long long)blockIdx.x * rows_per_block;
  const long long r1 = min(rows, r0 + rows_per_block);
  for (long long row = r0 + warp; row < r1; row += 8) {
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + row * dim);
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * dim);
    uint4* dxr = reinterpret_cast<uint4*>(dx + row * dim);
    const float r = rstd[row];
    uint4 kdy[kVec], kx[kVec];
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      const int v = lane + i * 32;
      if (v < nvec) {
        kdy[i] = dyr[v];
        kx[i] = xr[v];
      }
    }
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      const int v = lane + i * 32;
      if (v < nvec) {
        float a[8], b[8], w[8];
        unpack8(kdy[i], a);
        unpack8(kx[i], b);
        load_gain8(gain, gain_type, v * 8, w);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dot += a[j] * w[j] * b[j];
          mine[v * 8 + j] += a[j] * b[j] * r;  // this lane is the only writer of these eight columns
        }
      }
    }
    dot = warp_sum(dot);
    const float c = r * r * r * dot / (float)dim;
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      const int v = lane + i * 32;
      if (v < nvec) {
        float a[8], b[8], w[8], o[8];
        unpack8(kdy[i], a);
        unpack8(kx[i], b);
        load_gain8(gain, gain_type, v * 8, w);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = r * a[j] * w[j] - c * b[j];
        dxr[v] = pack8(o);
      }
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < dim; c += 256) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += acc[(long long)w * dim + c];
    partial[(long long)blockIdx.x * dim + c] = t;
  }
}

// h = silu(g) * u
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const uint4* __restrict__ g, const uint4* __restrict__ u,
                                                        uint4* __restrict__ h, long long nvec) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float a[8], b[8], o[8];
    unpack8(g[i], a);
    unpack8(u[i], b);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = a[j] / (1.f + __expf(-a[j])) * b[j];
    h[i] = pack8(o);
  }
}
// dg = dh * u * s * (1 + g * (1 - s)),  du = dh * g * s,  s = sigmoid(g)
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const uint4* __restrict__ dh, const uint4* __restrict__ g,
                                                        const uint4* __restrict__ u, uint4* __restrict__ dg,
                                                        uint4* __restrict__ du, long long nvec) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float d[8], a[8], b[8], og[8], ou[8];
    unpack8(dh[i], d);
    unpack8(g[i], a);
    unpack8(u[i], b);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = 1.f / (1.f + __expf(-a[j]));
      og[j] = d[j] * b[j] * s * (1.f + a[j] * (1.f - s));
      ou[j] = d[j] * a[j] * s;
    }
    dg[i] = pack8(og);
    du[i] = pack8(ou);
  }
}

bool norm_args_ok(const void* gain, int gain_type, int dim) {
  return dim % 8 == 0 && dim <= kMaxVec * 256 && gain != nullptr &&
         (reinterpret_cast<uintptr_t>(gain) & (gain_type == kElemF32 ? 15 : 15)) == 0;
}

}  // namespace

cudaError_t rmsnorm_gain_fwd_launch(const void* x, const void* gain, int gain_type, void* y, float* rstd,
                                    long long rows, int dim, float eps, cudaStream_t s) {
  if (rows == 0) return cudaSuccess;
  if (!norm_args_ok(gain, gain_type, dim)) return cudaErrorInvalidValue;
  const unsigned grid = (unsigned)((rows + 7) / 8);
#define DION_GAIN_FWD(V)                                                                                          \
  rmsnorm_gain_fwd_kernel<V><<<grid, 256, 0, s>>>(reinterpret_cast<const bf16*>(x), gain, gain_type,                 \
                                                  reinterpret_cast<bf16*>(y), rstd, rows, dim, eps)
  if (dim <= 4 * 256) DION_GAIN_FWD(4);
  else if (dim <= 8 * 256) DION_GAIN_FWD(8);
  else DION_GAIN_FWD(16);
#undef DION_GAIN_FWD
  return cudaGetLastError();
}

int rmsnorm_gain_bwd_blocks(long long rows) {
  long long b = (rows + 63) / 64;  // at least 64 rows per block, at most four blocks per SM
  if (b > 148 * 4) b = 148 * 4;
  if (b < 1) b = 1;
  return (int)b;
}

cudaError_t rmsnorm_gain_bwd_launch(const void* dy, const void* x, const float* rstd, const void* gain, int gain_type,
                                    void* dx, float* partial, int blocks, long long rows, int dim, cudaStream_t s) {
  if (rows == 0) return cudaSuccess;
  if (!norm_args_ok(gain, gain_type, dim) || blocks < 1 || partial == nullptr) return cudaErrorInvalidValue;
  const long long rpb = (rows + blocks - 1) / blocks;
  const size_t smem = (size_t)8 * dim * sizeof(float);
#define DION_GAIN_BWD(V)                                                                                           \
  do {                                                                                                             \
    if (smem > 48 * 1024) {                                                                                        \
      cudaError_t e = cudaFuncSetAttribute(rmsnorm_gain_bwd_kernel<V>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           (int)smem);                                                             \
      if (e != cudaSuccess) return e;                                                                              \
    }                                                                                                              \
    rmsnorm_gain_bwd_kernel<V><<<blocks, 256, smem, s>>>(reinterpret_cast<const bf16*>(dy),                         \
                                                         reinterpret_cast<const bf16*>(x), rstd, gain, gain_type,   \
                                                         reinterpret_cast<bf16*>(dx), partial, rows, dim, rpb);     \
  } while (0)
  if (dim <= 4 * 256) DION_GAIN_BWD(4);
  else if (dim <= 8 * 256) DION_GAIN_BWD(8);
  else DION_GAIN_BWD(16);
#undef DION_GAIN_BWD
  return cudaGetLastError();
}

cudaError_t swiglu_fwd_launch(const void* g, const void* u, void* h, long long n, cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  if (n % 8 != 0 || ((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(u) | reinterpret_cast<uintptr_t>(h)) & 15))
    return cudaErrorInvalidValue;
  const long long nvec = n / 8;
  long long grid = (nvec + 255) / 256;
  if (grid > 148 * 16) grid = 148 * 16;
  swiglu_fwd_kernel<<<(int)grid, 256, 0, s>>>(reinterpret_cast<const uint4*>(g), reinterpret_cast<const uint4*>(u),
                                              reinterpret_cast<uint4*>(h), nvec);
  return cudaGetLastError();
}

cudaError_t swiglu_bwd_launch(const void* dh, const void* g, const void* u, void* dg, void* du, long long n,
                              cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  if (n % 8 != 0 || ((reinterpret_cast<uintptr_t>(dh) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(u) |
                      reinterpret_cast<uintptr_t>(dg) | reinterpret_cast<uintptr_t>(du)) & 15))
    return cudaErrorInvalidValue;
  const long long nvec = n / 8;
  long long grid = (nvec + 255) / 256;
  if (grid > 148 * 16) grid = 148 * 16;
  swiglu_bwd_kernel<<<(int)grid, 256, 0, s>>>(reinterpret_cast<const uint4*>(dh), reinterpret_cast<const uint4*>(g),
                                              reinterpret_cast<const uint4*>(u), reinterpret_cast<uint4*>(dg),
                                              reinterpret_cast<uint4*>(du), nvec);
  return cudaGetLastError();
}

}  // namespace dion
