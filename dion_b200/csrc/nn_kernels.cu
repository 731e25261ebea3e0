// Bandwidth-bound model kernels: RMSNorm, rotary + QK-norm, ReLU^2, softmax
// cross-entropy (forward and gradient in one pass) and the embedding gather/scatter.
// bf16 activations, fp32 math.  They stand in for the Inductor-generated kernels the
// reference gets from model.compile() (models/gpt_model.py:54-61, 86-89, 106-112,
// 115-124, 171-179).
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdlib.h>

#include <initializer_list>

#include "kernels.h"

namespace dion {

namespace {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
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

// ------------------------------------------------------------------ RMSNorm
// One warp per row; the row is kept in registers between the two passes.  kVec = 16-byte vectors
// per lane (dim <= kVec * 256): instantiated for 4, 8 and 16 so that narrow rows do not pay the
// registers, and with them the occupancy, of the widest case.
constexpr int kNormMaxVec = 16;  // 16 * 32 lanes * 8 elements = 4096 columns at most

template <int kVec>
__global__ void __launch_bounds__(256) rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ res,
                                                         bf16* __restrict__ x_out, bf16* __restrict__ y,
                                                         float* __restrict__ rstd, long long rows, int dim,
                                                         float eps) {
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int nvec = dim >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * dim);
  const uint4* rr = res ? reinterpret_cast<const uint4*>(res + row * dim) : nullptr;
  uint4* xo = x_out ? reinterpret_cast<uint4*>(x_out + row * dim) : nullptr;
  uint4* yr = reinterpret_cast<uint4*>(y + row * dim);
  uint4 keep[kVec];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const int v = lane + i * 32;
    if (v < nvec) {
      uint4 q = xr[v];
      float f[8];
      unpack8(q, f);
      if (rr) {
        float g[8];
        unpack8(rr[v], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += g[j];
        q = pack8(f);
        unpack8(q, f);  // normalise exactly what is stored as the new residual stream
        if (xo) xo[v] = q;
      }
      keep[i] = q;
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
    }
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / (float)dim + eps);
  if (lane == 0 && rstd) rstd[row] = r;
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const int v = lane + i * 32;
    if (v < nvec) {
      float f[8];
      unpack8(keep[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] *= r;
      yr[v] = pack8(f);
    }
  }
}

template <int kVec>
__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                                         const float* __restrict__ rstd,
                                                         const bf16* __restrict__ dx_add, bf16* __restrict__ dx,
                                                         long long rows, int dim) {
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int nvec = dim >> 3;
  const uint4* dyr = reinterpret_cast<const uint4*>(dy + row * dim);
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * dim);
  const uint4* ar = dx_add ? reinterpret_cast<const uint4*>(dx_add + row * dim) : nullptr;
  uint4* dxr = reinterpret_cast<uint4*>(dx + row * dim);
  const float r = rstd[row];
  // all loads of the row are issued before the first use
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
    if (lane + i * 32 < nvec) {
      float a[8], b[8];
      unpack8(kdy[i], a);
      unpack8(kx[i], b);
#pragma unroll
      for (int j = 0; j < 8; ++j) dot += a[j] * b[j];
    }
  }
  dot = warp_sum(dot);
  // dx = r * dy - x * r^3 * mean(dy * x)
  const float c = r * r * r * dot / (float)dim;
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const int v = lane + i * 32;
    if (v < nvec) {
      float a[8], b[8], o[8];
      unpack8(kdy[i], a);
      unpack8(kx[i], b);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = r * a[j] - c * b[j];
      if (ar) {
        float e[8];
        unpack8(ar[v], e);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += e[j];
      }
      dxr[v] = pack8(o);
    }
  }
}

// ------------------------------------------------------------------ rotary + QK norm
// HD / 8 lanes share one (token, head) row of q or k: every lane owns four consecutive
// rotation pairs (p, p + HD/2), i.e. one 8-byte load from each half of the row.
__device__ __forceinline__ void unpack4(const uint2& q, float (&f)[4]) {
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q.y));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ uint2 pack4(const float (&f)[4]) {
  uint2 q;
  *reinterpret_cast<__nv_bfloat162*>(&q.x) = __floats2bfloat162_rn(f[0], f[1]);
  *reinterpret_cast<__nv_bfloat162*>(&q.y) = __floats2bfloat162_rn(f[2], f[3]);
  return q;
}
template <int LPR>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int HD>
__global__ void __launch_bounds__(256) rope_qknorm_fwd_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k,
                                                             bf16* __restrict__ qo, bf16* __restrict__ ko,
                                                             const bf16* __restrict__ cosb,
                                                             const bf16* __restrict__ sinb, long long tokens,
                                                             int seq_len, int heads, long long in_pitch,
                                                             long long out_pitch, float eps) {
  constexpr int HALF = HD / 2;
  constexpr int LPR = HD / 8;  // lanes per row
  const long long gid = (long long)blockIdx.x * 256 + threadIdx.x;
  const long long rid = gid / LPR;
  const int sub = (int)(gid - rid * LPR);
  const long long nrows = tokens * heads * (k ? 2 : 1);
  const bool live = rid < nrows;
  const long long r = live ? rid : 0;
  const int which = k ? (int)(r & 1) : 0;  // 0 = q, 1 = k
  const long long th = k ? (r >> 1) : r;
  const long long tok = th / heads;
  const int head = (int)(th - tok * heads);
  const int pos = (int)(tok % seq_len);
  const int p = sub * 4;
  const bf16* src = (which ? k : q) + tok * in_pitch + (long long)head * HD;
  float x1[4], x2[4], c[4], sn[4], y1[4], y2[4];
  unpack4(*reinterpret_cast<const uint2*>(src + p), x1);
  unpack4(*reinterpret_cast<const uint2*>(src + p + HALF), x2);
  unpack4(*reinterpret_cast<const uint2*>(cosb + (long long)pos * HALF + p), c);
  unpack4(*reinterpret_cast<const uint2*>(sinb + (long long)pos * HALF + p), sn);
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    y1[i] = x1[i] * c[i] + x2[i] * sn[i];
    y2[i] = x2[i] * c[i] - x1[i] * sn[i];
    ss += y1[i] * y1[i] + y2[i] * y2[i];
  }
  ss = group_sum<LPR>(ss);
  const float rs = eps < 0.f ? 1.f : rsqrtf(ss / (float)HD + eps);  // eps < 0: rotary only, no norm
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    y1[i] *= rs;
    y2[i] *= rs;
  }
  if (live) {
    bf16* dst = (which ? ko : qo) + tok * out_pitch + (long long)head * HD;
    *reinterpret_cast<uint2*>(dst + p) = pack4(y1);
    *reinterpret_cast<uint2*>(dst + p + HALF) = pack4(y2);
  }
}

template <int HD>
__global__ void __launch_bounds__(256) rope_qknorm_bwd_kernel(const bf16* __restrict__ dqo,
                                                             const bf16* __restrict__ dko,
                                                             const bf16* __restrict__ q, const bf16* __restrict__ k,
                                                             bf16* __restrict__ dq, bf16* __restrict__ dk,
                                                             const bf16* __restrict__ cosb,
                                                             const bf16* __restrict__ sinb, long long tokens,
                                                             int seq_len, int heads, long long in_pitch,
                                                             long long out_pitch, float eps) {
  constexpr int HALF = HD / 2;
  constexpr int LPR = HD / 8;
  const long long gid = (long long)blockIdx.x * 256 + threadIdx.x;
  const long long rid = gid / LPR;
  const int sub = (int)(gid - rid * LPR);
  const long long nrows = tokens * heads * (k ? 2 : 1);
  const bool live = rid < nrows;
  const long long r = live ? rid : 0;
  const int which = k ? (int)(r & 1) : 0;
  const long long th = k ? (r >> 1) : r;
  const long long tok = th / heads;
  const int head = (int)(th - tok * heads);
  const int pos = (int)(tok % seq_len);
  const int p = sub * 4;
  const bf16* src = (which ? k : q) + tok * in_pitch + (long long)head * HD;
  const bf16* gsrc = (which ? dko : dqo) + tok * out_pitch + (long long)head * HD;
  float x1[4], x2[4], c[4], sn[4], y1[4], y2[4], g1[4], g2[4];
  unpack4(*reinterpret_cast<const uint2*>(src + p), x1);
  unpack4(*reinterpret_cast<const uint2*>(src + p + HALF), x2);
  unpack4(*reinterpret_cast<const uint2*>(cosb + (long long)pos * HALF + p), c);
  unpack4(*reinterpret_cast<const uint2*>(sinb + (long long)pos * HALF + p), sn);
  unpack4(*reinterpret_cast<const uint2*>(gsrc + p), g1);
  unpack4(*reinterpret_cast<const uint2*>(gsrc + p + HALF), g2);
  float ss = 0.f, dot = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    y1[i] = x1[i] * c[i] + x2[i] * sn[i];
    y2[i] = x2[i] * c[i] - x1[i] * sn[i];
    ss += y1[i] * y1[i] + y2[i] * y2[i];
    dot += g1[i] * y1[i] + g2[i] * y2[i];
  }
  ss = group_sum<LPR>(ss);
  dot = group_sum<LPR>(dot);
  const float rs = eps < 0.f ? 1.f : rsqrtf(ss / (float)HD + eps);
  const float c3 = eps < 0.f ? 0.f : rs * rs * rs * dot / (float)HD;
  float o1[4], o2[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float d1 = rs * g1[i] - c3 * y1[i];  // gradient w.r.t. the rotated values
    const float d2 = rs * g2[i] - c3 * y2[i];
    o1[i] = d1 * c[i] - d2 * sn[i];
    o2[i] = d1 * sn[i] + d2 * c[i];
  }
  if (live) {
    bf16* gdst = (which ? dk : dq) + tok * in_pitch + (long long)head * HD;
    *reinterpret_cast<uint2*>(gdst + p) = pack4(o1);
    *reinterpret_cast<uint2*>(gdst + p + HALF) = pack4(o2);
  }
}

// Wide variants (every pointer 16-byte aligned, pitches multiples of 8 elements): HD / 16 lanes share one
// (token, head); a lane owns eight consecutive rotation pairs - one 16-byte load from each half of the row -
// of q AND of k, which use the same cos / sin values.  Twice the bytes per load and two independent rows per
// thread keep more of the memory system busy than the 8-byte kernel above, which stays for unaligned views.
template <int LPR>
__device__ __forceinline__ void rope_rotate_norm(const float (&x1)[8], const float (&x2)[8], const float (&c)[8],
                                                 const float (&sn)[8], float eps, int hd, float (&y1)[8],
                                                 float (&y2)[8], float& rs) {
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    y1[i] = x1[i] * c[i] + x2[i] * sn[i];
    y2[i] = x2[i] * c[i] - x1[i] * sn[i];
    ss += y1[i] * y1[i] + y2[i] * y2[i];
  }
  ss = group_sum<LPR>(ss);
  rs = eps < 0.f ? 1.f : rsqrtf(ss / (float)hd + eps);
}

template <int HD>
__global__ void __launch_bounds__(256) rope_qknorm_fwd_wide_kernel(const bf16* __restrict__ q,
                                                                  const bf16* __restrict__ k, bf16* __restrict__ qo,
                                                                  bf16* __restrict__ ko,
                                                                  const bf16* __restrict__ cosb,
                                                                  const bf16* __restrict__ sinb, long long tokens,
                                                                  int seq_len, int heads, long long in_pitch,
                                                                  long long out_pitch, float eps) {
  constexpr int HALF = HD / 2;
  constexpr int LPR = HD / 16;  // lanes per (token, head)
  const long long gid = (long long)blockIdx.x * 256 + threadIdx.x;
  const long long rid = gid / LPR;
  const int sub = (int)(gid - rid * LPR);
  const long long nrows = tokens * heads;
  const bool live = rid < nrows;  // dead lanes compute on row 0 so that the shuffles stay converged
  const long long th = live ? rid : 0;
  const long long tok = th / heads;
  const int head = (int)(th - tok * heads);
  const int pos = (int)(tok % seq_len);
  const int p = sub * 8;
  const long long in_off = tok * in_pitch + (long long)head * HD + p;
  const long long out_off = tok * out_pitch + (long long)head * HD + p;
  // all loads first
  const uint4 q1 = *reinterpret_cast<const uint4*>(q + in_off);
  const uint4 q2 = *reinterpret_cast<const uint4*>(q + in_off + HALF);
  uint4 k1 = make_uint4(0, 0, 0, 0), k2 = k1;
  if (k) {
    k1 = *reinterpret_cast<const uint4*>(k + in_off);
    k2 = *reinterpret_cast<const uint4*>(k + in_off + HALF);
  }
  const uint4 cq = *reinterpret_cast<const uint4*>(cosb + (long long)pos * HALF + p);
  const uint4 sq = *reinterpret_cast<const uint4*>(sinb + (long long)pos * HALF + p);
  float c[8], sn[8], x1[8], x2[8], y1[8], y2[8], rs;
  unpack8(cq, c);
  unpack8(sq, sn);
  unpack8(q1, x1);
  unpack8(q2, x2);
  rope_rotate_norm<LPR>(x1, x2, c, sn, eps, HD, y1, y2, rs);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    y1[i] *= rs;
    y2[i] *= rs;
  }
  if (live) {
    *reinterpret_cast<uint4*>(qo + out_off) = pack8(y1);
    *reinterpret_cast<uint4*>(qo + out_off + HALF) = pack8(y2);
  }
  if (k) {
    unpack8(k1, x1);
    unpack8(k2, x2);
    rope_rotate_norm<LPR>(x1, x2, c, sn, eps, HD, y1, y2, rs);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      y1[i] *= rs;
      y2[i] *= rs;
    }
    if (live) {
      *reinterpret_cast<uint4*>(ko + out_off) = pack8(y1);
      *reinterpret_cast<uint4*>(ko + out_off + HALF) = pack8(y2);
    }
  }
}

template <int LPR>
__device__ __forceinline__ void rope_backward_row(const uint4& xa, const uint4& xb, const uint4& ga, const uint4& gb,
                                                  const float (&c)[8], const float (&sn)[8], float eps, int hd,
                                                  uint4& oa, uint4& ob) {
  float x1[8], x2[8], g1[8], g2[8], y1[8], y2[8], rs;
  unpack8(xa, x1);
  unpack8(xb, x2);
  unpack8(ga, g1);
  unpack8(gb, g2);
  rope_rotate_norm<LPR>(x1, x2, c, sn, eps, hd, y1, y2, rs);
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) dot += g1[i] * y1[i] + g2[i] * y2[i];
  dot = group_sum<LPR>(dot);
  const float c3 = eps < 0.f ? 0.f : rs * rs * rs * dot / (float)hd;
  float o1[8], o2[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float d1 = rs * g1[i] - c3 * y1[i];  // gradient w.r.t. the rotated values
    const float d2 = rs * g2[i] - c3 * y2[i];
    o1[i] = d1 * c[i] - d2 * sn[i];
    o2[i] = d1 * sn[i] + d2 * c[i];
  }
  oa = pack8(o1);
  ob = pack8(o2);
}

template <int HD>
__global__ void __launch_bounds__(256) rope_qknorm_bwd_wide_kernel(const bf16* __restrict__ dqo,
                                                                  const bf16* __restrict__ dko,
                                                                  const bf16* __restrict__ q,
                                                                  const bf16* __restrict__ k, bf16* __restrict__ dq,
                                                                  bf16* __restrict__ dk,
                                                                  const bf16* __restrict__ cosb,
                                                                  const bf16* __restrict__ sinb, long long tokens,
                                                                  int seq_len, int heads, long long in_pitch,
                                                                  long long out_pitch, float eps) {
  constexpr int HALF = HD / 2;
  constexpr int LPR = HD / 16;
  const long long gid = (long long)blockIdx.x * 256 + threadIdx.x;
  const long long rid = gid / LPR;
  const int sub = (int)(gid - rid * LPR);
  const long long nrows = tokens * heads;
  const bool live = rid < nrows;
  const long long th = live ? rid : 0;
  const long long tok = th / heads;
  const int head = (int)(th - tok * heads);
  const int pos = (int)(tok % seq_len);
  const int p = sub * 8;
  const long long in_off = tok * in_pitch + (long long)head * HD + p;    // q, k and their gradients
  const long long out_off = tok * out_pitch + (long long)head * HD + p;  // gradients of the rotated outputs
  const uint4 q1 = *reinterpret_cast<const uint4*>(q + in_off);
  const uint4 q2 = *reinterpret_cast<const uint4*>(q + in_off + HALF);
  const uint4 gq1 = *reinterpret_cast<const uint4*>(dqo + out_off);
  const uint4 gq2 = *reinterpret_cast<const uint4*>(dqo + out_off + HALF);
  uint4 k1 = make_uint4(0, 0, 0, 0), k2 = k1, gk1 = k1, gk2 = k1;
  if (k) {
    k1 = *reinterpret_cast<const uint4*>(k + in_off);
    k2 = *reinterpret_cast<const uint4*>(k + in_off + HALF);
    gk1 = *reinterpret_cast<const uint4*>(dko + out_off);
    gk2 = *reinterpret_cast<const uint4*>(dko + out_off + HALF);
  }
  float c[8], sn[8];
  unpack8(*reinterpret_cast<const uint4*>(cosb + (long long)pos * HALF + p), c);
  unpack8(*reinterpret_cast<const uint4*>(sinb + (long long)pos * HALF + p), sn);
  uint4 oa, ob;
  rope_backward_row<LPR>(q1, q2, gq1, gq2, c, sn, eps, HD, oa, ob);
  if (live) {
    *reinterpret_cast<uint4*>(dq + in_off) = oa;
    *reinterpret_cast<uint4*>(dq + in_off + HALF) = ob;
  }
  if (k) {
    rope_backward_row<LPR>(k1, k2, gk1, gk2, c, sn, eps, HD, oa, ob);
    if (live) {
      *reinterpret_cast<uint4*>(dk + in_off) = oa;
      *reinterpret_cast<uint4*>(dk + in_off + HALF) = ob;
    }
  }
}

// ------------------------------------------------------------------ ReLU^2
__global__ void __launch_bounds__(256) relu2_fwd_kernel(const uint4* __restrict__ x, uint4* __restrict__ h,
                                                       long long nvec) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= nvec) return;
  float f[8];
  unpack8(x[i], f);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float r = fmaxf(f[j], 0.f);
    f[j] = r * r;
  }
  h[i] = pack8(f);
}
__global__ void __launch_bounds__(256) relu2_bwd_kernel(const uint4* __restrict__ dh, const uint4* __restrict__ x,
                                                       uint4* __restrict__ dx, long long nvec) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= nvec) return;
  float f[8], g[8];
  unpack8(x[i], f);
  unpack8(dh[i], g);
#pragma unroll
  for (int j = 0; j < 8; ++j) g[j] = g[j] * 2.f * fmaxf(f[j], 0.f);
  dx[i] = pack8(g);
}

// ------------------------------------------------------------------ cross entropy
// One 256-thread block per row.  Pass 1 streams the bf16 row once and keeps an online
// (max, sum-exp) pair per thread; pass 2 re-reads the row and writes the gradient in place.  Nothing
// is kept in registers, so any vocabulary size works and eight rows are resident per SM.  For
// 50304-wide rows the second read mostly comes from DRAM again (1.4x the algorithmic traffic); a
// variant that kept the row in shared memory instead was slower, because with two exponentials per
// element the kernel is bound as much by the special-function unit as by DRAM and needs many small
// blocks per SM to overlap the two.
constexpr int kCeThreads = 256;

__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
  const float mx = fmaxf(m, m2);
  if (mx == -INFINITY) {
    s = 0.f;
  } else {
    s = s * __expf(m - mx) + s2 * __expf(m2 - mx);
  }
  m = mx;
}

__global__ void __launch_bounds__(kCeThreads) cross_entropy_kernel(bf16* __restrict__ logits,
                                                                  const long long* __restrict__ targets,
                                                                  float* __restrict__ row_loss,
                                                                  const float* __restrict__ scale_ptr,
                                                                  int vocab, long long pitch, float grad_scale,
                                                                  long long ignore_index, int write_grad) {
  __shared__ float red_m[kCeThreads / 32], red_s[kCeThreads / 32];
  const long long row = blockIdx.x;
  const long long tgt = targets[row];
  uint4* lr = reinterpret_cast<uint4*>(logits + row * pitch);
  const int nvec = vocab >> 3;
  if (tgt == ignore_index) {
    if (threadIdx.x == 0) row_loss[row] = 0.f;
    if (write_grad) {
      const uint4 z = make_uint4(0, 0, 0, 0);
      for (int v = threadIdx.x; v < nvec; v += kCeThreads) lr[v] = z;
    }
    return;
  }
  // pass 1: online softmax statistics
  float m = -INFINITY, ssum = 0.f;
  for (int v = threadIdx.x; v < nvec; v += kCeThreads) {
    float f[8];
    unpack8(lr[v], f);
    float mv = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) mv = fmaxf(mv, f[j]);
    const float mx = fmaxf(m, mv);
    float acc = ssum * __expf(m - mx);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += __expf(f[j] - mx);
    ssum = acc;
    m = mx;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    const float s2 = __shfl_xor_sync(0xffffffffu, ssum, o);
    online_merge(m, ssum, m2, s2);
  }
  if ((threadIdx.x & 31) == 0) {
    red_m[threadIdx.x >> 5] = m;
    red_s[threadIdx.x >> 5] = ssum;
  }
  __syncthreads();
  m = red_m[0];
  ssum = red_s[0];
#pragma unroll
  for (int w = 1; w < kCeThreads / 32; ++w) online_merge(m, ssum, red_m[w], red_s[w]);
  const float tl = __bfloat162float(logits[row * pitch + tgt]);
  if (threadIdx.x == 0) row_loss[row] = m + __logf(ssum) - tl;
  if (!write_grad) return;
  __syncthreads();  // every thread has read the target logit before the row is overwritten
  // pass 2: gradient, in place
  const float gs = grad_scale * (scale_ptr ? *scale_ptr : 1.f);
  const float inv = gs / ssum;
  const int tv = (int)(tgt >> 3), tj = (int)(tgt & 7);
  for (int v = threadIdx.x; v < nvec; v += kCeThreads) {
    float f[8];
    unpack8(lr[v], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = __expf(f[j] - m) * inv;
    if (v == tv) f[tj] -= gs;
    lr[v] = pack8(f);
  }
}

// ------------------------------------------------------------------ embedding
__global__ void __launch_bounds__(256) embedding_fwd_kernel(const void* __restrict__ table, int table_type,
                                                           const long long* __restrict__ idx, bf16* __restrict__ out,
                                                           long long tokens, int dim) {
  const long long tok = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (tok >= tokens) return;
  const int lane = threadIdx.x & 31;
  const long long id = idx[tok];
  bf16* o = out + tok * dim;
  if (table_type == kElemF32) {
    const float* t = reinterpret_cast<const float*>(table) + id * dim;
    for (int c = lane * 4; c < dim; c += 128) {
      const float4 f = *reinterpret_cast<const float4*>(t + c);
      uint2 q;
      *reinterpret_cast<__nv_bfloat162*>(&q.x) = __floats2bfloat162_rn(f.x, f.y);
      *reinterpret_cast<__nv_bfloat162*>(&q.y) = __floats2bfloat162_rn(f.z, f.w);
      *reinterpret_cast<uint2*>(o + c) = q;
    }
  } else {
    const bf16* t = reinterpret_cast<const bf16*>(table) + id * dim;
    for (int c = lane * 8; c < dim; c += 256) *reinterpret_cast<uint4*>(o + c) = *reinterpret_cast<const uint4*>(t + c);
  }
}

__global__ void __launch_bounds__(256) embedding_bwd_kernel(const bf16* __restrict__ dout,
                                                           const long long* __restrict__ idx,
                                                           float* __restrict__ dtable, long long tokens, int dim) {
  const long long tok = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (tok >= tokens) return;
  const int lane = threadIdx.x & 31;
  const long long id = idx[tok];
  const bf16* g = dout + tok * dim;
  float* t = dtable + id * dim;
  for (int c = lane * 2; c < dim; c += 64) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(g + c));
    atomicAdd(t + c, f.x);
    atomicAdd(t + c + 1, f.y);
  }
}

}  // namespace

cudaError_t rmsnorm_fwd_launch(const void* x, const void* residual, void* x_out, void* y, float* rstd,
                               long long rows, int dim, float eps, cudaStream_t s) {
  if (rows == 0) return cudaSuccess;
  if (dim % 8 != 0 || dim > kNormMaxVec * 256) return cudaErrorInvalidValue;
  const unsigned grid = (unsigned)((rows + 7) / 8);
#define DION_NORM_FWD(V)                                                                                          \
  rmsnorm_fwd_kernel<V><<<grid, 256, 0, s>>>(reinterpret_cast<const bf16*>(x), reinterpret_cast<const bf16*>(residual), \
                                             reinterpret_cast<bf16*>(x_out), reinterpret_cast<bf16*>(y), rstd, rows, \
                                             dim, eps)
  if (dim <= 4 * 256) DION_NORM_FWD(4);
  else if (dim <= 8 * 256) DION_NORM_FWD(8);
  else DION_NORM_FWD(16);
#undef DION_NORM_FWD
  return cudaGetLastError();
}
cudaError_t rmsnorm_bwd_launch(const void* dy, const void* x, const float* rstd, const void* dx_add, void* dx,
                               long long rows, int dim, cudaStream_t s) {
  if (rows == 0) return cudaSuccess;
  if (dim % 8 != 0 || dim > kNormMaxVec * 256) return cudaErrorInvalidValue;
  const unsigned grid = (unsigned)((rows + 7) / 8);
#define DION_NORM_BWD(V)                                                                                          \
  rmsnorm_bwd_kernel<V><<<grid, 256, 0, s>>>(reinterpret_cast<const bf16*>(dy), reinterpret_cast<const bf16*>(x), rstd, \
                                             reinterpret_cast<const bf16*>(dx_add), reinterpret_cast<bf16*>(dx), rows, dim)
  if (dim <= 4 * 256) DION_NORM_BWD(4);
  else if (dim <= 8 * 256) DION_NORM_BWD(8);
  else DION_NORM_BWD(16);
#undef DION_NORM_BWD
  return cudaGetLastError();
}

// 16-byte accesses need every base pointer on a 16-byte boundary and pitches that keep it there
static bool rope_wide_ok(std::initializer_list<const void*> ptrs, long long in_pitch, long long out_pitch) {
  static const bool enabled = [] {  // DION_B200_ROPE_WIDE=0 keeps the 8-byte kernels
    const char* e = getenv("DION_B200_ROPE_WIDE");
    return !(e && e[0] == '0');
  }();
  if (!enabled) return false;
  for (const void* p : ptrs)
    if (reinterpret_cast<uintptr_t>(p) & 15) return false;
  return in_pitch % 8 == 0 && out_pitch % 8 == 0;
}

cudaError_t rope_qknorm_fwd_launch(const void* q, const void* k, void* q_out, void* k_out, const void* cos,
                                   const void* sin, long long tokens, int seq_len, int heads, int head_dim,
                                   long long in_pitch, long long out_pitch, float eps, cudaStream_t s) {
  const long long nrows = tokens * heads * (k ? 2 : 1);
  if (nrows == 0) return cudaSuccess;
  if (in_pitch % 4 != 0 || out_pitch % 4 != 0) return cudaErrorInvalidValue;
  if (head_dim != 64 && head_dim != 128) return cudaErrorInvalidValue;
  const bool wide = rope_wide_ok({q, k, q_out, k_out, cos, sin}, in_pitch, out_pitch);
  const unsigned grid = wide ? (unsigned)((tokens * heads * (head_dim / 16) + 255) / 256)
                             : (unsigned)((nrows * (head_dim / 8) + 255) / 256);
#define DION_ROPE_FWD(KERNEL, HD)                                                                                 \
  KERNEL<HD><<<grid, 256, 0, s>>>(                                                                                \
      reinterpret_cast<const bf16*>(q), reinterpret_cast<const bf16*>(k), reinterpret_cast<bf16*>(q_out),         \
      reinterpret_cast<bf16*>(k_out), reinterpret_cast<const bf16*>(cos), reinterpret_cast<const bf16*>(sin),     \
      tokens, seq_len, heads, in_pitch, out_pitch, eps)
  if (wide) {
    if (head_dim == 64) DION_ROPE_FWD(rope_qknorm_fwd_wide_kernel, 64);
    else DION_ROPE_FWD(rope_qknorm_fwd_wide_kernel, 128);
  } else {
    if (head_dim == 64) DION_ROPE_FWD(rope_qknorm_fwd_kernel, 64);
    else DION_ROPE_FWD(rope_qknorm_fwd_kernel, 128);
  }
#undef DION_ROPE_FWD
  return cudaGetLastError();
}
cudaError_t rope_qknorm_bwd_launch(const void* dq_out, const void* dk_out, const void* q, const void* k, void* dq,
                                   void* dk, const void* cos, const void* sin, long long tokens, int seq_len,
                                   int heads, int head_dim, long long in_pitch, long long out_pitch, float eps,
                                   cudaStream_t s) {
  const long long nrows = tokens * heads * (k ? 2 : 1);
  if (nrows == 0) return cudaSuccess;
  if (in_pitch % 4 != 0 || out_pitch % 4 != 0) return cudaErrorInvalidValue;
  if (head_dim != 64 && head_dim != 128) return cudaErrorInvalidValue;
  const bool wide = rope_wide_ok({dq_out, dk_out, q, k, dq, dk, cos, sin}, in_pitch, out_pitch);
  const unsigned grid = wide ? (unsigned)((tokens * heads * (head_dim / 16) + 255) / 256)
                             : (unsigned)((nrows * (head_dim / 8) + 255) / 256);
#define DION_ROPE_BWD(KERNEL, HD)                                                                                 \
  KERNEL<HD><<<grid, 256, 0, s>>>(                                                                                \
      reinterpret_cast<const bf16*>(dq_out), reinterpret_cast<const bf16*>(dk_out),                               \
      reinterpret_cast<const bf16*>(q), reinterpret_cast<const bf16*>(k), reinterpret_cast<bf16*>(dq),            \
      reinterpret_cast<bf16*>(dk), reinterpret_cast<const bf16*>(cos), reinterpret_cast<const bf16*>(sin),        \
      tokens, seq_len, heads, in_pitch, out_pitch, eps)
  if (wide) {
    if (head_dim == 64) DION_ROPE_BWD(rope_qknorm_bwd_wide_kernel, 64);
    else DION_ROPE_BWD(rope_qknorm_bwd_wide_kernel, 128);
  } else {
    if (head_dim == 64) DION_ROPE_BWD(rope_qknorm_bwd_kernel, 64);
    else DION_ROPE_BWD(rope_qknorm_bwd_kernel, 128);
  }
#undef DION_ROPE_BWD
  return cudaGetLastError();
}

cudaError_t relu2_fwd_launch(const void* x, void* h, long long n, cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  if (n % 8 != 0) return cudaErrorInvalidValue;
  const long long nvec = n / 8;
  relu2_fwd_kernel<<<(unsigned)((nvec + 255) / 256), 256, 0, s>>>(reinterpret_cast<const uint4*>(x),
                                                                 reinterpret_cast<uint4*>(h), nvec);
  return cudaGetLastError();
}
cudaError_t relu2_bwd_launch(const void* dh, const void* x, void* dx, long long n, cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  if (n % 8 != 0) return cudaErrorInvalidValue;
  const long long nvec = n / 8;
  relu2_bwd_kernel<<<(unsigned)((nvec + 255) / 256), 256, 0, s>>>(
      reinterpret_cast<const uint4*>(dh), reinterpret_cast<const uint4*>(x), reinterpret_cast<uint4*>(dx), nvec);
  return cudaGetLastError();
}

cudaError_t cross_entropy_fwd_bwd_launch(void* logits, const long long* targets, float* row_loss,
                                         const float* scale_ptr, long long rows, int vocab, long long pitch,
                                         float grad_scale, long long ignore_index, bool write_grad, cudaStream_t s) {
  if (rows == 0) return cudaSuccess;
  if (vocab % 8 != 0 || pitch % 8 != 0) return cudaErrorInvalidValue;
  cross_entropy_kernel<<<(unsigned)rows, kCeThreads, 0, s>>>(reinterpret_cast<bf16*>(logits), targets, row_loss,
                                                            scale_ptr, vocab, pitch, grad_scale, ignore_index,
                                                            write_grad ? 1 : 0);
  return cudaGetLastError();
}

cudaError_t embedding_fwd_launch(const void* table, int table_type, const long long* idx, void* out,
                                 long long tokens, int dim, cudaStream_t s) {
  if (tokens == 0) return cudaSuccess;
  if (dim % 8 != 0) return cudaErrorInvalidValue;
  embedding_fwd_kernel<<<(unsigned)((tokens + 7) / 8), 256, 0, s>>>(table, table_type, idx,
                                                                   reinterpret_cast<bf16*>(out), tokens, dim);
  return cudaGetLastError();
}
cudaError_t embedding_bwd_launch(const void* dout, const long long* idx, float* dtable, long long tokens, int dim,
                                 cudaStream_t s) {
  if (tokens == 0) return cudaSuccess;
  if (dim % 2 != 0) return cudaErrorInvalidValue;
  embedding_bwd_kernel<<<(unsigned)((tokens + 7) / 8), 256, 0, s>>>(reinterpret_cast<const bf16*>(dout), idx, dtable,
                                                                   tokens, dim);
  return cudaGetLastError();
}

}  // namespace dion
