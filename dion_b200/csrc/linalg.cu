// Small dense factorizations that the Dion orthonormalisation needs, one CTA per
// matrix, fp32 throughout.
//
// chol_inverse: for a symmetric positive semi-definite Gram matrix G = P^T P it
// produces Z = L^{-1} with G ~= L L^T, after a Jacobi (unit-diagonal) scaling of G,
// so that P * Z^T has orthonormal columns.  It is the device-side replacement for the
// cuSOLVER geqrf / potrf + cuBLAS trsm sequence of the reference
// (dion/dion.py:1284-1303, 1366-1406).  A pivot that is not safely positive is
// replaced by 1 and its column eliminates nothing (the column is treated as dependent on the earlier
// ones) instead of failing; the count of such pivots is reported per matrix.
//
// Algorithm (right-looking, block size NB): per block column k
//   1. factor the NB x NB diagonal block in shared memory, invert it (Linv)
//   2. Z[k,:]   = Linv * B[k,:]                (B starts as the identity)
//   3. panel    = A[k+1:, k] * Linv^T          (kept transposed in shared memory)
//   4. A[k+1:, k+1:] -= panel * panel^T        (lower triangle, 64x64 register tiles)
//      B[k+1:, :]    -= panel * Z[k,:]
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "kernels.h"
#include "umma.cuh"

namespace dion {

namespace {

constexpr int kCholThreads = 1024;  // four 256-thread groups, each updating its own 64 x 64 tile

// out[row0 + i][col0 + j] -= sum_a At[a][i] * Bt[a][j]   for a 64 x 64 tile; each of the
// 256 threads owns a 4 x 4 sub-tile.  At / Bt are shared-memory arrays indexed [a][.]
// whose rows are 16-byte aligned and the offsets multiples of 4.
template <int NB>
__device__ __forceinline__ void tile_update(float* __restrict__ out, long long ld, int row0, int col0,
                                            const float* __restrict__ At, int a_stride,
                                            const float* __restrict__ Bt, int b_stride, int row_end, int col_end) {
  const int t = threadIdx.x & 255;
  const int ty = t >> 4, tx = t & 15;
  const int i0 = ty * 4, j0 = tx * 4;
  const bool vec = (col0 + j0 + 3 < col_end) && ((ld & 3) == 0);
  // fetch the output tile first so that its latency hides behind the multiply loop
  float4 cur[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = row0 + i0 + i;
    cur[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < row_end && vec) cur[i] = *reinterpret_cast<const float4*>(out + (long long)r * ld + col0 + j0);
  }
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
#pragma unroll 8
  for (int a = 0; a < NB; ++a) {
    const float4 av = *reinterpret_cast<const float4*>(At + (long long)a * a_stride + i0);
    const float4 bv = *reinterpret_cast<const float4*>(Bt + (long long)a * b_stride + j0);
    const float ar[4] = {av.x, av.y, av.z, av.w};
    const float br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = row0 + i0 + i;
    if (r >= row_end) continue;
    float* o = out + (long long)r * ld + col0 + j0;
    if (vec) {
      float4 v = cur[i];
      v.x -= acc[i][0];
      v.y -= acc[i][1];
      v.z -= acc[i][2];
      v.w -= acc[i][3];
      *reinterpret_cast<float4*>(o) = v;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (col0 + j0 + j < col_end) o[j] -= acc[i][j];
    }
  }
}

template <int NB>
__global__ void __launch_bounds__(kCholThreads, 1)
chol_inverse_kernel(const float* __restrict__ Gall, float* __restrict__ Zall, float* __restrict__ Wall,
                    int* __restrict__ info, int r, long long ldg, long long g_batch_stride, int rp,
                    float pivot_floor, int jacobi, float* __restrict__ colmask) {
  extern __shared__ __align__(16) float sm[];
  // rp = r rounded up to a multiple of 64 (+4 pad keeps rows 16-byte aligned)
  float* panelT = sm;                         // [NB][rp]   panel, transposed
  float* zrow = panelT + (size_t)NB * rp;     // [NB][rp]   current block row of Z
  float* dblk = zrow + (size_t)NB * rp;       // [NB][NB+1]
  float* linv = dblk + NB * (NB + 1);         // [NB][NB+1]
  float* dscale = linv + NB * (NB + 1);       // [rp] Jacobi scaling 1/sqrt(G_ii)
  int& clamp_count = *reinterpret_cast<int*>(dscale + rp);

  const int b = blockIdx.x;
  const float* G = Gall + (long long)b * g_batch_stride;
  float* Z = Zall + (long long)b * r * r;
  float* W = Wall + (long long)b * r * r;
  const int tid = threadIdx.x;

  if (tid == 0) clamp_count = 0;
  for (int i = tid; i < rp; i += kCholThreads) {
    float d = 0.f;
    if (i < r) {
      const float g = G[(long long)i * ldg + i];
      d = !jacobi ? 1.f : ((g > 1e-30f) ? rsqrtf(g) : 0.f);
    }
    dscale[i] = d;
  }
  __syncthreads();
  // W = D G D (lower triangle is what gets used), Z = I
  for (long long e = tid; e < (long long)r * r; e += kCholThreads) {
    const int i = (int)(e / r), j = (int)(e - (long long)i * r);
    W[e] = G[(long long)i * ldg + j] * dscale[i] * dscale[j];
    Z[e] = (i == j) ? 1.f : 0.f;
  }
  __syncthreads();

  for (int k0 = 0; k0 < r; k0 += NB) {
    const int nb = min(NB, r - k0);
    // ---- 1. diagonal block -> shared, unblocked Cholesky with pivot clamping
    for (int e = tid; e < NB * NB; e += kCholThreads) {
      const int i = e / NB, j = e - i * NB;
      float v = 0.f;
      if (i < nb && j < nb && j <= i) v = W[(long long)(k0 + i) * r + k0 + j];
      dblk[i * (NB + 1) + j] = v;
    }
    __syncthreads();
    for (int j = 0; j < nb; ++j) {
      if (tid == 0) {
        const float d = dblk[j * (NB + 1) + j];
        if (!(d > pivot_floor)) {
          ++clamp_count;
          dblk[j * (NB + 1) + j] = -1.f;  // marks the column for the other threads, replaced by 1 below
        } else {
          dblk[j * (NB + 1) + j] = sqrtf(d);
        }
        if (colmask) colmask[(long long)b * r + k0 + j] = (d > pivot_floor) ? 1.f : 0.f;
      }
      __syncthreads();
      const float piv = dblk[j * (NB + 1) + j];
      // a pivot that is not safely positive belongs to a column that depends on the earlier ones: it
      // gets a unit pivot and eliminates nothing, so that rounding noise is never divided by a tiny number
      const bool bad = piv < 0.f;
      for (int i = j + 1 + tid; i < nb; i += kCholThreads)
        dblk[i * (NB + 1) + j] = bad ? 0.f : dblk[i * (NB + 1) + j] / piv;
      __syncthreads();
      if (bad && tid == 0) dblk[j * (NB + 1) + j] = 1.f;
      // rank-1 update of the remaining lower triangle
      const int rem = nb - j - 1;
      for (int e = tid; e < rem * rem; e += kCholThreads) {
        const int ii = e / rem, jj = e - ii * rem;
        if (jj <= ii) {
          const int i = j + 1 + ii, c = j + 1 + jj;
          dblk[i * (NB + 1) + c] -= dblk[i * (NB + 1) + j] * dblk[c * (NB + 1) + j];
        }
      }
      __syncthreads();
    }
    // ---- inverse of the diagonal factor: column c of Linv by forward substitution
    for (int e = tid; e < NB * (NB + 1); e += kCholThreads) linv[e] = 0.f;
    __syncthreads();
    if (tid < nb) {
      const int c = tid;
      for (int i = c; i < nb; ++i) {
        float s = (i == c) ? 1.f : 0.f;
        for (int k = c; k < i; ++k) s -= dblk[i * (NB + 1) + k] * linv[k * (NB + 1) + c];
        linv[i * (NB + 1) + c] = s / dblk[i * (NB + 1) + i];
      }
    }
    __syncthreads();

    // ---- 2. Z[k,:] = Linv * B[k,:] for columns < k0 + nb
    const int zc = k0 + nb;
    for (int c = tid; c < rp; c += kCholThreads) {
      float bcol[NB];
#pragma unroll
      for (int a = 0; a < NB; ++a) bcol[a] = (a < nb && c < zc) ? Z[(long long)(k0 + a) * r + c] : 0.f;
#pragma unroll
      for (int a = 0; a < NB; ++a) {
        float s = 0.f;
#pragma unroll
        for (int bb = 0; bb < NB; ++bb)
          if (bb <= a) s = fmaf(linv[a * (NB + 1) + bb], bcol[bb], s);
        zrow[(size_t)a * rp + c] = s;
        if (a < nb && c < zc) Z[(long long)(k0 + a) * r + c] = s;
      }
    }
    // ---- 3. panel = A[k+1:, k] * Linv^T, stored transposed: panelT[a][i - p0]
    const int p0 = k0 + nb;  // first trailing row
    const int tr = r - p0;   // trailing rows
    for (int ii = tid; ii < rp; ii += kCholThreads) {
      float arow[NB];
      const bool live = ii < tr;
#pragma unroll
      for (int a = 0; a < NB; ++a) arow[a] = (live && a < nb) ? W[(long long)(p0 + ii) * r + k0 + a] : 0.f;
#pragma unroll
      for (int a = 0; a < NB; ++a) {
        float s = 0.f;
#pragma unroll
        for (int bb = 0; bb < NB; ++bb)
          if (bb <= a) s = fmaf(arow[bb], linv[a * (NB + 1) + bb], s);
        panelT[(size_t)a * rp + ii] = s;
      }
    }
    __syncthreads();
    if (tr <= 0) break;

    // ---- 4. trailing updates with 64 x 64 tiles, one tile per 256-thread group at a time:
    //         first the lower-triangular tiles of the Gram part, then the right-hand side
    const int nt = (tr + 63) / 64;
    const int nc = (zc + 63) / 64;
    const int gram_tiles = nt * (nt + 1) / 2;
    const int total_tiles = gram_tiles + nt * nc;
    for (int idx = tid >> 8; idx < total_tiles; idx += kCholThreads / 256) {
      if (idx < gram_tiles) {
        int ti = 0, rem = idx;
        while (rem > ti) {  // row ti of the lower triangle holds ti + 1 tiles
          rem -= ti + 1;
          ++ti;
        }
        const int tj = rem;
        tile_update<NB>(W, r, p0 + ti * 64, p0 + tj * 64, panelT + ti * 64, rp, panelT + tj * 64, rp, r, r);
      } else {
        const int q = idx - gram_tiles;
        const int ti = q / nc, tc = q - ti * nc;
        tile_update<NB>(Z, r, p0 + ti * 64, tc * 64, panelT + ti * 64, rp, zrow + tc * 64, rp, r, zc);
      }
    }
    __syncthreads();
  }

  // undo the Jacobi scaling: G = D^-1 L' L'^T D^-1  =>  L^{-1} = L'^{-1} D, i.e. scale column j by d_j
  __syncthreads();
  for (long long e = tid; e < (long long)r * r; e += kCholThreads) {
    const int i = (int)(e / r), j = (int)(e - (long long)i * r);
    Z[e] = (j <= i) ? Z[e] * dscale[j] : 0.f;
  }
  if (tid == 0 && info) info[b] = clamp_count;
}

// One block per (batch, 32 columns): out[b][j] = sum_i X[b][i][j]^2
__global__ void __launch_bounds__(256) col_sumsq_kernel(const void* __restrict__ X, int x_type,
                                                       float* __restrict__ out, long long rows, int cols,
                                                       long long ldx, long long batch_stride) {
  __shared__ float red[8][33];
  const int b = blockIdx.y;
  const int col = blockIdx.x * 32 + (threadIdx.x & 31);
  const int rlane = threadIdx.x >> 5;  // 8 row lanes
  float s = 0.f;
  if (col < cols) {
    if (x_type == kElemF32) {
      const float* x = reinterpret_cast<const float*>(X) + (long long)b * batch_stride;
      for (long long i = rlane; i < rows; i += 8) {
        const float v = x[i * ldx + col];
        s = fmaf(v, v, s);
      }
    } else {
      const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(X) + (long long)b * batch_stride;
      for (long long i = rlane; i < rows; i += 8) {
        const float v = __bfloat162float(x[i * ldx + col]);
        s = fmaf(v, v, s);
      }
    }
  }
  red[rlane][threadIdx.x & 31] = s;
  __syncthreads();
  if (rlane == 0 && col < cols) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += red[k][threadIdx.x & 31];
    out[(long long)b * cols + col] = t;
  }
}

// ---------------------------------------------------------------------------------------------
// Second-generation kernel: the same algorithm run by a cluster of two CTAs per matrix, so that
// 72 matrices occupy 144 SMs instead of 72.  Both CTAs factor the diagonal block and build the
// panel / block row redundantly (a few percent of the work, warp-synchronous in registers for the
// 32 x 32 factorisation), then share the trailing 128 x 128 tiles, each 256-thread group
// computing one tile with 8 x 8 register sub-tiles; a cluster barrier (release / acquire) ends
// every block step so that each CTA sees the other's updates of W and Z in global memory.
constexpr int kChol2Threads = 512;

__device__ __forceinline__ uint32_t chol_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void chol_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// out[row0 + i][col0 + j] -= sum_a At[a][i] * Bt[a][j] for a 128 x 128 tile; thread t of the
// 256-thread group owns rows {4 ty .. 4 ty + 3} and {64 + 4 ty ..}, columns likewise with tx.
template <int NB>
__device__ __forceinline__ void tile_update128(float* __restrict__ out, long long ld, int row0, int col0,
                                               const float* __restrict__ At, int a_stride,
                                               const float* __restrict__ Bt, int b_stride, int row_end,
                                               int col_end, int t) {
  const int ty = t >> 4, tx = t & 15;
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
  const float* ap = At + ty * 4;
  const float* bp = Bt + tx * 4;
#pragma unroll 4
  for (int a = 0; a < NB; ++a) {
    const float4 a0 = *reinterpret_cast<const float4*>(ap + (long long)a * a_stride);
    const float4 a1 = *reinterpret_cast<const float4*>(ap + (long long)a * a_stride + 64);
    const float4 b0 = *reinterpret_cast<const float4*>(bp + (long long)a * b_stride);
    const float4 b1 = *reinterpret_cast<const float4*>(bp + (long long)a * b_stride + 64);
    const float ar[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    const float br[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
  }
  const bool ld_vec = (ld & 3) == 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = row0 + (i >> 2) * 64 + ty * 4 + (i & 3);
    if (r >= row_end) continue;
#pragma unroll
    for (int jh = 0; jh < 2; ++jh) {
      const int c = col0 + jh * 64 + tx * 4;
      float* o = out + (long long)r * ld + c;
      if (ld_vec && c + 3 < col_end) {
        float4 v = *reinterpret_cast<const float4*>(o);
        v.x -= acc[i][jh * 4 + 0];
        v.y -= acc[i][jh * 4 + 1];
        v.z -= acc[i][jh * 4 + 2];
        v.w -= acc[i][jh * 4 + 3];
        *reinterpret_cast<float4*>(o) = v;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (c + j < col_end) o[j] -= acc[i][jh * 4 + j];
      }
    }
  }
}

// Cholesky factor L of the NB x NB block in `dblk` (lower triangle, row pitch NB + 1) and its
// inverse, written to `linv` (pitch NB + 1) and `linv_al` (pitch NB, rows 16-byte aligned), upper
// parts zero.  One warp, lane i owns row i of the block and of the right-hand side in registers;
// rows >= nb are treated as rows of the identity.  Column step j (a rolled loop, so that this
// single-warp code is not bound by instruction fetch; everything indexed by a column c inside
// it is unrolled to keep the rows in registers):
//   L[:, j] = A[:, j] / sqrt(A_jj);  A[i, c] -= L[i, j] L[c, j]  (c > j)
//   X[j, :] /= L_jj;                 X[i, :] -= L[i, j] X[j, :]  (i > j), X starting as I
// Returns the number of clamped pivots (valid in every lane).
template <int NB>
__device__ __forceinline__ int warp_factor_block(const float* dblk, float* linv, float* linv_al, int nb,
                                                 float pivot_floor, int lane, float* colmask) {
  static_assert(NB <= 32, "one lane per row");
  constexpr int P = NB + 1;
  float a[NB], x[NB];
#pragma unroll
  for (int c = 0; c < NB; ++c) {
    float v = (c == lane) ? 1.f : 0.f;
    if (lane < nb && c < nb) v = dblk[lane * P + c];
    a[c] = v;
    x[c] = (c == lane) ? 1.f : 0.f;
  }
  int clamped = 0;
#pragma unroll 1
  for (int j = 0; j < NB; ++j) {
    float aj = 0.f;  // A[lane][j]
#pragma unroll
    for (int c = 0; c < NB; ++c) aj = (c == j) ? a[c] : aj;
    const float d = __shfl_sync(0xffffffffu, aj, j);
    // a pivot that is not safely positive belongs to a column that depends on the earlier ones: it gets
    // a unit pivot and eliminates nothing, so that rounding noise is never divided by a tiny number
    const bool bad = !(d > pivot_floor);
    if (bad && j < nb) ++clamped;
    if (colmask != nullptr && lane == 0 && j < nb) colmask[j] = bad ? 0.f : 1.f;
    const float inv_s = bad ? 1.f : rsqrtf(d);
    const float l = (lane > j && !bad) ? aj * inv_s : 0.f;  // L[lane][j] below the diagonal
#pragma unroll
    for (int c = 0; c < NB; ++c) {
      const float lc = __shfl_sync(0xffffffffu, l, c);
      if (c > j && lane >= c) a[c] = fmaf(-l, lc, a[c]);
      const float xs = (lane == j) ? x[c] * inv_s : x[c];
      const float xj = __shfl_sync(0xffffffffu, xs, j);
      x[c] = (lane > j) ? fmaf(-l, xj, xs) : xs;
    }
  }
  if (lane < NB) {
#pragma unroll
    for (int c = 0; c < NB; ++c) {
      const float v = (c <= lane) ? x[c] : 0.f;
      linv[lane * P + c] = v;
      linv_al[lane * NB + c] = v;
    }
  }
  return clamped;
}

template <int NB>
__global__ void __launch_bounds__(kChol2Threads, 1)
chol_inverse_pair_kernel(const float* __restrict__ Gall, float* __restrict__ Zall, float* __restrict__ Wall,
                         int* __restrict__ info, int r, long long ldg, long long g_batch_stride, int rp,
                         float pivot_floor, int jacobi, float* __restrict__ colmask) {
  extern __shared__ __align__(16) float sm[];
  // rp = r rounded up to a multiple of 128
  float* panelT = sm;                         // [NB][rp]   panel, transposed
  float* zrow = panelT + (size_t)NB * rp;     // [NB][rp]   current block row of Z
  float* dblk = zrow + (size_t)NB * rp;       // [NB][NB+1]
  float* linv = dblk + NB * (NB + 1);         // [NB][NB+1]
  float* linv_al = linv + NB * (NB + 1);      // [NB][NB], rows 16-byte aligned (NB * (NB + 1) is a multiple of 4)
  float* dscale = linv_al + NB * NB;          // [rp] Jacobi scaling 1/sqrt(G_ii)

  const int cta = (int)chol_cluster_rank();
  const int b = blockIdx.x >> 1;
  const float* G = Gall + (long long)b * g_batch_stride;
  float* Z = Zall + (long long)b * r * r;
  float* W = Wall + (long long)b * r * r;
  const int tid = threadIdx.x;
  int clamp_count = 0;  // meaningful in warp 0

  for (int i = tid; i < rp; i += kChol2Threads) {
    float d = 0.f;
    if (i < r) {
      const float g = G[(long long)i * ldg + i];
      d = !jacobi ? 1.f : ((g > 1e-30f) ? rsqrtf(g) : 0.f);
    }
    dscale[i] = d;
  }
  __syncthreads();
  // W = D G D (lower triangle is what gets used), Z = I; the two CTAs take alternate rows
  for (int i = cta; i < r; i += 2) {
    const float di = dscale[i];
    for (int j = tid; j < r; j += kChol2Threads) {
      W[(long long)i * r + j] = G[(long long)i * ldg + j] * di * dscale[j];
      Z[(long long)i * r + j] = (i == j) ? 1.f : 0.f;
    }
  }
  chol_cluster_sync();

  // debug build: the padded rank covers the rank and the shared-memory layout was sized for it
  if (!DION_DBG_OK(rp >= r && (rp & 127) == 0 && r > 0, nullptr)) return;
  for (int k0 = 0; k0 < r; k0 += NB) {
    const int nb = min(NB, r - k0);
    // ---- 1. diagonal block -> shared, factor and invert it in warp 0
    for (int e = tid; e < NB * NB; e += kChol2Threads) {
      const int i = e / NB, j = e - i * NB;
      float v = 0.f;
      if (i < nb && j < nb && j <= i) v = W[(long long)(k0 + i) * r + k0 + j];
      dblk[i * (NB + 1) + j] = v;
    }
    __syncthreads();
    if (tid < 32)
      clamp_count += warp_factor_block<NB>(dblk, linv, linv_al, nb, pivot_floor, tid,
                                           (colmask != nullptr && cta == 0) ? colmask + (long long)b * r + k0 : nullptr);
    __syncthreads();

    // ---- 2. Z[k,:] = Linv * B[k,:] for columns < k0 + nb.  Both CTAs need the old block row, so
    //         the result stays in `zrow` here; CTA 0 writes it back after the cluster barrier that
    //         ends the step, when the other CTA can no longer be reading the old values.
    const int zc = k0 + nb;
    for (int c = tid; c < rp; c += kChol2Threads) {
      float bcol[NB];
#pragma unroll
      for (int a = 0; a < NB; ++a) bcol[a] = (a < nb && c < zc) ? Z[(long long)(k0 + a) * r + c] : 0.f;
#pragma unroll 1
      for (int a = 0; a < NB; ++a) {
        const float4* lrow = reinterpret_cast<const float4*>(linv_al + a * NB);  // lower triangular, zeros above
        float s = 0.f;
#pragma unroll
        for (int q = 0; q < NB / 4; ++q) {
          const float4 lv = lrow[q];
          s = fmaf(lv.x, bcol[4 * q], s);
          s = fmaf(lv.y, bcol[4 * q + 1], s);
          s = fmaf(lv.z, bcol[4 * q + 2], s);
          s = fmaf(lv.w, bcol[4 * q + 3], s);
        }
        zrow[(size_t)a * rp + c] = s;
      }
    }
    // ---- 3. panel = A[k+1:, k] * Linv^T, stored transposed: panelT[a][i - p0]
    const int p0 = k0 + nb;  // first trailing row
    const int tr = r - p0;   // trailing rows
    for (int ii = tid; ii < rp; ii += kChol2Threads) {
      float arow[NB];
      const bool live = ii < tr;
#pragma unroll
      for (int a = 0; a < NB; ++a) arow[a] = (live && a < nb) ? W[(long long)(p0 + ii) * r + k0 + a] : 0.f;
#pragma unroll 1
      for (int a = 0; a < NB; ++a) {
        const float4* lrow = reinterpret_cast<const float4*>(linv_al + a * NB);
        float s = 0.f;
#pragma unroll
        for (int q = 0; q < NB / 4; ++q) {
          const float4 lv = lrow[q];
          s = fmaf(arow[4 * q], lv.x, s);
          s = fmaf(arow[4 * q + 1], lv.y, s);
          s = fmaf(arow[4 * q + 2], lv.z, s);
          s = fmaf(arow[4 * q + 3], lv.w, s);
        }
        panelT[(size_t)a * rp + ii] = s;
      }
    }
    __syncthreads();

    // ---- 4. trailing updates with 128 x 128 tiles, spread over the four 256-thread groups of
    //         the cluster: lower-triangular tiles of the Gram part, then the right-hand side
    const int nt = tr > 0 ? (tr + 127) / 128 : 0;
    const int nc = (zc + 127) / 128;
    const int gram_tiles = nt * (nt + 1) / 2;
    const int total_tiles = gram_tiles + nt * nc;
    const int t = tid & 255;
    for (int idx = cta * 2 + (tid >> 8); idx < total_tiles; idx += 4) {
      if (idx < gram_tiles) {
        int ti = 0, rem = idx;
        while (rem > ti) {  // row ti of the lower triangle holds ti + 1 tiles
          rem -= ti + 1;
          ++ti;
        }
        const int tj = rem;
        tile_update128<NB>(W, r, p0 + ti * 128, p0 + tj * 128, panelT + ti * 128, rp, panelT + tj * 128, rp, r, r,
                           t);
      } else {
        const int q = idx - gram_tiles;
        const int ti = q / nc, tc = q - ti * nc;
        tile_update128<NB>(Z, r, p0 + ti * 128, tc * 128, panelT + ti * 128, rp, zrow + tc * 128, rp, r, zc, t);
      }
    }
    chol_cluster_sync();
    // rows k0 .. k0 + nb of Z: nobody reads them from global memory again before the final scaling,
    // and every read of their old values (step 2 of both CTAs) lies before the barrier above
    if (cta == 0) {
      for (int c = tid; c < zc; c += kChol2Threads)
        for (int a = 0; a < nb; ++a) Z[(long long)(k0 + a) * r + c] = zrow[(size_t)a * rp + c];
    }
    __syncthreads();  // zrow is rewritten by the next step
    if (tr <= 0) break;  // uniform over the cluster
  }

  // undo the Jacobi scaling: G = D^-1 L' L'^T D^-1  =>  L^{-1} = L'^{-1} D, i.e. scale column j by d_j
  // (the barrier also hands CTA 0's last block row to CTA 1)
  chol_cluster_sync();
  for (int i = cta; i < r; i += 2) {
    for (int j = tid; j < r; j += kChol2Threads) {
      const long long e = (long long)i * r + j;
      Z[e] = (j <= i) ? Z[e] * dscale[j] : 0.f;
    }
  }
  if (cta == 0 && tid == 0 && info) info[b] = clamp_count;
}


// x = hi + lo with hi exactly representable in tf32 (low 13 mantissa bits cleared): the two
// operands of a 3xTF32 product, written in one pass over x.
__global__ void __launch_bounds__(256) split_tf32_kernel(const float4* __restrict__ x, float4* __restrict__ hi,
                                                        float4* __restrict__ lo, long long nvec,
                                                        const float* __restrict__ xs, float* __restrict__ his,
                                                        float* __restrict__ los, long long ntail) {
  auto split = [](float v, float& h, float& l) {
    h = __int_as_float(__float_as_int(v) & 0xffffe000);
    l = v - h;
  };
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const float4 v = x[i];
    float4 h, l;
    split(v.x, h.x, l.x);
    split(v.y, h.y, l.y);
    split(v.z, h.z, l.z);
    split(v.w, h.w, l.w);
    hi[i] = h;
    lo[i] = l;
  }
  if (blockIdx.x == 0 && threadIdx.x < ntail) split(xs[threadIdx.x], his[threadIdx.x], los[threadIdx.x]);
}

// Preparation of one triangular Newton correction from a Gram matrix G (r x r per batch entry):
//   d_i  = G_ii > tiny ? rsqrt(G_ii) : 0
//   C_ij = i > j ? d_i * G_ij * d_j : 0          (strictly lower part of D G D - I)
// One block per (row block of 8, batch entry); d is written by the blocks of the first column tile.
// With `fold` the columns of C are scaled by d once more (C_ij = d_i G_ij d_j^2), which lets the correction
// X D (I - C^T) run as one product on the unscaled X: X diag(d) - X (C diag(d))^T.
__global__ void __launch_bounds__(256) refine_prep_kernel(const float* __restrict__ G, float* __restrict__ C,
                                                         float* __restrict__ d, int r, float dead_below,
                                                         const int* __restrict__ skip, int fold) {
  const long long b = blockIdx.y;
  // matrices flagged in `skip` get C = 0: they are only rescaled, not corrected
  const bool no_correction = skip != nullptr && skip[b] != 0;
  const float* g = G + b * (long long)r * r;
  float* c = C + b * (long long)r * r;
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= r) return;
  const int lane = threadIdx.x & 31;
  const float gii = g[(long long)row * r + row];
  const float di = gii > dead_below ? rsqrtf(gii) : 0.f;
  if (lane == 0) d[b * r + row] = di;
  for (int j = lane; j < r; j += 32) {
    float v = 0.f;
    if (j < row && !no_correction) {
      const float gjj = g[(long long)j * r + j];
      const float dj = gjj > dead_below ? rsqrtf(gjj) : 0.f;
      v = di * g[(long long)row * r + j] * dj;
      if (fold) v *= dj;
    }
    c[(long long)row * r + j] = v;
  }
}

}  // namespace

cudaError_t chol_inverse_launch(const float* G, float* Z, float* work, int* info, int batch, int r, long long ldg,
                                long long g_batch_stride, float pivot_floor, cudaStream_t s, bool jacobi,
                                float* colmask) {
  const int jac = jacobi ? 1 : 0;
  if (batch == 0 || r == 0) return cudaSuccess;
  constexpr int kMaxDevices = 64;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) dev = 0;
  {
    // cluster-pair kernel (two CTAs per matrix); DION_B200_CHOL_PAIR=0 selects the single-CTA one
    static const int pair_env = [] {
      const char* e = getenv("DION_B200_CHOL_PAIR");
      return (e && e[0] == '0') ? 0 : 1;
    }();
    const int rp2 = ((r + 127) / 128) * 128;
    const size_t smem2 = (size_t)(2 * 32 * rp2 + 2 * 32 * 33 + 32 * 32 + rp2 + 4) * sizeof(float);
    if (pair_env && smem2 <= 227 * 1024) {
      // the attribute belongs to the device that is current, so it is tracked per device
      static bool granted[kMaxDevices] = {};
      if (!granted[dev]) {
        cudaError_t e2 = cudaFuncSetAttribute(chol_inverse_pair_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              227 * 1024);
        if (e2 != cudaSuccess) return e2;
        granted[dev] = true;
      }
      cudaLaunchConfig_t cfg;
      memset(&cfg, 0, sizeof(cfg));
      cfg.gridDim = dim3(2 * batch, 1, 1);
      cfg.blockDim = dim3(kChol2Threads, 1, 1);
      cfg.dynamicSmemBytes = smem2;
      cfg.stream = s;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 2;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      return cudaLaunchKernelEx(&cfg, chol_inverse_pair_kernel<32>, G, Z, work, info, r, ldg, g_batch_stride, rp2,
                                pivot_floor, jac, colmask);
    }
  }
  const int rp = ((r + 63) / 64) * 64;
  auto smem_for = [&](int nb) { return (size_t)(2 * nb * rp + 2 * nb * (nb + 1) + rp + 4) * sizeof(float); };
  constexpr size_t kMaxSmem = 227 * 1024;
  cudaError_t e;
  if (smem_for(32) <= kMaxSmem) {
    static bool granted32[kMaxDevices] = {};
    if (smem_for(32) > 48 * 1024 && !granted32[dev]) {
      e = cudaFuncSetAttribute(chol_inverse_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxSmem);
      if (e != cudaSuccess) return e;
      granted32[dev] = true;
    }
    chol_inverse_kernel<32><<<batch, kCholThreads, smem_for(32), s>>>(G, Z, work, info, r, ldg, g_batch_stride, rp,
                                                                     pivot_floor, jac, colmask);
  } else if (smem_for(16) <= kMaxSmem) {
    static bool granted16[kMaxDevices] = {};
    if (smem_for(16) > 48 * 1024 && !granted16[dev]) {
      e = cudaFuncSetAttribute(chol_inverse_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxSmem);
      if (e != cudaSuccess) return e;
      granted16[dev] = true;
    }
    chol_inverse_kernel<16><<<batch, kCholThreads, smem_for(16), s>>>(G, Z, work, info, r, ldg, g_batch_stride, rp,
                                                                     pivot_floor, jac, colmask);
  } else {
    return cudaErrorNotSupported;  // rank too large for the kernels' shared memory: the caller falls back
  }
  return cudaGetLastError();
}

cudaError_t col_sumsq_launch(const void* X, int x_type, float* out, int batch, long long rows, int cols,
                             long long ldx, long long batch_stride, cudaStream_t s) {
  if (batch == 0 || cols == 0) return cudaSuccess;
  dim3 grid((cols + 31) / 32, batch);
  col_sumsq_kernel<<<grid, 256, 0, s>>>(X, x_type, out, rows, cols, ldx, batch_stride);
  return cudaGetLastError();
}

// Rows of a strided [batch][rows][cols] array (element (b, i, j) at b * bs + i * ld + j) into contiguous hi / lo.
__global__ void __launch_bounds__(256) split_tf32_rows_kernel(const float* __restrict__ x, float* __restrict__ hi,
                                                             float* __restrict__ lo, long long rows_total, int rows,
                                                             int cols, long long ld, long long bs) {
  const int vpr = cols >> 2;  // float4 per row (cols is a multiple of 4)
  const long long nvec = rows_total * vpr;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (long long)gridDim.x * blockDim.x) {
    const long long row = v / vpr;
    const int c = (int)(v - row * vpr) << 2;
    const long long b = row / rows;
    const long long i = row - b * rows;
    const float4 q = *reinterpret_cast<const float4*>(x + b * bs + i * ld + c);
    float4 h, l;
    h.x = __int_as_float(__float_as_int(q.x) & 0xffffe000);
    h.y = __int_as_float(__float_as_int(q.y) & 0xffffe000);
    h.z = __int_as_float(__float_as_int(q.z) & 0xffffe000);
    h.w = __int_as_float(__float_as_int(q.w) & 0xffffe000);
    l.x = q.x - h.x;
    l.y = q.y - h.y;
    l.z = q.z - h.z;
    l.w = q.w - h.w;
    reinterpret_cast<float4*>(hi)[v] = h;
    reinterpret_cast<float4*>(lo)[v] = l;
  }
}

// Unit-diagonal (Jacobi) scaling of Gram matrices: d_i = rsqrt(G_ii) (0 where G_ii is not positive),
// W = D G D.  One block per (8 rows, matrix).
__global__ void __launch_bounds__(256) jacobi_scale_kernel(const float* __restrict__ G, float* __restrict__ W,
                                                          float* __restrict__ d, int r, long long ldg,
                                                          long long g_batch_stride) {
  const long long b = blockIdx.y;
  const float* g = G + b * g_batch_stride;
  float* w = W + b * (long long)r * r;
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= r) return;
  const int lane = threadIdx.x & 31;
  const float gii = g[(long long)row * ldg + row];
  const float di = gii > 1e-30f ? rsqrtf(gii) : 0.f;
  if (lane == 0) d[b * r + row] = di;
  for (int j = lane; j < r; j += 32) {
    const float gjj = g[(long long)j * ldg + j];
    const float dj = gjj > 1e-30f ? rsqrtf(gjj) : 0.f;
    w[(long long)row * r + j] = g[(long long)row * ldg + j] * di * dj;
  }
}

// Zd (contiguous [batch][nb][nb]) into the diagonal block of Z at (k0, k0) (pitch r), and Zm = Zd with the
// rows of clamped pivots (mask == 0) zeroed.  One block per (8 rows, matrix).
__global__ void __launch_bounds__(256) place_block_kernel(const float* __restrict__ Zd, const float* __restrict__ mask,
                                                         float* __restrict__ Z, float* __restrict__ Zm, int nb, int r,
                                                         int k0) {
  const long long b = blockIdx.y;
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= nb) return;
  const int lane = threadIdx.x & 31;
  const float m = mask[b * nb + row];
  const float* src = Zd + (b * nb + row) * (long long)nb;
  float* dst = Z + b * (long long)r * r + (long long)(k0 + row) * r + k0;
  float* dm = Zm + (b * nb + row) * (long long)nb;
  for (int j = lane; j < nb; j += 32) {
    const float v = src[j];
    dst[j] = v;
    dm[j] = v * m;
  }
}

cudaError_t jacobi_scale_launch(const float* G, float* W, float* d, int batch, int r, long long ldg,
                                long long g_batch_stride, cudaStream_t s) {
  if (batch == 0 || r == 0) return cudaSuccess;
  if (batch > 65535) return cudaErrorInvalidValue;
  jacobi_scale_kernel<<<dim3((r + 7) / 8, batch), 256, 0, s>>>(G, W, d, r, ldg, g_batch_stride);
  return cudaGetLastError();
}

cudaError_t place_block_launch(const float* Zd, const float* mask, float* Z, float* Zm, int batch, int nb, int r, int k0,
                               cudaStream_t s) {
  if (batch == 0 || nb == 0) return cudaSuccess;
  if (batch > 65535 || k0 < 0 || k0 + nb > r) return cudaErrorInvalidValue;
  place_block_kernel<<<dim3((nb + 7) / 8, batch), 256, 0, s>>>(Zd, mask, Z, Zm, nb, r, k0);
  return cudaGetLastError();
}

cudaError_t split_tf32_rows_launch(const float* x, float* hi, float* lo, int batch, int rows, int cols, long long ld,
                                   long long bs, cudaStream_t s) {
  if (batch == 0 || rows == 0 || cols == 0) return cudaSuccess;
  if ((cols & 3) || (ld & 3) || (bs & 3) ||
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(hi) | reinterpret_cast<uintptr_t>(lo)) & 15))
    return cudaErrorInvalidValue;
  const long long rows_total = (long long)batch * rows;
  const long long nvec = rows_total * (cols >> 2);
  long long grid = (nvec + 255) / 256;
  if (grid > 148 * 16) grid = 148 * 16;
  split_tf32_rows_kernel<<<(int)grid, 256, 0, s>>>(x, hi, lo, rows_total, rows, cols, ld, bs);
  return cudaGetLastError();
}

cudaError_t split_tf32_launch(const float* x, float* hi, float* lo, long long numel, cudaStream_t s) {
  if (numel == 0) return cudaSuccess;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(hi) | reinterpret_cast<uintptr_t>(lo)) & 15)
    return cudaErrorInvalidValue;
  const long long nvec = numel / 4, ntail = numel - nvec * 4;
  long long grid = (nvec + 255) / 256;
  if (grid > 148 * 16) grid = 148 * 16;
  if (grid < 1) grid = 1;
  split_tf32_kernel<<<(int)grid, 256, 0, s>>>(reinterpret_cast<const float4*>(x), reinterpret_cast<float4*>(hi),
                                              reinterpret_cast<float4*>(lo), nvec, x + nvec * 4, hi + nvec * 4,
                                              lo + nvec * 4, ntail);
  return cudaGetLastError();
}

cudaError_t refine_prep_launch(const float* G, float* C, float* d, int batch, int r, float dead_below,
                               const int* skip, bool fold, cudaStream_t s) {
  if (batch == 0 || r == 0) return cudaSuccess;
  if (batch > 65535) return cudaErrorInvalidValue;
  refine_prep_kernel<<<dim3((r + 7) / 8, batch), 256, 0, s>>>(G, C, d, r, dead_below, skip, fold ? 1 : 0);
  return cudaGetLastError();
}

}  // namespace dion
