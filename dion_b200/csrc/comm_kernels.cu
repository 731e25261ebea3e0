// Collectives written as kernels over symmetric memory (same-offset buffers on every
// GPU of a group, reachable through NVLink peer pointers and, when the group has an
// NVSwitch multicast object, through one multicast address).
//
//   barrier           - release/acquire flags in every peer's flag block, bounded spin
//   all_reduce        - in place: every rank reduces one slice (peer loads in rank order,
//                       or multimem.ld_reduce in the switch) and writes it to every peer
//                       (peer stores or multimem.st); results are bit-identical everywhere
//   reduce_into       - one shot: dst (+)= scale * sum_p src_p, every rank reads all peers
//
// These stand in for the NCCL all-reduce / reduce-scatter / all-gather calls the reference
// issues through funcol and DTensor redistribute around its power iteration
// (dion/dion.py:806-844, 925-960, 1076-1110, 1165-1197).
//
// Every wait is bounded (kWaitBudgetNs); a wait that gives up sets the status word and the
// kernel finishes normally.  Nothing here uses TMA or cluster multicast.
#include <cuda_bf16.h>

#include "kernels.h"
#include "symm_flags.cuh"
#include "umma.cuh"

namespace dion {

namespace {

__global__ void barrier_kernel(PeerTable t, long long flag_off, int channel, int rank, int world, unsigned epoch,
                               int* status) {
  const int lane = threadIdx.x;
  __threadfence_system();
  signal_peers(t, flag_off, channel, rank, world, epoch, lane);
  if (!wait_peers(t, flag_off, channel, rank, world, epoch, lane) && status) atomicCAS(status, 0, kStatusPeerTimeout);
}

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

template <typename T>
struct Vec16;
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float (&f)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&f)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  }
  // sum over the multicast group, performed by the switch
  static __device__ __forceinline__ void mc_load_reduce(const float* p, float (&f)[4]) {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(f[0]), "=f"(f[1]), "=f"(f[2]), "=f"(f[3])
                 : "l"(p)
                 : "memory");
  }
  static __device__ __forceinline__ void mc_store(float* p, const float (&f)[4]) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(f[0]), "f"(f[1]),
                 "f"(f[2]), "f"(f[3])
                 : "memory");
  }
};
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 q = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 v = __bfloat1622float2(h[j]);
      f[2 * j] = v.x;
      f[2 * j + 1] = v.y;
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&f)[8]) {
    uint4 q;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
    *reinterpret_cast<uint4*>(p) = q;
  }
  static __device__ __forceinline__ void mc_load_reduce(const __nv_bfloat16* p, float (&f)[8]) {
    uint4 q;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w)
                 : "l"(p)
                 : "memory");
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 v = __bfloat1622float2(h[j]);
      f[2 * j] = v.x;
      f[2 * j + 1] = v.y;
    }
  }
  static __device__ __forceinline__ void mc_store(__nv_bfloat16* p, const float (&f)[8]) {
    uint4 q;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
    asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(q.x), "r"(q.y),
                 "r"(q.z), "r"(q.w)
                 : "memory");
  }
};

// In-place all-reduce of `numel` elements at byte offset `data_off` of every peer's arena.
// Phase 0: all ranks' inputs are complete (flags, channel 0).
// Phase 1: rank r reduces elements [r * slice, (r + 1) * slice) and writes the result to
//          all peers.  Phase 2: all slices are written (flags, channel 1), after which the
//          kernel retires, so stream order hands complete data to the next kernel.
template <typename T, bool kMulticast>
__global__ void __launch_bounds__(512) all_reduce_kernel(PeerTable t, long long flag_off, long long data_off,
                                                        char* mc_base, long long numel, float scale, int rank,
                                                        int world, unsigned epoch, unsigned* done_counter,
                                                        int* status) {
  using V = Vec16<T>;
  constexpr int N = V::N;
  __shared__ int ok_flag;
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();
  // debug build: rank and group size are consistent and the buffer keeps the alignment of the vector accesses
  if (threadIdx.x == 0 && !DION_DBG_OK(world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world && (data_off & 15) == 0 &&
                                           t.ptrs[rank] != nullptr, status))
    ok_flag = 0;
  __syncthreads();
  if (ok_flag && threadIdx.x < 32) {
    if (blockIdx.x == 0) {
      __threadfence_system();
      signal_peers(t, flag_off, 0, rank, world, epoch, threadIdx.x);
    }
    if (!wait_peers(t, flag_off, 0, rank, world, epoch, threadIdx.x)) {
      ok_flag = 0;
      if (status) atomicCAS(status, 0, kStatusPeerTimeout);
    }
  }
  __syncthreads();
  if (ok_flag) {
    // slice boundaries in vectors, the last rank also takes the remainder
    const long long nvec = numel / N;
    const long long per = (nvec + world - 1) / world;
    const long long v0 = per * rank;
    const long long v1 = min(v0 + per, nvec);
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long vb = v0 + (long long)blockIdx.x * blockDim.x + threadIdx.x; vb < v1; vb += 4 * stride) {
      float acc[4][N];
      // up to four vectors per thread, so that several peer / switch loads are in flight
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const long long v = vb + u * stride;
        if (v >= v1) break;
        if (kMulticast) {
          V::mc_load_reduce(reinterpret_cast<const T*>(mc_base + data_off) + v * N, acc[u]);
        } else {
#pragma unroll
          for (int j = 0; j < N; ++j) acc[u][j] = 0.f;
          for (int p = 0; p < world; ++p) {
            float f[N];
            V::load(reinterpret_cast<const T*>(reinterpret_cast<const char*>(t.ptrs[p]) + data_off) + v * N, f);
#pragma unroll
            for (int j = 0; j < N; ++j) acc[u][j] += f[j];
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const long long v = vb + u * stride;
        if (v >= v1) break;
#pragma unroll
        for (int j = 0; j < N; ++j) acc[u][j] *= scale;
        if (kMulticast) {
          V::mc_store(reinterpret_cast<T*>(mc_base + data_off) + v * N, acc[u]);
        } else {
          for (int p = 0; p < world; ++p)
            V::store(reinterpret_cast<T*>(reinterpret_cast<char*>(t.ptrs[p]) + data_off) + v * N, acc[u]);
        }
      }
    }
    // scalar tail (numel not a multiple of the vector width): rank 0 handles it with peer accesses
    if (rank == 0 && blockIdx.x == 0) {
      for (long long i = nvec * N + threadIdx.x; i < numel; i += blockDim.x) {
        float a = 0.f;
        for (int p = 0; p < world; ++p)
          a += to_f(reinterpret_cast<const T*>(reinterpret_cast<const char*>(t.ptrs[p]) + data_off)[i]);
        a *= scale;
        for (int p = 0; p < world; ++p)
          reinterpret_cast<T*>(reinterpret_cast<char*>(t.ptrs[p]) + data_off)[i] = from_f<T>(a);
      }
    }
  }
  // the last CTA of this rank to finish announces it and waits for the other ranks
  __threadfence_system();
  __syncthreads();
  __shared__ int is_last;
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(done_counter, 1u);
    is_last = (prev == gridDim.x - 1);
    if (is_last) *done_counter = 0;  // ready for the next launch on this stream
  }
  __syncthreads();
  if (is_last && threadIdx.x < 32) {
    __threadfence_system();
    signal_peers(t, flag_off, 1, rank, world, epoch, threadIdx.x);
    if (!wait_peers(t, flag_off, 1, rank, world, epoch, threadIdx.x) && status)
      atomicCAS(status, 0, kStatusPeerTimeout);
  }
}

// dst[i] = beta * dst[i] + scale * sum_p src_p[i]; src at `data_off` of every peer's arena,
// dst an ordinary local fp32 / bf16 buffer.  Channel 2 says "inputs complete", channel 3
// "this rank finished reading", so the sources may be overwritten once the kernel retired.
template <typename T, typename D>
__global__ void __launch_bounds__(512) reduce_into_kernel(PeerTable t, long long flag_off, long long data_off,
                                                         D* __restrict__ dst, long long numel, float scale,
                                                         float beta, int rank, int world, unsigned epoch,
                                                         unsigned* done_counter, int* status) {
  __shared__ int ok_flag;
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();
  if (threadIdx.x < 32) {
    if (blockIdx.x == 0) {
      __threadfence_system();
      signal_peers(t, flag_off, 2, rank, world, epoch, threadIdx.x);
    }
    if (!wait_peers(t, flag_off, 2, rank, world, epoch, threadIdx.x)) {
      ok_flag = 0;
      if (status) atomicCAS(status, 0, kStatusPeerTimeout);
    }
  }
  __syncthreads();
  if (ok_flag) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < numel;
         i += (long long)gridDim.x * blockDim.x) {
      float a = 0.f;
      for (int p = 0; p < world; ++p)
        a += to_f(reinterpret_cast<const T*>(reinterpret_cast<const char*>(t.ptrs[p]) + data_off)[i]);
      a *= scale;
      if (beta != 0.f) a += beta * to_f(dst[i]);
      dst[i] = from_f<D>(a);
    }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int is_last;
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(done_counter, 1u);
    is_last = (prev == gridDim.x - 1);
    if (is_last) *done_counter = 0;
  }
  __syncthreads();
  if (is_last && threadIdx.x < 32) {
    signal_peers(t, flag_off, 3, rank, world, epoch, threadIdx.x);
    if (!wait_peers(t, flag_off, 3, rank, world, epoch, threadIdx.x) && status)
      atomicCAS(status, 0, kStatusPeerTimeout);
  }
}

// All-gather for parameter shards (the collective FSDP2 issues before a block runs,
// models/gpt_model.py:336-376 in the reference).  `out` (world * bytes) and `in` (bytes) are
// ordinary local buffers; only a staging slot of the arena is symmetric:
//   1. copy `in` to this rank's staging slot (and to out[rank] unless it already lives there),
//   2. the last CTA to finish announces it on `channel`,
//   3. every CTA pulls peer p's slot into out[p] as soon as p announced.
// Slots alternate with the parity of `epoch`: a rank can only start writing slot e+2 after its
// launch e+1 saw every peer's announcement e+1, which peers make after their launch e retired,
// so no closing barrier is needed.  Launches of one arena must be stream-ordered on every rank.
__global__ void __launch_bounds__(512) all_gather_kernel(PeerTable t, long long flag_off, long long slot_off,
                                                        const char* __restrict__ in, char* __restrict__ out,
                                                        long long bytes, int rank, int world, unsigned epoch,
                                                        int channel, unsigned* done_counter, int* status,
                                                        unsigned long long budget_ns) {
  const long long nvec = bytes / 16;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  {
    const uint4* src = reinterpret_cast<const uint4*>(in);
    uint4* slot = reinterpret_cast<uint4*>(reinterpret_cast<char*>(t.ptrs[rank]) + slot_off);
    uint4* own = reinterpret_cast<uint4*>(out + (long long)rank * bytes);
    const bool copy_own = reinterpret_cast<const char*>(own) != in;
    for (long long v = tid; v < nvec; v += 4 * nthreads) {
      uint4 q[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (v + u * nthreads < nvec) q[u] = src[v + u * nthreads];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (v + u * nthreads < nvec) {
          slot[v + u * nthreads] = q[u];
          if (copy_own) own[v + u * nthreads] = q[u];
        }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(done_counter, 1u);
    if (prev == gridDim.x - 1) {
      *done_counter = 0;
      __threadfence_system();
      for (int p = 0; p < world; ++p) {
        unsigned* f = reinterpret_cast<unsigned*>(reinterpret_cast<char*>(t.ptrs[p]) + flag_off);
        st_release_sys(f + channel * kMaxPeers + rank, epoch);
      }
    }
  }
  __shared__ int ok_flag;
  for (int i = 1; i < world; ++i) {
    const int p = (rank + i) % world;
    if (threadIdx.x == 0) {
      ok_flag = wait_peer(t, flag_off, channel, rank, p, epoch, budget_ns) ? 1 : 0;
      if (!ok_flag && status) atomicCAS(status, 0, kStatusPeerTimeout);
    }
    __syncthreads();
    if (ok_flag) {
      const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(t.ptrs[p]) + slot_off);
      uint4* dst = reinterpret_cast<uint4*>(out + (long long)p * bytes);
      // eight independent 16-byte peer loads in flight per thread: a load over NVLink takes a few
      // microseconds, and the bytes in flight have to cover that at link speed
      for (long long v = tid; v < nvec; v += 8 * nthreads) {
        uint4 q[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (v + u * nthreads < nvec) q[u] = src[v + u * nthreads];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (v + u * nthreads < nvec) dst[v + u * nthreads] = q[u];
      }
    }
    __syncthreads();
  }
}

// Reduce-scatter for gradients: every rank's input (world * numel elements at `data_off` of its
// arena) is complete when the kernel starts in stream order; rank r writes
// out[i] = scale * sum_p in_p[r * numel + i], summing in rank order (or in the switch).  The
// kernel retires only after every peer finished reading this rank's input, so the input may be
// overwritten by the next kernel in the stream.
template <typename T, bool kMulticast>
__global__ void __launch_bounds__(512) reduce_scatter_kernel(PeerTable t, long long flag_off, long long data_off,
                                                            char* mc_base, T* __restrict__ out, long long numel,
                                                            float scale, int rank, int world, unsigned epoch,
                                                            int ch_start, int ch_end, unsigned* done_counter,
                                                            int* status, unsigned long long budget_ns) {
  using V = Vec16<T>;
  constexpr int N = V::N;
  __shared__ int ok_flag;
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();
  if (threadIdx.x < 32) {
    if (blockIdx.x == 0) {
      __threadfence_system();
      signal_peers(t, flag_off, ch_start, rank, world, epoch, threadIdx.x);
    }
    if (!wait_peers(t, flag_off, ch_start, rank, world, epoch, threadIdx.x, budget_ns)) {
      ok_flag = 0;
      if (status) atomicCAS(status, 0, kStatusPeerTimeout);
    }
  }
  __syncthreads();
  if (ok_flag) {
    const long long slice_off = data_off + (long long)rank * numel * (long long)sizeof(T);
    const long long nvec = numel / N;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long v0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; v0 < nvec; v0 += 4 * stride) {
      float acc[4][N];
      // up to four vectors per thread: their peer loads are independent and overlap
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const long long v = v0 + u * stride;
        if (v >= nvec) break;
        if (kMulticast) {
          V::mc_load_reduce(reinterpret_cast<const T*>(mc_base + slice_off) + v * N, acc[u]);
        } else {
#pragma unroll
          for (int j = 0; j < N; ++j) acc[u][j] = 0.f;
          for (int p = 0; p < world; ++p) {
            float f[N];
            V::load(reinterpret_cast<const T*>(reinterpret_cast<const char*>(t.ptrs[p]) + slice_off) + v * N, f);
#pragma unroll
            for (int j = 0; j < N; ++j) acc[u][j] += f[j];
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const long long v = v0 + u * stride;
        if (v >= nvec) break;
#pragma unroll
        for (int j = 0; j < N; ++j) acc[u][j] *= scale;
        V::store(out + v * N, acc[u]);
      }
    }
    if (blockIdx.x == 0) {
      for (long long i = nvec * N + threadIdx.x; i < numel; i += blockDim.x) {
        float a = 0.f;
        for (int p = 0; p < world; ++p)
          a += to_f(reinterpret_cast<const T*>(reinterpret_cast<const char*>(t.ptrs[p]) + slice_off)[i]);
        out[i] = from_f<T>(a * scale);
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int is_last;
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(done_counter, 1u);
    is_last = (prev == gridDim.x - 1);
    if (is_last) *done_counter = 0;
  }
  __syncthreads();
  if (is_last && threadIdx.x < 32) {
    signal_peers(t, flag_off, ch_end, rank, world, epoch, threadIdx.x);
    if (!wait_peers(t, flag_off, ch_end, rank, world, epoch, threadIdx.x, budget_ns) && status)
      atomicCAS(status, 0, kStatusPeerTimeout);
  }
}

int comm_grid(long long work_items, int threads) {
  long long g = (work_items + threads - 1) / threads;
  if (g < 1) g = 1;
  if (g > 96) g = 96;  // enough CTAs to keep NVLink busy; the rest of the GPU stays free for compute
  return (int)g;
}

}  // namespace

cudaError_t symm_barrier_launch(const PeerTable& t, long long flag_off, int channel, int rank, int world,
                                unsigned epoch, int* status, cudaStream_t s) {
  if (world > kMaxPeers) return cudaErrorInvalidValue;
  barrier_kernel<<<1, 32, 0, s>>>(t, flag_off, channel, rank, world, epoch, status);
  return cudaGetLastError();
}

cudaError_t symm_all_reduce_launch(const PeerTable& t, long long flag_off, long long data_off, void* mc_base,
                                   int elem_type, long long numel, float scale, int rank, int world, unsigned epoch,
                                   unsigned* done_counter, int* status, cudaStream_t s) {
  if (world > kMaxPeers || (data_off & 15)) return cudaErrorInvalidValue;
  const int threads = 512;
  const int vecn = elem_type == kElemF32 ? 4 : 8;
  const int grid = comm_grid((numel / vecn + world - 1) / world, threads);
  char* mc = reinterpret_cast<char*>(mc_base);
  if (elem_type == kElemF32) {
    if (mc)
      all_reduce_kernel<float, true><<<grid, threads, 0, s>>>(t, flag_off, data_off, mc, numel, scale, rank, world,
                                                             epoch, done_counter, status);
    else
      all_reduce_kernel<float, false><<<grid, threads, 0, s>>>(t, flag_off, data_off, mc, numel, scale, rank, world,
                                                              epoch, done_counter, status);
  } else {
    if (mc)
      all_reduce_kernel<__nv_bfloat16, true><<<grid, threads, 0, s>>>(t, flag_off, data_off, mc, numel, scale, rank,
                                                                     world, epoch, done_counter, status);
    else
      all_reduce_kernel<__nv_bfloat16, false><<<grid, threads, 0, s>>>(t, flag_off, data_off, mc, numel, scale,
                                                                      rank, world, epoch, done_counter, status);
  }
  return cudaGetLastError();
}

cudaError_t symm_reduce_into_launch(const PeerTable& t, long long flag_off, long long data_off, int src_type,
                                    void* dst, int dst_type, long long numel, float scale, float beta, int rank,
                                    int world, unsigned epoch, unsigned* done_counter, int* status, cudaStream_t s) {
  if (world > kMaxPeers) return cudaErrorInvalidValue;
  const int threads = 512;
  const int grid = comm_grid(numel, threads);
#define DION_RI(T, D)                                                                                            \
  reduce_into_kernel<T, D><<<grid, threads, 0, s>>>(t, flag_off, data_off, reinterpret_cast<D*>(dst), numel, scale, \
                                                    beta, rank, world, epoch, done_counter, status)
  if (src_type == kElemF32 && dst_type == kElemF32) DION_RI(float, float);
  else if (src_type == kElemF32 && dst_type == kElemBF16) DION_RI(float, __nv_bfloat16);
  else if (src_type == kElemBF16 && dst_type == kElemF32) DION_RI(__nv_bfloat16, float);
  else DION_RI(__nv_bfloat16, __nv_bfloat16);
#undef DION_RI
  return cudaGetLastError();
}

cudaError_t symm_all_gather_launch(const PeerTable& t, long long flag_off, long long slot_off, const void* in,
                                   void* out, long long bytes, int rank, int world, unsigned epoch, int channel,
                                   unsigned* done_counter, int* status, long long budget_ns, cudaStream_t s) {
  if (world > kMaxPeers || (bytes & 15) || (slot_off & 15) || (reinterpret_cast<uintptr_t>(in) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return cudaErrorInvalidValue;
  const int threads = 512;
  // the copies of this kernel are pure loads and stores; with more than two ranks it pays to use most SMs
  int grid = comm_grid(bytes / 16, threads);
  if (world > 2) {
    long long g = (bytes / 16 + threads - 1) / threads;
    grid = (int)(g < 1 ? 1 : (g > 132 ? 132 : g));
  }
  all_gather_kernel<<<grid, threads, 0, s>>>(t, flag_off, slot_off, reinterpret_cast<const char*>(in),
                                             reinterpret_cast<char*>(out), bytes, rank, world, epoch, channel,
                                             done_counter, status, (unsigned long long)budget_ns);
  return cudaGetLastError();
}

cudaError_t symm_reduce_scatter_launch(const PeerTable& t, long long flag_off, long long data_off, void* mc_base,
                                       int elem_type, void* out, long long numel, float scale, int rank, int world,
                                       unsigned epoch, int ch_start, int ch_end, unsigned* done_counter, int* status,
                                       long long budget_ns, cudaStream_t s) {
  const int es = elem_type == kElemF32 ? 4 : 2;
  if (world > kMaxPeers || (data_off & 15) || ((numel * es) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return cudaErrorInvalidValue;
  const int threads = 512;
  const int grid = comm_grid(numel / (16 / es), threads);
  char* mc = reinterpret_cast<char*>(mc_base);
  const unsigned long long b = (unsigned long long)budget_ns;
#define DION_RS(T, MC)                                                                                           \
  reduce_scatter_kernel<T, MC><<<grid, threads, 0, s>>>(t, flag_off, data_off, mc, reinterpret_cast<T*>(out), numel, \
                                                        scale, rank, world, epoch, ch_start, ch_end, done_counter,   \
                                                        status, b)
  if (elem_type == kElemF32) {
    if (mc) DION_RS(float, true);
    else DION_RS(float, false);
  } else {
    if (mc) DION_RS(__nv_bfloat16, true);
    else DION_RS(__nv_bfloat16, false);
  }
#undef DION_RS
  return cudaGetLastError();
}

}  // namespace dion
