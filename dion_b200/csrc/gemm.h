// Host interface of the tcgen05 GEMM.  Plain C++/CUDA types only, so that the
// same entry points serve the torch bindings and C callers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace dion {

enum GemmDType : int { kBF16 = 0, kF32 = 1 };  // kF32 operands run as TF32 on the tensor cores
enum GemmMajor : int { kMajorK = 0, kMajorMN = 1 };
enum GemmEpilogue : int {
  kEpiStore = 0,      // D = act(alpha * acc) + beta * C
  kEpiAtomicAdd = 1,  // D += alpha * acc   (fp32 D, red.global.add; used with split-K)
};
constexpr int kGatherMaxPeers = 8;  // ranks of a symmetric-memory group (width of its flag block)

enum GemmAct : int {
  kActNone = 0,
  kActRelu2 = 1,         // D = relu(alpha * acc)^2 (+ beta * C)
  kActRelu2SavePre = 2,  // as kActRelu2, and D2 receives the pre-activation alpha * acc
  kActMulRelu2Grad = 3,  // D = alpha * acc * 2 * relu(C): backward of ReLU^2 with C the saved pre-activation
  kActMulRelu2GradSq = 4,  // D = alpha * acc * 2 * sqrt(max(C, 0)): the same with C = relu(pre)^2, the saved activation
};

// D[b] = alpha * op(A[b]) * op(B[b]) (+ beta * C[b]),  op(A) is M x K, op(B) is K x N.
//
// Operand storage:
//   a_major == kMajorK  : A is stored M x K row-major (K contiguous), row pitch lda
//   a_major == kMajorMN : A is stored K x M row-major (M contiguous), row pitch lda
//   b_major == kMajorK  : B is stored N x K row-major (K contiguous), row pitch ldb
//   b_major == kMajorMN : B is stored K x N row-major (N contiguous), row pitch ldb
// Pitches and batch strides are in elements.  Base pointers must be 16-byte
// aligned and pitches a multiple of 16 bytes (TMA requirement).
struct GemmArgs {
  const void* A = nullptr;
  const void* B = nullptr;
  // Optional low halves of fp32 operands that were split as x = hi + lo with hi exactly representable
  // in tf32 (A and B then hold the hi halves; same shapes, pitches and strides).  The product runs as
  // three K-segments into one accumulator, A B + A_lo B + A B_lo - a 3xTF32 product (close to fp32
  // accuracy) in a single launch.  Both or neither; fp32 operands, split_k == 1.
  const void* A_lo = nullptr;
  const void* B_lo = nullptr;
  // fp32 operands multiplied with 3xTF32 accuracy, the hi / lo halves being formed in shared memory by the
  // kernel itself (no copies in global memory; tiles of up to 128 columns).  Excludes A_lo / B_lo.
  int split3 = 0;
  int ab_dtype = kBF16;
  int a_major = kMajorK;
  int b_major = kMajorK;
  int64_t lda = 0, ldb = 0;
  int64_t a_batch_stride = 0, b_batch_stride = 0;
  int M = 0, N = 0, K = 0, batch = 1;
  int split_k = 1;  // > 1 requires kEpiAtomicAdd

  float alpha = 1.f, beta = 0.f;
  // C (optional addend) and D (output); row-major M x N with pitches ldc / ldd.
  const void* C = nullptr;
  int c_dtype = kF32;
  int64_t ldc = 0, c_batch_stride = 0;
  const void* const* c_ptrs = nullptr;  // optional device array of per-batch C pointers
  // Optional per-column factor of the addend: D = alpha * acc + beta * C * diag(c_col_scale[b]);
  // fp32 [batch][N], contiguous.
  const float* c_col_scale = nullptr;
  void* D = nullptr;
  int d_dtype = kF32;
  int64_t ldd = 0, d_batch_stride = 0;
  void* const* d_ptrs = nullptr;  // optional device array of per-batch D pointers
  // With d_ptrs: every batch element is stored to `d_dup` destinations, d_ptrs[b * d_dup + k] (k < d_dup) -
  // e.g. the same slot of a symmetric buffer on every rank of a group, written with peer stores.
  int d_dup = 1;
  // Optional second output: bf16 copy of what was stored to D.
  void* D2 = nullptr;
  int64_t ldd2 = 0, d2_batch_stride = 0;
  void* const* d2_ptrs = nullptr;

  int epilogue = kEpiStore;
  int act = kActNone;
  // Symmetric mode (M == N, result known symmetric, e.g. X * X^T): only tiles on or
  // above the diagonal are computed and each off-diagonal tile is also stored transposed.
  int symmetric = 0;
  // Scatter epilogue: D is not one matrix but `scatter_dests` blocks per batch element, each
  // in its own buffer (typically another GPU's memory, written with peer stores):
  //   mode 1: block k holds rows    [k * scatter_block, (k + 1) * scatter_block)
  //   mode 2: block k holds columns [k * scatter_block, (k + 1) * scatter_block)  (multiple of 32)
  // `scatter_ptrs` is a device array of batch * scatter_dests base pointers; ldd is the row
  // pitch inside a block; d_dtype its element type.
  int scatter_mode = 0;
  int scatter_block = 0;
  int scatter_dests = 0;
  void* const* scatter_ptrs = nullptr;
  int block_n = 0;  // 0 = choose automatically (64 / 128 / 256)
  int max_ctas = 0;  // 0 = one CTA per SM
  int pair = 0;      // CTA pairs (256-row tiles): 0 = choose automatically, 1 = force (needs block_n 256), -1 = never

  int* status = nullptr;  // device int, set to a non-zero code on a device-side failure

  // All-gather of operand A inside the kernel (bf16, K-major A and B, one batch, lda == K): A is
  // `gather.world` row blocks of `gather.rows` rows, block k produced by rank k.  Two extra warps of
  // every CTA copy this rank's block from `gather.in` into its staging slot in symmetric memory
  // (`peers[rank] + slot_off`) and into A, announce it on `channel` of every peer's flag block, and
  // then pull the other ranks' slots into A with peer loads, in units handed out by a counter, raising
  // one counter per chunk of rows; the TMA producer waits for the counter of a tile's chunk before it
  // loads from A, and the tiles are visited starting with this rank's own rows.  `counters`
  // (`counter_words` >= 2 + M / tile rows unsigned words) is cleared by the launch.  Waits are bounded
  // by `budget_ns`.
  struct Gather {
    int world = 0;  // 0 = off
    int rank = 0;
    int rows = 0;
    const void* in = nullptr;
    void* peers[kGatherMaxPeers] = {};
    long long flag_off = 0, slot_off = 0;
    unsigned epoch = 0;
    int channel = 0;
    unsigned* counters = nullptr;
    int counter_words = 0;
    long long budget_ns = 0;
  } gather;
};

// Returns cudaSuccess or the launch error; argument errors return cudaErrorInvalidValue
// and write a message retrievable with gemm_last_error().
cudaError_t gemm_launch(const GemmArgs& args, cudaStream_t stream);
const char* gemm_last_error();

// Host only, no launch: what the all-gather variant would do for `args` (sizes, majors and the
// `gather` fields world / rank / rows are read).  out = {tile rows, tile columns, CTA pairs (0 / 1),
// rows per readiness counter, copy units per counter, first m-tile of the schedule, m-tiles, n-tiles}.
bool gemm_gather_plan(const GemmArgs& args, int (&out)[8]);

}  // namespace dion
