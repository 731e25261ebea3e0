// Host launchers of the non-GEMM sm_100a kernels (plain CUDA types only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace dion {

enum ElemType : int { kElemF32 = 0, kElemBF16 = 1 };

// ---------------------------------------------------------------------------
// Multi-tensor launches: up to kMaxTensorsPerLaunch tensors travel in the kernel
// parameter block (no device-side tables, no host-to-device copies).
// ---------------------------------------------------------------------------
constexpr int kMaxTensorsPerLaunch = 40;
constexpr int kMaxLists = 5;

struct TensorListChunk {
  void* ptrs[kMaxLists][kMaxTensorsPerLaunch];
  long long numel[kMaxTensorsPerLaunch];
  int block_start[kMaxTensorsPerLaunch + 1];  // prefix sum of thread blocks per tensor
  int num_tensors;
};

struct AdamWHyper {
  float lr, beta1, beta2, weight_decay, eps;
  float bias_correction1, bias_correction2_sqrt;
};
struct LionHyper {
  float lr, beta1, beta2, weight_decay;
};

// lists: 0 = X (fp32), 1 = G, 2 = M, 3 = V, 4 = optional bf16 shadow of X
cudaError_t adamw_multi_launch(const TensorListChunk& tl, int g_type, int m_type, int v_type, bool has_shadow,
                               const AdamWHyper& h, cudaStream_t s);
// lists: 0 = X (fp32), 1 = G, 2 = M, 4 = optional bf16 shadow of X
cudaError_t lion_multi_launch(const TensorListChunk& tl, int g_type, int m_type, bool has_shadow,
                              const LionHyper& h, cudaStream_t s);
// Muon momentum: M = mu*M + G; U = nesterov ? mu*M + G : M  (bf16 out); sumsq[t] += sum(U^2)
// lists: 0 = G, 1 = M (fp32), 2 = U (bf16);  sumsq: fp32[num_tensors] or null
cudaError_t muon_pre_multi_launch(const TensorListChunk& tl, int g_type, float mu, bool nesterov, float* sumsq,
                                  cudaStream_t s);
// Muon apply: X = decay * X - step * U ; lists: 0 = X (fp32), 1 = U (bf16), 4 = optional bf16 shadow
cudaError_t muon_post_multi_launch(const TensorListChunk& tl, bool has_shadow, float decay, float step,
                                   cudaStream_t s);
// Dion momentum accumulate: M += G; nonzero[t] |= any(M != 0)
// lists: 0 = G, 1 = M ; nonzero: int[num_tensors] or null
cudaError_t dion_accum_multi_launch(const TensorListChunk& tl, int g_type, int m_type, int* nonzero,
                                    cudaStream_t s);
// dst = (dst_type) src ; lists: 0 = src, 1 = dst
cudaError_t cast_multi_launch(const TensorListChunk& tl, int src_type, int dst_type, cudaStream_t s);

int multi_tensor_block_elems();

// out[b] = x[b] / (||x[b]||_F + eps) for a contiguous batch of bf16 matrices of `per` elements each (the
// scaling in front of Newton-Schulz).  With `sumsq` (fp32 [batch], the squared norms) one launch; without,
// a first launch writes per-chunk partial sums to `partial` (batch * frob_chunks(per) floats), which the
// scaling launch adds up in a fixed order.
int frob_chunks(long long per);
cudaError_t frob_scale_launch(const void* x, void* out, float* partial, const float* sumsq, float eps, int batch,
                              long long per, cudaStream_t s);

// ---------------------------------------------------------------------------
// Model kernels (bf16 activations, fp32 math)
// ---------------------------------------------------------------------------
// y = x * rsqrt(mean(x^2) + eps)  over the last dim (weightless RMSNorm); rstd saved for backward.
// When `residual` is given: x_out = x + residual is written first and normalised.
cudaError_t rmsnorm_fwd_launch(const void* x, const void* residual, void* x_out, void* y, float* rstd,
                               long long rows, int dim, float eps, cudaStream_t s);
// dx = rstd * (dy - y_hat * mean(dy * y_hat)) (+ dx_add when given), y_hat = x * rstd
cudaError_t rmsnorm_bwd_launch(const void* dy, const void* x, const float* rstd, const void* dx_add, void* dx,
                               long long rows, int dim, cudaStream_t s);
// Rotary embedding (half-split) followed by RMS norm over head_dim, for q and k together.
// k (with k_out / dk / dk_out) may be null to process a single tensor; eps < 0 skips the norm.
// in/out: [tokens, heads, head_dim] bf16 rows with arbitrary row pitch; cos/sin: [seq, head_dim/2] bf16.
cudaError_t rope_qknorm_fwd_launch(const void* q, const void* k, void* q_out, void* k_out, const void* cos,
                                   const void* sin, long long tokens, int seq_len, int heads, int head_dim,
                                   long long in_pitch, long long out_pitch, float eps, cudaStream_t s);
cudaError_t rope_qknorm_bwd_launch(const void* dq_out, const void* dk_out, const void* q, const void* k, void* dq,
                                   void* dk, const void* cos, const void* sin, long long tokens, int seq_len,
                                   int heads, int head_dim, long long in_pitch, long long out_pitch, float eps,
                                   cudaStream_t s);
// h = relu(x)^2 ; dx = dh * 2 * relu(x)
cudaError_t relu2_fwd_launch(const void* x, void* h, long long n, cudaStream_t s);
cudaError_t relu2_bwd_launch(const void* dh, const void* x, void* dx, long long n, cudaStream_t s);
// Softmax cross-entropy over bf16 logits [rows, vocab] with row pitch `pitch`:
//   row_loss[i] = lse_i - logit_i[target_i]  (0 for rows whose target == ignore_index)
//   when write_grad: logits are overwritten with grad_scale * (*scale_ptr) * (softmax - onehot)
//   (zero for ignored rows); scale_ptr is an optional device scalar, e.g. 1 / valid rows.
cudaError_t cross_entropy_fwd_bwd_launch(void* logits, const long long* targets, float* row_loss,
                                         const float* scale_ptr, long long rows, int vocab, long long pitch,
                                         float grad_scale, long long ignore_index, bool write_grad, cudaStream_t s);
// out[t, :] = (bf16) table[idx[t], :]   (table fp32 or bf16)
cudaError_t embedding_fwd_launch(const void* table, int table_type, const long long* idx, void* out,
                                 long long tokens, int dim, cudaStream_t s);
// dtable[idx[t], :] += dout[t, :]  (fp32 atomic accumulation)
cudaError_t embedding_bwd_launch(const void* dout, const long long* idx, float* dtable, long long tokens, int dim,
                                 cudaStream_t s);

// RMSNorm with a learnable gain (fp32 or bf16 vector of `dim`): y = x * rstd * gain; the backward pass writes
// dx and per-block partial sums of the gain's gradient, partial[blocks][dim] (fp32), which the caller
// adds up; `blocks` = rmsnorm_gain_bwd_blocks(rows).  dim a multiple of 8, at most 4096.
cudaError_t rmsnorm_gain_fwd_launch(const void* x, const void* gain, int gain_type, void* y, float* rstd,
                                    long long rows, int dim, float eps, cudaStream_t s);
int rmsnorm_gain_bwd_blocks(long long rows);
cudaError_t rmsnorm_gain_bwd_launch(const void* dy, const void* x, const float* rstd, const void* gain, int gain_type,
                                    void* dx, float* partial, int blocks, long long rows, int dim, cudaStream_t s);
// SwiGLU gate on bf16: h = silu(g) * u;  dg = dh * u * s * (1 + g * (1 - s)), du = dh * g * s, s = sigmoid(g)
cudaError_t swiglu_fwd_launch(const void* g, const void* u, void* h, long long n, cudaStream_t s);
cudaError_t swiglu_bwd_launch(const void* dh, const void* g, const void* u, void* dg, void* du, long long n,
                              cudaStream_t s);

// ---------------------------------------------------------------------------
// Dense linear algebra on small matrices (one CTA per matrix, fp32)
// ---------------------------------------------------------------------------
// For each of `batch` symmetric positive (semi-)definite r x r matrices G (row-major,
// pitch ldg): computes the upper Cholesky factor R (G = R^T R) with pivot clamping and
// writes Rinv = R^{-1} (upper triangular, zeros below the diagonal).
// `info[b]` counts clamped pivots.  `work` is scratch of batch * r * r floats.
// `jacobi` = false skips the unit-diagonal scaling (the pivot floor is then absolute); `colmask` (optional,
// fp32 [batch][r]) receives 1 for every column that was factorised and 0 for every clamped pivot.
cudaError_t chol_inverse_launch(const float* G, float* Rinv, float* work, int* info, int batch, int r,
                                long long ldg, long long g_batch_stride, float pivot_floor_rel, cudaStream_t s,
                                bool jacobi = true, float* colmask = nullptr);

// Column sums of squares: out[b, j] = sum_i X[b, i, j]^2  (X fp32/bf16, row-major [batch, rows, cols])
cudaError_t col_sumsq_launch(const void* X, int x_type, float* out, int batch, long long rows, int cols,
                             long long ldx, long long batch_stride, cudaStream_t s);
// Causal flash attention forward on tcgen05: q [B*T, H*D], k / v [B*T, Hkv*D], out [B*T, H*D] bf16,
// lse [B, H, T] fp32 (natural log of the softmax denominator, for the backward pass); D is 64 or 128,
// T a multiple of 128.
cudaError_t attn_fwd_launch(const void* q, const void* k, const void* v, void* out, float* lse, int B, int T, int H,
                            int Hkv, int D, float scale, int* status, cudaStream_t stream);
// Backward of the same attention: dq [B*T, H*D], dk / dv [B*T, Hkv*D] (bf16) from q, k, v, the forward's
// output `o` and log-sum-exp `lse`, and the output gradient `d_o`; `delta` is a [B, H, T] fp32 workspace.
cudaError_t attn_bwd_launch(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                            const float* lse, float* delta, void* dq, void* dk, void* dv, int B, int T, int H, int Hkv,
                            int D, float scale, int* status, cudaStream_t stream);
// Pieces of the blocked Cholesky-inverse: W = D G D with d = rsqrt(diag G) (contiguous W [batch][r][r], d
// [batch][r]); and the placement of a diagonal block's inverse factor Zd ([batch][nb][nb]) into Z at (k0, k0)
// together with its copy Zm whose rows of clamped pivots (mask == 0) are zero.
cudaError_t jacobi_scale_launch(const float* G, float* W, float* d, int batch, int r, long long ldg,
                                long long g_batch_stride, cudaStream_t s);
cudaError_t place_block_launch(const float* Zd, const float* mask, float* Z, float* Zm, int batch, int nb, int r, int k0,
                               cudaStream_t s);
// hi / lo halves of fp32 data for 3xTF32 products; all three pointers 16-byte aligned
cudaError_t split_tf32_launch(const float* x, float* hi, float* lo, long long numel, cudaStream_t s);
// the same for a strided [batch][rows][cols] source (element (b, i, j) at b * bs + i * ld + j; cols, ld and bs
// multiples of 4) into contiguous hi / lo
cudaError_t split_tf32_rows_launch(const float* x, float* hi, float* lo, int batch, int rows, int cols, long long ld,
                                   long long bs, cudaStream_t s);
// d = rsqrt(diag G) (0 where the diagonal is not above `dead_below`), C = strictly lower part of D G D
// (all zero for matrices b with skip[b] != 0, `skip` may be null); contiguous [batch, r, r]
// With `fold`, column j of C is scaled by d_j once more (see the kernel).
cudaError_t refine_prep_launch(const float* G, float* C, float* d, int batch, int r, float dead_below,
                               const int* skip, bool fold, cudaStream_t s);

// ---------------------------------------------------------------------------
// Collectives over symmetric memory (one arena per process group; the same offset names
// the same logical buffer on every rank).  `PeerTable` holds the arena base address of
// every rank as seen from this GPU; `flag_off` is the byte offset of the arena's flag
// block (4 channels x kMaxPeers unsigned words, zeroed at creation); epochs grow by one
// per collective on a channel.
// ---------------------------------------------------------------------------
constexpr int kMaxPeers = 8;
struct PeerTable {
  void* ptrs[kMaxPeers];
};
cudaError_t symm_barrier_launch(const PeerTable& t, long long flag_off, int channel, int rank, int world,
                                unsigned epoch, int* status, cudaStream_t s);
// In-place sum (times `scale`) over all ranks of `numel` elements at `data_off`; `mc_base`
// is the multicast address of the arena or null for plain peer loads and stores.
cudaError_t symm_all_reduce_launch(const PeerTable& t, long long flag_off, long long data_off, void* mc_base,
                                   int elem_type, long long numel, float scale, int rank, int world, unsigned epoch,
                                   unsigned* done_counter, int* status, cudaStream_t s);
// dst = beta * dst + scale * sum over ranks of the buffer at `data_off`; dst is local memory.
cudaError_t symm_reduce_into_launch(const PeerTable& t, long long flag_off, long long data_off, int src_type,
                                    void* dst, int dst_type, long long numel, float scale, float beta, int rank,
                                    int world, unsigned epoch, unsigned* done_counter, int* status, cudaStream_t s);
// FSDP-style collectives: all-gather through a double-buffered symmetric staging slot (in / out
// are ordinary local buffers) and reduce-scatter of a symmetric input into an ordinary output.
// `budget_ns` bounds every wait on a peer.
cudaError_t symm_all_gather_launch(const PeerTable& t, long long flag_off, long long slot_off, const void* in,
                                   void* out, long long bytes, int rank, int world, unsigned epoch, int channel,
                                   unsigned* done_counter, int* status, long long budget_ns, cudaStream_t s);
cudaError_t symm_reduce_scatter_launch(const PeerTable& t, long long flag_off, long long data_off, void* mc_base,
                                       int elem_type, void* out, long long numel, float scale, int rank, int world,
                                       unsigned epoch, int ch_start, int ch_end, unsigned* done_counter, int* status,
                                       long long budget_ns, cudaStream_t s);

// ---------------------------------------------------------------------------
// Reductions over ranks fused with Dion's arithmetic (dion_fused.cu).  A "slot buffer" is
// `nslots` equally shaped fp32 arrays, `slot_stride` elements apart, in this GPU's part of a
// symmetric arena: slot s holds what rank s contributed (stored there by that rank's GEMM
// epilogue or reduction kernel with peer stores).  `SlotWait` describes the flag exchange that
// tells the consumer the slots are complete (world <= 1: nothing to wait for).
// ---------------------------------------------------------------------------
struct SlotWait {
  PeerTable peers;
  long long flag_off;
  int channel, rank, world;
  unsigned epoch;
  unsigned long long budget_ns;
};

// out = scale * (slot 0 + slot 1 + ...), summed in slot order; optionally also its tf32 halves
// (hi = low 13 mantissa bits cleared, lo = out - hi) and copies to `ndest` further addresses
// (slots of a second group, for a hierarchical reduction).  numel and slot_stride multiples of 4.
struct SlotReduceArgs {
  SlotWait wait;
  const float* slots;
  long long slot_stride;
  int nslots;
  long long numel;
  float scale;
  float* out;  // may be null
  float* hi;   // both or neither
  float* lo;
  int ndest;
  float* dest[kMaxPeers];
  int* status;
};
cudaError_t slot_reduce_launch(const SlotReduceArgs& a, cudaStream_t s);

// The same for bf16 activations: out = slot 0 + slot 1 + ... (+ residual), accumulated in fp32 in slot
// order; numel and slot_stride multiples of 8, 16-byte aligned pointers.
struct SlotReduceBf16Args {
  SlotWait wait;
  const void* slots;
  long long slot_stride;
  int nslots;
  long long numel;
  const void* residual;  // may be null
  void* out;
  int* status;
};
cudaError_t slot_reduce_bf16_launch(const SlotReduceBf16Args& a, cudaStream_t s);

// After R = A^T P (contiguous [B][n][r] per slot): R <- scale * sum of slots; for a matrix whose
// momentum is all zero (nonzero[b] == 0) R <- previous Q and P <- 0, otherwise NaN / inf are
// replaced in R and P (dion/dion.py:1416-1444); R32 (fp32, optional) and Rm (momentum dtype,
// optional) receive R, ss[b][j] the column sums of squares.  With `finish` the kernel also writes
// the new Q = R / (sqrt(ss) + eps) per column (previous Q where ss == 0) to Qn ([B][n][r], optional)
// and columns [qs_col0, qs_col0 + qs_cols) of it to Qs ([B][n][qs_cols], optional).
// Qm: previous Q with all r columns, element (b, i, j) at b * q_bs + i * q_ld + j.
// P: [B][p_rows][r] with pitches p_ld / p_bs, modified in place (may be null).
struct RPostArgs {
  SlotWait wait;
  const float* slots;
  long long slot_stride;
  int nslots;
  float scale;
  int B, n, r;
  const int* nonzero;
  const void* Qm;
  int q_type;
  long long q_ld, q_bs;
  void* P;
  int p_type;
  long long p_rows, p_ld, p_bs;
  float* R32;
  void* Rm;
  int rm_type;
  float* ss;
  int finish;
  float eps;
  void* Qn;
  int qn_type;
  void* Qs;
  int qs_type;
  int qs_col0, qs_cols;
  int* status;
};
cudaError_t r_post_launch(const RPostArgs& a, cudaStream_t s);

// The column normalisation alone: Qn / Qs from R32 and the (already reduced) ss.
struct QNormArgs {
  const float* R32;
  const float* ss;
  int B, n, r;
  float eps;
  const void* Qm;
  int q_type;
  long long q_ld, q_bs;
  void* Qn;
  int qn_type;
  void* Qs;
  int qs_type;
  int qs_col0, qs_cols;
};
cudaError_t q_norm_launch(const QNormArgs& a, cudaStream_t s);

}  // namespace dion
