// torch bindings for the sm_100a kernels of dion_b200.  Registered as
// torch.ops.dion_b200.* by loading the shared library; no Python C-API use.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/torch.h>

#include "gemm.h"
#include "kernels.h"

#include <atomic>

namespace {

using at::Tensor;

// Number of kernel launches issued through this library (for benchmarks and tests).
std::atomic<long long> g_launches{0};
int64_t launch_count() { return (int64_t)g_launches.load(); }

// host only: the tiling and copy schedule the all-gather GEMM would use (empty if the shapes do not fit)
std::vector<int64_t> gemm_gather_plan(int64_t M, int64_t N, int64_t K, int64_t rows, int64_t world, int64_t rank) {
  dion::GemmArgs g;
  g.ab_dtype = dion::kBF16;
  g.M = (int)M;
  g.N = (int)N;
  g.K = (int)K;
  g.lda = K;
  g.ldb = K;
  g.gather.world = (int)world;
  g.gather.rank = (int)rank;
  g.gather.rows = (int)rows;
  int out[8];
  if (!dion::gemm_gather_plan(g, out)) return {};
  return std::vector<int64_t>(out, out + 8);
}

int gemm_dtype(const Tensor& t, const char* what) {
  if (t.scalar_type() == at::kBFloat16) return dion::kBF16;
  if (t.scalar_type() == at::kFloat) return dion::kF32;
  TORCH_CHECK(false, what, " must be bfloat16 or float32, got ", t.scalar_type());
}

// Describe a logical (rows x cols) matrix view: returns major + pitch.
// `contract_last` says whether the contraction (K) dimension is the last logical dim.
void describe_operand(const Tensor& t, bool contract_last, int* major, int64_t* ld, int64_t* bstride,
                      const char* what) {
  TORCH_CHECK(t.dim() == 2 || t.dim() == 3, what, " must be 2-D or 3-D");
  const int64_t s_row = t.stride(-2), s_col = t.stride(-1);
  const int64_t rows = t.size(-2), cols = t.size(-1);
  bool last_contig;
  if (s_col == 1 && (s_row >= cols || rows == 1)) {
    last_contig = true;
    *ld = rows == 1 ? std::max<int64_t>(s_row, cols) : s_row;
  } else if (s_row == 1 && (s_col >= rows || cols == 1)) {
    last_contig = false;
    *ld = cols == 1 ? std::max<int64_t>(s_col, rows) : s_col;
  } else {
    TORCH_CHECK(false, what, " needs a unit stride in one of its last two dimensions; strides = ", t.strides());
  }
  // K-major means the contraction dimension is the contiguous one.
  *major = (last_contig == contract_last) ? dion::kMajorK : dion::kMajorMN;
  *bstride = t.dim() == 3 ? t.stride(0) : 0;
}

void check_out(const Tensor& t, int64_t batch, int64_t M, int64_t N, const char* what) {
  TORCH_CHECK(t.is_cuda(), what, " must be a CUDA tensor");
  TORCH_CHECK(t.dim() == 2 || t.dim() == 3, what, " must be 2-D or 3-D");
  TORCH_CHECK(t.size(-2) == M && t.size(-1) == N, what, " has shape ", t.sizes(), ", expected (.., ", M, ", ", N, ")");
  TORCH_CHECK((t.dim() == 3 ? t.size(0) : 1) == batch, what, " batch mismatch");
  TORCH_CHECK(t.stride(-1) == 1, what, " must be row-major");
}

// d = act(alpha * a @ b) + beta * c   (a: [B,]M,K   b: [B,]K,N, any transposed views)
void gemm(const Tensor& a, const Tensor& b, const std::optional<Tensor>& c, Tensor d,
          const std::optional<Tensor>& d2, const std::optional<Tensor>& c_ptrs,
          const std::optional<Tensor>& d_ptrs, const std::optional<Tensor>& d2_ptrs, double alpha, double beta,
          int64_t act, int64_t epilogue, int64_t split_k, bool symmetric, int64_t block_n, int64_t pair,
          const std::optional<Tensor>& status, int64_t d_dup, const std::optional<Tensor>& a_lo,
          const std::optional<Tensor>& b_lo, const std::optional<Tensor>& c_col_scale, bool split3) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda(), "gemm operands must be CUDA tensors");
  TORCH_CHECK(a.scalar_type() == b.scalar_type(), "gemm operands must share a dtype");
  TORCH_CHECK(a.dim() == b.dim(), "gemm operands must both be 2-D or both 3-D");
  const c10::cuda::CUDAGuard guard(a.device());
  dion::GemmArgs g;
  g.ab_dtype = gemm_dtype(a, "a");
  g.M = (int)a.size(-2);
  g.K = (int)a.size(-1);
  g.N = (int)b.size(-1);
  TORCH_CHECK(b.size(-2) == g.K, "gemm inner dimensions differ: ", a.sizes(), " x ", b.sizes());
  g.batch = a.dim() == 3 ? (int)a.size(0) : 1;
  if (a.dim() == 3) TORCH_CHECK(b.size(0) == g.batch, "gemm batch sizes differ");
  describe_operand(a, /*contract_last=*/true, &g.a_major, &g.lda, &g.a_batch_stride, "a");
  describe_operand(b, /*contract_last=*/false, &g.b_major, &g.ldb, &g.b_batch_stride, "b");
  g.A = a.data_ptr();
  g.B = b.data_ptr();
  TORCH_CHECK(a_lo.has_value() == b_lo.has_value(), "hi / lo operands need both low halves");
  if (split3) {
    TORCH_CHECK(a.scalar_type() == at::kFloat && !a_lo.has_value(), "split3 takes fp32 operands without low halves");
    g.split3 = 1;
  }
  if (a_lo.has_value()) {
    TORCH_CHECK(a.scalar_type() == at::kFloat, "hi / lo operands are fp32");
    TORCH_CHECK(a_lo->is_cuda() && b_lo->is_cuda() && a_lo->scalar_type() == at::kFloat && b_lo->scalar_type() == at::kFloat &&
                a_lo->sizes() == a.sizes() && a_lo->strides() == a.strides() && b_lo->sizes() == b.sizes() &&
                b_lo->strides() == b.strides(), "low halves must have the layout of the high halves");
    g.A_lo = a_lo->data_ptr();
    g.B_lo = b_lo->data_ptr();
  }
  g.alpha = (float)alpha;
  g.beta = (float)beta;
  g.act = (int)act;
  g.epilogue = (int)epilogue;
  g.split_k = (int)split_k;
  g.symmetric = symmetric ? 1 : 0;
  g.block_n = (int)block_n;
  g.pair = (int)pair;

  // Per-batch pointer arrays (int64 CUDA tensors) describe outputs that are separate
  // allocations; `d` / `c` then only supply dtype, shape and pitch of one element.
  if (d_ptrs.has_value()) {
    TORCH_CHECK(d_dup >= 1 && d_dup <= dion::kMaxPeers, "d_dup out of range");
    TORCH_CHECK(d_ptrs->scalar_type() == at::kLong && d_ptrs->is_cuda() && d_ptrs->is_contiguous() &&
                d_ptrs->numel() >= g.batch * d_dup);
    TORCH_CHECK(d.dim() == 2 && d.size(0) == g.M && d.size(1) == g.N && d.stride(1) == 1);
    g.d_ptrs = reinterpret_cast<void* const*>(d_ptrs->data_ptr<int64_t>());
    g.d_dup = (int)d_dup;
  } else {
    check_out(d, g.batch, g.M, g.N, "d");
    g.d_batch_stride = d.dim() == 3 ? d.stride(0) : 0;
  }
  g.D = d.data_ptr();
  g.d_dtype = gemm_dtype(d, "d");
  g.ldd = d.stride(-2);
  if (c.has_value()) {
    const Tensor& ct = *c;
    if (c_ptrs.has_value()) {
      TORCH_CHECK(c_ptrs->scalar_type() == at::kLong && c_ptrs->is_cuda() && c_ptrs->numel() >= g.batch);
      g.c_ptrs = reinterpret_cast<const void* const*>(c_ptrs->data_ptr<int64_t>());
    } else {
      check_out(ct, g.batch, g.M, g.N, "c");
      g.c_batch_stride = ct.dim() == 3 ? ct.stride(0) : 0;
    }
    g.C = ct.data_ptr();
    g.c_dtype = gemm_dtype(ct, "c");
    g.ldc = ct.stride(-2);
  }
  if (c_col_scale.has_value()) {
    TORCH_CHECK(c.has_value(), "a column scale needs the addend c");
    TORCH_CHECK(c_col_scale->is_cuda() && c_col_scale->scalar_type() == at::kFloat && c_col_scale->is_contiguous() &&
                c_col_scale->numel() == (int64_t)g.batch * g.N, "c_col_scale must be contiguous fp32 [batch, N]");
    g.c_col_scale = c_col_scale->data_ptr<float>();
  }
  if (d2.has_value()) {
    const Tensor& t = *d2;
    TORCH_CHECK(t.scalar_type() == at::kBFloat16, "d2 must be bfloat16");
    if (d2_ptrs.has_value()) {
      TORCH_CHECK(d2_ptrs->scalar_type() == at::kLong && d2_ptrs->is_cuda() && d2_ptrs->numel() >= g.batch);
      g.d2_ptrs = reinterpret_cast<void* const*>(d2_ptrs->data_ptr<int64_t>());
    } else {
      check_out(t, g.batch, g.M, g.N, "d2");
      g.d2_batch_stride = t.dim() == 3 ? t.stride(0) : 0;
    }
    g.D2 = t.data_ptr();
    g.ldd2 = t.stride(-2);
  }
  if (status.has_value()) {
    TORCH_CHECK(status->scalar_type() == at::kInt && status->is_cuda());
    g.status = status->data_ptr<int>();
  }
  cudaError_t e = dion::gemm_launch(g, at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(e == cudaSuccess, "dion_b200 gemm launch failed: ", cudaGetErrorString(e), " ",
              dion::gemm_last_error());
  g_launches.fetch_add(1, std::memory_order_relaxed);
}


// out-of-place product whose result tiles are scattered to per-destination blocks:
//   mode 1: block k = rows [k*block, (k+1)*block), mode 2: block k = columns [k*block, (k+1)*block).
// `block_like` gives dtype and row pitch of one block; `scatter_ptrs` holds batch * dests addresses.
void gemm_scatter(const Tensor& a, const Tensor& b, const std::optional<Tensor>& c, const Tensor& block_like,
                  const Tensor& scatter_ptrs, int64_t mode, int64_t block, int64_t dests, double alpha, double beta,
                  const std::optional<Tensor>& status) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.scalar_type() == b.scalar_type() && a.dim() == b.dim());
  const c10::cuda::CUDAGuard guard(a.device());
  dion::GemmArgs g;
  g.ab_dtype = gemm_dtype(a, "a");
  g.M = (int)a.size(-2);
  g.K = (int)a.size(-1);
  g.N = (int)b.size(-1);
  TORCH_CHECK(b.size(-2) == g.K, "gemm inner dimensions differ");
  g.batch = a.dim() == 3 ? (int)a.size(0) : 1;
  describe_operand(a, true, &g.a_major, &g.lda, &g.a_batch_stride, "a");
  describe_operand(b, false, &g.b_major, &g.ldb, &g.b_batch_stride, "b");
  g.A = a.data_ptr();
  g.B = b.data_ptr();
  g.alpha = (float)alpha;
  g.beta = (float)beta;
  if (c.has_value()) {
    check_out(*c, g.batch, g.M, g.N, "c");
    g.C = c->data_ptr();
    g.c_dtype = gemm_dtype(*c, "c");
    g.ldc = c->stride(-2);
    g.c_batch_stride = c->dim() == 3 ? c->stride(0) : 0;
  }
  TORCH_CHECK(block_like.dim() == 2 && block_like.stride(1) == 1);
  g.d_dtype = gemm_dtype(block_like, "block_like");
  g.ldd = block_like.stride(0);
  TORCH_CHECK(scatter_ptrs.scalar_type() == at::kLong && scatter_ptrs.is_cuda() &&
              scatter_ptrs.numel() >= (int64_t)g.batch * dests);
  g.scatter_ptrs = reinterpret_cast<void* const*>(scatter_ptrs.data_ptr<int64_t>());
  g.scatter_mode = (int)mode;
  g.scatter_block = (int)block;
  g.scatter_dests = (int)dests;
  if (status.has_value()) g.status = status->data_ptr<int>();
  cudaError_t e = dion::gemm_launch(g, at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(e == cudaSuccess, "dion_b200 gemm_scatter launch failed: ", cudaGetErrorString(e), " ",
              dion::gemm_last_error());
  g_launches.fetch_add(1, std::memory_order_relaxed);
}

// d = gathered(a) @ b with the all-gather of a's row blocks running inside the GEMM kernel:
// `x_local` [rows, K] are this rank's rows, `a_full` [world * rows, K] receives every rank's rows (it
// is the GEMM's operand, and stays valid afterwards), `b` is [K, N] K-major, `d` [world * rows, N].
void gemm_gather(const Tensor& x_local, Tensor a_full, const Tensor& b, Tensor d, at::IntArrayRef peers,
                 int64_t flag_off, int64_t slot_off, int64_t rank, int64_t epoch, int64_t channel, Tensor counters,
                 const std::optional<Tensor>& status, int64_t budget_ns) {
  TORCH_CHECK(x_local.is_cuda() && a_full.is_cuda() && b.is_cuda() && d.is_cuda());
  TORCH_CHECK(x_local.scalar_type() == at::kBFloat16 && a_full.scalar_type() == at::kBFloat16 &&
              b.scalar_type() == at::kBFloat16, "gemm_gather operands must be bfloat16");
  TORCH_CHECK(x_local.dim() == 2 && a_full.dim() == 2 && b.dim() == 2 && d.dim() == 2);
  TORCH_CHECK(x_local.is_contiguous() && a_full.is_contiguous());
  const int64_t world = (int64_t)peers.size();
  TORCH_CHECK(world >= 1 && world <= dion::kGatherMaxPeers && rank >= 0 && rank < world);
  TORCH_CHECK(a_full.size(0) == x_local.size(0) * world && a_full.size(1) == x_local.size(1),
              "a_full must hold every rank's rows");
  TORCH_CHECK(counters.scalar_type() == at::kInt && counters.is_cuda() && counters.is_contiguous());
  const c10::cuda::CUDAGuard guard(x_local.device());
  dion::GemmArgs g;
  g.ab_dtype = dion::kBF16;
  g.M = (int)a_full.size(0);
  g.K = (int)a_full.size(1);
  g.N = (int)b.size(1);
  TORCH_CHECK(b.size(0) == g.K, "gemm inner dimensions differ");
  describe_operand(a_full, true, &g.a_major, &g.lda, &g.a_batch_stride, "a_full");
  describe_operand(b, false, &g.b_major, &g.ldb, &g.b_batch_stride, "b");
  g.A = a_full.data_ptr();
  g.B = b.data_ptr();
  check_out(d, 1, g.M, g.N, "d");
  g.D = d.data_ptr();
  g.d_dtype = gemm_dtype(d, "d");
  g.ldd = d.stride(-2);
  g.gather.world = (int)world;
  g.gather.rank = (int)rank;
  g.gather.rows = (int)x_local.size(0);
  g.gather.in = x_local.data_ptr();
  for (int64_t i = 0; i < world; ++i) g.gather.peers[i] = reinterpret_cast<void*>(peers[i]);
  g.gather.flag_off = flag_off;
  g.gather.slot_off = slot_off;
  g.gather.epoch = (unsigned)epoch;
  g.gather.channel = (int)channel;
  g.gather.counters = reinterpret_cast<unsigned*>(counters.data_ptr<int>());
  g.gather.counter_words = (int)counters.numel();
  g.gather.budget_ns = budget_ns;
  if (status.has_value()) g.status = status->data_ptr<int>();
  cudaError_t e = dion::gemm_launch(g, at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(e == cudaSuccess, "dion_b200 gemm_gather launch failed: ", cudaGetErrorString(e), " ",
              dion::gemm_last_error());
  g_launches.fetch_add(1, std::memory_order_relaxed);
}

// ----------------------------------------------------------------------------- multi-tensor helpers

int elem_type(const Tensor& t, const char* what) {
  if (t.scalar_type() == at::kFloat) return dion::kElemF32;
  if (t.scalar_type() == at::kBFloat16) return dion::kElemBF16;
  TORCH_CHECK(false, what, " must be float32 or bfloat16, got ", t.scalar_type());
}

void check_list(at::TensorList ref, at::TensorList other, const char* what) {
  TORCH_CHECK(ref.size() == other.size(), what, ": list length mismatch");
  for (size_t i = 0; i < ref.size(); ++i) {
    TORCH_CHECK(other[i].is_cuda() && other[i].is_contiguous(), what, ": tensors must be contiguous CUDA tensors");
    TORCH_CHECK(other[i].numel() == ref[i].numel(), what, ": element count mismatch at index ", i);
    TORCH_CHECK(other[i].scalar_type() == other[0].scalar_type(), what, ": mixed dtypes in one list");
  }
}

// Calls fn(chunk, first_tensor_index) for consecutive groups of tensors.
template <typename Fn>
void for_each_chunk(std::initializer_list<std::pair<int, at::TensorList>> lists, Fn fn) {
  const at::TensorList& ref = lists.begin()->second;
  const int64_t n = (int64_t)ref.size();
  const int block_elems = dion::multi_tensor_block_elems();
  int64_t i = 0;
  while (i < n) {
    dion::TensorListChunk c;
    memset(&c, 0, sizeof(c));
    int k = 0;
    int blocks = 0;
    const int64_t first = i;
    while (i < n && k < dion::kMaxTensorsPerLaunch) {
      const int64_t numel = ref[i].numel();
      for (const auto& l : lists) c.ptrs[l.first][k] = l.second[i].data_ptr();
      c.numel[k] = numel;
      c.block_start[k] = blocks;
      blocks += (int)((numel + block_elems - 1) / block_elems);
      ++k;
      ++i;
    }
    c.block_start[k] = blocks;
    c.num_tensors = k;
    fn(c, first);
  }
}

#define DION_CUDA_CHECK(expr)                                                           \
  do {                                                                                  \
    cudaError_t _e = (expr);                                                            \
    TORCH_CHECK(_e == cudaSuccess, "dion_b200 kernel launch failed: ", cudaGetErrorString(_e)); \
    g_launches.fetch_add(1, std::memory_order_relaxed);                                 \
  } while (0)

void adamw_multi(at::TensorList X, at::TensorList G, at::TensorList M, at::TensorList V, at::TensorList shadow,
                 double lr, double beta1, double beta2, double weight_decay, double eps, int64_t step) {
  if (X.empty()) return;
  const c10::cuda::CUDAGuard guard(X[0].device());
  check_list(X, X, "X");
  check_list(X, G, "G");
  check_list(X, M, "M");
  check_list(X, V, "V");
  TORCH_CHECK(X[0].scalar_type() == at::kFloat, "adamw_multi updates float32 parameters");
  const bool has_shadow = !shadow.empty();
  if (has_shadow) {
    check_list(X, shadow, "shadow");
    TORCH_CHECK(shadow[0].scalar_type() == at::kBFloat16);
  }
  dion::AdamWHyper h;
  h.lr = (float)lr;
  h.beta1 = (float)beta1;
  h.beta2 = (float)beta2;
  h.weight_decay = (float)weight_decay;
  h.eps = (float)eps;
  h.bias_correction1 = (float)(1.0 - std::pow(beta1, (double)step));
  h.bias_correction2_sqrt = (float)std::sqrt(1.0 - std::pow(beta2, (double)step));
  auto stream = at::cuda::getCurrentCUDAStream();
  const int gt = elem_type(G[0], "G"), mt = elem_type(M[0], "M"), vt = elem_type(V[0], "V");
  auto run = [&](const dion::TensorListChunk& c, int64_t) {
    DION_CUDA_CHECK(dion::adamw_multi_launch(c, gt, mt, vt, has_shadow, h, stream));
  };
  if (has_shadow) for_each_chunk({{0, X}, {1, G}, {2, M}, {3, V}, {4, shadow}}, run);
  else for_each_chunk({{0, X}, {1, G}, {2, M}, {3, V}}, run);
}

void lion_multi(at::TensorList X, at::TensorList G, at::TensorList M, at::TensorList shadow, double lr,
                double beta1, double beta2, double weight_decay) {
  if (X.empty()) return;
  const c10::cuda::CUDAGuard guard(X[0].device());
  check_list(X, X, "X");
  check_list(X, G, "G");
  check_list(X, M, "M");
  TORCH_CHECK(X[0].scalar_type() == at::kFloat, "lion_multi updates float32 parameters");
  const bool has_shadow = !shadow.empty();
  if (has_shadow) {
    check_list(X, shadow, "shadow");
    TORCH_CHECK(shadow[0].scalar_type() == at::kBFloat16);
  }
  dion::LionHyper h{(float)lr, (float)beta1, (float)beta2, (float)weight_decay};
  auto stream = at::cuda::getCurrentCUDAStream();
  const int gt = elem_type(G[0], "G"), mt = elem_type(M[0], "M");
  auto run = [&](const dion::TensorListChunk& c, int64_t) {
    DION_CUDA_CHECK(dion::lion_multi_launch(c, gt, mt, has_shadow, h, stream));
  };
  if (has_shadow) for_each_chunk({{0, X}, {1, G}, {2, M}, {4, shadow}}, run);
  else for_each_chunk({{0, X}, {1, G}, {2, M}}, run);
}

void muon_pre_multi(at::TensorList G, at::TensorList M, at::TensorList U, double mu, bool nesterov,
                    const std::optional<Tensor>& sumsq) {
  if (G.empty()) return;
  const c10::cuda::CUDAGuard guard(G[0].device());
  check_list(G, G, "G");
  check_list(G, M, "M");
  check_list(G, U, "U");
  TORCH_CHECK(M[0].scalar_type() == at::kFloat && U[0].scalar_type() == at::kBFloat16);
  float* ss = nullptr;
  if (sumsq.has_value()) {
    TORCH_CHECK(sumsq->scalar_type() == at::kFloat && sumsq->is_cuda() && sumsq->numel() >= (int64_t)G.size());
    ss = sumsq->data_ptr<float>();
  }
  auto stream = at::cuda::getCurrentCUDAStream();
  const int gt = elem_type(G[0], "G");
  for_each_chunk({{0, G}, {1, M}, {2, U}}, [&](const dion::TensorListChunk& c, int64_t first) {
    DION_CUDA_CHECK(dion::muon_pre_multi_launch(c, gt, (float)mu, nesterov, ss ? ss + first : nullptr, stream));
  });
}

// x, out: contiguous bf16 [B, ...]; sumsq: optional fp32 [B] squared Frobenius norms
void frob_scale(const Tensor& x, Tensor out, const std::optional<Tensor>& sumsq, double eps) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16 && x.dim() >= 2 &&
              x.is_contiguous() && out.is_contiguous() && out.numel() == x.numel());
  const int64_t B = x.size(0), per = x.numel() / std::max<int64_t>(B, 1);
  const float* ss = nullptr;
  Tensor partial;
  if (sumsq.has_value()) {
    TORCH_CHECK(sumsq->scalar_type() == at::kFloat && sumsq->is_contiguous() && sumsq->numel() >= B);
    ss = sumsq->data_ptr<float>();
    g_launches += 1;
  } else {
    partial = at::empty({B * dion::frob_chunks(per)}, x.options().dtype(at::kFloat));
    g_launches += 2;
  }
  DION_CUDA_CHECK(dion::frob_scale_launch(x.data_ptr(), out.data_ptr(), ss ? nullptr : partial.data_ptr<float>(), ss,
                                          (float)eps, (int)B, per, at::cuda::getCurrentCUDAStream()));
}

void muon_post_multi(at::TensorList X, at::TensorList U, at::TensorList shadow, double decay, double step) {
  if (X.empty()) return;
  const c10::cuda::CUDAGuard guard(X[0].device());
  check_list(X, X, "X");
  check_list(X, U, "U");
  TORCH_CHECK(X[0].scalar_type() == at::kFloat && U[0].scalar_type() == at::kBFloat16);
  const bool has_shadow = !shadow.empty();
  if (has_shadow) check_list(X, shadow, "shadow");
  auto stream = at::cuda::getCurrentCUDAStream();
  auto run = [&](const dion::TensorListChunk& c, int64_t) {
    DION_CUDA_CHECK(dion::muon_post_multi_launch(c, has_shadow, (float)decay, (float)step, stream));
  };
  if (has_shadow) for_each_chunk({{0, X}, {1, U}, {4, shadow}}, run);
  else for_each_chunk({{0, X}, {1, U}}, run);
}

void dion_accum_multi(at::TensorList G, at::TensorList M, const std::optional<Tensor>& nonzero) {
  if (G.empty()) return;
  const c10::cuda::CUDAGuard guard(G[0].device());
  check_list(G, G, "G");
  check_list(G, M, "M");
  int* nz = nullptr;
  if (nonzero.has_value()) {
    TORCH_CHECK(nonzero->scalar_type() == at::kInt && nonzero->is_cuda() && nonzero->numel() >= (int64_t)G.size());
    nz = nonzero->data_ptr<int>();
  }
  auto stream = at::cuda::getCurrentCUDAStream();
  const int gt = elem_type(G[0], "G"), mt = elem_type(M[0], "M");
  for_each_chunk({{0, G}, {1, M}}, [&](const dion::TensorListChunk& c, int64_t first) {
    DION_CUDA_CHECK(dion::dion_accum_multi_launch(c, gt, mt, nz ? nz + first : nullptr, stream));
  });
}

void cast_multi(at::TensorList src, at::TensorList dst) {
  if (src.empty()) return;
  const c10::cuda::CUDAGuard guard(src[0].device());
  check_list(src, src, "src");
  check_list(src, dst, "dst");
  auto stream = at::cuda::getCurrentCUDAStream();
  const int st = elem_type(src[0], "src"), dt = elem_type(dst[0], "dst");
  for_each_chunk({{0, src}, {1, dst}}, [&](const dion::TensorListChunk& c, int64_t) {
    DION_CUDA_CHECK(dion::cast_multi_launch(c, st, dt, stream));
  });
}

// ----------------------------------------------------------------------------- model kernels

void check_bf16(const Tensor& t, const char* what) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.is_contiguous(), what,
              " must be a contiguous CUDA bfloat16 tensor");
}

void rmsnorm_fwd(const Tensor& x, const std::optional<Tensor>& residual, const std::optional<Tensor>& x_out,
                 Tensor y, Tensor rstd, double eps) {
  check_bf16(x, "x");
  check_bf16(y, "y");
  const c10::cuda::CUDAGuard guard(x.device());
  const int dim = (int)x.size(-1);
  const int64_t rows = x.numel() / dim;
  TORCH_CHECK(rstd.scalar_type() == at::kFloat && rstd.numel() == rows);
  const void* res = nullptr;
  void* xo = nullptr;
  if (residual.has_value()) {
    check_bf16(*residual, "residual");
    res = residual->data_ptr();
  }
  if (x_out.has_value()) {
    check_bf16(*x_out, "x_out");
    xo = x_out->data_ptr();
  }
  DION_CUDA_CHECK(dion::rmsnorm_fwd_launch(x.data_ptr(), res, xo, y.data_ptr(), rstd.data_ptr<float>(), rows, dim,
                                           (float)eps, at::cuda::getCurrentCUDAStream()));
}

void rmsnorm_gain_fwd(const Tensor& x, const Tensor& gain, Tensor y, Tensor rstd, double eps) {
  check_bf16(x, "x");
  check_bf16(y, "y");
  const c10::cuda::CUDAGuard guard(x.device());
  const int dim = (int)x.size(-1);
  const int64_t rows = x.numel() / dim;
  TORCH_CHECK(x.is_contiguous() && y.is_contiguous() && gain.is_contiguous() && gain.numel() == dim);
  TORCH_CHECK(rstd.scalar_type() == at::kFloat && rstd.numel() == rows);
  ++g_launches;
  DION_CUDA_CHECK(dion::rmsnorm_gain_fwd_launch(x.data_ptr(), gain.data_ptr(), elem_type(gain, "gain"), y.data_ptr(),
                                                rstd.data_ptr<float>(), rows, dim, (float)eps,
                                                at::cuda::getCurrentCUDAStream()));
}

// returns the per-block partial sums of the gain's gradient, [blocks, dim] fp32
Tensor rmsnorm_gain_bwd(const Tensor& dy, const Tensor& x, const Tensor& rstd, const Tensor& gain, Tensor dx) {
  check_bf16(dy, "dy");
  check_bf16(x, "x");
  check_bf16(dx, "dx");
  const c10::cuda::CUDAGuard guard(x.device());
  const int dim = (int)x.size(-1);
  const int64_t rows = x.numel() / dim;
  TORCH_CHECK(dy.is_contiguous() && x.is_contiguous() && dx.is_contiguous() && gain.is_contiguous() && gain.numel() == dim);
  const int blocks = dion::rmsnorm_gain_bwd_blocks(rows);
  Tensor partial = at::empty({blocks, dim}, x.options().dtype(at::kFloat));
  ++g_launches;
  DION_CUDA_CHECK(dion::rmsnorm_gain_bwd_launch(dy.data_ptr(), x.data_ptr(), rstd.data_ptr<float>(), gain.data_ptr(),
                                                elem_type(gain, "gain"), dx.data_ptr(), partial.data_ptr<float>(), blocks,
                                                rows, dim, at::cuda::getCurrentCUDAStream()));
  return partial;
}

void swiglu_fwd(const Tensor& g, const Tensor& u, Tensor h) {
  check_bf16(g, "g");
  check_bf16(u, "u");
  check_bf16(h, "h");
  const c10::cuda::CUDAGuard guard(g.device());
  TORCH_CHECK(g.is_contiguous() && u.is_contiguous() && h.is_contiguous() && u.numel() == g.numel() && h.numel() == g.numel());
  ++g_launches;
  DION_CUDA_CHECK(dion::swiglu_fwd_launch(g.data_ptr(), u.data_ptr(), h.data_ptr(), g.numel(), at::cuda::getCurrentCUDAStream()));
}

void swiglu_bwd(const Tensor& dh, const Tensor& g, const Tensor& u, Tensor dg, Tensor du) {
  check_bf16(dh, "dh");
  check_bf16(g, "g");
  check_bf16(u, "u");
  check_bf16(dg, "dg");
  check_bf16(du, "du");
  const c10::cuda::CUDAGuard guard(g.device());
  TORCH_CHECK(dh.is_contiguous() && g.is_contiguous() && u.is_contiguous() && dg.is_contiguous() && du.is_contiguous());
  TORCH_CHECK(dh.numel() == g.numel() && u.numel() == g.numel() && dg.numel() == g.numel() && du.numel() == g.numel());
  ++g_launches;
  DION_CUDA_CHECK(dion::swiglu_bwd_launch(dh.data_ptr(), g.data_ptr(), u.data_ptr(), dg.data_ptr(), du.data_ptr(), g.numel(),
                                          at::cuda::getCurrentCUDAStream()));
}

void rmsnorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& rstd, const std::optional<Tensor>& dx_add,
                 Tensor dx) {
  check_bf16(dy, "dy");
  check_bf16(x, "x");
  check_bf16(dx, "dx");
  const c10::cuda::CUDAGuard guard(x.device());
  const int dim = (int)x.size(-1);
  const int64_t rows = x.numel() / dim;
  const void* add = nullptr;
  if (dx_add.has_value()) {
    check_bf16(*dx_add, "dx_add");
    add = dx_add->data_ptr();
  }
  DION_CUDA_CHECK(dion::rmsnorm_bwd_launch(dy.data_ptr(), x.data_ptr(), rstd.data_ptr<float>(), add, dx.data_ptr(),
                                           rows, dim, at::cuda::getCurrentCUDAStream()));
}

// q, k: [tokens, heads * head_dim] (row pitch = stride(0)); outputs contiguous [tokens, heads, head_dim]
void rope_qknorm_fwd(const Tensor& q, const Tensor& k, Tensor q_out, Tensor k_out, const Tensor& cos,
                     const Tensor& sin, int64_t seq_len, int64_t heads, int64_t head_dim, double eps) {
  const c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(q.dim() == 2 && k.dim() == 2 && q.stride(1) == 1 && k.stride(1) == 1 && q.stride(0) == k.stride(0));
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16);
  check_bf16(q_out, "q_out");
  check_bf16(k_out, "k_out");
  check_bf16(cos, "cos");
  check_bf16(sin, "sin");
  const int64_t tokens = q.size(0);
  TORCH_CHECK(q.size(1) == heads * head_dim && cos.size(-1) == head_dim / 2 && cos.numel() >= seq_len * head_dim / 2);
  DION_CUDA_CHECK(dion::rope_qknorm_fwd_launch(q.data_ptr(), k.data_ptr(), q_out.data_ptr(), k_out.data_ptr(),
                                               cos.data_ptr(), sin.data_ptr(), tokens, (int)seq_len, (int)heads,
                                               (int)head_dim, q.stride(0), heads * head_dim, (float)eps,
                                               at::cuda::getCurrentCUDAStream()));
}

void rope_qknorm_bwd(const Tensor& dq_out, const Tensor& dk_out, const Tensor& q, const Tensor& k, Tensor dq,
                     Tensor dk, const Tensor& cos, const Tensor& sin, int64_t seq_len, int64_t heads,
                     int64_t head_dim, double eps) {
  const c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(q.dim() == 2 && k.dim() == 2 && q.stride(1) == 1 && k.stride(1) == 1 && q.stride(0) == k.stride(0));
  TORCH_CHECK(dq.dim() == 2 && dk.dim() == 2 && dq.stride(1) == 1 && dk.stride(1) == 1 &&
              dq.stride(0) == q.stride(0) && dk.stride(0) == q.stride(0));
  check_bf16(dq_out, "dq_out");
  check_bf16(dk_out, "dk_out");
  const int64_t tokens = q.size(0);
  DION_CUDA_CHECK(dion::rope_qknorm_bwd_launch(dq_out.data_ptr(), dk_out.data_ptr(), q.data_ptr(), k.data_ptr(),
                                               dq.data_ptr(), dk.data_ptr(), cos.data_ptr(), sin.data_ptr(), tokens,
                                               (int)seq_len, (int)heads, (int)head_dim, q.stride(0),
                                               heads * head_dim, (float)eps, at::cuda::getCurrentCUDAStream()));
}

// rotary embedding of one tensor [tokens, heads * head_dim], no normalisation
void rope_fwd(const Tensor& x, Tensor out, const Tensor& cos, const Tensor& sin, int64_t seq_len, int64_t heads,
              int64_t head_dim) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && x.scalar_type() == at::kBFloat16 && x.size(1) == heads * head_dim);
  check_bf16(out, "out");
  check_bf16(cos, "cos");
  check_bf16(sin, "sin");
  DION_CUDA_CHECK(dion::rope_qknorm_fwd_launch(x.data_ptr(), nullptr, out.data_ptr(), nullptr, cos.data_ptr(),
                                               sin.data_ptr(), x.size(0), (int)seq_len, (int)heads, (int)head_dim,
                                               x.stride(0), heads * head_dim, -1.f,
                                               at::cuda::getCurrentCUDAStream()));
}
void rope_bwd(const Tensor& dout, const Tensor& x, Tensor dx, const Tensor& cos, const Tensor& sin, int64_t seq_len,
              int64_t heads, int64_t head_dim) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && dx.dim() == 2 && dx.stride(1) == 1 && dx.stride(0) == x.stride(0));
  check_bf16(dout, "dout");
  DION_CUDA_CHECK(dion::rope_qknorm_bwd_launch(dout.data_ptr(), nullptr, x.data_ptr(), nullptr, dx.data_ptr(),
                                               nullptr, cos.data_ptr(), sin.data_ptr(), x.size(0), (int)seq_len,
                                               (int)heads, (int)head_dim, x.stride(0), heads * head_dim, -1.f,
                                               at::cuda::getCurrentCUDAStream()));
}

void relu2_fwd(const Tensor& x, Tensor h) {
  check_bf16(x, "x");
  check_bf16(h, "h");
  const c10::cuda::CUDAGuard guard(x.device());
  DION_CUDA_CHECK(dion::relu2_fwd_launch(x.data_ptr(), h.data_ptr(), x.numel(), at::cuda::getCurrentCUDAStream()));
}
void relu2_bwd(const Tensor& dh, const Tensor& x, Tensor dx) {
  check_bf16(dh, "dh");
  check_bf16(x, "x");
  check_bf16(dx, "dx");
  const c10::cuda::CUDAGuard guard(x.device());
  DION_CUDA_CHECK(dion::relu2_bwd_launch(dh.data_ptr(), x.data_ptr(), dx.data_ptr(), x.numel(),
                                         at::cuda::getCurrentCUDAStream()));
}

void cross_entropy_fwd_bwd(Tensor logits, const Tensor& targets, Tensor row_loss, const std::optional<Tensor>& scale,
                           double grad_scale, int64_t ignore_index, bool write_grad) {
  const c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.scalar_type() == at::kBFloat16 && logits.stride(1) == 1);
  TORCH_CHECK(targets.is_cuda() && targets.scalar_type() == at::kLong && targets.is_contiguous() &&
              targets.numel() == logits.size(0));
  TORCH_CHECK(row_loss.scalar_type() == at::kFloat && row_loss.numel() == logits.size(0) && row_loss.is_contiguous());
  const float* sp = nullptr;
  if (scale.has_value()) {
    TORCH_CHECK(scale->scalar_type() == at::kFloat && scale->is_cuda());
    sp = scale->data_ptr<float>();
  }
  DION_CUDA_CHECK(dion::cross_entropy_fwd_bwd_launch(logits.data_ptr(), (const long long*)targets.data_ptr<int64_t>(),
                                                     row_loss.data_ptr<float>(), sp, logits.size(0),
                                                     (int)logits.size(1), logits.stride(0), (float)grad_scale,
                                                     ignore_index, write_grad, at::cuda::getCurrentCUDAStream()));
}

void embedding_fwd(const Tensor& table, const Tensor& idx, Tensor out) {
  const c10::cuda::CUDAGuard guard(table.device());
  TORCH_CHECK(table.is_cuda() && table.is_contiguous() && table.dim() == 2);
  TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == at::kLong && idx.is_contiguous());
  check_bf16(out, "out");
  DION_CUDA_CHECK(dion::embedding_fwd_launch(table.data_ptr(), elem_type(table, "table"),
                                             (const long long*)idx.data_ptr<int64_t>(), out.data_ptr(), idx.numel(),
                                             (int)table.size(1), at::cuda::getCurrentCUDAStream()));
}
void embedding_bwd(const Tensor& dout, const Tensor& idx, Tensor dtable) {
  const c10::cuda::CUDAGuard guard(dout.device());
  check_bf16(dout, "dout");
  TORCH_CHECK(dtable.is_cuda() && dtable.scalar_type() == at::kFloat && dtable.is_contiguous());
  DION_CUDA_CHECK(dion::embedding_bwd_launch(dout.data_ptr(), (const long long*)idx.data_ptr<int64_t>(),
                                             dtable.data_ptr<float>(), idx.numel(), (int)dtable.size(1),
                                             at::cuda::getCurrentCUDAStream()));
}

// ----------------------------------------------------------------------------- linear algebra

void chol_inverse(const Tensor& G, Tensor Z, Tensor work, Tensor info, double pivot_floor, bool jacobi,
                  const std::optional<Tensor>& colmask) {
  const c10::cuda::CUDAGuard guard(G.device());
  TORCH_CHECK(G.is_cuda() && G.scalar_type() == at::kFloat && G.dim() == 3 && G.size(1) == G.size(2) &&
              G.stride(2) == 1);
  const int batch = (int)G.size(0), r = (int)G.size(1);
  TORCH_CHECK(Z.is_contiguous() && Z.scalar_type() == at::kFloat && Z.numel() == (int64_t)batch * r * r);
  TORCH_CHECK(work.is_contiguous() && work.scalar_type() == at::kFloat && work.numel() >= (int64_t)batch * r * r);
  TORCH_CHECK(info.scalar_type() == at::kInt && info.numel() >= batch);
  float* mask = nullptr;
  if (colmask.has_value()) {
    TORCH_CHECK(colmask->scalar_type() == at::kFloat && colmask->is_contiguous() && colmask->numel() == (int64_t)batch * r);
    mask = colmask->data_ptr<float>();
  }
  cudaError_t e = dion::chol_inverse_launch(G.data_ptr<float>(), Z.data_ptr<float>(), work.data_ptr<float>(),
                                            info.data_ptr<int>(), batch, r, G.stride(1), G.stride(0),
                                            (float)pivot_floor, at::cuda::getCurrentCUDAStream(), jacobi, mask);
  TORCH_CHECK(e == cudaSuccess, "chol_inverse launch failed (rank ", r, "): ", cudaGetErrorString(e));
  g_launches.fetch_add(1, std::memory_order_relaxed);
}

void col_sumsq(const Tensor& X, Tensor out) {
  const c10::cuda::CUDAGuard guard(X.device());
  TORCH_CHECK(X.is_cuda() && X.dim() == 3 && X.stride(2) == 1);
  TORCH_CHECK(out.scalar_type() == at::kFloat && out.is_contiguous() && out.numel() == X.size(0) * X.size(2));
  DION_CUDA_CHECK(dion::col_sumsq_launch(X.data_ptr(), elem_type(X, "X"), out.data_ptr<float>(), (int)X.size(0),
                                         X.size(1), (int)X.size(2), X.stride(1), X.stride(0),
                                         at::cuda::getCurrentCUDAStream()));
}

// ----------------------------------------------------------------------------- symmetric-memory collectives

dion::PeerTable peer_table(at::IntArrayRef peers) {
  TORCH_CHECK(!peers.empty() && (int)peers.size() <= dion::kMaxPeers, "between 1 and ", dion::kMaxPeers,
              " peers are supported, got ", peers.size());
  dion::PeerTable t;
  memset(&t, 0, sizeof(t));
  for (size_t i = 0; i < peers.size(); ++i) t.ptrs[i] = reinterpret_cast<void*>(peers[i]);
  return t;
}

// `anchor` is any tensor on the device the kernel runs on (it selects the CUDA backend and stream).
void symm_barrier(const Tensor& anchor, at::IntArrayRef peers, int64_t flag_off, int64_t channel, int64_t rank,
                  int64_t epoch, Tensor status) {
  const c10::cuda::CUDAGuard guard(anchor.device());
  DION_CUDA_CHECK(dion::symm_barrier_launch(peer_table(peers), flag_off, (int)channel, (int)rank, (int)peers.size(),
                                            (unsigned)epoch, status.data_ptr<int>(),
                                            at::cuda::getCurrentCUDAStream()));
}

// In-place all-reduce of `buf`, a view into this rank's arena at byte offset `data_off`.
void symm_all_reduce(Tensor buf, at::IntArrayRef peers, int64_t flag_off, int64_t data_off, int64_t mc_base,
                     double scale, int64_t rank, int64_t epoch, Tensor counter, Tensor status) {
  const c10::cuda::CUDAGuard guard(buf.device());
  TORCH_CHECK(buf.is_contiguous(), "symm_all_reduce needs a contiguous arena view");
  TORCH_CHECK(reinterpret_cast<int64_t>(buf.data_ptr()) == peers[rank] + data_off,
              "buffer is not at the stated offset of this rank's arena");
  DION_CUDA_CHECK(dion::symm_all_reduce_launch(peer_table(peers), flag_off, data_off,
                                               reinterpret_cast<void*>(mc_base), elem_type(buf, "buf"), buf.numel(),
                                               (float)scale, (int)rank, (int)peers.size(), (unsigned)epoch,
                                               reinterpret_cast<unsigned*>(counter.data_ptr<int>()),
                                               status.data_ptr<int>(), at::cuda::getCurrentCUDAStream()));
}

// dst = beta * dst + scale * sum over ranks of `src` (arena view at `data_off`)
void symm_reduce_into(const Tensor& src, Tensor dst, at::IntArrayRef peers, int64_t flag_off, int64_t data_off,
                      double scale, double beta, int64_t rank, int64_t epoch, Tensor counter, Tensor status) {
  const c10::cuda::CUDAGuard guard(src.device());
  TORCH_CHECK(src.is_contiguous() && dst.is_contiguous() && src.numel() == dst.numel());
  TORCH_CHECK(reinterpret_cast<int64_t>(src.data_ptr()) == peers[rank] + data_off,
              "source is not at the stated offset of this rank's arena");
  DION_CUDA_CHECK(dion::symm_reduce_into_launch(peer_table(peers), flag_off, data_off, elem_type(src, "src"),
                                                dst.data_ptr(), elem_type(dst, "dst"), src.numel(), (float)scale,
                                                (float)beta, (int)rank, (int)peers.size(), (unsigned)epoch,
                                                reinterpret_cast<unsigned*>(counter.data_ptr<int>()),
                                                status.data_ptr<int>(), at::cuda::getCurrentCUDAStream()));
}

// ----------------------------------------------------------------------------- fused reductions of Dion

dion::SlotWait slot_wait(at::IntArrayRef peers, int64_t flag_off, int64_t channel, int64_t rank, int64_t epoch,
                         int64_t budget_ns) {
  dion::SlotWait w;
  memset(&w, 0, sizeof(w));
  TORCH_CHECK((int)peers.size() <= dion::kMaxPeers, "at most ", dion::kMaxPeers, " peers are supported");
  for (size_t i = 0; i < peers.size(); ++i) w.peers.ptrs[i] = reinterpret_cast<void*>(peers[i]);
  w.flag_off = flag_off;
  w.channel = (int)channel;
  w.rank = (int)rank;
  w.world = (int)peers.size();
  w.epoch = (unsigned)epoch;
  w.budget_ns = (unsigned long long)budget_ns;
  return w;
}

// slots: fp32 [nslots, ...] (a view into this rank's arena); out / hi / lo: fp32 tensors of one slot's size;
// dests: raw addresses that also receive the sum (peer memory); peers empty = nothing to wait for.
void slot_reduce(const Tensor& slots, const std::optional<Tensor>& out, const std::optional<Tensor>& hi,
                 const std::optional<Tensor>& lo, at::IntArrayRef dests, double scale, at::IntArrayRef peers,
                 int64_t flag_off, int64_t channel, int64_t rank, int64_t epoch, int64_t budget_ns, Tensor status) {
  const c10::cuda::CUDAGuard guard(slots.device());
  // slot s may be a leading part of a larger slot (stride(0) is free), but is contiguous in itself
  TORCH_CHECK(slots.is_cuda() && slots.scalar_type() == at::kFloat && slots.dim() >= 2 && slots.size(0) >= 1 &&
              (slots.numel() == 0 || slots.select(0, 0).is_contiguous()));
  dion::SlotReduceArgs a;
  memset(&a, 0, sizeof(a));
  a.wait = slot_wait(peers, flag_off, channel, rank, epoch, budget_ns);
  a.slots = slots.data_ptr<float>();
  a.nslots = (int)slots.size(0);
  a.slot_stride = slots.stride(0);
  a.numel = slots.numel() / slots.size(0);
  a.scale = (float)scale;
  auto local = [&](const std::optional<Tensor>& t, const char* what) -> float* {
    if (!t.has_value()) return nullptr;
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat && t->is_contiguous() && t->numel() == a.numel, what,
                " must be a contiguous fp32 tensor of one slot's size");
    return t->data_ptr<float>();
  };
  a.out = local(out, "out");
  a.hi = local(hi, "hi");
  a.lo = local(lo, "lo");
  TORCH_CHECK((int)dests.size() <= dion::kMaxPeers);
  a.ndest = (int)dests.size();
  for (size_t i = 0; i < dests.size(); ++i) a.dest[i] = reinterpret_cast<float*>(dests[i]);
  a.status = status.data_ptr<int>();
  ++g_launches;
  DION_CUDA_CHECK(dion::slot_reduce_launch(a, at::cuda::getCurrentCUDAStream()));
}

// slots: bf16 [nslots, ...]; out (and the optional residual): bf16 tensors of one slot's size
void slot_reduce_bf16(const Tensor& slots, Tensor out, const std::optional<Tensor>& residual, at::IntArrayRef peers,
                      int64_t flag_off, int64_t channel, int64_t rank, int64_t epoch, int64_t budget_ns, Tensor status) {
  const c10::cuda::CUDAGuard guard(slots.device());
  TORCH_CHECK(slots.is_cuda() && slots.scalar_type() == at::kBFloat16 && slots.dim() >= 2 && slots.size(0) >= 1 &&
              slots.select(0, 0).is_contiguous());
  dion::SlotReduceBf16Args a;
  memset(&a, 0, sizeof(a));
  a.wait = slot_wait(peers, flag_off, channel, rank, epoch, budget_ns);
  a.slots = slots.data_ptr();
  a.nslots = (int)slots.size(0);
  a.slot_stride = slots.stride(0);
  a.numel = slots.numel() / slots.size(0);
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.is_contiguous() && out.numel() == a.numel);
  a.out = out.data_ptr();
  if (residual.has_value()) {
    TORCH_CHECK(residual->scalar_type() == at::kBFloat16 && residual->is_contiguous() && residual->numel() == a.numel);
    a.residual = residual->data_ptr();
  }
  a.status = status.data_ptr<int>();
  ++g_launches;
  DION_CUDA_CHECK(dion::slot_reduce_bf16_launch(a, at::cuda::getCurrentCUDAStream()));
}

void dion_r_post(const Tensor& slots, double scale, const std::optional<Tensor>& nonzero, const Tensor& Qm,
                 const std::optional<Tensor>& P, const std::optional<Tensor>& R32, const std::optional<Tensor>& Rm,
                 const std::optional<Tensor>& ss, bool finish, double eps, const std::optional<Tensor>& Qn,
                 const std::optional<Tensor>& Qs, int64_t qs_col0, at::IntArrayRef peers, int64_t flag_off,
                 int64_t channel, int64_t rank, int64_t epoch, int64_t budget_ns, Tensor status) {
  const c10::cuda::CUDAGuard guard(slots.device());
  TORCH_CHECK(slots.is_cuda() && slots.scalar_type() == at::kFloat && slots.dim() == 4 && slots.is_contiguous(),
              "slots must be contiguous fp32 [nslots, B, n, r]");
  dion::RPostArgs a;
  memset(&a, 0, sizeof(a));
  a.wait = slot_wait(peers, flag_off, channel, rank, epoch, budget_ns);
  a.slots = slots.data_ptr<float>();
  a.nslots = (int)slots.size(0);
  a.slot_stride = slots.stride(0);
  a.scale = (float)scale;
  a.B = (int)slots.size(1);
  a.n = (int)slots.size(2);
  a.r = (int)slots.size(3);
  const int64_t numel = (int64_t)a.B * a.n * a.r;
  if (nonzero.has_value()) {
    TORCH_CHECK(nonzero->scalar_type() == at::kInt && nonzero->numel() >= a.B && nonzero->is_contiguous());
    a.nonzero = nonzero->data_ptr<int>();
  }
  TORCH_CHECK(Qm.dim() == 3 && Qm.size(0) == a.B && Qm.size(1) == a.n && Qm.size(2) == a.r && Qm.stride(2) == 1,
              "Qm must be [B, n, r] with unit column stride");
  a.Qm = Qm.data_ptr();
  a.q_type = elem_type(Qm, "Qm");
  a.q_ld = Qm.stride(1);
  a.q_bs = Qm.stride(0);
  if (P.has_value()) {
    TORCH_CHECK(P->dim() == 3 && P->size(0) == a.B && P->size(2) == a.r && P->stride(2) == 1,
                "P must be [B, m, r] with unit column stride");
    a.P = P->data_ptr();
    a.p_type = elem_type(*P, "P");
    a.p_rows = P->size(1);
    a.p_ld = P->stride(1);
    a.p_bs = P->stride(0);
  }
  if (R32.has_value()) {
    TORCH_CHECK(R32->scalar_type() == at::kFloat && R32->is_contiguous() && R32->numel() == numel);
    a.R32 = R32->data_ptr<float>();
  }
  if (Rm.has_value()) {
    TORCH_CHECK(Rm->is_contiguous() && Rm->numel() == numel);
    a.Rm = Rm->data_ptr();
    a.rm_type = elem_type(*Rm, "Rm");
  }
  if (ss.has_value()) {
    TORCH_CHECK(ss->scalar_type() == at::kFloat && ss->is_contiguous() && ss->numel() == (int64_t)a.B * a.r);
    a.ss = ss->data_ptr<float>();
  }
  a.finish = finish ? 1 : 0;
  a.eps = (float)eps;
  if (Qn.has_value()) {
    TORCH_CHECK(Qn->is_contiguous() && Qn->numel() == numel);
    a.Qn = Qn->data_ptr();
    a.qn_type = elem_type(*Qn, "Qn");
  }
  if (Qs.has_value()) {
    TORCH_CHECK(Qs->dim() == 3 && Qs->is_contiguous() && Qs->size(0) == a.B && Qs->size(1) == a.n);
    a.Qs = Qs->data_ptr();
    a.qs_type = elem_type(*Qs, "Qs");
    a.qs_col0 = (int)qs_col0;
    a.qs_cols = (int)Qs->size(2);
  }
  a.status = status.data_ptr<int>();
  ++g_launches;
  DION_CUDA_CHECK(dion::r_post_launch(a, at::cuda::getCurrentCUDAStream()));
}

void dion_q_norm(const Tensor& R32, const Tensor& ss, const Tensor& Qm, double eps, const std::optional<Tensor>& Qn,
                 const std::optional<Tensor>& Qs, int64_t qs_col0) {
  const c10::cuda::CUDAGuard guard(R32.device());
  TORCH_CHECK(R32.is_cuda() && R32.scalar_type() == at::kFloat && R32.dim() == 3 && R32.is_contiguous());
  dion::QNormArgs a;
  memset(&a, 0, sizeof(a));
  a.R32 = R32.data_ptr<float>();
  a.B = (int)R32.size(0);
  a.n = (int)R32.size(1);
  a.r = (int)R32.size(2);
  TORCH_CHECK(ss.scalar_type() == at::kFloat && ss.is_contiguous() && ss.numel() == (int64_t)a.B * a.r);
  a.ss = ss.data_ptr<float>();
  a.eps = (float)eps;
  TORCH_CHECK(Qm.dim() == 3 && Qm.size(0) == a.B && Qm.size(1) == a.n && Qm.size(2) == a.r && Qm.stride(2) == 1);
  a.Qm = Qm.data_ptr();
  a.q_type = elem_type(Qm, "Qm");
  a.q_ld = Qm.stride(1);
  a.q_bs = Qm.stride(0);
  if (Qn.has_value()) {
    TORCH_CHECK(Qn->is_contiguous() && Qn->numel() == R32.numel());
    a.Qn = Qn->data_ptr();
    a.qn_type = elem_type(*Qn, "Qn");
  }
  if (Qs.has_value()) {
    TORCH_CHECK(Qs->dim() == 3 && Qs->is_contiguous() && Qs->size(0) == a.B && Qs->size(1) == a.n);
    a.Qs = Qs->data_ptr();
    a.qs_type = elem_type(*Qs, "Qs");
    a.qs_col0 = (int)qs_col0;
    a.qs_cols = (int)Qs->size(2);
  }
  ++g_launches;
  DION_CUDA_CHECK(dion::q_norm_launch(a, at::cuda::getCurrentCUDAStream()));
}

// q [B, T, H, D], k / v [B, T, Hkv, D] (contiguous bf16) -> out [B, T, H, D], lse [B, H, T]
void attn_fwd(const Tensor& q, const Tensor& k, const Tensor& v, Tensor out, Tensor lse, double scale, Tensor status) {
  const c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4, "attention operands must be [B, T, H, D]");
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16 &&
              v.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16 && lse.scalar_type() == at::kFloat);
  TORCH_CHECK(q.is_contiguous() && k.is_contiguous() && v.is_contiguous() && out.is_contiguous() && lse.is_contiguous());
  const int64_t B = q.size(0), T = q.size(1), H = q.size(2), D = q.size(3), Hkv = k.size(2);
  TORCH_CHECK(k.size(0) == B && k.size(1) == T && k.size(3) == D && v.sizes() == k.sizes() && out.sizes() == q.sizes());
  TORCH_CHECK(lse.numel() == B * H * T);
  ++g_launches;
  DION_CUDA_CHECK(dion::attn_fwd_launch(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr<float>(),
                                        (int)B, (int)T, (int)H, (int)Hkv, (int)D, (float)scale, status.data_ptr<int>(),
                                        at::cuda::getCurrentCUDAStream()));
}

void attn_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o, const Tensor& d_o, const Tensor& lse,
              Tensor delta, Tensor dq, Tensor dk, Tensor dv, double scale, Tensor status) {
  const c10::cuda::CUDAGuard guard(q.device());
  for (const Tensor* t : std::initializer_list<const Tensor*>{&q, &k, &v, &o, &d_o, &dq, &dk, &dv})
    TORCH_CHECK(t->dim() == 4 && t->scalar_type() == at::kBFloat16 && t->is_contiguous(),
                "attention tensors must be contiguous bf16 [B, T, H, D]");
  TORCH_CHECK(lse.scalar_type() == at::kFloat && delta.scalar_type() == at::kFloat && lse.is_contiguous() &&
              delta.is_contiguous() && delta.numel() == lse.numel());
  const int64_t B = q.size(0), T = q.size(1), H = q.size(2), D = q.size(3), Hkv = k.size(2);
  TORCH_CHECK(o.sizes() == q.sizes() && d_o.sizes() == q.sizes() && dq.sizes() == q.sizes() && v.sizes() == k.sizes() &&
              dk.sizes() == k.sizes() && dv.sizes() == k.sizes() && lse.numel() == B * H * T);
  g_launches += 3;
  DION_CUDA_CHECK(dion::attn_bwd_launch(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr(),
                                        lse.data_ptr<float>(), delta.data_ptr<float>(), dq.data_ptr(), dk.data_ptr(),
                                        dv.data_ptr(), (int)B, (int)T, (int)H, (int)Hkv, (int)D, (float)scale,
                                        status.data_ptr<int>(), at::cuda::getCurrentCUDAStream()));
}

void split_tf32(const Tensor& x, Tensor hi, Tensor lo) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.scalar_type() == at::kFloat && hi.scalar_type() == at::kFloat && lo.scalar_type() == at::kFloat);
  TORCH_CHECK(x.is_contiguous() && hi.is_contiguous() && lo.is_contiguous() && hi.numel() == x.numel() &&
              lo.numel() == x.numel());
  ++g_launches;
  DION_CUDA_CHECK(dion::split_tf32_launch(x.data_ptr<float>(), hi.data_ptr<float>(), lo.data_ptr<float>(), x.numel(),
                                          at::cuda::getCurrentCUDAStream()));
}

void jacobi_scale(const Tensor& G, Tensor W, Tensor d) {
  const c10::cuda::CUDAGuard guard(G.device());
  TORCH_CHECK(G.is_cuda() && G.scalar_type() == at::kFloat && G.dim() == 3 && G.size(1) == G.size(2) && G.stride(2) == 1);
  const int64_t B = G.size(0), r = G.size(1);
  TORCH_CHECK(W.scalar_type() == at::kFloat && W.is_contiguous() && W.numel() == B * r * r);
  TORCH_CHECK(d.scalar_type() == at::kFloat && d.is_contiguous() && d.numel() == B * r);
  ++g_launches;
  DION_CUDA_CHECK(dion::jacobi_scale_launch(G.data_ptr<float>(), W.data_ptr<float>(), d.data_ptr<float>(), (int)B, (int)r,
                                            G.stride(1), G.stride(0), at::cuda::getCurrentCUDAStream()));
}

// Z: contiguous [B, r, r]; Zd, Zm: contiguous [B, nb, nb]; mask: [B, nb]
void place_block(const Tensor& Zd, const Tensor& mask, Tensor Z, Tensor Zm, int64_t k0) {
  const c10::cuda::CUDAGuard guard(Zd.device());
  TORCH_CHECK(Zd.is_cuda() && Zd.scalar_type() == at::kFloat && Zd.dim() == 3 && Zd.is_contiguous() && Zd.size(1) == Zd.size(2));
  const int64_t B = Zd.size(0), nb = Zd.size(1);
  TORCH_CHECK(Z.scalar_type() == at::kFloat && Z.dim() == 3 && Z.is_contiguous() && Z.size(0) == B && Z.size(1) == Z.size(2));
  TORCH_CHECK(Zm.scalar_type() == at::kFloat && Zm.is_contiguous() && Zm.numel() == Zd.numel());
  TORCH_CHECK(mask.scalar_type() == at::kFloat && mask.is_contiguous() && mask.numel() == B * nb);
  ++g_launches;
  DION_CUDA_CHECK(dion::place_block_launch(Zd.data_ptr<float>(), mask.data_ptr<float>(), Z.data_ptr<float>(),
                                           Zm.data_ptr<float>(), (int)B, (int)nb, (int)Z.size(1), (int)k0,
                                           at::cuda::getCurrentCUDAStream()));
}

// x: fp32 [B, rows, cols] view with unit column stride; hi / lo contiguous
void split_tf32_rows(const Tensor& x, Tensor hi, Tensor lo) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kFloat && x.dim() == 3 && x.stride(2) == 1);
  TORCH_CHECK(hi.scalar_type() == at::kFloat && lo.scalar_type() == at::kFloat && hi.is_contiguous() &&
              lo.is_contiguous() && hi.numel() == x.numel() && lo.numel() == x.numel());
  ++g_launches;
  DION_CUDA_CHECK(dion::split_tf32_rows_launch(x.data_ptr<float>(), hi.data_ptr<float>(), lo.data_ptr<float>(),
                                               (int)x.size(0), (int)x.size(1), (int)x.size(2), x.stride(1), x.stride(0),
                                               at::cuda::getCurrentCUDAStream()));
}

void refine_prep(const Tensor& G, Tensor C, Tensor d, double dead_below, const std::optional<Tensor>& skip,
                 bool fold) {
  const c10::cuda::CUDAGuard guard(G.device());
  TORCH_CHECK(G.scalar_type() == at::kFloat && C.scalar_type() == at::kFloat && d.scalar_type() == at::kFloat);
  TORCH_CHECK(G.dim() == 3 && G.size(1) == G.size(2) && G.is_contiguous() && C.is_contiguous() && d.is_contiguous());
  TORCH_CHECK(C.numel() == G.numel() && d.numel() == G.size(0) * G.size(1));
  if (skip.has_value())
    TORCH_CHECK(skip->scalar_type() == at::kInt && skip->is_cuda() && skip->is_contiguous() && skip->numel() == G.size(0),
                "skip must be one int32 per matrix");
  ++g_launches;
  DION_CUDA_CHECK(dion::refine_prep_launch(G.data_ptr<float>(), C.data_ptr<float>(), d.data_ptr<float>(),
                                           (int)G.size(0), (int)G.size(1), (float)dead_below,
                                           skip.has_value() ? skip->data_ptr<int>() : nullptr, fold,
                                           at::cuda::getCurrentCUDAStream()));
}

// out (world * n) = concatenation of every rank's `inp` (n), through the staging slot at `slot_off`
void symm_all_gather(const Tensor& inp, Tensor out, at::IntArrayRef peers, int64_t flag_off, int64_t slot_off,
                     int64_t rank, int64_t epoch, int64_t channel, Tensor counter, Tensor status, int64_t budget_ns) {
  const c10::cuda::CUDAGuard guard(inp.device());
  TORCH_CHECK(inp.is_contiguous() && out.is_contiguous() && inp.scalar_type() == out.scalar_type());
  TORCH_CHECK(out.numel() == inp.numel() * (int64_t)peers.size(), "all-gather output must hold every rank's input");
  ++g_launches;
  DION_CUDA_CHECK(dion::symm_all_gather_launch(peer_table(peers), flag_off, slot_off, inp.data_ptr(), out.data_ptr(),
                                               inp.numel() * inp.element_size(), (int)rank, (int)peers.size(),
                                               (unsigned)epoch, (int)channel,
                                               reinterpret_cast<unsigned*>(counter.data_ptr<int>()),
                                               status.data_ptr<int>(), budget_ns, at::cuda::getCurrentCUDAStream()));
}

// out (n) = scale * sum over ranks of slice `rank` of `inp` (world * n, an arena view at `data_off`)
void symm_reduce_scatter(const Tensor& inp, Tensor out, at::IntArrayRef peers, int64_t flag_off, int64_t data_off,
                         int64_t mc_base, double scale, int64_t rank, int64_t epoch, int64_t ch_start, int64_t ch_end,
                         Tensor counter, Tensor status, int64_t budget_ns) {
  const c10::cuda::CUDAGuard guard(inp.device());
  TORCH_CHECK(inp.is_contiguous() && out.is_contiguous() && inp.scalar_type() == out.scalar_type());
  TORCH_CHECK(inp.numel() == out.numel() * (int64_t)peers.size(), "reduce-scatter input must hold one slice per rank");
  TORCH_CHECK(reinterpret_cast<int64_t>(inp.data_ptr()) == peers[rank] + data_off,
              "input is not at the stated offset of this rank's arena");
  ++g_launches;
  DION_CUDA_CHECK(dion::symm_reduce_scatter_launch(
      peer_table(peers), flag_off, data_off, reinterpret_cast<void*>(mc_base), elem_type(inp, "input"), out.data_ptr(),
      out.numel(), (float)scale, (int)rank, (int)peers.size(), (unsigned)epoch, (int)ch_start, (int)ch_end,
      reinterpret_cast<unsigned*>(counter.data_ptr<int>()), status.data_ptr<int>(), budget_ns,
      at::cuda::getCurrentCUDAStream()));
}

}  // namespace

TORCH_LIBRARY(dion_b200, m) {
  m.def(
      "symm_all_gather(Tensor inp, Tensor(a!) out, int[] peers, int flag_off, int slot_off, int rank, int epoch, "
      "int channel, Tensor(b!) counter, Tensor(c!) status, int budget_ns) -> ()");
  m.def(
      "symm_reduce_scatter(Tensor inp, Tensor(a!) out, int[] peers, int flag_off, int data_off, int mc_base, "
      "float scale, int rank, int epoch, int ch_start, int ch_end, Tensor(b!) counter, Tensor(c!) status, "
      "int budget_ns) -> ()");
  m.def(
      "gemm_scatter(Tensor a, Tensor b, Tensor? c, Tensor block_like, Tensor scatter_ptrs, int mode, int block, "
      "int dests, float alpha, float beta, Tensor? status) -> ()");
  m.def(
      "gemm_gather(Tensor x_local, Tensor(a!) a_full, Tensor b, Tensor(b!) d, int[] peers, int flag_off, int slot_off, "
      "int rank, int epoch, int channel, Tensor(c!) counters, Tensor? status, int budget_ns) -> ()");
  m.def("symm_barrier(Tensor anchor, int[] peers, int flag_off, int channel, int rank, int epoch, Tensor(a!) status) -> ()");
  m.def(
      "symm_all_reduce(Tensor(a!) buf, int[] peers, int flag_off, int data_off, int mc_base, float scale, int rank, "
      "int epoch, Tensor(b!) counter, Tensor(c!) status) -> ()");
  m.def(
      "symm_reduce_into(Tensor src, Tensor(a!) dst, int[] peers, int flag_off, int data_off, float scale, float beta, "
      "int rank, int epoch, Tensor(b!) counter, Tensor(c!) status) -> ()");
  m.def(
      "gemm(Tensor a, Tensor b, Tensor? c, Tensor(a!) d, Tensor(b!)? d2, Tensor? c_ptrs, Tensor? d_ptrs, "
      "Tensor? d2_ptrs, float alpha, float beta, int act, int epilogue, int split_k, bool symmetric, "
      "int block_n, int pair, Tensor? status, int d_dup=1, Tensor? a_lo=None, Tensor? b_lo=None, "
      "Tensor? c_col_scale=None, bool split3=False) -> ()");
  m.def(
      "adamw_multi(Tensor(a!)[] X, Tensor[] G, Tensor(b!)[] M, Tensor(c!)[] V, Tensor(d!)[] shadow, float lr, "
      "float beta1, float beta2, float weight_decay, float eps, int step) -> ()");
  m.def(
      "lion_multi(Tensor(a!)[] X, Tensor[] G, Tensor(b!)[] M, Tensor(c!)[] shadow, float lr, float beta1, "
      "float beta2, float weight_decay) -> ()");
  m.def("muon_pre_multi(Tensor[] G, Tensor(a!)[] M, Tensor(b!)[] U, float mu, bool nesterov, Tensor(c!)? sumsq) -> ()");
  m.def("muon_post_multi(Tensor(a!)[] X, Tensor[] U, Tensor(b!)[] shadow, float decay, float step) -> ()");
  m.def("frob_scale(Tensor x, Tensor(a!) out, Tensor? sumsq, float eps) -> ()");
  m.def("dion_accum_multi(Tensor[] G, Tensor(a!)[] M, Tensor(b!)? nonzero) -> ()");
  m.def("cast_multi(Tensor[] src, Tensor(a!)[] dst) -> ()");
  m.def("rmsnorm_fwd(Tensor x, Tensor? residual, Tensor(a!)? x_out, Tensor(b!) y, Tensor(c!) rstd, float eps) -> ()");
  m.def("rmsnorm_bwd(Tensor dy, Tensor x, Tensor rstd, Tensor? dx_add, Tensor(a!) dx) -> ()");
  m.def("rmsnorm_gain_fwd(Tensor x, Tensor gain, Tensor(a!) y, Tensor(b!) rstd, float eps) -> ()");
  m.def("rmsnorm_gain_bwd(Tensor dy, Tensor x, Tensor rstd, Tensor gain, Tensor(a!) dx) -> Tensor");
  m.def("swiglu_fwd(Tensor g, Tensor u, Tensor(a!) h) -> ()");
  m.def("swiglu_bwd(Tensor dh, Tensor g, Tensor u, Tensor(a!) dg, Tensor(b!) du) -> ()");
  m.def(
      "rope_qknorm_fwd(Tensor q, Tensor k, Tensor(a!) q_out, Tensor(b!) k_out, Tensor cos, Tensor sin, int seq_len, "
      "int heads, int head_dim, float eps) -> ()");
  m.def(
      "rope_qknorm_bwd(Tensor dq_out, Tensor dk_out, Tensor q, Tensor k, Tensor(a!) dq, Tensor(b!) dk, Tensor cos, "
      "Tensor sin, int seq_len, int heads, int head_dim, float eps) -> ()");
  m.def("rope_fwd(Tensor x, Tensor(a!) out, Tensor cos, Tensor sin, int seq_len, int heads, int head_dim) -> ()");
  m.def("rope_bwd(Tensor dout, Tensor x, Tensor(a!) dx, Tensor cos, Tensor sin, int seq_len, int heads, int head_dim) -> ()");
  m.def("relu2_fwd(Tensor x, Tensor(a!) h) -> ()");
  m.def("relu2_bwd(Tensor dh, Tensor x, Tensor(a!) dx) -> ()");
  m.def(
      "cross_entropy_fwd_bwd(Tensor(a!) logits, Tensor targets, Tensor(b!) row_loss, Tensor? scale, float grad_scale, "
      "int ignore_index, bool write_grad) -> ()");
  m.def("embedding_fwd(Tensor table, Tensor idx, Tensor(a!) out) -> ()");
  m.def("embedding_bwd(Tensor dout, Tensor idx, Tensor(a!) dtable) -> ()");
  m.def(
      "chol_inverse(Tensor G, Tensor(a!) Z, Tensor(b!) work, Tensor(c!) info, float pivot_floor, bool jacobi=True, "
      "Tensor(d!)? colmask=None) -> ()");
  m.def("split_tf32_rows(Tensor x, Tensor(a!) hi, Tensor(b!) lo) -> ()");
  m.def("jacobi_scale(Tensor G, Tensor(a!) W, Tensor(b!) d) -> ()");
  m.def("place_block(Tensor Zd, Tensor mask, Tensor(a!) Z, Tensor(b!) Zm, int k0) -> ()");
  m.def("col_sumsq(Tensor X, Tensor(a!) out) -> ()");
  m.def("split_tf32(Tensor x, Tensor(a!) hi, Tensor(b!) lo) -> ()");
  m.def("attn_fwd(Tensor q, Tensor k, Tensor v, Tensor(a!) out, Tensor(b!) lse, float scale, Tensor(c!) status) -> ()");
  m.def(
      "attn_bwd(Tensor q, Tensor k, Tensor v, Tensor o, Tensor d_o, Tensor lse, Tensor(a!) delta, Tensor(b!) dq, "
      "Tensor(c!) dk, Tensor(d!) dv, float scale, Tensor(e!) status) -> ()");
  m.def("refine_prep(Tensor G, Tensor(a!) C, Tensor(b!) d, float dead_below, Tensor? skip, bool fold=False) -> ()");
  m.def(
      "slot_reduce(Tensor slots, Tensor(a!)? out, Tensor(b!)? hi, Tensor(c!)? lo, int[] dests, float scale, int[] peers, "
      "int flag_off, int channel, int rank, int epoch, int budget_ns, Tensor(d!) status) -> ()");
  m.def(
      "slot_reduce_bf16(Tensor slots, Tensor(a!) out, Tensor? residual, int[] peers, int flag_off, int channel, int rank, "
      "int epoch, int budget_ns, Tensor(b!) status) -> ()");
  m.def(
      "dion_r_post(Tensor slots, float scale, Tensor? nonzero, Tensor Qm, Tensor(a!)? P, Tensor(b!)? R32, Tensor(c!)? Rm, "
      "Tensor(d!)? ss, bool finish, float eps, Tensor(e!)? Qn, Tensor(f!)? Qs, int qs_col0, int[] peers, int flag_off, "
      "int channel, int rank, int epoch, int budget_ns, Tensor(g!) status) -> ()");
  m.def("dion_q_norm(Tensor R32, Tensor ss, Tensor Qm, float eps, Tensor(a!)? Qn, Tensor(b!)? Qs, int qs_col0) -> ()");
  m.def("launch_count() -> int", &launch_count);
  m.def("gemm_gather_plan(int M, int N, int K, int rows, int world, int rank) -> int[]", &gemm_gather_plan);
}

TORCH_LIBRARY_IMPL(dion_b200, CUDA, m) {
  m.impl("gemm", &gemm);
  m.impl("frob_scale", &frob_scale);
  m.impl("rmsnorm_fwd", &rmsnorm_fwd);
  m.impl("rmsnorm_bwd", &rmsnorm_bwd);
  m.impl("rmsnorm_gain_fwd", &rmsnorm_gain_fwd);
  m.impl("rmsnorm_gain_bwd", &rmsnorm_gain_bwd);
  m.impl("swiglu_fwd", &swiglu_fwd);
  m.impl("swiglu_bwd", &swiglu_bwd);
  m.impl("rope_qknorm_fwd", &rope_qknorm_fwd);
  m.impl("rope_qknorm_bwd", &rope_qknorm_bwd);
  m.impl("rope_fwd", &rope_fwd);
  m.impl("rope_bwd", &rope_bwd);
  m.impl("relu2_fwd", &relu2_fwd);
  m.impl("relu2_bwd", &relu2_bwd);
  m.impl("cross_entropy_fwd_bwd", &cross_entropy_fwd_bwd);
  m.impl("embedding_fwd", &embedding_fwd);
  m.impl("embedding_bwd", &embedding_bwd);
  m.impl("chol_inverse", &chol_inverse);
  m.impl("col_sumsq", &col_sumsq);
  m.impl("split_tf32", &split_tf32);
  m.impl("split_tf32_rows", &split_tf32_rows);
  m.impl("jacobi_scale", &jacobi_scale);
  m.impl("place_block", &place_block);
  m.impl("attn_fwd", &attn_fwd);
  m.impl("attn_bwd", &attn_bwd);
  m.impl("refine_prep", &refine_prep);
  m.impl("slot_reduce", &slot_reduce);
  m.impl("slot_reduce_bf16", &slot_reduce_bf16);
  m.impl("dion_r_post", &dion_r_post);
  m.impl("dion_q_norm", &dion_q_norm);
  m.impl("gemm_scatter", &gemm_scatter);
  m.impl("gemm_gather", &gemm_gather);
  m.impl("symm_barrier", &symm_barrier);
  m.impl("symm_all_reduce", &symm_all_reduce);
  m.impl("symm_reduce_into", &symm_reduce_into);
  m.impl("symm_all_gather", &symm_all_gather);
  m.impl("symm_reduce_scatter", &symm_reduce_scatter);
}

// Ops whose arguments are tensor lists have no dispatch key to select on when a list
// is empty, so they are registered for every backend and check devices themselves.
TORCH_LIBRARY_IMPL(dion_b200, CompositeExplicitAutograd, m) {
  m.impl("adamw_multi", &adamw_multi);
  m.impl("lion_multi", &lion_multi);
  m.impl("muon_pre_multi", &muon_pre_multi);
  m.impl("muon_post_multi", &muon_post_multi);
  m.impl("dion_accum_multi", &dion_accum_multi);
  m.impl("cast_multi", &cast_multi);
}
