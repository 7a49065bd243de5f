// torch.ops.fbgemm.* for CUDA tensors, implemented on the C ABI of libb200tbe.so.
//
// This is the host half of the plugin: it validates arguments with TORCH_CHECK, allocates outputs
// on the inputs' device, takes the caller's current CUDA stream and calls one extern "C" entry
// point per operator. It follows the pattern of the torchcodec-xpu plugin of intel/torchlib-xpu: a
// shared library whose static initialisers register it with the host framework when
// torch.ops.load_library() opens it (packages/torchcodec-xpu/src/torchcodec_xpu/
// XpuDeviceInterface.cpp:33-35, loaded by src/torchcodec_xpu/__init__.py:25-32), work enqueued on
// the current stream (XpuDeviceInterface.cpp:415), errors raised through TORCH_CHECK (ibid.
// :302-318), outputs allocated by the plugin or shape-checked when pre-allocated (ibid. :308-322).
//
// Operator names and argument lists are those of fbgemm_gpu's operators of the same name. fbgemm_gpu
// is not available to check them against, so the schemas below are written from its public
// documentation; arguments that select features outside this library (UVM / cache placements,
// stochastic rounding, gradient clipping, weight decay) are accepted and must be at their neutral
// value. There is no CPU implementation and no fallback: only the CUDA dispatch key is registered.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/csrc/autograd/custom_function.h>

#include <mutex>
#include <unordered_map>
#include <vector>

#include "b200tbe.h"

namespace {

using at::Tensor;
using torch::autograd::AutogradContext;
using torch::autograd::Variable;
using torch::autograd::variable_list;

b200tbe_stream_t current_stream() {
  return reinterpret_cast<b200tbe_stream_t>(at::cuda::getCurrentCUDAStream().stream());
}

void check_status(int status, const char* what) {
  TORCH_CHECK(status == B200TBE_OK, what, ": ", b200tbe_status_string(status), " (", status, ")");
}

int dtype_code(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return B200TBE_FP32;
    case at::kHalf: return B200TBE_FP16;
    case at::kBFloat16: return B200TBE_BF16;
    default: return -1;
  }
}

at::ScalarType output_scalar_type(int64_t sparse_type) {
  TORCH_CHECK(sparse_type == B200TBE_FP32 || sparse_type == B200TBE_FP16,
              "output_dtype must be 0 (fp32) or 1 (fp16), got ", sparse_type);
  return sparse_type == B200TBE_FP32 ? at::kFloat : at::kHalf;
}

void check_cuda_contig(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

int index_bytes_of(const Tensor& indices, const Tensor& offsets) {
  TORCH_CHECK(indices.scalar_type() == offsets.scalar_type(),
              "indices and offsets must have the same dtype");
  TORCH_CHECK(indices.scalar_type() == at::kLong || indices.scalar_type() == at::kInt,
              "indices and offsets must be int64 or int32");
  return static_cast<int>(indices.element_size());
}

bool is_empty_or_undefined(const Tensor& t) { return !t.defined() || t.numel() == 0; }

// ---- facts about long-lived index tables, read from the device once ----------------------------
// The lookup ops receive hash_size_cumsum, weights_placements and weights_offsets as DEVICE tensors
// on every call. What the kernels need from them on the host side (row counts for range checks, the
// largest table for the sort, "all placements are DEVICE") does not change while the tensor is not
// written, so it is read back once -- one synchronising copy on the first call -- and remembered
// under the tensor's storage address, size and version counter.
struct TensorKey {
  const void* ptr;
  int64_t numel;
  uint64_t version;
  int device;
  bool operator==(const TensorKey& o) const {
    return ptr == o.ptr && numel == o.numel && version == o.version && device == o.device;
  }
};
struct TensorKeyHash {
  size_t operator()(const TensorKey& k) const {
    return std::hash<const void*>()(k.ptr) ^ (std::hash<int64_t>()(k.numel) * 31) ^
           (std::hash<uint64_t>()(k.version) * 131) ^ static_cast<size_t>(k.device);
  }
};
TensorKey key_of(const Tensor& t) {
  return {t.data_ptr(), t.numel(), static_cast<uint64_t>(t._version()), t.get_device()};
}

template <typename V>
class FactCache {
 public:
  template <typename Make>
  V get(const Tensor& t, Make make) {
    const TensorKey k = key_of(t);
    {
      std::lock_guard<std::mutex> lock(mu_);
      auto it = map_.find(k);
      if (it != map_.end()) return it->second;
    }
    V v = make();
    std::lock_guard<std::mutex> lock(mu_);
    if (map_.size() >= 256) map_.clear();   // tables come and go; the facts are cheap to rebuild
    map_.emplace(k, v);
    return v;
  }

 private:
  std::mutex mu_;
  std::unordered_map<TensorKey, V, TensorKeyHash> map_;
};

struct TableRows {
  Tensor rows_per_table;   // [T] int64 on the device
  int64_t max_rows;
};

TableRows table_rows_of(const Tensor& hash_size_cumsum) {
  static FactCache<TableRows> cache;
  return cache.get(hash_size_cumsum, [&] {
    const int64_t n = hash_size_cumsum.numel();
    Tensor rows = (hash_size_cumsum.slice(0, 1, n) - hash_size_cumsum.slice(0, 0, n - 1)).contiguous();
    const int64_t max_rows = n > 1 ? rows.max().item<int64_t>() : 0;
    return TableRows{rows, max_rows};
  });
}

// One int32 per device that the kernels OR B200TBE_DEV_* bits into (an index out of range, a row
// shape a kernel cannot take). Nothing reads it on the hot path; fbgemm::b200tbe_pop_device_status
// returns and clears it.
Tensor device_status(const at::Device& device) {
  static std::mutex mu;
  static std::unordered_map<int, Tensor> words;
  std::lock_guard<std::mutex> lock(mu);
  auto it = words.find(device.index());
  if (it != words.end()) return it->second;
  Tensor w = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(device));
  words.emplace(device.index(), w);
  return w;
}

int64_t pop_device_status(const Tensor& like) {
  TORCH_CHECK(like.is_cuda(), "b200tbe_pop_device_status takes any CUDA tensor of the device to query");
  c10::cuda::CUDAGuard guard(like.device());
  Tensor w = device_status(like.device());
  const int64_t bits = w.item<int32_t>();   // synchronises with the current stream
  if (bits != 0) w.zero_();
  return bits;
}

// ---- jagged ---------------------------------------------------------------------------------

b200tbe_jagged_shape jagged_shape(const std::vector<Tensor>& offsets, at::IntArrayRef max_lengths,
                                  int64_t inner, int64_t total_rows, const Tensor& like) {
  TORCH_CHECK(!offsets.empty() && offsets.size() <= B200TBE_MAX_JAGGED_DIMS, "1 to ",
              B200TBE_MAX_JAGGED_DIMS, " jagged dimensions are supported, got ", offsets.size());
  TORCH_CHECK(offsets.size() == max_lengths.size(),
              "offsets and max_lengths must have the same length");
  b200tbe_jagged_shape s{};
  const auto otype = offsets[0].scalar_type();
  TORCH_CHECK(otype == at::kLong || otype == at::kInt, "offsets must be int64 or int32");
  for (size_t d = 0; d < offsets.size(); ++d) {
    check_cuda_contig(offsets[d], "offsets");
    TORCH_CHECK(offsets[d].scalar_type() == otype, "offsets must share one dtype");
    TORCH_CHECK(offsets[d].numel() >= 1, "offsets must have at least one entry");
    TORCH_CHECK(max_lengths[d] >= 0, "max_lengths must be non-negative");
    s.offsets[d] = offsets[d].data_ptr();
    s.max_lengths[d] = max_lengths[d];
  }
  s.num_jagged_dims = static_cast<int32_t>(offsets.size());
  s.offset_bytes = static_cast<int32_t>(offsets[0].element_size());
  s.outer_size = offsets[0].numel() - 1;
  s.inner_size = inner;
  s.total_rows = total_rows;
  s.elem_bytes = static_cast<int32_t>(like.element_size());
  s.dtype = dtype_code(like.scalar_type());
  return s;
}

uint64_t pad_bits(double value, at::ScalarType t) {
  Tensor one = at::full({1}, value, at::TensorOptions().dtype(t).device(at::kCPU));
  uint64_t bits = 0;
  std::memcpy(&bits, one.data_ptr(), one.element_size());
  return bits;
}

Tensor jagged_to_padded_dense(const Tensor& values, const std::vector<Tensor>& offsets,
                              at::IntArrayRef max_lengths, double padding_value) {
  check_cuda_contig(values, "values");
  TORCH_CHECK(values.dim() == 1 || values.dim() == 2, "values must be [total] or [total, D]");
  c10::cuda::CUDAGuard guard(values.device());
  const Tensor v2 = values.dim() == 1 ? values.unsqueeze(1) : values;
  const int64_t inner = v2.size(1);
  const auto s = jagged_shape(offsets, max_lengths, inner, v2.size(0), v2);
  std::vector<int64_t> shape{s.outer_size};
  for (auto m : max_lengths) shape.push_back(m);
  shape.push_back(inner);
  Tensor dense = at::empty(shape, values.options());
  check_status(b200tbe_jagged_to_padded_dense(&s, v2.data_ptr(), dense.data_ptr(),
                                              pad_bits(padding_value, values.scalar_type()),
                                              current_stream()),
               "jagged_to_padded_dense");
  return values.dim() == 1 ? dense.squeeze(-1) : dense;
}

std::tuple<Tensor, std::vector<Tensor>> dense_to_jagged(const Tensor& dense,
                                                        const std::vector<Tensor>& offsets,
                                                        c10::optional<int64_t> total_L) {
  check_cuda_contig(dense, "dense");
  TORCH_CHECK(!offsets.empty(), "offsets must not be empty");
  TORCH_CHECK(dense.dim() == static_cast<int64_t>(offsets.size()) + 2,
              "dense must be [B, max_lengths..., D]");
  c10::cuda::CUDAGuard guard(dense.device());
  int64_t total = 0;
  if (total_L.has_value()) {
    total = *total_L;
  } else {
    total = offsets.back()[-1].item<int64_t>();  // one synchronising read, as in fbgemm_gpu
  }
  TORCH_CHECK(total >= 0, "total_L must be non-negative");
  std::vector<int64_t> max_lengths(dense.sizes().begin() + 1, dense.sizes().end() - 1);
  const int64_t inner = dense.size(-1);
  const auto s = jagged_shape(offsets, max_lengths, inner, total, dense);
  TORCH_CHECK(s.outer_size == dense.size(0), "offsets[0] must have dense.size(0) + 1 entries");
  Tensor values = at::empty({total, inner}, dense.options());
  check_status(b200tbe_dense_to_jagged(&s, dense.data_ptr(), values.data_ptr(), current_stream()),
               "dense_to_jagged");
  return {values, offsets};
}

Tensor jagged_dense_elementwise_add(const Tensor& x_values, const std::vector<Tensor>& x_offsets,
                                    const Tensor& y) {
  check_cuda_contig(x_values, "x_values");
  check_cuda_contig(y, "y");
  TORCH_CHECK(x_values.scalar_type() == y.scalar_type(), "x_values and y must share a dtype");
  TORCH_CHECK(dtype_code(y.scalar_type()) >= 0, "supported dtypes: float32, float16, bfloat16");
  TORCH_CHECK(y.dim() == static_cast<int64_t>(x_offsets.size()) + 2 && x_values.dim() == 2,
              "y must be [B, max_lengths..., D] and x_values [total, D]");
  TORCH_CHECK(x_values.size(1) == y.size(-1), "inner dimensions differ");
  c10::cuda::CUDAGuard guard(y.device());
  std::vector<int64_t> max_lengths(y.sizes().begin() + 1, y.sizes().end() - 1);
  const auto s = jagged_shape(x_offsets, max_lengths, y.size(-1), x_values.size(0), y);
  TORCH_CHECK(s.outer_size == y.size(0), "x_offsets[0] must have y.size(0) + 1 entries");
  Tensor out = at::empty_like(y);
  check_status(b200tbe_jagged_dense_elementwise_add(&s, x_values.data_ptr(), y.data_ptr(),
                                                    out.data_ptr(), current_stream()),
               "jagged_dense_elementwise_add");
  return out;
}

Tensor jagged_2d_to_dense(const Tensor& values, const Tensor& offsets, int64_t max_sequence_length) {
  return jagged_to_padded_dense(values, {offsets}, {max_sequence_length}, 0.0);
}

// ---- autograd for the jagged ops --------------------------------------------------------------
// The two copies are each other's transpose: the gradient of jagged_to_padded_dense with respect to
// values is dense_to_jagged of the output gradient (padding positions receive none), and the
// gradient of dense_to_jagged with respect to dense is jagged_to_padded_dense of the output
// gradient with zero padding. jagged_dense_elementwise_add passes its gradient to y unchanged and
// to x_values through dense_to_jagged. Offsets carry no gradient. The backward passes are the same
// CUDA kernels, called below the autograd key so that they are not recorded again.
std::vector<int64_t> max_lengths_of(const Tensor& dense, size_t jagged_dims) {
  return std::vector<int64_t>(dense.sizes().begin() + 1, dense.sizes().begin() + 1 + jagged_dims);
}

class JaggedToPaddedDenseFunction : public torch::autograd::Function<JaggedToPaddedDenseFunction> {
 public:
  static Variable forward(AutogradContext* ctx, const Tensor& values, const std::vector<Tensor>& offsets,
                          std::vector<int64_t> max_lengths, double padding_value) {
    at::AutoDispatchBelowADInplaceOrView guard;
    ctx->save_for_backward(offsets);
    ctx->saved_data["total"] = values.size(0);
    ctx->saved_data["vector"] = values.dim() == 1;
    return jagged_to_padded_dense(values, offsets, max_lengths, padding_value);
  }
  static variable_list backward(AutogradContext* ctx, variable_list grads) {
    at::AutoDispatchBelowADInplaceOrView guard;
    const auto offsets = ctx->get_saved_variables();
    Tensor g = grads[0].contiguous();
    const bool vec = ctx->saved_data["vector"].toBool();
    if (vec) g = g.unsqueeze(-1);
    Tensor gv = std::get<0>(dense_to_jagged(g, offsets, ctx->saved_data["total"].toInt()));
    if (vec) gv = gv.squeeze(-1);
    return {gv, Tensor(), Tensor(), Tensor()};
  }
};

class DenseToJaggedFunction : public torch::autograd::Function<DenseToJaggedFunction> {
 public:
  static Variable forward(AutogradContext* ctx, const Tensor& dense, const std::vector<Tensor>& offsets,
                          c10::optional<int64_t> total_L) {
    at::AutoDispatchBelowADInplaceOrView guard;
    ctx->save_for_backward(offsets);
    ctx->saved_data["max_lengths"] = max_lengths_of(dense, offsets.size());
    return std::get<0>(dense_to_jagged(dense, offsets, total_L));
  }
  static variable_list backward(AutogradContext* ctx, variable_list grads) {
    at::AutoDispatchBelowADInplaceOrView guard;
    const auto offsets = ctx->get_saved_variables();
    const std::vector<int64_t> ml = ctx->saved_data["max_lengths"].toIntVector();
    return {jagged_to_padded_dense(grads[0].contiguous(), offsets, ml, 0.0), Tensor(), Tensor()};
  }
};

class JaggedDenseAddFunction : public torch::autograd::Function<JaggedDenseAddFunction> {
 public:
  static Variable forward(AutogradContext* ctx, const Tensor& x_values, const std::vector<Tensor>& x_offsets,
                          const Tensor& y) {
    at::AutoDispatchBelowADInplaceOrView guard;
    ctx->save_for_backward(x_offsets);
    ctx->saved_data["total"] = x_values.size(0);
    return jagged_dense_elementwise_add(x_values, x_offsets, y);
  }
  static variable_list backward(AutogradContext* ctx, variable_list grads) {
    at::AutoDispatchBelowADInplaceOrView guard;
    const auto offsets = ctx->get_saved_variables();
    const Tensor g = grads[0].contiguous();
    return {std::get<0>(dense_to_jagged(g, offsets, ctx->saved_data["total"].toInt())), Tensor(), g};
  }
};

Tensor jagged_to_padded_dense_autograd(const Tensor& values, const std::vector<Tensor>& offsets,
                                       at::IntArrayRef max_lengths, double padding_value) {
  return JaggedToPaddedDenseFunction::apply(values, offsets, max_lengths.vec(), padding_value);
}
std::tuple<Tensor, std::vector<Tensor>> dense_to_jagged_autograd(const Tensor& dense,
                                                                 const std::vector<Tensor>& offsets,
                                                                 c10::optional<int64_t> total_L) {
  return {DenseToJaggedFunction::apply(dense, offsets, total_L), offsets};
}
Tensor jagged_dense_elementwise_add_autograd(const Tensor& x_values, const std::vector<Tensor>& x_offsets,
                                             const Tensor& y) {
  return JaggedDenseAddFunction::apply(x_values, x_offsets, y);
}
Tensor jagged_2d_to_dense_autograd(const Tensor& values, const Tensor& offsets, int64_t max_sequence_length) {
  return JaggedToPaddedDenseFunction::apply(values, std::vector<Tensor>{offsets},
                                            std::vector<int64_t>{max_sequence_length}, 0.0);
}

// ---- permute_2D_sparse_data -----------------------------------------------------------------------
// lengths is [T, B], indices (and weights) hold the T rows' ids one row after the other; row j of
// the result is row permute[j] of the input (rows may repeat or be left out, so the result can be
// longer or shorter than the input). Whole rows move as segments of b200tbe_permute_segments.
std::tuple<Tensor, Tensor, c10::optional<Tensor>> permute_2d_sparse_data(
    const Tensor& permute, const Tensor& lengths, const Tensor& indices,
    const c10::optional<Tensor>& weights, c10::optional<int64_t> permuted_lengths_sum) {
  check_cuda_contig(permute, "permute");
  check_cuda_contig(lengths, "lengths");
  check_cuda_contig(indices, "indices");
  TORCH_CHECK(lengths.dim() == 2, "lengths must be [T, B]");
  TORCH_CHECK(permute.scalar_type() == at::kInt || permute.scalar_type() == at::kLong,
              "permute must be int32 or int64");
  c10::cuda::CUDAGuard guard(indices.device());
  const Tensor permuted_lengths = lengths.index_select(0, permute);
  const Tensor row_len = lengths.to(at::kLong).sum(1);
  Tensor in_off = at::zeros({row_len.numel() + 1}, row_len.options());
  in_off.slice(0, 1).copy_(row_len.cumsum(0));
  const Tensor out_len = row_len.index_select(0, permute);
  Tensor out_off = at::zeros({out_len.numel() + 1}, out_len.options());
  out_off.slice(0, 1).copy_(out_len.cumsum(0));
  int64_t total = 0;
  if (permuted_lengths_sum.has_value()) {
    total = *permuted_lengths_sum;
  } else {
    total = out_off[-1].item<int64_t>();  // one synchronising read, as in fbgemm_gpu
  }
  TORCH_CHECK(total >= 0, "permuted_lengths_sum must be non-negative");
  auto move = [&](const Tensor& src, const char* what) {
    Tensor dst = at::empty({total}, src.options());
    const int64_t eb = static_cast<int64_t>(src.element_size());
    TORCH_CHECK(eb == 2 || eb == 4 || eb == 8, what, ": elements of 2, 4 or 8 bytes");
    check_status(b200tbe_permute_segments(src.data_ptr(), dst.data_ptr(), in_off.data_ptr(),
                                          out_off.data_ptr(), permute.data_ptr(), permute.numel(),
                                          total, static_cast<int32_t>(eb), 8,
                                          static_cast<int32_t>(permute.element_size()), current_stream()),
                 "permute_2D_sparse_data");
    return dst;
  };
  Tensor permuted_indices = move(indices, "indices");
  c10::optional<Tensor> permuted_weights;
  if (weights.has_value() && weights->defined()) {
    check_cuda_contig(*weights, "weights");
    TORCH_CHECK(weights->numel() == indices.numel(), "weights and indices differ in length");
    permuted_weights = move(*weights, "weights");
  }
  return {permuted_lengths, permuted_indices, permuted_weights};
}

// ---- TBE forward / backward -----------------------------------------------------------------

struct TbeCommon {
  Tensor dev_weights, weights_offsets, D_offsets, hash_size_cumsum, indices, offsets;
  c10::optional<Tensor> indice_weights;
  int64_t total_D, max_D, total_hash_size_bits, pooling_mode, output_dtype;
};

void check_placements(const Tensor& uvm_weights, const Tensor& lxu_cache_weights,
                      const Tensor& weights_placements) {
  TORCH_CHECK(is_empty_or_undefined(uvm_weights),
              "uvm_weights must be empty: all tables live in dev_weights (HBM)");
  TORCH_CHECK(is_empty_or_undefined(lxu_cache_weights), "lxu_cache_weights must be empty: no cache");
  if (weights_placements.defined() && weights_placements.numel() > 0) {
    static FactCache<bool> cache;   // read back once per placements tensor, not once per call
    const bool all_device = cache.get(
        weights_placements, [&] { return weights_placements.to(at::kCPU).eq(0).all().item<bool>(); });
    TORCH_CHECK(all_device, "weights_placements must be all DEVICE (0)");
  }
}

Tensor tbe_forward(const TbeCommon& c) {
  check_cuda_contig(c.dev_weights, "dev_weights");
  check_cuda_contig(c.weights_offsets, "weights_offsets");
  check_cuda_contig(c.D_offsets, "D_offsets");
  check_cuda_contig(c.indices, "indices");
  check_cuda_contig(c.offsets, "offsets");
  TORCH_CHECK(c.weights_offsets.scalar_type() == at::kLong, "weights_offsets must be int64");
  TORCH_CHECK(c.D_offsets.scalar_type() == at::kInt, "D_offsets must be int32");
  TORCH_CHECK(c.pooling_mode == B200TBE_POOL_SUM || c.pooling_mode == B200TBE_POOL_MEAN,
              "pooling_mode must be SUM (0) or MEAN (1)");
  const int64_t T = c.D_offsets.numel() - 1;
  TORCH_CHECK(T >= 0 && c.weights_offsets.numel() == T, "weights_offsets must have one entry per table");
  const int64_t B = T > 0 ? (c.offsets.numel() - 1) / T : 0;
  TORCH_CHECK(T == 0 || c.offsets.numel() == T * B + 1, "offsets must have T*B+1 entries");
  c10::cuda::CUDAGuard guard(c.dev_weights.device());
  Tensor out = at::empty({B, c.total_D},
                         c.dev_weights.options().dtype(output_scalar_type(c.output_dtype)));
  b200tbe_forward_params p{};
  p.dev_weights = c.dev_weights.data_ptr();
  p.weights_offsets = c.weights_offsets.data_ptr<int64_t>();
  p.D_offsets = c.D_offsets.data_ptr<int32_t>();
  p.indices = c.indices.data_ptr();
  p.offsets = c.offsets.data_ptr();
  if (c.indice_weights.has_value() && c.indice_weights->defined()) {
    check_cuda_contig(*c.indice_weights, "indice_weights");
    TORCH_CHECK(c.indice_weights->scalar_type() == at::kFloat, "indice_weights must be float32");
    TORCH_CHECK(c.indice_weights->numel() == c.indices.numel(), "one weight per index");
    p.per_sample_weights = c.indice_weights->data_ptr<float>();
  }
  // ids are range-checked against the tables' row counts; a bad id is skipped and flagged
  Tensor rows_keepalive, status_word;
  if (c.hash_size_cumsum.defined() && c.hash_size_cumsum.numel() == T + 1 && T > 0) {
    check_cuda_contig(c.hash_size_cumsum, "hash_size_cumsum");
    TORCH_CHECK(c.hash_size_cumsum.scalar_type() == at::kLong, "hash_size_cumsum must be int64");
    rows_keepalive = table_rows_of(c.hash_size_cumsum).rows_per_table;
    status_word = device_status(c.dev_weights.device());
    p.rows_per_table = rows_keepalive.data_ptr<int64_t>();
    p.status = status_word.data_ptr<int32_t>();
  }
  p.outputs[0] = out.data_ptr();
  p.output_stride = c.total_D;
  p.rows_per_dest = B > 0 ? B : 1;
  p.num_dests = 1;
  p.T = static_cast<int32_t>(T);
  p.B = static_cast<int32_t>(B);
  p.max_D = static_cast<int32_t>(c.max_D);
  p.weights_dtype = dtype_code(c.dev_weights.scalar_type());
  TORCH_CHECK(p.weights_dtype == B200TBE_FP32 || p.weights_dtype == B200TBE_FP16,
              "dev_weights must be float32 or float16");
  p.output_dtype = static_cast<int32_t>(c.output_dtype);
  p.index_bytes = index_bytes_of(c.indices, c.offsets);
  p.pooling_mode = static_cast<int32_t>(c.pooling_mode);
  check_status(b200tbe_forward(&p, current_stream()), "split_embedding lookup forward");
  return out;
}

struct OptimizerArgs {
  int optimizer;
  double learning_rate, eps;
  Tensor momentum1, momentum1_offsets;
};

void tbe_backward(const TbeCommon& c, const Tensor& grad_in, const OptimizerArgs& o) {
  Tensor grad = grad_in.contiguous();
  if (grad.scalar_type() != at::kFloat && grad.scalar_type() != at::kHalf) grad = grad.to(at::kFloat);
  const int64_t T = c.D_offsets.numel() - 1;
  const int64_t B = T > 0 ? (c.offsets.numel() - 1) / T : 0;
  if (T == 0 || B == 0 || c.indices.numel() == 0) return;
  check_cuda_contig(c.hash_size_cumsum, "hash_size_cumsum");
  TORCH_CHECK(c.hash_size_cumsum.scalar_type() == at::kLong && c.hash_size_cumsum.numel() == T + 1,
              "hash_size_cumsum must be int64 with T+1 entries");
  c10::cuda::CUDAGuard guard(c.dev_weights.device());
  const size_t need = b200tbe_backward_scratch_bytes(c.indices.numel(),
                                                     static_cast<int32_t>(c.total_hash_size_bits),
                                                     static_cast<int32_t>(c.max_D),
                                                     static_cast<int32_t>(T));
  Tensor scratch = at::empty({static_cast<int64_t>(need)}, c.dev_weights.options().dtype(at::kByte));
  b200tbe_backward_params p{};
  p.dev_weights = c.dev_weights.data_ptr();
  p.weights_offsets = c.weights_offsets.data_ptr<int64_t>();
  p.D_offsets = c.D_offsets.data_ptr<int32_t>();
  p.hash_size_cumsum = c.hash_size_cumsum.data_ptr<int64_t>();
  p.indices = c.indices.data_ptr();
  p.offsets = c.offsets.data_ptr();
  if (c.indice_weights.has_value() && c.indice_weights->defined())
    p.per_sample_weights = c.indice_weights->data_ptr<float>();
  p.grad_output = grad.data_ptr();
  p.grad_stride = grad.stride(0);
  p.grad_col_offset = 0;
  if (o.optimizer == B200TBE_OPT_ROWWISE_ADAGRAD) {
    check_cuda_contig(o.momentum1, "momentum1_dev");
    check_cuda_contig(o.momentum1_offsets, "momentum1_offsets");
    TORCH_CHECK(o.momentum1.scalar_type() == at::kFloat, "momentum1_dev must be float32");
    TORCH_CHECK(o.momentum1_offsets.scalar_type() == at::kLong, "momentum1_offsets must be int64");
    p.momentum1 = o.momentum1.data_ptr<float>();
    p.momentum1_offsets = o.momentum1_offsets.data_ptr<int64_t>();
  }
  p.num_indices = c.indices.numel();
  p.T = static_cast<int32_t>(T);
  p.B = static_cast<int32_t>(B);
  p.max_D = static_cast<int32_t>(c.max_D);
  p.total_hash_size_bits = static_cast<int32_t>(c.total_hash_size_bits);
  p.weights_dtype = dtype_code(c.dev_weights.scalar_type());
  p.grad_dtype = dtype_code(grad.scalar_type());
  p.index_bytes = index_bytes_of(c.indices, c.offsets);
  p.pooling_mode = static_cast<int32_t>(c.pooling_mode);
  p.optimizer = o.optimizer;
  p.learning_rate = static_cast<float>(o.learning_rate);
  p.eps = static_cast<float>(o.eps);
  p.scratch = scratch.data_ptr();
  p.scratch_bytes = need;
  p.max_table_rows = table_rows_of(c.hash_size_cumsum).max_rows;
  Tensor status_word = device_status(c.dev_weights.device());
  p.status = status_word.data_ptr<int32_t>();
  check_status(b200tbe_backward(&p, current_stream()), "split_embedding lookup backward");
}

// One autograd node for both optimizers: forward pools, backward applies the fused update in
// place and hands no gradient to any input (the placeholder tensor only exists to get this node
// into the graph).
class TbeLookupFunction : public torch::autograd::Function<TbeLookupFunction> {
 public:
  static Variable forward(AutogradContext* ctx, const Tensor& placeholder_autograd_tensor,
                          const Tensor& dev_weights, const Tensor& weights_offsets,
                          const Tensor& D_offsets, int64_t total_D, int64_t max_D,
                          const Tensor& hash_size_cumsum, int64_t total_hash_size_bits,
                          const Tensor& indices, const Tensor& offsets, int64_t pooling_mode,
                          const c10::optional<Tensor>& indice_weights, int64_t output_dtype,
                          int64_t optimizer, double learning_rate, double eps,
                          const Tensor& momentum1, const Tensor& momentum1_offsets) {
    (void)placeholder_autograd_tensor;
    TbeCommon c{dev_weights, weights_offsets, D_offsets, hash_size_cumsum, indices, offsets,
                indice_weights, total_D, max_D, total_hash_size_bits, pooling_mode, output_dtype};
    ctx->save_for_backward({dev_weights, weights_offsets, D_offsets, hash_size_cumsum, indices,
                            offsets, indice_weights.value_or(Tensor()), momentum1,
                            momentum1_offsets});
    ctx->saved_data["total_D"] = total_D;
    ctx->saved_data["max_D"] = max_D;
    ctx->saved_data["total_hash_size_bits"] = total_hash_size_bits;
    ctx->saved_data["pooling_mode"] = pooling_mode;
    ctx->saved_data["output_dtype"] = output_dtype;
    ctx->saved_data["optimizer"] = optimizer;
    ctx->saved_data["learning_rate"] = learning_rate;
    ctx->saved_data["eps"] = eps;
    return tbe_forward(c);
  }

  static variable_list backward(AutogradContext* ctx, variable_list grad_outputs) {
    const auto saved = ctx->get_saved_variables();
    TbeCommon c{saved[0], saved[1], saved[2], saved[3], saved[4], saved[5],
                saved[6].defined() ? c10::optional<Tensor>(saved[6]) : c10::nullopt,
                ctx->saved_data["total_D"].toInt(), ctx->saved_data["max_D"].toInt(),
                ctx->saved_data["total_hash_size_bits"].toInt(),
                ctx->saved_data["pooling_mode"].toInt(), ctx->saved_data["output_dtype"].toInt()};
    OptimizerArgs o{static_cast<int>(ctx->saved_data["optimizer"].toInt()),
                    ctx->saved_data["learning_rate"].toDouble(), ctx->saved_data["eps"].toDouble(),
                    saved[7], saved[8]};
    TORCH_CHECK(grad_outputs.size() == 1 && grad_outputs[0].defined(), "missing output gradient");
    tbe_backward(c, grad_outputs[0], o);
    return variable_list(18);
  }
};

void check_training_neutral(bool gradient_clipping, bool stochastic_rounding,
                            const c10::optional<Tensor>& feature_requires_grad,
                            const Tensor& lxu_cache_locations) {
  TORCH_CHECK(!gradient_clipping, "gradient_clipping is not supported");
  TORCH_CHECK(!stochastic_rounding,
              "stochastic_rounding must be false: fp16 weights are written round-to-nearest");
  TORCH_CHECK(!feature_requires_grad.has_value() || !feature_requires_grad->defined() ||
                  feature_requires_grad->numel() == 0,
              "feature_requires_grad is not supported");
  (void)lxu_cache_locations;
}

Tensor split_embedding_codegen_lookup_rowwise_adagrad_function(
    const Tensor& placeholder_autograd_tensor, const Tensor& dev_weights, const Tensor& uvm_weights,
    const Tensor& lxu_cache_weights, const Tensor& weights_placements,
    const Tensor& weights_offsets, const Tensor& D_offsets, int64_t total_D, int64_t max_D,
    const Tensor& hash_size_cumsum, int64_t total_hash_size_bits, const Tensor& indices,
    const Tensor& offsets, int64_t pooling_mode, const c10::optional<Tensor>& indice_weights,
    const c10::optional<Tensor>& feature_requires_grad, const Tensor& lxu_cache_locations,
    bool gradient_clipping, double max_gradient, bool stochastic_rounding,
    const Tensor& momentum1_dev, const Tensor& momentum1_uvm, const Tensor& momentum1_placements,
    const Tensor& momentum1_offsets, double eps, double learning_rate, double weight_decay,
    int64_t weight_decay_mode, double max_norm, int64_t output_dtype) {
  (void)max_gradient;
  (void)weight_decay_mode;
  check_placements(uvm_weights, lxu_cache_weights, weights_placements);
  check_placements(momentum1_uvm, Tensor(), momentum1_placements);
  check_training_neutral(gradient_clipping, stochastic_rounding, feature_requires_grad,
                         lxu_cache_locations);
  TORCH_CHECK(weight_decay == 0.0, "weight_decay is not supported");
  TORCH_CHECK(max_norm == 0.0, "max_norm is not supported");
  return TbeLookupFunction::apply(placeholder_autograd_tensor, dev_weights, weights_offsets,
                                  D_offsets, total_D, max_D, hash_size_cumsum,
                                  total_hash_size_bits, indices, offsets, pooling_mode,
                                  indice_weights, output_dtype,
                                  static_cast<int64_t>(B200TBE_OPT_ROWWISE_ADAGRAD), learning_rate,
                                  eps, momentum1_dev, momentum1_offsets);
}

Tensor split_embedding_codegen_lookup_sgd_function(
    const Tensor& placeholder_autograd_tensor, const Tensor& dev_weights, const Tensor& uvm_weights,
    const Tensor& lxu_cache_weights, const Tensor& weights_placements,
    const Tensor& weights_offsets, const Tensor& D_offsets, int64_t total_D, int64_t max_D,
    const Tensor& hash_size_cumsum, int64_t total_hash_size_bits, const Tensor& indices,
    const Tensor& offsets, int64_t pooling_mode, const c10::optional<Tensor>& indice_weights,
    const c10::optional<Tensor>& feature_requires_grad, const Tensor& lxu_cache_locations,
    bool gradient_clipping, double max_gradient, bool stochastic_rounding, double learning_rate,
    int64_t output_dtype) {
  (void)max_gradient;
  check_placements(uvm_weights, lxu_cache_weights, weights_placements);
  check_training_neutral(gradient_clipping, stochastic_rounding, feature_requires_grad,
                         lxu_cache_locations);
  return TbeLookupFunction::apply(placeholder_autograd_tensor, dev_weights, weights_offsets,
                                  D_offsets, total_D, max_D, hash_size_cumsum,
                                  total_hash_size_bits, indices, offsets, pooling_mode,
                                  indice_weights, output_dtype,
                                  static_cast<int64_t>(B200TBE_OPT_SGD), learning_rate, 0.0,
                                  at::empty({0}, dev_weights.options().dtype(at::kFloat)),
                                  at::empty({0}, dev_weights.options().dtype(at::kLong)));
}

// ---- quantised inference lookup ----------------------------------------------------------------

Tensor int_nbit_split_embedding_codegen_lookup_function(
    const Tensor& dev_weights, const Tensor& uvm_weights, const Tensor& weights_placements,
    const Tensor& weights_offsets, const Tensor& weights_tys, const Tensor& D_offsets,
    int64_t total_D, int64_t max_int2_D, int64_t max_int4_D, int64_t max_int8_D,
    int64_t max_float16_D, int64_t max_float32_D, const Tensor& indices, const Tensor& offsets,
    int64_t pooling_mode, const c10::optional<Tensor>& indice_weights, int64_t output_dtype,
    const c10::optional<Tensor>& lxu_cache_weights,
    const c10::optional<Tensor>& lxu_cache_locations, c10::optional<int64_t> row_alignment,
    c10::optional<int64_t> max_float8_D, c10::optional<int64_t> fp8_exponent_bits,
    c10::optional<int64_t> fp8_exponent_bias) {
  (void)lxu_cache_locations;
  (void)fp8_exponent_bits;
  (void)fp8_exponent_bias;
  check_placements(uvm_weights, lxu_cache_weights.value_or(Tensor()), weights_placements);
  TORCH_CHECK(max_float8_D.value_or(0) == 0, "FP8 tables are not supported");
  check_cuda_contig(dev_weights, "dev_weights");
  check_cuda_contig(weights_offsets, "weights_offsets");
  check_cuda_contig(weights_tys, "weights_tys");
  check_cuda_contig(D_offsets, "D_offsets");
  check_cuda_contig(indices, "indices");
  check_cuda_contig(offsets, "offsets");
  TORCH_CHECK(dev_weights.scalar_type() == at::kByte, "dev_weights must be uint8");
  TORCH_CHECK(weights_tys.scalar_type() == at::kByte, "weights_tys must be uint8");
  TORCH_CHECK(weights_offsets.scalar_type() == at::kLong, "weights_offsets must be int64");
  TORCH_CHECK(D_offsets.scalar_type() == at::kInt, "D_offsets must be int32");
  TORCH_CHECK(pooling_mode == B200TBE_POOL_SUM || pooling_mode == B200TBE_POOL_MEAN,
              "pooling_mode must be SUM (0) or MEAN (1)");
  const int64_t T = D_offsets.numel() - 1;
  TORCH_CHECK(T >= 0 && weights_offsets.numel() == T && weights_tys.numel() == T,
              "weights_offsets and weights_tys must have one entry per table");
  const int64_t B = T > 0 ? (offsets.numel() - 1) / T : 0;
  TORCH_CHECK(T == 0 || offsets.numel() == T * B + 1, "offsets must have T*B+1 entries");
  c10::cuda::CUDAGuard guard(dev_weights.device());
  Tensor out =
      at::empty({B, total_D}, dev_weights.options().dtype(output_scalar_type(output_dtype)));
  b200tbe_nbit_forward_params p{};
  p.dev_weights = dev_weights.data_ptr<uint8_t>();
  p.weights_offsets = weights_offsets.data_ptr<int64_t>();
  p.weights_tys = weights_tys.data_ptr<uint8_t>();
  p.D_offsets = D_offsets.data_ptr<int32_t>();
  p.indices = indices.data_ptr();
  p.offsets = offsets.data_ptr();
  if (indice_weights.has_value() && indice_weights->defined()) {
    check_cuda_contig(*indice_weights, "indice_weights");
    TORCH_CHECK(indice_weights->scalar_type() == at::kFloat, "indice_weights must be float32");
    p.per_sample_weights = indice_weights->data_ptr<float>();
  }
  p.outputs[0] = out.data_ptr();
  p.output_stride = total_D;
  p.rows_per_dest = B > 0 ? B : 1;
  p.num_dests = 1;
  p.T = static_cast<int32_t>(T);
  p.B = static_cast<int32_t>(B);
  p.max_D = static_cast<int32_t>(std::max({max_int2_D, max_int4_D, max_int8_D, max_float16_D,
                                           max_float32_D}));
  p.row_alignment = static_cast<int32_t>(row_alignment.value_or(16));
  // the per-type maxima say which types exist at all
  p.table_type_mask = (max_int2_D > 0 ? 1u << B200TBE_INT2 : 0u) | (max_int4_D > 0 ? 1u << B200TBE_INT4 : 0u) |
                      (max_int8_D > 0 ? 1u << B200TBE_INT8 : 0u) | (max_float16_D > 0 ? 1u << B200TBE_FP16 : 0u) |
                      (max_float32_D > 0 ? 1u << B200TBE_FP32 : 0u);
  // Row counts for the range check: the op's argument list does not carry them, but a table ends no
  // later than where the nearest following table begins (or dev_weights ends), so
  // rows_t <= bytes_t / stride_t: an id beyond that would read another table's bytes.
  Tensor rows_keepalive, status_word;
  if (T > 0) {
    static FactCache<Tensor> cache;
    const int64_t total_bytes = dev_weights.numel();
    const int32_t align = p.row_alignment;
    rows_keepalive = cache.get(weights_offsets, [&] {
      const Tensor wo = weights_offsets.to(at::kCPU), ty = weights_tys.to(at::kCPU), Do = D_offsets.to(at::kCPU);
      Tensor rows = at::empty({T}, at::TensorOptions().dtype(at::kLong));
      for (int64_t t = 0; t < T; ++t) {
        const int64_t begin = wo.data_ptr<int64_t>()[t];
        int64_t end = total_bytes;   // tables need not be stored in table order
        for (int64_t u = 0; u < T; ++u) {
          const int64_t b = wo.data_ptr<int64_t>()[u];
          if (b > begin && b < end) end = b;
        }
        const int32_t D = Do.data_ptr<int32_t>()[t + 1] - Do.data_ptr<int32_t>()[t];
        const int code = ty.data_ptr<uint8_t>()[t];
        int64_t stride = b200tbe_quantized_row_bytes(D, code, align);
        if (stride <= 0) {   // float tables: no header
          const int64_t raw = static_cast<int64_t>(D) * (code == B200TBE_FP16 ? 2 : 4);
          stride = (raw + align - 1) / align * align;
        }
        rows.data_ptr<int64_t>()[t] = stride > 0 && end > begin ? (end - begin) / stride : 0;
      }
      return rows.to(dev_weights.device());
    });
    status_word = device_status(dev_weights.device());
    p.rows_per_table = rows_keepalive.data_ptr<int64_t>();
    p.status = status_word.data_ptr<int32_t>();
  }
  p.output_dtype = static_cast<int32_t>(output_dtype);
  p.index_bytes = index_bytes_of(indices, offsets);
  p.pooling_mode = static_cast<int32_t>(pooling_mode);
  check_status(b200tbe_nbit_forward(&p, current_stream()), "int_nbit_split_embedding lookup");
  return out;
}

// ---- fused N-bit row-wise quantisation ops -----------------------------------------------------
// Layout of FBGEMM's fused N-bit row-wise ops: [rows, payload + 4], fp16 scale and bias BEHIND the
// payload, rows unpadded.

int nbit_type(int64_t bit_rate) {
  TORCH_CHECK(bit_rate == 2 || bit_rate == 4 || bit_rate == 8, "bit_rate must be 2, 4 or 8");
  return bit_rate == 8 ? B200TBE_INT8 : (bit_rate == 4 ? B200TBE_INT4 : B200TBE_INT2);
}

Tensor float_or_half_to_fused_nbit(const Tensor& input, int64_t bit_rate) {
  check_cuda_contig(input, "input");
  TORCH_CHECK(input.dim() == 2, "input must be [rows, columns]");
  TORCH_CHECK(input.scalar_type() == at::kFloat || input.scalar_type() == at::kHalf,
              "input must be float32 or float16");
  const int ty = nbit_type(bit_rate);
  const int64_t rows = input.size(0), D = input.size(1);
  TORCH_CHECK(D % (8 / bit_rate) == 0, "columns must be a multiple of ", 8 / bit_rate);
  c10::cuda::CUDAGuard guard(input.device());
  const int64_t stride = b200tbe_quantized_row_bytes(static_cast<int32_t>(D), ty, 1);
  Tensor out = at::empty({rows, stride}, input.options().dtype(at::kByte));
  check_status(b200tbe_quantize_rows(input.data_ptr(), dtype_code(input.scalar_type()), rows,
                                     static_cast<int32_t>(D), ty, 1, /*header_first=*/0,
                                     out.data_ptr<uint8_t>(), current_stream()),
               "FloatOrHalfToFusedNBitRowwiseQuantizedSBHalf");
  return out;
}

Tensor fused_nbit_to_float_or_half(const Tensor& input, int64_t bit_rate, int64_t output_dtype) {
  check_cuda_contig(input, "input");
  TORCH_CHECK(input.dim() == 2 && input.scalar_type() == at::kByte, "input must be uint8 [rows, bytes]");
  TORCH_CHECK(input.size(1) >= 4, "rows must hold the 4-byte scale/bias");
  const int ty = nbit_type(bit_rate);
  const int64_t rows = input.size(0), D = (input.size(1) - 4) * (8 / bit_rate);
  c10::cuda::CUDAGuard guard(input.device());
  Tensor out = at::empty({rows, D}, input.options().dtype(output_scalar_type(output_dtype)));
  check_status(b200tbe_dequantize_rows(input.data_ptr<uint8_t>(), rows, static_cast<int32_t>(D), ty,
                                       1, /*header_first=*/0, out.data_ptr(),
                                       static_cast<int32_t>(output_dtype), current_stream()),
               "FusedNBitRowwiseQuantizedSBHalfToFloatOrHalf");
  return out;
}

Tensor fused_nbit_to_float(const Tensor& input, int64_t bit_rate) {
  return fused_nbit_to_float_or_half(input, bit_rate, B200TBE_FP32);
}
Tensor fused_nbit_to_half(const Tensor& input, int64_t bit_rate) {
  return fused_nbit_to_float_or_half(input, bit_rate, B200TBE_FP16);
}

}  // namespace

// A second definition of these schemas (an fbgemm_gpu install in the same process) makes
// TORCH_LIBRARY_FRAGMENT's def() throw at load time, which is the loud failure wanted here.
TORCH_LIBRARY_FRAGMENT(fbgemm, m) {
  m.def(
      "jagged_to_padded_dense(Tensor values, Tensor[] offsets, int[] max_lengths, "
      "float padding_value=0) -> Tensor");
  m.def("dense_to_jagged(Tensor dense, Tensor[] x_offsets, int? total_L=None) -> (Tensor, Tensor[])");
  m.def("jagged_dense_elementwise_add(Tensor x_values, Tensor[] x_offsets, Tensor y) -> Tensor");
  m.def("jagged_2d_to_dense(Tensor values, Tensor offsets, int max_sequence_length) -> Tensor");
  m.def(
      "permute_2D_sparse_data(Tensor permute, Tensor lengths, Tensor indices, Tensor? weights=None, "
      "int? permuted_lengths_sum=None) -> (Tensor, Tensor, Tensor?)");
  m.def("FloatToFusedNBitRowwiseQuantizedSBHalf(Tensor input, int bit_rate) -> Tensor");
  m.def("HalfToFusedNBitRowwiseQuantizedSBHalf(Tensor input, int bit_rate) -> Tensor");
  m.def("FloatOrHalfToFusedNBitRowwiseQuantizedSBHalf(Tensor input, int bit_rate) -> Tensor");
  m.def("FusedNBitRowwiseQuantizedSBHalfToFloat(Tensor input, int bit_rate) -> Tensor");
  m.def("FusedNBitRowwiseQuantizedSBHalfToHalf(Tensor input, int bit_rate) -> Tensor");
  m.def(
      "FusedNBitRowwiseQuantizedSBHalfToFloatOrHalf(Tensor input, int bit_rate, int output_dtype=0) "
      "-> Tensor");
  m.def(
      "split_embedding_codegen_lookup_rowwise_adagrad_function(Tensor placeholder_autograd_tensor, "
      "Tensor dev_weights, Tensor uvm_weights, Tensor lxu_cache_weights, Tensor weights_placements, "
      "Tensor weights_offsets, Tensor D_offsets, int total_D, int max_D, Tensor hash_size_cumsum, "
      "int total_hash_size_bits, Tensor indices, Tensor offsets, int pooling_mode, "
      "Tensor? indice_weights, Tensor? feature_requires_grad, Tensor lxu_cache_locations, "
      "bool gradient_clipping, float max_gradient, bool stochastic_rounding, Tensor momentum1_dev, "
      "Tensor momentum1_uvm, Tensor momentum1_placements, Tensor momentum1_offsets, float eps=0, "
      "float learning_rate=0, float weight_decay=0.0, int weight_decay_mode=0, float max_norm=0.0, "
      "int output_dtype=0) -> Tensor");
  m.def(
      "split_embedding_codegen_lookup_sgd_function(Tensor placeholder_autograd_tensor, "
      "Tensor dev_weights, Tensor uvm_weights, Tensor lxu_cache_weights, Tensor weights_placements, "
      "Tensor weights_offsets, Tensor D_offsets, int total_D, int max_D, Tensor hash_size_cumsum, "
      "int total_hash_size_bits, Tensor indices, Tensor offsets, int pooling_mode, "
      "Tensor? indice_weights, Tensor? feature_requires_grad, Tensor lxu_cache_locations, "
      "bool gradient_clipping, float max_gradient, bool stochastic_rounding, "
      "float learning_rate=0, int output_dtype=0) -> Tensor");
  m.def(
      "int_nbit_split_embedding_codegen_lookup_function(Tensor dev_weights, Tensor uvm_weights, "
      "Tensor weights_placements, Tensor weights_offsets, Tensor weights_tys, Tensor D_offsets, "
      "int total_D, int max_int2_D, int max_int4_D, int max_int8_D, int max_float16_D, "
      "int max_float32_D, Tensor indices, Tensor offsets, int pooling_mode, "
      "Tensor? indice_weights, int output_dtype=1, Tensor? lxu_cache_weights=None, "
      "Tensor? lxu_cache_locations=None, int? row_alignment=None, int? max_float8_D=0, "
      "int? fp8_exponent_bits=-1, int? fp8_exponent_bias=-1) -> Tensor");
  // Not an fbgemm_gpu operator: returns, and clears, the B200TBE_DEV_* bits the lookup kernels have
  // raised on the device of `like` since the last call (0: none). Synchronises.
  m.def("b200tbe_pop_device_status(Tensor like) -> int");
}

TORCH_LIBRARY_IMPL(fbgemm, CUDA, m) {
  m.impl("jagged_to_padded_dense", TORCH_FN(jagged_to_padded_dense));
  m.impl("dense_to_jagged", TORCH_FN(dense_to_jagged));
  m.impl("jagged_dense_elementwise_add", TORCH_FN(jagged_dense_elementwise_add));
  m.impl("jagged_2d_to_dense", TORCH_FN(jagged_2d_to_dense));
  m.impl("permute_2D_sparse_data", TORCH_FN(permute_2d_sparse_data));
  m.impl("FloatToFusedNBitRowwiseQuantizedSBHalf", TORCH_FN(float_or_half_to_fused_nbit));
  m.impl("HalfToFusedNBitRowwiseQuantizedSBHalf", TORCH_FN(float_or_half_to_fused_nbit));
  m.impl("FloatOrHalfToFusedNBitRowwiseQuantizedSBHalf", TORCH_FN(float_or_half_to_fused_nbit));
  m.impl("FusedNBitRowwiseQuantizedSBHalfToFloat", TORCH_FN(fused_nbit_to_float));
  m.impl("FusedNBitRowwiseQuantizedSBHalfToHalf", TORCH_FN(fused_nbit_to_half));
  m.impl("FusedNBitRowwiseQuantizedSBHalfToFloatOrHalf", TORCH_FN(fused_nbit_to_float_or_half));
  m.impl("int_nbit_split_embedding_codegen_lookup_function",
         TORCH_FN(int_nbit_split_embedding_codegen_lookup_function));
  m.impl("b200tbe_pop_device_status", TORCH_FN(pop_device_status));
}

// The training lookups and the jagged ops carry their own autograd nodes, so they also sit on the
// Autograd key (the jagged ops' CUDA registrations above are what those nodes call).
TORCH_LIBRARY_IMPL(fbgemm, AutogradCUDA, m) {
  m.impl("jagged_to_padded_dense", TORCH_FN(jagged_to_padded_dense_autograd));
  m.impl("dense_to_jagged", TORCH_FN(dense_to_jagged_autograd));
  m.impl("jagged_dense_elementwise_add", TORCH_FN(jagged_dense_elementwise_add_autograd));
  m.impl("jagged_2d_to_dense", TORCH_FN(jagged_2d_to_dense_autograd));
  m.impl("split_embedding_codegen_lookup_rowwise_adagrad_function",
         TORCH_FN(split_embedding_codegen_lookup_rowwise_adagrad_function));
  m.impl("split_embedding_codegen_lookup_sgd_function",
         TORCH_FN(split_embedding_codegen_lookup_sgd_function));
}
