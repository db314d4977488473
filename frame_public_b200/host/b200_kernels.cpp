// One KernelFn per op of the compiled-graph path, registered for backend "cuda" with
// FRAME_REGISTER_KERNEL (include/frame/ops/kernel_registry.h:46-51,104-107 of the reference).
// These are what Backend::launch (eager, unit tests) and the backend_lowering pass see
// (src/compiler/passes/backend_lowering.cpp:26-82: every op of a graph needs an (op, "cuda")
// kernel or the whole graph drops to the eager fallback).  Each function only unpacks the
// borrowed KernelContext and calls the C ABI; dtype dispatch happens inside the library.
// They replace src/backends/cuda/kernels/*.cpp|*.cu of the reference.
#include <cmath>
#include <string>
#include <variant>
#include <vector>

#include <frame/core/tensor.h>
#include <frame/hal/backend.h>
#include <frame/hal/stream.h>
#include <frame/ops/fused_elementwise_utils.h>
#include <frame/ops/kernel_registry.h>

#include "b200_status.h"
#include "frame_b200.h"

namespace {

using frame::ErrorCode;
using frame::Status;
using frame::Tensor;
using frame::ops::KernelContext;

fb200_stream stream_of(const KernelContext& ctx) {
  return ctx.stream != nullptr ? ctx.stream->native_handle() : nullptr;
}
int dtype_of(const Tensor& t) { return static_cast<int>(t.dtype().code()); }
int allow_tf32(const KernelContext& ctx) {
  return (ctx.compile_options != nullptr && ctx.compile_options->allow_tf32) ? 1 : 0;
}

Status arity(const KernelContext& ctx, std::string_view op, size_t min_in, size_t max_in) {
  if (ctx.inputs.size() < min_in || ctx.inputs.size() > max_in) {
    return Status::make(ErrorCode::kInvalidArgument,
                        "op '" + std::string(op) + "' cuda kernel expects " +
                            std::to_string(min_in) + (max_in != min_in ? ".." + std::to_string(max_in) : "") +
                            " inputs, got " + std::to_string(ctx.inputs.size()));
  }
  if (ctx.outputs.size() != 1) {
    return Status::make(ErrorCode::kInvalidArgument,
                        "op '" + std::string(op) + "' cuda kernel expects 1 output, got " +
                            std::to_string(ctx.outputs.size()));
  }
  for (const Tensor& t : ctx.inputs) {
    if (!(t.dtype() == ctx.outputs[0].dtype())) {
      return Status::make(ErrorCode::kInvalidArgument,
                          "op '" + std::string(op) + "' cuda kernel requires one dtype for all operands");
    }
  }
  return Status::ok();
}

template <typename T>
const T* attr(const KernelContext& ctx, const char* name) {
  if (ctx.attrs == nullptr) return nullptr;
  const auto it = ctx.attrs->find(name);
  if (it == ctx.attrs->end()) return nullptr;
  return std::get_if<T>(&it->second);
}

Status missing(std::string_view op, const char* name) {
  return Status::make(ErrorCode::kInvalidArgument, "op '" + std::string(op) +
                                                       "' cuda kernel is missing required attribute '" +
                                                       name + "'");
}

// ---- elementwise --------------------------------------------------------------------------------
template <int CODE, int ARITY>
Status elementwise(KernelContext& ctx, const char* op) {
  FRAME_RETURN_IF_ERROR(arity(ctx, op, ARITY, ARITY));
  for (const Tensor& t : ctx.inputs) {
    if (!(t.shape() == ctx.outputs[0].shape())) {
      return Status::make(ErrorCode::kInvalidArgument,
                          "op '" + std::string(op) + "' cuda kernel requires identical shapes, got " +
                              t.shape().to_string() + " and " + ctx.outputs[0].shape().to_string());
    }
  }
  const void* in[2] = {ctx.inputs[0].raw_data(), ARITY == 2 ? ctx.inputs[1].raw_data() : nullptr};
  const int ops[1] = {CODE};
  const int ar[1] = {ARITY};
  return frame_b200::to_status(
      fb200_fused_elementwise(in, ARITY, ctx.outputs[0].raw_data(), ctx.outputs[0].numel(),
                              dtype_of(ctx.outputs[0]), ops, ar, 1, stream_of(ctx)),
      op);
}

int code_of(std::string_view name) {
  static const char* names[] = {"", "add", "mul", "relu", "square", "sigmoid", "tanh", "rsqrt",
                                "gelu", "silu", "softplus", "exp", "heaviside_surrogate", "relu_grad_internal"};
  for (int i = 1; i <= 13; ++i) if (name == names[i]) return i;
  return 0;
}

// fused_elementwise_internal{ops="add;mul;relu", arities=[2,2,1]}: one launch for the group
// (the reference calls each sub-kernel in turn, src/ops/fused_elementwise_utils.cpp:122-206).
Status fused_elementwise(KernelContext& ctx) {
  if (ctx.outputs.size() != 1) {
    return Status::make(ErrorCode::kInvalidArgument,
                        "op 'fused_elementwise_internal' cuda kernel expects 1 output");
  }
  const std::string* ops_attr = attr<std::string>(ctx, "ops");
  const std::vector<int64_t>* ar_attr = attr<std::vector<int64_t>>(ctx, "arities");
  if (ops_attr == nullptr) return missing("fused_elementwise_internal", "ops");
  if (ar_attr == nullptr) return missing("fused_elementwise_internal", "arities");
  std::vector<int> codes, arities;
  size_t start = 0;
  while (start <= ops_attr->size()) {
    const size_t semi = ops_attr->find(';', start);
    const std::string name = ops_attr->substr(start, semi == std::string::npos ? std::string::npos : semi - start);
    const int code = code_of(name);
    if (code == 0) {
      return Status::make(ErrorCode::kUnimplemented,
                          "op 'fused_elementwise_internal': sub-op '" + name + "' has no cuda kernel");
    }
    codes.push_back(code);
    if (semi == std::string::npos) break;
    start = semi + 1;
  }
  for (const int64_t a : *ar_attr) arities.push_back(static_cast<int>(a));
  if (arities.size() != codes.size()) {
    return Status::make(ErrorCode::kInvalidArgument,
                        "op 'fused_elementwise_internal': ops and arities differ in length");
  }
  std::vector<const void*> in(ctx.inputs.size());
  for (size_t i = 0; i < ctx.inputs.size(); ++i) {
    if (!(ctx.inputs[i].shape() == ctx.outputs[0].shape()) ||
        !(ctx.inputs[i].dtype() == ctx.outputs[0].dtype())) {
      return Status::make(ErrorCode::kInvalidArgument,
                          "op 'fused_elementwise_internal' cuda kernel requires identical shapes and dtypes");
    }
    in[i] = ctx.inputs[i].raw_data();
  }
  return frame_b200::to_status(
      fb200_fused_elementwise(in.data(), static_cast<int>(in.size()), ctx.outputs[0].raw_data(),
                              ctx.outputs[0].numel(), dtype_of(ctx.outputs[0]), codes.data(),
                              arities.data(), static_cast<int>(codes.size()), stream_of(ctx)),
      "fused_elementwise_internal");
}

// ---- contractions ---------------------------------------------------------------------------------
Status matmul(KernelContext& ctx) {
  FRAME_RETURN_IF_ERROR(arity(ctx, "matmul", 2, 2));
  const Tensor& a = ctx.inputs[0];
  const Tensor& b = ctx.inputs[1];
  Tensor& c = ctx.outputs[0];
  if (a.shape().rank() != 2 || b.shape().rank() != 2 || c.shape().rank() != 2) {
    return Status::make(ErrorCode::kInvalidArgument, "op 'matmul' cuda kernel requires rank-2 operands");
  }
  const int64_t m = a.shape().dim(0), k = a.shape().dim(1), n = b.shape().dim(1);
  if (b.shape().dim(0) != k || c.shape().dim(0) != m || c.shape().dim(1) != n) {
    return Status::make(ErrorCode::kInvalidArgument,
                        "op 'matmul' cuda kernel shape mismatch: " + a.shape().to_string() + " x " +
                            b.shape().to_string() + " -> " + c.shape().to_string());
  }
  return frame_b200::to_status(fb200_matmul(a.raw_data(), b.raw_data(), c.raw_data(), m, n, k,
                                            dtype_of(c), allow_tf32(ctx), nullptr, stream_of(ctx)),
                               "matmul");
}

Status conv2d(KernelContext& ctx) {
  FRAME_RETURN_IF_ERROR(arity(ctx, "conv2d", 2, 3));
  const auto* stride = attr<std::vector<int64_t>>(ctx, "stride");
  const auto* padding = attr<std::vector<int64_t>>(ctx, "padding");
  const auto* groups = attr<int64_t>(ctx, "groups");
  if (stride == nullptr || stride->size() != 2) return missing("conv2d", "stride");
  if (padding == nullptr || padding->size() != 2) return missing("conv2d", "padding");
  if (groups == nullptr) return missing("conv2d", "groups");
  const Tensor& x = ctx.inputs[0];
  const Tensor& w = ctx.inputs[1];
  if (x.shape().rank() != 4 || w.shape().rank() != 4) {
    return Status::make(ErrorCode::kInvalidArgument, "op 'conv2d' cuda kernel requires rank-4 x and w");
  }
  fb200_conv2d_params p{};
  p.n = x.shape().dim(0); p.cin = x.shape().dim(1); p.h = x.shape().dim(2); p.w = x.shape().dim(3);
  p.cout = w.shape().dim(0); p.kh = w.shape().dim(2); p.kw = w.shape().dim(3);
  p.stride_h = (*stride)[0]; p.stride_w = (*stride)[1];
  p.pad_h = (*padding)[0]; p.pad_w = (*padding)[1];
  p.groups = *groups;
  if (w.shape().dim(1) * p.groups != p.cin) {
    return Status::make(ErrorCode::kInvalidArgument, "op 'conv2d' cuda kernel: w.dim(1)*groups != Cin");
  }
  const void* bias = ctx.inputs.size() == 3 ? ctx.inputs[2].raw_data() : nullptr;
  return frame_b200::to_status(
      fb200_conv2d(x.raw_data(), w.raw_data(), bias, ctx.outputs[0].raw_data(), &p,
                   dtype_of(ctx.outputs[0]), allow_tf32(ctx), nullptr, stream_of(ctx)),
      "conv2d");
}

Status conv1d(KernelContext& ctx) {
  FRAME_RETURN_IF_ERROR(arity(ctx, "conv1d", 2, 3));
  const auto* stride = attr<int64_t>(ctx, "stride");
  const auto* padding = attr<int64_t>(ctx, "padding");
  const auto* groups = attr<int64_t>(ctx, "groups");
  if (stride == nullptr) return missing("conv1d", "stride");
  if (padding == nullptr) return missing("conv1d", "padding");
  if (groups == nullptr) return missing("conv1d", "groups");
  const Tensor& x = ctx.inputs[0];
  const Tensor& w = ctx.inputs[1];
  if (x.shape().rank() != 3 || w.shape().rank() != 3) {
    return Status::make(ErrorCode::kInvalidArgument, "op 'conv1d' cuda kernel requires rank-3 x and w");
  }
  const void* bias = ctx.inputs.size() == 3 ? ctx.inputs[2].raw_data() : nullptr;
  return frame_b200::to_status(
      fb200_conv1d(x.raw_data(), w.raw_data(), bias, ctx.outputs[0].raw_data(), x.shape().dim(0),
                   x.shape().dim(1), x.shape().dim(2), w.shape().dim(0), w.shape().dim(2), *stride,
                   *padding, *groups, dtype_of(ctx.outputs[0]), stream_of(ctx)),
      "conv1d");
}

Status max_pool2d(KernelContext& ctx) {
  FRAME_RETURN_IF_ERROR(arity(ctx, "max_pool2d", 1, 1));
  const auto* kernel = attr<std::vector<int64_t>>(ctx, "kernel");
  const auto* stride = attr<std::vector<int64_t>>(ctx, "stride");
  const auto* padding = attr<std::vector<int64_t>>(ctx, "padding");
  if (kernel == nullptr || kernel->size() != 2) return missing("max_pool2d", "kernel");
  if (stride == nullptr || stride->size() != 2) return missing("max_pool2d", "stride");
  if (padding == nullptr || padding->size() != 2) return missing("max_pool2d", "padding");
  const Tensor& x = ctx.inputs[0];
  if (x.shape().rank() != 4) {
    return Status::make(ErrorCode::kInvalidArgument, "op 'max_pool2d' cuda kernel requires rank-4 x");
  }
  return frame_b200::to_status(
      fb200_max_pool2d(x.raw_data(), ctx.outputs[0].raw_data(), x.shape().dim(0), x.shape().dim(1),
                       x.shape().dim(2), x.shape().dim(3), (*kernel)[0], (*kernel)[1], (*stride)[0],
                       (*stride)[1], (*padding)[0], (*padding)[1], dtype_of(x), stream_of(ctx)),
      "max_pool2d");
}

Status avg_pool2d(KernelContext& ctx) {
  FRAME_RETURN_IF_ERROR(arity(ctx, "avg_pool2d", 1, 1));
  const auto* kernel = attr<std::vector<int64_t>>(ctx, "kernel");
  const auto* stride = attr<std::vector<int64_t>>(ctx, "stride");
  const auto* padding = attr<std::vector<int64_t>>(ctx, "padding");
  if (kernel == nullptr || kernel->size() != 2) return missing("avg_pool2d", "kernel");
  if (stride == nullptr || stride->size() != 2) return missing("avg_pool2d", "stride");
  if (padding == nullptr || padding->size() != 2) return missing("avg_pool2d", "padding");
  const Tensor& x = ctx.inputs[0];
  if (x.shape().rank() != 4) {
    return Status::make(ErrorCode::kInvalidArgument, "op 'avg_pool2d' cuda kernel requires rank-4 x");
  }
  return frame_b200::to_status(
      fb200_avg_pool2d(x.raw_data(), ctx.outputs[0].raw_data(), x.shape().dim(0), x.shape().dim(1),
                       x.shape().dim(2), x.shape().dim(3), (*kernel)[0], (*kernel)[1], (*stride)[0],
                       (*stride)[1], (*padding)[0], (*padding)[1], dtype_of(x), stream_of(ctx)),
      "avg_pool2d");
}

// Gradient-side internals of pooling and convolution (gathers in the CPU reference's order).  The
// geometry comes from the tensors themselves: the forward op's input is operand 1 of the max-pool
// ops, the result of avg_pool2d_grad_internal / conv2d_grad_input_internal, operand 0 of
// conv2d_grad_filter_internal; the filter is operand 1 resp. the result.
struct PoolAttrs3 {
  const std::vector<int64_t>* kernel;
  const std::vector<int64_t>* stride;
  const std::vector<int64_t>* padding;
};
Status pool_attrs(KernelContext& ctx, const char* op, PoolAttrs3* a) {
  a->kernel = attr<std::vector<int64_t>>(ctx, "kernel");
  a->stride = attr<std::vector<int64_t>>(ctx, "stride");
  a->padding = attr<std::vector<int64_t>>(ctx, "padding");
  if (a->kernel == nullptr || a->kernel->size() != 2) return missing(op, "kernel");
  if (a->stride == nullptr || a->stride->size() != 2) return missing(op, "stride");
  if (a->padding == nullptr || a->padding->size() != 2) return missing(op, "padding");
  return Status::ok();
}

Status max_pool2d_select_or_grad(KernelContext& ctx, const char* op, bool select) {
  FRAME_RETURN_IF_ERROR(arity(ctx, op, 2, 2));
  PoolAttrs3 a{};
  FRAME_RETURN_IF_ERROR(pool_attrs(ctx, op, &a));
  const Tensor& x = ctx.inputs[1];
  if (x.shape().rank() != 4) {
    return Status::make(ErrorCode::kInvalidArgument, std::string("op '") + op + "' cuda kernel requires rank-4 x");
  }
  auto fn = select ? fb200_max_pool2d_select : fb200_max_pool2d_grad;
  return frame_b200::to_status(
      fn(ctx.inputs[0].raw_data(), x.raw_data(), ctx.outputs[0].raw_data(), x.shape().dim(0), x.shape().dim(1),
         x.shape().dim(2), x.shape().dim(3), (*a.kernel)[0], (*a.kernel)[1], (*a.stride)[0], (*a.stride)[1],
         (*a.padding)[0], (*a.padding)[1], dtype_of(x), stream_of(ctx)),
      op);
}
Status max_pool2d_select_internal(KernelContext& ctx) {
  return max_pool2d_select_or_grad(ctx, "max_pool2d_select_internal", true);
}
Status max_pool2d_grad_internal(KernelContext& ctx) {
  return max_pool2d_select_or_grad(ctx, "max_pool2d_grad_internal", false);
}

Status avg_pool2d_grad_internal(KernelContext& ctx) {
  FRAME_RETURN_IF_ERROR(arity(ctx, "avg_pool2d_grad_internal", 1, 1));
  PoolAttrs3 a{};
  FRAME_RETURN_IF_ERROR(pool_attrs(ctx, "avg_pool2d_grad_internal", &a));
  const Tensor& dx = ctx.outputs[0];
  if (dx.shape().rank() != 4) {
    return Status::make(ErrorCode::kInvalidArgument, "op 'avg_pool2d_grad_internal' cuda kernel requires a rank-4 result");
  }
  return frame_b200::to_status(
      fb200_avg_pool2d_grad(ctx.inputs[0].raw_data(), ctx.outputs[0].raw_data(), dx.shape().dim(0), dx.shape().dim(1),
                            dx.shape().dim(2), dx.shape().dim(3), (*a.kernel)[0], (*a.kernel)[1], (*a.stride)[0],
                            (*a.stride)[1], (*a.padding)[0], (*a.padding)[1], dtype_of(dx), stream_of(ctx)),
      "avg_pool2d_grad_internal");
}

Status conv2d_grad(KernelContext& ctx, const char* op, bool wrt_input) {
  FRAME_RETURN_IF_ERROR(arity(ctx, op, 2, 2));
  const auto* stride = attr<std::vector<int64_t>>(ctx, "stride");
  const auto* padding = attr<std::vector<int64_t>>(ctx, "padding");
  const auto* groups = attr<int64_t>(ctx, "groups");
  if (stride == nullptr || stride->size() != 2) return missing(op, "stride");
  if (padding == nullptr || padding->size() != 2) return missing(op, "padding");
  if (groups == nullptr) return missing(op, "groups");
  const Tensor& xt = wrt_input ? ctx.outputs[0] : ctx.inputs[0];
  const Tensor& wt = wrt_input ? ctx.inputs[1] : ctx.outputs[0];
  if (xt.shape().rank() != 4 || wt.shape().rank() != 4) {
    return Status::make(ErrorCode::kInvalidArgument, std::string("op '") + op + "' cuda kernel requires rank-4 tensors");
  }
  fb200_conv2d_params p{};
  p.n = xt.shape().dim(0); p.cin = xt.shape().dim(1); p.h = xt.shape().dim(2); p.w = xt.shape().dim(3);
  p.cout = wt.shape().dim(0); p.kh = wt.shape().dim(2); p.kw = wt.shape().dim(3);
  p.stride_h = (*stride)[0]; p.stride_w = (*stride)[1];
  p.pad_h = (*padding)[0]; p.pad_w = (*padding)[1];
  p.groups = *groups;
  if (wt.shape().dim(1) * p.groups != p.cin) {
    return Status::make(ErrorCode::kInvalidArgument, std::string("op '") + op + "' cuda kernel: w.dim(1)*groups != Cin");
  }
  const int rc = wrt_input ? fb200_conv2d_grad_input(ctx.inputs[0].raw_data(), ctx.inputs[1].raw_data(),
                                                     ctx.outputs[0].raw_data(), &p, dtype_of(ctx.outputs[0]), stream_of(ctx))
                           : fb200_conv2d_grad_filter(ctx.inputs[0].raw_data(), ctx.inputs[1].raw_data(),
                                                      ctx.outputs[0].raw_data(), &p, dtype_of(ctx.outputs[0]), stream_of(ctx));
  return frame_b200::to_status(rc, op);
}
Status conv2d_grad_input_internal(KernelContext& ctx) { return conv2d_grad(ctx, "conv2d_grad_input_internal", true); }
Status conv2d_grad_filter_internal(KernelContext& ctx) { return conv2d_grad(ctx, "conv2d_grad_filter_internal", false); }

// Gradients of matmul and the MSE loss pair: ops the reference's own CUDA table lacks (a graph built by
// build_backward_graph would otherwise take the fallback chain).
Status matmul_grad_lhs_internal(KernelContext& ctx) {
  FRAME_RETURN_IF_ERROR(arity(ctx, "matmul_grad_lhs_internal", 2, 2));
  const Tensor& gy = ctx.inputs[0];
  const Tensor& b = ctx.inputs[1];
  if (gy.shape().rank() != 2 || b.shape().rank() != 2 || gy.shape().dim(1) != b.shape().dim(1)) {
    return Status::make(ErrorCode::kInvalidArgument,
                        "op 'matmul_grad_lhs_internal' cuda kernel requires gy [m, n] and b [k, n], got " +
                            gy.shape().to_string() + " and " + b.shape().to_string());
  }
  return frame_b200::to_status(
      fb200_matmul_grad_lhs(gy.raw_data(), b.raw_data(), ctx.outputs[0].raw_data(), gy.shape().dim(0),
                            gy.shape().dim(1), b.shape().dim(0), dtype_of(gy), allow_tf32(ctx), stream_of(ctx)),
      "matmul_grad_lhs_internal");
}

Status matmul_grad_rhs_internal(KernelContext& ctx) {
  FRAME_RETURN_IF_ERROR(arity(ctx, "matmul_grad_rhs_internal", 2, 2));
  const Tensor& a = ctx.inputs[0];
  const Tensor& gy = ctx.inputs[1];
  if (a.shape().rank() != 2 || gy.shape().rank() != 2 || a.shape().dim(0) != gy.shape().dim(0)) {
    return Status::make(ErrorCode::kInvalidArgument,
                        "op 'matmul_grad_rhs_internal' cuda kernel requires a [m, k] and gy [m, n], got " +
                            a.shape().to_string() + " and " + gy.shape().to_string());
  }
  return frame_b200::to_status(
      fb200_matmul_grad_rhs(a.raw_data(), gy.raw_data(), ctx.outputs[0].raw_data(), a.shape().dim(0),
                            gy.shape().dim(1), a.shape().dim(1), dtype_of(a), allow_tf32(ctx), stream_of(ctx)),
      "matmul_grad_rhs_internal");
}

Status mse_loss(KernelContext& ctx) {
  FRAME_RETURN_IF_ERROR(arity(ctx, "mse_loss", 2, 2));
  const Tensor& pred = ctx.inputs[0];
  if (!(pred.shape() == ctx.inputs[1].shape())) {
    return Status::make(ErrorCode::kInvalidArgument,
                        "op 'mse_loss' cuda kernel requires pred and target of the same shape, got " +
                            pred.shape().to_string() + ", " + ctx.inputs[1].shape().to_string());
  }
  return frame_b200::to_status(
      fb200_mse_loss(pred.raw_data(), ctx.inputs[1].raw_data(), ctx.outputs[0].raw_data(), pred.numel(),
                     dtype_of(pred), stream_of(ctx)),
      "mse_loss");
}

Status mse_loss_grad_internal(KernelContext& ctx) {
  FRAME_RETURN_IF_ERROR(arity(ctx, "mse_loss_grad_internal", 3, 3));
  const Tensor& pred = ctx.inputs[0];
  if (!(pred.shape() == ctx.inputs[1].shape()) || ctx.inputs[2].numel() != 1) {
    return Status::make(ErrorCode::kInvalidArgument,
                        "op 'mse_loss_grad_internal' cuda kernel requires pred and target of the same shape "
                        "and a scalar gy");
  }
  return frame_b200::to_status(
      fb200_mse_loss_grad(pred.raw_data(), ctx.inputs[1].raw_data(), ctx.inputs[2].raw_data(),
                          ctx.outputs[0].raw_data(), pred.numel(), dtype_of(pred), stream_of(ctx)),
      "mse_loss_grad_internal");
}

// rfft / irfft along the last axis, float32 only as in the reference (src/ops/schemas/fft.cpp).
Status rfft(KernelContext& ctx) {
  FRAME_RETURN_IF_ERROR(arity(ctx, "rfft", 1, 1));
  const Tensor& x = ctx.inputs[0];
  const size_t rank = x.shape().rank();
  if (rank < 1 || x.shape().dim(rank - 1) < 2) {
    return Status::make(ErrorCode::kInvalidArgument, "op 'rfft' cuda kernel requires rank >= 1 and n >= 2");
  }
  const int64_t n = x.shape().dim(rank - 1);
  const int64_t rows = n > 0 ? x.numel() / n : 0;
  return frame_b200::to_status(
      fb200_rfft(x.raw_data(), ctx.outputs[0].raw_data(), rows, n, dtype_of(x), stream_of(ctx)), "rfft");
}

Status irfft(KernelContext& ctx) {
  FRAME_RETURN_IF_ERROR(arity(ctx, "irfft", 1, 1));
  const auto* n = attr<int64_t>(ctx, "n");
  if (n == nullptr) return missing("irfft", "n");
  const Tensor& z = ctx.inputs[0];
  const size_t rank = z.shape().rank();
  if (rank < 2 || z.shape().dim(rank - 1) != 2 || z.shape().dim(rank - 2) != *n / 2 + 1) {
    return Status::make(ErrorCode::kInvalidArgument,
                        "op 'irfft' cuda kernel requires z [..., n/2+1, 2] for attribute n=" + std::to_string(*n));
  }
  const int64_t per_row = z.shape().dim(rank - 2) * 2;
  const int64_t rows = z.numel() / per_row;
  return frame_b200::to_status(
      fb200_irfft(z.raw_data(), ctx.outputs[0].raw_data(), rows, *n, dtype_of(z), stream_of(ctx)), "irfft");
}

// heaviside_surrogate: alpha only shapes the backward graph, but a bad alpha is an error here too
// (src/backends/cpu/kernels/elementwise.cpp, read_heaviside_alpha).
Status heaviside_surrogate(KernelContext& ctx) {
  const double* alpha = attr<double>(ctx, "alpha");
  if (alpha == nullptr) return missing("heaviside_surrogate", "alpha");
  if (!std::isfinite(*alpha) || !(*alpha > 0.0)) {
    return Status::make(ErrorCode::kInvalidArgument,
                        "op 'heaviside_surrogate' cuda kernel attribute 'alpha' must be finite and positive, got " +
                            std::to_string(*alpha));
  }
  return elementwise<FB200_EW_HEAVISIDE, 1>(ctx, "heaviside_surrogate");
}

// gather along axis 0 and scatter_add / gather_grad_internal (src/ops/schemas/gather.cpp:86-216).
Status gather(KernelContext& ctx) {
  FRAME_RETURN_IF_ERROR(arity(ctx, "gather", 2, 1));
  const Tensor& x = ctx.inputs[0];
  const Tensor& idx = ctx.inputs[1];
  if (x.shape().rank() != 2 || idx.shape().rank() != 1) {
    return Status::make(ErrorCode::kInvalidArgument, "op 'gather' cuda kernel requires x [N, F] and indices [K]");
  }
  return frame_b200::to_status(
      fb200_gather(x.raw_data(), idx.raw_data(), ctx.outputs[0].raw_data(), x.shape().dim(0), x.shape().dim(1),
                   idx.shape().dim(0), dtype_of(x), dtype_of(idx), stream_of(ctx)),
      "gather");
}

Status scatter_add_like(KernelContext& ctx, const char* op) {
  FRAME_RETURN_IF_ERROR(arity(ctx, op, 2, 1));
  const Tensor& u = ctx.inputs[0];
  const Tensor& idx = ctx.inputs[1];
  const Tensor& out = ctx.outputs[0];
  if (u.shape().rank() != 2 || idx.shape().rank() != 1 || out.shape().rank() != 2 ||
      idx.shape().dim(0) != u.shape().dim(0) || out.shape().dim(1) != u.shape().dim(1)) {
    return Status::make(ErrorCode::kInvalidArgument,
                        std::string("op '") + op + "' cuda kernel requires updates [K, F], indices [K], out [V, F]");
  }
  return frame_b200::to_status(
      fb200_scatter_add(u.raw_data(), idx.raw_data(), ctx.outputs[0].raw_data(), u.shape().dim(0), u.shape().dim(1),
                        out.shape().dim(0), dtype_of(u), dtype_of(idx), stream_of(ctx)),
      op);
}
Status scatter_add(KernelContext& ctx) { return scatter_add_like(ctx, "scatter_add"); }
Status gather_grad_internal(KernelContext& ctx) { return scatter_add_like(ctx, "gather_grad_internal"); }

// ---- row kernels -----------------------------------------------------------------------------------
Status softmax(KernelContext& ctx) {
  FRAME_RETURN_IF_ERROR(arity(ctx, "softmax", 1, 1));
  const Tensor& x = ctx.inputs[0];
  if (x.shape().rank() != 2 || !(x.shape() == ctx.outputs[0].shape())) {
    return Status::make(ErrorCode::kInvalidArgument,
                        "op 'softmax' cuda kernel requires x to be rank-2 [N, D] and out to match");
  }
  return frame_b200::to_status(fb200_softmax(x.raw_data(), ctx.outputs[0].raw_data(), x.shape().dim(0),
                                             x.shape().dim(1), dtype_of(x), stream_of(ctx)),
                               "softmax");
}

Status layer_norm(KernelContext& ctx) {
  FRAME_RETURN_IF_ERROR(arity(ctx, "layer_norm", 3, 3));
  const double* eps = attr<double>(ctx, "eps");
  if (eps == nullptr) return missing("layer_norm", "eps");
  const Tensor& x = ctx.inputs[0];
  if (x.shape().rank() != 2 || ctx.inputs[1].shape().rank() != 1 || ctx.inputs[2].shape().rank() != 1 ||
      ctx.inputs[1].shape().dim(0) != x.shape().dim(1) || ctx.inputs[2].shape().dim(0) != x.shape().dim(1) ||
      !(x.shape() == ctx.outputs[0].shape())) {
    return Status::make(ErrorCode::kInvalidArgument,
                        "op 'layer_norm' cuda kernel requires x [N, D], gamma [D], beta [D], out [N, D]");
  }
  return frame_b200::to_status(
      fb200_layer_norm(x.raw_data(), ctx.inputs[1].raw_data(), ctx.inputs[2].raw_data(),
                       ctx.outputs[0].raw_data(), x.shape().dim(0), x.shape().dim(1), *eps, dtype_of(x),
                       stream_of(ctx)),
      "layer_norm");
}

Status selective_scan(KernelContext& ctx) {
  FRAME_RETURN_IF_ERROR(arity(ctx, "selective_scan", 5, 5));
  const Tensor& x = ctx.inputs[0];
  if (x.shape().rank() < 1) {
    return Status::make(ErrorCode::kInvalidArgument, "op 'selective_scan' cuda kernel requires rank >= 1, got rank 0");
  }
  for (const Tensor& t : ctx.inputs) {
    if (!(t.shape() == x.shape())) {
      return Status::make(ErrorCode::kInvalidArgument,
                          "op 'selective_scan' cuda kernel requires all input shapes to match x " +
                              x.shape().to_string() + ", got " + t.shape().to_string());
    }
  }
  const int64_t steps = x.shape().dim(x.shape().rank() - 1);
  if (steps < 1) {
    return Status::make(ErrorCode::kInvalidArgument,
                        "op 'selective_scan' cuda kernel requires the last dimension (steps) to be >= 1, got " +
                            std::to_string(steps));
  }
  return frame_b200::to_status(
      fb200_selective_scan(x.raw_data(), ctx.inputs[1].raw_data(), ctx.inputs[2].raw_data(),
                           ctx.inputs[3].raw_data(), ctx.inputs[4].raw_data(), ctx.outputs[0].raw_data(),
                           x.numel() / steps, steps, dtype_of(x), stream_of(ctx)),
      "selective_scan");
}

// ---- data movement -----------------------------------------------------------------------------------
Status reshape(KernelContext& ctx) {
  if (ctx.inputs.size() != 1 || ctx.outputs.size() != 1 || ctx.inputs[0].numel() != ctx.outputs[0].numel()) {
    return Status::make(ErrorCode::kInvalidArgument, "op 'reshape' cuda kernel expects 1 input and 1 output of equal numel");
  }
  const size_t bytes = static_cast<size_t>(ctx.inputs[0].numel()) * ctx.inputs[0].dtype().itemsize();
  return frame_b200::to_status(fb200_memcpy(ctx.device.index, ctx.outputs[0].raw_data(), ctx.inputs[0].raw_data(),
                                            bytes, FB200_D2D, stream_of(ctx), 0),
                               "reshape");
}

Status transpose(KernelContext& ctx) {
  if (ctx.inputs.size() != 1 || ctx.outputs.size() != 1) {
    return Status::make(ErrorCode::kInvalidArgument, "op 'transpose' cuda kernel expects 1 input and 1 output");
  }
  const auto* perm = attr<std::vector<int64_t>>(ctx, "perm");
  if (perm == nullptr) return missing("transpose", "perm");
  const Tensor& x = ctx.inputs[0];
  if (static_cast<int64_t>(perm->size()) != x.shape().rank()) {
    return Status::make(ErrorCode::kInvalidArgument, "op 'transpose' cuda kernel: perm length differs from rank");
  }
  return frame_b200::to_status(
      fb200_transpose(x.raw_data(), ctx.outputs[0].raw_data(), static_cast<int>(x.shape().rank()),
                      x.shape().dims().data(), perm->data(), static_cast<int>(x.dtype().itemsize()),
                      stream_of(ctx)),
      "transpose");
}

Status slice(KernelContext& ctx) {
  if (ctx.inputs.size() != 1 || ctx.outputs.size() != 1) {
    return Status::make(ErrorCode::kInvalidArgument, "op 'slice' cuda kernel expects 1 input and 1 output");
  }
  const auto* axis = attr<int64_t>(ctx, "axis");
  const auto* start = attr<int64_t>(ctx, "start");
  const auto* stop = attr<int64_t>(ctx, "stop");
  if (axis == nullptr) return missing("slice", "axis");
  if (start == nullptr) return missing("slice", "start");
  if (stop == nullptr) return missing("slice", "stop");
  const Tensor& x = ctx.inputs[0];
  return frame_b200::to_status(
      fb200_slice(x.raw_data(), ctx.outputs[0].raw_data(), static_cast<int>(x.shape().rank()),
                  x.shape().dims().data(), *axis, *start, *stop, static_cast<int>(x.dtype().itemsize()),
                  stream_of(ctx)),
      "slice");
}

Status concat(KernelContext& ctx) {
  if (ctx.inputs.empty() || ctx.outputs.size() != 1) {
    return Status::make(ErrorCode::kInvalidArgument, "op 'concat' cuda kernel expects >= 1 input and 1 output");
  }
  const auto* axis = attr<int64_t>(ctx, "axis");
  if (axis == nullptr) return missing("concat", "axis");
  Tensor& out = ctx.outputs[0];
  if (*axis < 0 || *axis >= out.shape().rank()) {
    return Status::make(ErrorCode::kInvalidArgument, "op 'concat' cuda kernel: axis out of range");
  }
  std::vector<const void*> in(ctx.inputs.size());
  std::vector<int64_t> sizes(ctx.inputs.size());
  for (size_t i = 0; i < ctx.inputs.size(); ++i) {
    if (ctx.inputs[i].shape().rank() != out.shape().rank()) {
      return Status::make(ErrorCode::kInvalidArgument, "op 'concat' cuda kernel: rank mismatch");
    }
    in[i] = ctx.inputs[i].raw_data();
    sizes[i] = ctx.inputs[i].shape().dim(*axis);
  }
  return frame_b200::to_status(
      fb200_concat(in.data(), static_cast<int>(in.size()), sizes.data(), out.raw_data(),
                   static_cast<int>(out.shape().rank()), out.shape().dims().data(), *axis,
                   static_cast<int>(out.dtype().itemsize()), stream_of(ctx)),
      "concat");
}

Status sum(KernelContext& ctx) {
  if (ctx.inputs.size() != 1 || ctx.outputs.size() != 1) {
    return Status::make(ErrorCode::kInvalidArgument, "op 'sum' cuda kernel expects 1 input and 1 output");
  }
  const auto* axes = attr<std::vector<int64_t>>(ctx, "axes");
  if (axes == nullptr) return missing("sum", "axes");
  const Tensor& x = ctx.inputs[0];
  return frame_b200::to_status(
      fb200_sum_axes(x.raw_data(), ctx.outputs[0].raw_data(), static_cast<int>(x.shape().rank()),
                     x.shape().dims().data(), axes->data(), static_cast<int>(axes->size()), dtype_of(x),
                     stream_of(ctx)),
      "sum");
}

// constant: decoded on the host and uploaded.  Inside a compiled executable constants are
// materialised once at compile time by the plan; this eager form exists for Backend::launch.
Status constant(KernelContext& ctx) {
  if (!ctx.inputs.empty() || ctx.outputs.size() != 1) {
    return Status::make(ErrorCode::kInvalidArgument, "op 'constant' cuda kernel expects 0 inputs and 1 output");
  }
  const auto* value = attr<std::vector<double>>(ctx, "value");
  if (value == nullptr) return missing("constant", "value");
  Tensor& out = ctx.outputs[0];
  const int64_t n = out.numel();
  if (n == 0) return Status::ok();
  if (static_cast<int64_t>(value->size()) != n && value->size() != 1) {
    return Status::make(ErrorCode::kInvalidArgument, "op 'constant' cuda kernel: value length differs from numel");
  }
  std::vector<unsigned char> host(static_cast<size_t>(n) * out.dtype().itemsize());
  for (int64_t i = 0; i < n; ++i) {
    const double d = (*value)[value->size() == 1 ? 0 : static_cast<size_t>(i)];
    switch (out.dtype().code()) {
      case frame::DTypeCode::kFloat32: reinterpret_cast<float*>(host.data())[i] = static_cast<float>(d); break;
      case frame::DTypeCode::kFloat64: reinterpret_cast<double*>(host.data())[i] = d; break;
      case frame::DTypeCode::kBFloat16:
        reinterpret_cast<frame::bfloat16_t*>(host.data())[i] = frame::float_to_bfloat16(static_cast<float>(d));
        break;
      case frame::DTypeCode::kFloat16:
        reinterpret_cast<frame::float16_t*>(host.data())[i] = frame::float_to_float16(static_cast<float>(d));
        break;
      case frame::DTypeCode::kInt32: reinterpret_cast<int32_t*>(host.data())[i] = static_cast<int32_t>(d); break;
      case frame::DTypeCode::kInt64: reinterpret_cast<int64_t*>(host.data())[i] = static_cast<int64_t>(d); break;
      default:
        return Status::make(ErrorCode::kUnimplemented, "op 'constant' cuda kernel: unsupported dtype");
    }
  }
  const fb200_stream s = stream_of(ctx);
  // The staging vector dies at return: make the upload synchronous with respect to the host.
  return frame_b200::to_status(
      fb200_memcpy(ctx.device.index, out.raw_data(), host.data(), host.size(), FB200_H2D, s, 1), "constant");
}

}  // namespace

#define B200_ELEMENTWISE(name, code, ar)                                                  \
  static Status b200_ew_##code(KernelContext& c) { return elementwise<code, ar>(c, name); } \
  FRAME_REGISTER_KERNEL(name, "cuda", &b200_ew_##code)

B200_ELEMENTWISE("add", FB200_EW_ADD, 2);
B200_ELEMENTWISE("mul", FB200_EW_MUL, 2);
B200_ELEMENTWISE("relu_grad_internal", FB200_EW_RELU_GRAD, 2);
B200_ELEMENTWISE("relu", FB200_EW_RELU, 1);
B200_ELEMENTWISE("square", FB200_EW_SQUARE, 1);
B200_ELEMENTWISE("sigmoid", FB200_EW_SIGMOID, 1);
B200_ELEMENTWISE("tanh", FB200_EW_TANH, 1);
B200_ELEMENTWISE("rsqrt", FB200_EW_RSQRT, 1);
B200_ELEMENTWISE("gelu", FB200_EW_GELU, 1);
B200_ELEMENTWISE("silu", FB200_EW_SILU, 1);
B200_ELEMENTWISE("softplus", FB200_EW_SOFTPLUS, 1);
B200_ELEMENTWISE("exp", FB200_EW_EXP, 1);
FRAME_REGISTER_KERNEL(frame::ops::kFusedElementwiseOpName, "cuda", &fused_elementwise);
FRAME_REGISTER_KERNEL("matmul", "cuda", &matmul);
FRAME_REGISTER_KERNEL("conv2d", "cuda", &conv2d);
FRAME_REGISTER_KERNEL("conv1d", "cuda", &conv1d);
FRAME_REGISTER_KERNEL("max_pool2d", "cuda", &max_pool2d);
FRAME_REGISTER_KERNEL("avg_pool2d", "cuda", &avg_pool2d);
FRAME_REGISTER_KERNEL("matmul_grad_lhs_internal", "cuda", &matmul_grad_lhs_internal);
FRAME_REGISTER_KERNEL("matmul_grad_rhs_internal", "cuda", &matmul_grad_rhs_internal);
FRAME_REGISTER_KERNEL("mse_loss", "cuda", &mse_loss);
FRAME_REGISTER_KERNEL("mse_loss_grad_internal", "cuda", &mse_loss_grad_internal);
FRAME_REGISTER_KERNEL("rfft", "cuda", &rfft);
FRAME_REGISTER_KERNEL("irfft", "cuda", &irfft);
FRAME_REGISTER_KERNEL("max_pool2d_select_internal", "cuda", &max_pool2d_select_internal);
FRAME_REGISTER_KERNEL("max_pool2d_grad_internal", "cuda", &max_pool2d_grad_internal);
FRAME_REGISTER_KERNEL("avg_pool2d_grad_internal", "cuda", &avg_pool2d_grad_internal);
FRAME_REGISTER_KERNEL("conv2d_grad_input_internal", "cuda", &conv2d_grad_input_internal);
FRAME_REGISTER_KERNEL("conv2d_grad_filter_internal", "cuda", &conv2d_grad_filter_internal);
FRAME_REGISTER_KERNEL("heaviside_surrogate", "cuda", &heaviside_surrogate);
FRAME_REGISTER_KERNEL("gather", "cuda", &gather);
FRAME_REGISTER_KERNEL("scatter_add", "cuda", &scatter_add);
FRAME_REGISTER_KERNEL("gather_grad_internal", "cuda", &gather_grad_internal);
FRAME_REGISTER_KERNEL("softmax", "cuda", &softmax);
FRAME_REGISTER_KERNEL("layer_norm", "cuda", &layer_norm);
FRAME_REGISTER_KERNEL("selective_scan", "cuda", &selective_scan);
FRAME_REGISTER_KERNEL("reshape", "cuda", &reshape);
FRAME_REGISTER_KERNEL("transpose", "cuda", &transpose);
FRAME_REGISTER_KERNEL("slice", "cuda", &slice);
FRAME_REGISTER_KERNEL("concat", "cuda", &concat);
FRAME_REGISTER_KERNEL("sum", "cuda", &sum);
FRAME_REGISTER_KERNEL("constant", "cuda", &constant);
