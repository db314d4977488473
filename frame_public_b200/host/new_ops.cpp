// Ops the compiled-graph configs need that the reference does not have, added through the
// reference's own public extension API: schema with FRAME_REGISTER_OP, a CPU reference kernel and
// a "cuda" kernel with FRAME_REGISTER_KERNEL (the custom-op recipe of
// examples/03_custom_op/main.cpp:20-143 and docs/architecture/operator-system.md:62,88 of the
// reference).  gelu / silu / softplus / exp are attribute-free, kElementwise | kFusable, so the
// reference's own operator_fusion pass groups them (src/compiler/passes/operator_fusion.cpp:50-58);
// a CPU kernel is mandatory because that pass and constant_folding look it up
// (operator_fusion.cpp:159-168, constant_folding.cpp:85-89).
//
// None of these has a counterpart in the reference: their CPU kernels below are written in the
// style of src/backends/cpu/kernels/elementwise.cpp:265-321 (fp32 math through libm, one
// round-to-nearest-even store) and are the semantic definition the sm_100a kernels follow.
#include <cmath>
#include <string>
#include <vector>

#include <frame/core/dtype.h>
#include <frame/core/tensor.h>
#include <frame/hal/stream.h>
#include <frame/ops/kernel_registry.h>
#include <frame/ops/op_registry.h>

#include "b200_status.h"
#include "frame_b200.h"

namespace {

using frame::ErrorCode;
using frame::Result;
using frame::Shape;
using frame::Status;
using frame::Tensor;
using frame::ops::KernelContext;
using frame::ops::NodeContext;

// ---- schemas -------------------------------------------------------------------------------------
Result<std::vector<Shape>> infer_unary(const NodeContext& ctx) {
  if (ctx.input_types.size() != 1) {
    return Status::make(ErrorCode::kInvalidArgument, "op '" + std::string(ctx.op) +
                                                         "' expects 1 input, got " +
                                                         std::to_string(ctx.input_types.size()));
  }
  return std::vector<Shape>{ctx.input_types[0].shape};
}

Result<std::vector<Shape>> infer_bias_add(const NodeContext& ctx) {
  if (ctx.input_types.size() != 2) {
    return Status::make(ErrorCode::kInvalidArgument, "op 'bias_add' expects 2 inputs (x, bias)");
  }
  const Shape& x = ctx.input_types[0].shape;
  const Shape& b = ctx.input_types[1].shape;
  if (x.rank() < 1 || b.rank() != 1 || b.dim(0) != x.dim(x.rank() - 1)) {
    return Status::make(ErrorCode::kInvalidArgument,
                        "op 'bias_add' requires bias of shape [x.last_dim], got x " + x.to_string() +
                            " and bias " + b.to_string());
  }
  return std::vector<Shape>{x};
}

Result<std::vector<Shape>> infer_mamba_scan(const NodeContext& ctx) {
  if (ctx.input_types.size() != 7) {
    return Status::make(ErrorCode::kInvalidArgument,
                        "op 'mamba_scan' expects 7 inputs (u, delta, A, B, C, D, z)");
  }
  const Shape& u = ctx.input_types[0].shape;
  const Shape& a = ctx.input_types[2].shape;
  const Shape& b = ctx.input_types[3].shape;
  if (u.rank() != 3 || a.rank() != 2 || b.rank() != 3 || !(ctx.input_types[1].shape == u) ||
      !(ctx.input_types[6].shape == u) || a.dim(0) != u.dim(2) || b.dim(0) != u.dim(0) ||
      b.dim(1) != u.dim(1) || b.dim(2) != a.dim(1) || !(ctx.input_types[4].shape == b) ||
      ctx.input_types[5].shape.rank() != 1 || ctx.input_types[5].shape.dim(0) != u.dim(2)) {
    return Status::make(ErrorCode::kInvalidArgument,
                        "op 'mamba_scan' requires u/delta/z [B,L,D], A [D,N], B/C [B,L,N], D [D]");
  }
  return std::vector<Shape>{u};
}

// ---- CPU reference kernels -------------------------------------------------------------------------
template <typename T> float to_accum(T v) {
  if constexpr (std::is_same_v<T, float>) return v;
  else if constexpr (std::is_same_v<T, frame::float16_t>) return frame::float16_to_float(v);
  else return frame::bfloat16_to_float(v);
}
template <typename T> T from_accum(float v) {
  if constexpr (std::is_same_v<T, float>) return v;
  else if constexpr (std::is_same_v<T, frame::float16_t>) return frame::float_to_float16(v);
  else return frame::float_to_bfloat16(v);
}

float sigmoid_ref(float x) {  // the reference's two-branch form, cpu/kernels/elementwise.cpp:346-354
  if (x >= 0.0F) return 1.0F / (1.0F + std::exp(-x));
  const float e = std::exp(x);
  return e / (1.0F + e);
}
float gelu_ref(float x) {
  const float inner = 0.7978845608028654F * (x + 0.044715F * (x * x * x));
  return 0.5F * x * (1.0F + std::tanh(inner));
}
float silu_ref(float x) { return x * sigmoid_ref(x); }
float softplus_ref(float x) { return x > 20.0F ? x : std::log1p(std::exp(x)); }
float exp_ref(float x) { return std::exp(x); }

Status check_float_same(const char* op, const Tensor& a, const Tensor& b) {
  const frame::DTypeCode c = a.dtype().code();
  if (!(a.dtype() == b.dtype()) || (c != frame::DTypeCode::kFloat32 && c != frame::DTypeCode::kFloat16 &&
                                    c != frame::DTypeCode::kBFloat16)) {
    return Status::make(ErrorCode::kInvalidArgument,
                        std::string("op '") + op + "' cpu kernel supports float32/float16/bfloat16 with one dtype");
  }
  return Status::ok();
}

template <float (*FN)(float)>
Status unary_cpu(KernelContext& ctx, const char* op) {
  if (ctx.inputs.size() != 1 || ctx.outputs.size() != 1) {
    return Status::make(ErrorCode::kInvalidArgument, std::string("op '") + op + "' cpu kernel expects 1 input and 1 output");
  }
  const Tensor& x = ctx.inputs[0];
  Tensor& y = ctx.outputs[0];
  FRAME_RETURN_IF_ERROR(check_float_same(op, x, y));
  if (!(x.shape() == y.shape())) {
    return Status::make(ErrorCode::kInvalidArgument, std::string("op '") + op + "' cpu kernel requires x/y of the same shape");
  }
  const int64_t n = x.numel();
  return frame::dispatch_dtype(x.dtype().code(), [&]<typename T>() -> Status {
    if constexpr (std::is_same_v<T, float> || std::is_same_v<T, frame::float16_t> ||
                  std::is_same_v<T, frame::bfloat16_t>) {
      const T* in = static_cast<const T*>(x.raw_data());
      T* out = static_cast<T*>(y.raw_data());
      for (int64_t i = 0; i < n; ++i) out[i] = from_accum<T>(FN(to_accum<T>(in[i])));
    }
    return Status::ok();
  });
}

Status bias_add_cpu(KernelContext& ctx) {
  if (ctx.inputs.size() != 2 || ctx.outputs.size() != 1) {
    return Status::make(ErrorCode::kInvalidArgument, "op 'bias_add' cpu kernel expects 2 inputs and 1 output");
  }
  const Tensor& x = ctx.inputs[0];
  const Tensor& b = ctx.inputs[1];
  Tensor& y = ctx.outputs[0];
  FRAME_RETURN_IF_ERROR(check_float_same("bias_add", x, y));
  FRAME_RETURN_IF_ERROR(check_float_same("bias_add", x, b));
  const int64_t cols = b.numel();
  const int64_t n = x.numel();
  if (cols == 0 || n % cols != 0 || !(x.shape() == y.shape())) {
    return Status::make(ErrorCode::kInvalidArgument, "op 'bias_add' cpu kernel shape mismatch");
  }
  return frame::dispatch_dtype(x.dtype().code(), [&]<typename T>() -> Status {
    if constexpr (std::is_same_v<T, float> || std::is_same_v<T, frame::float16_t> ||
                  std::is_same_v<T, frame::bfloat16_t>) {
      const T* in = static_cast<const T*>(x.raw_data());
      const T* bias = static_cast<const T*>(b.raw_data());
      T* out = static_cast<T*>(y.raw_data());
      for (int64_t i = 0; i < n; ++i) out[i] = from_accum<T>(to_accum<T>(in[i]) + to_accum<T>(bias[i % cols]));
    }
    return Status::ok();
  });
}

// h[n] = exp(delta*A[d,n])*h[n] + (delta*B[n])*u ; y = sum_n C[n]*h[n] (n increasing) + D[d]*u ;
// y *= silu(z).  fp32 only.
Status mamba_scan_cpu(KernelContext& ctx) {
  if (ctx.inputs.size() != 7 || ctx.outputs.size() != 1) {
    return Status::make(ErrorCode::kInvalidArgument, "op 'mamba_scan' cpu kernel expects 7 inputs and 1 output");
  }
  for (const Tensor& t : ctx.inputs) {
    if (t.dtype().code() != frame::DTypeCode::kFloat32) {
      return Status::make(ErrorCode::kInvalidArgument, "op 'mamba_scan' cpu kernel supports float32 only");
    }
  }
  const Tensor& u = ctx.inputs[0];
  const int64_t bt = u.shape().dim(0), len = u.shape().dim(1), dm = u.shape().dim(2);
  const int64_t ns = ctx.inputs[2].shape().dim(1);
  const float* up = static_cast<const float*>(u.raw_data());
  const float* dp = static_cast<const float*>(ctx.inputs[1].raw_data());
  const float* Ap = static_cast<const float*>(ctx.inputs[2].raw_data());
  const float* Bp = static_cast<const float*>(ctx.inputs[3].raw_data());
  const float* Cp = static_cast<const float*>(ctx.inputs[4].raw_data());
  const float* Dp = static_cast<const float*>(ctx.inputs[5].raw_data());
  const float* zp = static_cast<const float*>(ctx.inputs[6].raw_data());
  float* yp = static_cast<float*>(ctx.outputs[0].raw_data());
  std::vector<float> h(static_cast<size_t>(ns));
  for (int64_t b = 0; b < bt; ++b) {
    for (int64_t d = 0; d < dm; ++d) {
      for (auto& v : h) v = 0.0F;
      for (int64_t t = 0; t < len; ++t) {
        const int64_t idx = (b * len + t) * dm + d;
        const float uv = up[idx];
        const float dt = dp[idx];
        float acc = 0.0F;
        for (int64_t n = 0; n < ns; ++n) {
          const float da = std::exp(dt * Ap[d * ns + n]);
          const float db = dt * Bp[(b * len + t) * ns + n];
          h[static_cast<size_t>(n)] = da * h[static_cast<size_t>(n)] + db * uv;
          acc = acc + Cp[(b * len + t) * ns + n] * h[static_cast<size_t>(n)];
        }
        float out = acc + Dp[d] * uv;
        const float zv = zp[idx];
        out = out * (zv * sigmoid_ref(zv));
        yp[idx] = out;
      }
    }
  }
  return Status::ok();
}

// ---- "cuda" kernels for the two non-elementwise new ops (the unary ones are registered with the
// other elementwise kernels) ----------------------------------------------------------------------------
fb200_stream stream_of(const KernelContext& ctx) {
  return ctx.stream != nullptr ? ctx.stream->native_handle() : nullptr;
}

Status bias_add_cuda(KernelContext& ctx) {
  if (ctx.inputs.size() != 2 || ctx.outputs.size() != 1) {
    return Status::make(ErrorCode::kInvalidArgument, "op 'bias_add' cuda kernel expects 2 inputs and 1 output");
  }
  const Tensor& x = ctx.inputs[0];
  const int64_t cols = ctx.inputs[1].numel();
  if (cols == 0 || x.numel() % cols != 0) {
    return Status::make(ErrorCode::kInvalidArgument, "op 'bias_add' cuda kernel shape mismatch");
  }
  return frame_b200::to_status(
      fb200_bias_add(x.raw_data(), ctx.inputs[1].raw_data(), ctx.outputs[0].raw_data(), x.numel() / cols,
                     cols, static_cast<int>(x.dtype().code()), stream_of(ctx)),
      "bias_add");
}

Status mamba_scan_cuda(KernelContext& ctx) {
  if (ctx.inputs.size() != 7 || ctx.outputs.size() != 1) {
    return Status::make(ErrorCode::kInvalidArgument, "op 'mamba_scan' cuda kernel expects 7 inputs and 1 output");
  }
  for (const Tensor& t : ctx.inputs) {
    if (t.dtype().code() != frame::DTypeCode::kFloat32) {
      return Status::make(ErrorCode::kInvalidArgument, "op 'mamba_scan' cuda kernel supports float32 only");
    }
  }
  const Tensor& u = ctx.inputs[0];
  return frame_b200::to_status(
      fb200_mamba_scan(u.raw_data(), ctx.inputs[1].raw_data(), ctx.inputs[2].raw_data(),
                       ctx.inputs[3].raw_data(), ctx.inputs[4].raw_data(), ctx.inputs[5].raw_data(),
                       ctx.inputs[6].raw_data(), ctx.outputs[0].raw_data(), u.shape().dim(0),
                       u.shape().dim(1), u.shape().dim(2), ctx.inputs[2].shape().dim(1), stream_of(ctx)),
      "mamba_scan");
}

}  // namespace

#define B200_NEW_UNARY_OP(name, doc)                          \
  FRAME_REGISTER_OP(name)                                     \
      .input("x", "input tensor")                             \
      .output("y", doc)                                       \
      .trait(frame::ops::OpTrait::kElementwise)               \
      .trait(frame::ops::OpTrait::kFusable)                   \
      .shape_infer(&infer_unary)

B200_NEW_UNARY_OP("gelu", "tanh-form GELU: 0.5*x*(1+tanh(sqrt(2/pi)*(x+0.044715*x^3)))");
B200_NEW_UNARY_OP("silu", "x*sigmoid(x)");
B200_NEW_UNARY_OP("softplus", "log1p(exp(x)), identity above 20");
B200_NEW_UNARY_OP("exp", "exp(x)");

FRAME_REGISTER_OP("bias_add")
    .input("x", "tensor [..., D]")
    .input("bias", "vector [D]")
    .output("y", "x + bias broadcast over the leading axes")
    .shape_infer(&infer_bias_add);

FRAME_REGISTER_OP("mamba_scan")
    .input("u", "[B,L,D]")
    .input("delta", "[B,L,D]")
    .input("A", "[D,N]")
    .input("B", "[B,L,N]")
    .input("C", "[B,L,N]")
    .input("D", "[D]")
    .input("z", "[B,L,D] gate")
    .output("y", "[B,L,D]")
    .shape_infer(&infer_mamba_scan);

static Status gelu_cpu(KernelContext& c) { return unary_cpu<&gelu_ref>(c, "gelu"); }
FRAME_REGISTER_KERNEL("gelu", "cpu", &gelu_cpu);
static Status silu_cpu(KernelContext& c) { return unary_cpu<&silu_ref>(c, "silu"); }
FRAME_REGISTER_KERNEL("silu", "cpu", &silu_cpu);
static Status softplus_cpu(KernelContext& c) { return unary_cpu<&softplus_ref>(c, "softplus"); }
FRAME_REGISTER_KERNEL("softplus", "cpu", &softplus_cpu);
static Status exp_cpu(KernelContext& c) { return unary_cpu<&exp_ref>(c, "exp"); }
FRAME_REGISTER_KERNEL("exp", "cpu", &exp_cpu);
FRAME_REGISTER_KERNEL("bias_add", "cpu", &bias_add_cpu);
FRAME_REGISTER_KERNEL("mamba_scan", "cpu", &mamba_scan_cpu);
FRAME_REGISTER_KERNEL("bias_add", "cuda", &bias_add_cuda);
FRAME_REGISTER_KERNEL("mamba_scan", "cuda", &mamba_scan_cuda);
