// TEST INFRASTRUCTURE — extern "C" shim over the reference framework's own
// public C++ API, so that Python (ctypes) can drive the UNMODIFIED reference:
// parse an IR text, run the nine-pass pipeline, compile on a named backend and
// run with host buffers.  With backend "cpu" this is the parity oracle and the
// timed CPU baseline; with backend "cuda" (the sm_100a backend of this
// repository loaded into the same process) it is the end-to-end product path.
// Nothing here computes anything itself.
//
// Reference API used (paths inside the reference project):
//   ir::parse_text / dump_text            include/frame/ir/serialization.h:77-81
//   runtime::compile                      src/runtime/compile.cpp:128-178
//   compiler::standard_pipeline           src/compiler/pipeline.cpp:9-28
//   ops::build_executable_plan            src/ops/executable_plan.cpp:16-121
//   hal::Backend::{allocator,copy,create_stream}  include/frame/hal/backend.h:77-109
//   runtime::FallbackStats                include/frame/runtime/fallback_stats.h:21-41
#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <memory>
#include <span>
#include <string>
#include <string_view>
#include <variant>
#include <vector>

#include <frame/compiler/autograd.h>
#include <frame/compiler/pipeline.h>
#include <frame/core/tensor.h>
#include <frame/hal/allocator.h>
#include <frame/hal/backend.h>
#include <frame/hal/event.h>
#include <frame/hal/executable.h>
#include <frame/hal/stream.h>
#include <frame/ir/graph.h>
#include <frame/ir/serialization.h>
#include <frame/nn/layers.h>
#include <frame/nn/module.h>
#include <frame/ops/executable_plan.h>
#include <frame/ops/kernel_registry.h>
#include <frame/ops/op_registry.h>
#include <frame/runtime/compile.h>
#include <frame/runtime/fallback_stats.h>

namespace {

using frame::Device;
using frame::Result;
using frame::Status;
using frame::Tensor;

void set_err(char* err, int errlen, const std::string& msg) {
  if (err == nullptr || errlen <= 0) return;
  std::snprintf(err, static_cast<size_t>(errlen), "%s", msg.c_str());
}

std::string_view static_backend_name(std::string_view name) {
  if (name == frame::kCpuBackendName) return frame::kCpuBackendName;
  if (name == frame::kCudaBackendName) return frame::kCudaBackendName;
  return {};
}

struct Handle {
  std::shared_ptr<frame::hal::Executable> exe;
  frame::hal::Backend* backend = nullptr;
  Device device;
  std::vector<frame::hal::IoSpec> in_sig;
  std::vector<frame::hal::IoSpec> out_sig;
  std::vector<Tensor> dev_in;
  std::vector<Tensor> dev_out;
  std::unique_ptr<frame::hal::Stream> stream;
};

Status ensure_buffers(Handle& h) {
  if (!h.dev_in.empty() || !h.dev_out.empty()) return Status::ok();
  frame::hal::Allocator* alloc = h.backend->allocator(h.device);
  if (alloc == nullptr) {
    return Status::make(frame::ErrorCode::kInternal, "shim: null allocator");
  }
  for (const auto& spec : h.in_sig) {
    Result<Tensor> t = Tensor::empty(spec.shape, spec.dtype, h.device, *alloc);
    if (!t.is_ok()) return t.status();
    h.dev_in.push_back(t.value());
  }
  for (const auto& spec : h.out_sig) {
    Result<Tensor> t = Tensor::empty(spec.shape, spec.dtype, h.device, *alloc);
    if (!t.is_ok()) return t.status();
    h.dev_out.push_back(t.value());
  }
  Result<std::unique_ptr<frame::hal::Stream>> s = h.backend->create_stream(h.device);
  if (!s.is_ok()) return s.status();
  h.stream = std::move(s.value());
  return Status::ok();
}

size_t spec_bytes(const frame::hal::IoSpec& spec) {
  return static_cast<size_t>(spec.shape.numel()) * spec.dtype.itemsize();
}

// An op with a schema and no kernel on any backend: what Backend::compile must reject by name.
constexpr std::string_view kOrphanOp = "fref_shim_op_without_kernel";

Result<std::vector<frame::Shape>> infer_orphan(const frame::ops::NodeContext& ctx) {
  if (ctx.input_types.size() != 1) {
    return Status::make(frame::ErrorCode::kInvalidArgument, "op 'fref_shim_op_without_kernel' expects 1 input");
  }
  return std::vector<frame::Shape>{ctx.input_types[0].shape};
}

}  // namespace

FRAME_REGISTER_OP(kOrphanOp).input("x", "input").output("out", "never given a kernel").shape_infer(&infer_orphan);

extern "C" {

// Parses `ir_text`, compiles it for `backend` through runtime::compile (cache,
// nine-pass pipeline, Backend::compile, fallback chain) and returns a handle.
void* fref_compile(const char* ir_text, const char* backend, int device_index, int allow_tf32,
                   char* err, int errlen) {
  const std::string_view bname = static_backend_name(backend);
  if (bname.empty()) {
    set_err(err, errlen, "shim: backend must be cpu or cuda");
    return nullptr;
  }
  Result<frame::ir::Graph> graph = frame::ir::parse_text(ir_text);
  if (!graph.is_ok()) {
    set_err(err, errlen, std::string(graph.status().message()));
    return nullptr;
  }
  frame::hal::CompileOptions options;
  options.allow_tf32 = allow_tf32 != 0;
  Result<std::shared_ptr<frame::hal::Executable>> exe =
      frame::runtime::compile(graph.value(), bname, options);
  if (!exe.is_ok()) {
    set_err(err, errlen, std::string(exe.status().message()));
    return nullptr;
  }
  Result<frame::hal::Backend*> be = frame::hal::BackendRegistry::instance().get(bname);
  if (!be.is_ok()) {
    set_err(err, errlen, std::string(be.status().message()));
    return nullptr;
  }
  auto* h = new Handle();
  h->exe = exe.value();
  h->backend = be.value();
  h->device = Device{bname, device_index};
  h->in_sig = h->exe->input_signature();
  h->out_sig = h->exe->output_signature();
  return h;
}

void fref_free(void* handle) { delete static_cast<Handle*>(handle); }

int fref_num_io(void* handle, int is_output) {
  auto* h = static_cast<Handle*>(handle);
  return static_cast<int>(is_output ? h->out_sig.size() : h->in_sig.size());
}

// dtype code (reference DTypeCode numbering), rank and dims of one signature entry.
int fref_io_spec(void* handle, int is_output, int index, int* dtype, int* rank, int64_t* dims,
                 int dims_cap) {
  auto* h = static_cast<Handle*>(handle);
  const auto& sig = is_output ? h->out_sig : h->in_sig;
  if (index < 0 || static_cast<size_t>(index) >= sig.size()) return -1;
  const auto& spec = sig[static_cast<size_t>(index)];
  *dtype = static_cast<int>(spec.dtype.code());
  *rank = static_cast<int>(spec.shape.rank());
  for (int i = 0; i < *rank && i < dims_cap; ++i) dims[i] = spec.shape.dims()[static_cast<size_t>(i)];
  return 0;
}

// One run with HOST buffers: copy in through Backend::copy, Executable::run on a
// persistent stream, synchronise, copy out.
int fref_run(void* handle, const void* const* host_in, void* const* host_out, char* err,
             int errlen) {
  auto* h = static_cast<Handle*>(handle);
  Status st = ensure_buffers(*h);
  if (!st.is_ok()) {
    set_err(err, errlen, std::string(st.message()));
    return 1;
  }
  for (size_t i = 0; i < h->in_sig.size(); ++i) {
    const size_t bytes = spec_bytes(h->in_sig[i]);
    if (bytes == 0) continue;
    st = h->backend->copy(h->dev_in[i].raw_data(), h->device, host_in[i], frame::cpu_device(),
                          bytes, h->stream.get());
    if (!st.is_ok()) {
      set_err(err, errlen, std::string(st.message()));
      return 2;
    }
  }
  st = h->exe->run(h->dev_in, h->dev_out, *h->stream);
  if (!st.is_ok()) {
    set_err(err, errlen, std::string(st.message()));
    return 3;
  }
  for (size_t i = 0; i < h->out_sig.size(); ++i) {
    const size_t bytes = spec_bytes(h->out_sig[i]);
    if (bytes == 0) continue;
    st = h->backend->copy(host_out[i], frame::cpu_device(), h->dev_out[i].raw_data(), h->device,
                          bytes, h->stream.get());
    if (!st.is_ok()) {
      set_err(err, errlen, std::string(st.message()));
      return 4;
    }
  }
  st = h->stream->synchronize();
  if (!st.is_ok()) {
    set_err(err, errlen, std::string(st.message()));
    return 5;
  }
  return 0;
}

// Seconds per Executable::run (inputs already resident), averaged over `iters`
// back-to-back runs followed by one stream synchronise; one untimed warm-up.
double fref_time_run(void* handle, int iters, char* err, int errlen) {
  auto* h = static_cast<Handle*>(handle);
  Status st = ensure_buffers(*h);
  if (!st.is_ok()) {
    set_err(err, errlen, std::string(st.message()));
    return -1.0;
  }
  st = h->exe->run(h->dev_in, h->dev_out, *h->stream);
  if (st.is_ok()) st = h->stream->synchronize();
  if (!st.is_ok()) {
    set_err(err, errlen, std::string(st.message()));
    return -1.0;
  }
  const auto t0 = std::chrono::steady_clock::now();
  for (int i = 0; i < iters; ++i) {
    st = h->exe->run(h->dev_in, h->dev_out, *h->stream);
    if (!st.is_ok()) {
      set_err(err, errlen, std::string(st.message()));
      return -1.0;
    }
  }
  st = h->stream->synchronize();
  const auto t1 = std::chrono::steady_clock::now();
  if (!st.is_ok()) {
    set_err(err, errlen, std::string(st.message()));
    return -1.0;
  }
  return std::chrono::duration<double>(t1 - t0).count() / (iters > 0 ? iters : 1);
}

// Device pointer of a resident input/output buffer (for harness-side timing).
void* fref_device_buffer(void* handle, int is_output, int index) {
  auto* h = static_cast<Handle*>(handle);
  if (!ensure_buffers(*h).is_ok()) return nullptr;
  auto& v = is_output ? h->dev_out : h->dev_in;
  if (index < 0 || static_cast<size_t>(index) >= v.size()) return nullptr;
  return v[static_cast<size_t>(index)].raw_data();
}

// IR text of one of the reference's own nn:: modules, built by the reference's builder
// (include/frame/nn/layers.h:157-234, src/nn/layers.cpp): graph input 0 is the activation, the
// module's parameters follow in Module::parameters() order.  kind: "transformer" =
// nn::TransformerEncoderBlock(batch, seq, embed, heads, ffn, with_bias), x: [batch*seq, embed];
// "mha" = nn::MultiheadAttention(batch, seq, embed, heads, with_bias); "mamba" =
// nn::Mamba(batch, channels = p2, steps = p1, kernel = p3), x: [batch, channels, steps]; "cnn" =
// nn::Sequential of Conv2d, Relu, MaxPool2d, Flatten, Linear, x: [batch, p1, p2, p2].
// Returns the number of bytes needed, -1 on error.
int64_t fref_nn_graph_text(const char* kind, int64_t batch, int64_t p1, int64_t p2, int64_t p3,
                           int64_t p4, int with_bias, int dtype_code, const char* backend,
                           int device_index, char* out, int64_t cap, char* err, int errlen) {
  const std::string_view bname = static_backend_name(backend);
  if (bname.empty()) {
    set_err(err, errlen, "unknown backend");
    return -1;
  }
  const frame::DType dtype(static_cast<frame::DTypeCode>(dtype_code));
  const Device device{bname, device_index};
  const std::string k(kind);
  frame::nn::Module module;
  frame::Shape x_shape;
  if (k == "transformer") {
    module = frame::nn::TransformerEncoderBlock("block", batch, p1, p2, p3, p4, with_bias != 0, dtype);
    x_shape = frame::Shape({batch * p1, p2});
  } else if (k == "mha") {
    module = frame::nn::MultiheadAttention("mha", batch, p1, p2, p3, with_bias != 0, dtype);
    x_shape = frame::Shape({batch * p1, p2});
  } else if (k == "mamba") {
    module = frame::nn::Mamba("mamba", batch, p2, p1, p3, dtype);
    x_shape = frame::Shape({batch, p2, p1});
  } else if (k == "cnn") {
    // nn::Sequential{Conv2d 3x3 s1 p1 + bias, Relu, MaxPool2d 2x2 s2, Flatten, Linear}: the reference's
    // own CNN (tests/cpp/nn/test_cnn_convergence.cpp:83-100; golden cnn_forward_expected.txt).
    // p1 = input channels, p2 = image height = width, p3 = conv output channels, p4 = classes
    const int64_t flat = p3 * (p2 / 2) * (p2 / 2);
    module = frame::nn::Sequential(
        "cnn", {frame::nn::Conv2d("conv", p1, p3, {3, 3}, {1, 1}, {1, 1}, 1, true, dtype), frame::nn::Relu("relu"),
                frame::nn::MaxPool2d("pool", {2, 2}, {2, 2}, {0, 0}), frame::nn::Flatten("flatten"),
                frame::nn::Linear("linear", batch, flat, p4, with_bias != 0, dtype)});
    x_shape = frame::Shape({batch, p1, p2, p2});
  } else {
    set_err(err, errlen, "unknown module kind");
    return -1;
  }
  frame::ir::Graph graph("nn_" + k);
  frame::ir::TensorType xt;
  xt.dtype = dtype;
  xt.shape = x_shape;
  xt.layout = frame::ir::Layout::kRowMajor;
  xt.device = device;
  Result<frame::ir::Value*> x = graph.add_graph_input(xt);
  if (!x.is_ok()) {
    set_err(err, errlen, std::string(x.status().message()));
    return -1;
  }
  std::vector<frame::nn::ParamSpec> specs = module.parameters();
  for (auto& spec : specs) spec.type.device = device;
  Result<std::vector<frame::ir::Value*>> params = frame::nn::add_parameter_inputs(graph, specs);
  if (!params.is_ok()) {
    set_err(err, errlen, std::string(params.status().message()));
    return -1;
  }
  Result<std::vector<frame::ir::Value*>> outs =
      module.build(graph, std::vector<frame::ir::Value*>{x.value()}, params.value());
  if (!outs.is_ok()) {
    set_err(err, errlen, std::string(outs.status().message()));
    return -1;
  }
  for (frame::ir::Value* v : outs.value()) {
    const Status st = graph.mark_output(v);
    if (!st.is_ok()) {
      set_err(err, errlen, std::string(st.message()));
      return -1;
    }
  }
  const std::string text = frame::ir::dump_text(graph);
  if (out != nullptr && cap > 0) std::snprintf(out, static_cast<size_t>(cap), "%s", text.c_str());
  return static_cast<int64_t>(text.size()) + 1;
}

// IR text of the training graph compiler::build_backward_graph derives from `ir_text`: the forward
// outputs followed by the gradients w.r.t. the listed graph inputs
// (include/frame/compiler/autograd.h:44).  Returns the number of bytes needed.
int64_t fref_backward_text(const char* ir_text, int32_t loss_output_index, const int32_t* wrt,
                           int32_t n_wrt, char* out, int64_t cap, char* err, int errlen) {
  Result<frame::ir::Graph> graph = frame::ir::parse_text(ir_text);
  if (!graph.is_ok()) {
    set_err(err, errlen, std::string(graph.status().message()));
    return -1;
  }
  Result<frame::ir::Graph> train = frame::compiler::build_backward_graph(
      graph.value(), loss_output_index, std::span<const int32_t>(wrt, static_cast<size_t>(n_wrt)));
  if (!train.is_ok()) {
    set_err(err, errlen, std::string(train.status().message()));
    return -1;
  }
  const std::string text = frame::ir::dump_text(train.value());
  if (out != nullptr && cap > 0) std::snprintf(out, static_cast<size_t>(cap), "%s", text.c_str());
  return static_cast<int64_t>(text.size()) + 1;
}

// IR text after the standard nine-pass pipeline for `backend` (what
// Backend::compile receives).  Returns the number of bytes needed.
int64_t fref_pipeline_text(const char* ir_text, const char* backend, char* out, int64_t cap,
                           char* err, int errlen) {
  const std::string_view bname = static_backend_name(backend);
  Result<frame::ir::Graph> graph = frame::ir::parse_text(ir_text);
  if (!graph.is_ok()) {
    set_err(err, errlen, std::string(graph.status().message()));
    return -1;
  }
  Result<frame::compiler::PassManager> pm = frame::compiler::standard_pipeline(bname);
  if (!pm.is_ok()) {
    set_err(err, errlen, std::string(pm.status().message()));
    return -1;
  }
  const Status st = pm.value().run(graph.value());
  if (!st.is_ok()) {
    set_err(err, errlen, std::string(st.message()));
    return -1;
  }
  const std::string text = frame::ir::dump_text(graph.value());
  if (out != nullptr && cap > 0) {
    std::snprintf(out, static_cast<size_t>(cap), "%s", text.c_str());
  }
  return static_cast<int64_t>(text.size()) + 1;
}

// The executable plan the reference builds for the pipeline's output (steps,
// slots, arena offsets of the memory planner), as line-oriented text:
//   plan slots=<n> arena=<bytes>
//   in <slot> <dtype> <rank> <dims...>
//   step <op> nin=<k> <slots...> nout=<m> (<slot> <dtype> <offset|-1> <rank> <dims...>)* attrs=<k>
//   attr <name> <kind> <value text in the IR's own attribute format>
//   out <slot>
int64_t fref_plan_text(const char* ir_text, const char* backend, int run_pipeline, char* out,
                       int64_t cap, char* err, int errlen) {
  const std::string_view bname = static_backend_name(backend);
  Result<frame::ir::Graph> graph = frame::ir::parse_text(ir_text);
  if (!graph.is_ok()) {
    set_err(err, errlen, std::string(graph.status().message()));
    return -1;
  }
  if (run_pipeline != 0) {
    Result<frame::compiler::PassManager> pm = frame::compiler::standard_pipeline(bname);
    if (!pm.is_ok()) {
      set_err(err, errlen, std::string(pm.status().message()));
      return -1;
    }
    const Status st = pm.value().run(graph.value());
    if (!st.is_ok()) {
      set_err(err, errlen, std::string(st.message()));
      return -1;
    }
  }
  Result<frame::ops::ExecutablePlan> plan = frame::ops::build_executable_plan(graph.value(), bname);
  if (!plan.is_ok()) {
    set_err(err, errlen, std::string(plan.status().message()));
    return -1;
  }
  const frame::ops::ExecutablePlan& p = plan.value();
  // Plain string appends: no iostreams in this translation unit.
  std::string text;
  auto num = [&](long long v) { text += ' '; text += std::to_string(v); };
  text += "plan slots=" + std::to_string(p.slot_count) + " arena=" + std::to_string(p.arena_total_bytes) + "\n";
  for (size_t i = 0; i < p.input_types.size(); ++i) {
    const auto& t = p.input_types[i];
    text += "in";
    num(static_cast<long long>(i));
    num(static_cast<int>(t.dtype.code()));
    num(t.shape.rank());
    for (const int64_t d : t.shape.dims()) num(d);
    text += '\n';
  }
  for (const auto& step : p.steps) {
    text += "step " + step.op + " nin=" + std::to_string(step.input_slots.size());
    for (const int32_t s : step.input_slots) num(s);
    text += " nout=" + std::to_string(step.output_slots.size());
    for (size_t i = 0; i < step.output_slots.size(); ++i) {
      const auto& t = step.output_types[i];
      const long long off = step.output_arena_offsets[i].has_value()
                                ? static_cast<long long>(*step.output_arena_offsets[i])
                                : -1LL;
      num(step.output_slots[i]);
      num(static_cast<int>(t.dtype.code()));
      num(off);
      num(t.shape.rank());
      for (const int64_t d : t.shape.dims()) num(d);
    }
    text += " attrs=" + std::to_string(step.attrs.size()) + "\n";
    std::vector<std::string> names;
    for (const auto& kv : step.attrs) names.push_back(kv.first);
    std::sort(names.begin(), names.end());
    for (const auto& name : names) {
      const auto& v = step.attrs.at(name);
      text += "attr " + name + " " + std::string(frame::ir::attr_type_name(frame::ir::attr_type_of(v))) +
              " " + frame::ir::format_attr_value(v) + "\n";
    }
  }
  for (const int32_t s : p.output_slots) text += "out " + std::to_string(s) + "\n";
  if (out != nullptr && cap > 0) {
    std::snprintf(out, static_cast<size_t>(cap), "%s", text.c_str());
  }
  return static_cast<int64_t>(text.size()) + 1;
}

int64_t fref_fallback_count(const char* op, const char* backend) {
  return frame::runtime::FallbackStats::instance().count(op, backend);
}

void fref_fallback_reset() { frame::runtime::FallbackStats::instance().reset(); }

int fref_has_kernel(const char* op, const char* backend) {
  return frame::ops::KernelRegistry::instance().find(op, backend).is_ok() ? 1 : 0;
}

// The contract every registered hal::Backend must meet, checked on the C++ classes behind
// BackendRegistry::get(backend): the eight cases of the reference's parameterised conformance suite
// (tests/cpp/hal_conformance/test_hal_conformance.cpp:96-269), restated here because that suite needs
// GoogleTest.  Returns the number of failed cases; `report` receives one "ok <case>" or
// "FAIL <case>: <why>" line per case.
int fref_hal_conformance(const char* backend, char* report, int cap) {
  std::string text;
  int failed = 0;
  auto note = [&](const char* name, bool ok, const std::string& why = "") {
    text += (ok ? std::string("ok ") : std::string("FAIL ")) + name + (ok || why.empty() ? "" : ": " + why) + "\n";
    if (!ok) ++failed;
  };
  Result<frame::hal::Backend*> got = frame::hal::BackendRegistry::instance().get(backend);
  note("get_returns_backend_with_matching_name", got.is_ok() && got.value()->name() == std::string_view(backend));
  if (!got.is_ok()) {
    if (report != nullptr && cap > 0) std::snprintf(report, static_cast<size_t>(cap), "%s", text.c_str());
    return failed + 7;
  }
  frame::hal::Backend* b = got.value();
  const Device dev{b->name(), 0};
  {
    Result<int32_t> n = b->device_count();
    note("device_count_is_at_least_one", n.is_ok() && n.value() >= 1);
  }
  {
    auto s = b->create_stream(dev);
    note("create_stream_succeeds", s.is_ok(), s.is_ok() ? "" : std::string(s.status().message()));
  }
  {
    auto e = b->create_event(dev);
    const bool ok = e.is_ok() && e.value()->query() && e.value()->synchronize().is_ok();
    note("unrecorded_event_reports_complete", ok);
  }
  {
    auto s = b->create_stream(dev);
    auto e = b->create_event(dev);
    const bool ok = s.is_ok() && e.is_ok() && s.value()->record(*e.value()).is_ok() &&
                    s.value()->wait(*e.value()).is_ok() && s.value()->synchronize().is_ok();
    note("record_wait_synchronize_succeed", ok);
  }
  frame::hal::Allocator* alloc = b->allocator(dev);
  {
    bool ok = alloc != nullptr;
    std::string why = ok ? "" : "null allocator";
    if (ok) {
      constexpr size_t kBytes = 256;
      Result<void*> p = alloc->allocate(kBytes, 64);
      ok = p.is_ok() && p.value() != nullptr && reinterpret_cast<std::uintptr_t>(p.value()) % 64 == 0;
      if (ok) {
        auto s = b->create_stream(dev);
        std::vector<unsigned char> pattern(kBytes), back(kBytes, 0);
        for (size_t i = 0; i < kBytes; ++i) pattern[i] = static_cast<unsigned char>(i * 13 + 0x21);
        ok = s.is_ok() && b->copy(p.value(), dev, pattern.data(), frame::cpu_device(), kBytes, s.value().get()).is_ok() &&
             b->copy(back.data(), frame::cpu_device(), p.value(), dev, kBytes, s.value().get()).is_ok() &&
             s.value()->synchronize().is_ok() && std::memcmp(back.data(), pattern.data(), kBytes) == 0;
        if (!ok) why = "bytes did not survive host -> device -> host";
        alloc->deallocate(p.value());
      } else {
        why = "allocation failed or is not 64-byte aligned";
      }
    }
    note("allocator_round_trip_at_alignment_64", ok, why);
  }
  {
    bool ok = alloc != nullptr;
    if (ok) {
      constexpr size_t kBytes = 128;
      Result<void*> a = alloc->allocate(kBytes, 64), c = alloc->allocate(kBytes, 64), d = alloc->allocate(kBytes, 64);
      ok = a.is_ok() && c.is_ok() && d.is_ok();
      if (ok) {
        auto s = b->create_stream(dev);
        std::vector<unsigned char> pattern(kBytes), back(kBytes, 0);
        for (size_t i = 0; i < kBytes; ++i) pattern[i] = static_cast<unsigned char>(i * 5 + 9);
        ok = s.is_ok() && b->copy(a.value(), dev, pattern.data(), frame::cpu_device(), kBytes, s.value().get()).is_ok() &&
             b->copy(c.value(), dev, a.value(), dev, kBytes, s.value().get()).is_ok() &&
             b->copy(d.value(), dev, c.value(), dev, kBytes, s.value().get()).is_ok() &&
             b->copy(back.data(), frame::cpu_device(), d.value(), dev, kBytes, s.value().get()).is_ok() &&
             s.value()->synchronize().is_ok() && std::memcmp(back.data(), pattern.data(), kBytes) == 0;
      }
      if (a.is_ok()) alloc->deallocate(a.value());
      if (c.is_ok()) alloc->deallocate(c.value());
      if (d.is_ok()) alloc->deallocate(d.value());
    }
    note("device_to_device_copies_preserve_bytes", ok);
  }
  {
    frame::ir::Graph graph;
    frame::ir::TensorType type;
    type.dtype = frame::DType::of<float>();
    type.shape = frame::Shape({4});
    type.layout = frame::ir::Layout::kRowMajor;
    type.device = dev;
    bool ok = false;
    std::string why = "graph construction failed";
    auto in = graph.add_graph_input(type);
    if (in.is_ok()) {
      auto node = graph.create_node(std::string(kOrphanOp), {in.value()}, {type});
      if (node.is_ok() && graph.mark_output(node.value(), 0).is_ok()) {
        auto compiled = b->compile(graph, frame::hal::CompileOptions{});
        ok = !compiled.is_ok() && compiled.status().code() == frame::ErrorCode::kUnimplemented &&
             std::string(compiled.status().message()).find(std::string(kOrphanOp)) != std::string::npos;
        why = compiled.is_ok() ? "compile accepted an op without a kernel" : std::string(compiled.status().message());
      }
    }
    note("compile_rejects_unsupported_op_as_unimplemented_with_its_name", ok, why);
  }
  if (report != nullptr && cap > 0) std::snprintf(report, static_cast<size_t>(cap), "%s", text.c_str());
  return failed;
}

int fref_has_backend(const char* backend) {
  return frame::hal::BackendRegistry::instance().get(backend).is_ok() ? 1 : 0;
}

}  // extern "C"
