// Frame HAL backend "cuda" for B200 (sm_100a): hal::Backend / Allocator / Stream / Event /
// Executable implemented over the C ABI of libframe_b200 (include/frame_b200.h).
//
// This translation unit is the reference-side binding: it includes Frame's own headers,
// registers itself with FRAME_REGISTER_BACKEND under the key "cuda" and converts the C ABI's
// integer statuses into frame::Status.  It replaces src/backends/cuda/cuda_backend.cpp,
// cuda_allocator.cpp and cuda_executable.cpp of the reference (which must then be built with
// FRAME_ENABLE_CUDA=OFF: a second backend or kernel registered under "cuda" aborts at start-up,
// src/runtime/backend_registry.cpp:39-48, src/ops/kernel_registry.cpp:23-43).
//
// Interface contracts mirrored here (paths inside the reference project):
//   include/frame/hal/backend.h:77-109     Backend: name, device_count, create_stream/event,
//                                          allocator (nullptr + one stderr line on a bad
//                                          device, src/backends/cuda/cuda_backend.cpp:162-167),
//                                          copy (direction from the two Devices, stream==nullptr
//                                          blocks, bytes==0 ok, null pointer -> kInvalidArgument,
//                                          cuda_backend.cpp:185-204), compile, launch
//   include/frame/hal/allocator.h:13-21    allocate(bytes > 0, alignment <= 256) / deallocate
//                                          (src/backends/cuda/cuda_allocator.cpp:26-66)
//   include/frame/hal/stream.h:13-29, event.h:16-24   un-recorded event reports complete
//   include/frame/hal/executable.h:28-59   run validates counts/dtypes/shapes/devices
#include <cstdio>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include <frame/core/device.h>
#include <frame/core/status.h>
#include <frame/core/tensor.h>
#include <frame/hal/allocator.h>
#include <frame/hal/backend.h>
#include <frame/hal/event.h>
#include <frame/hal/executable.h>
#include <frame/hal/stream.h>
#include <frame/ir/graph.h>
#include <frame/ir/serialization.h>
#include <frame/ops/executable_plan.h>
#include <frame/ops/kernel_registry.h>

#include "b200_status.h"
#include "frame_b200.h"

namespace frame_b200 {

using frame::Device;
using frame::ErrorCode;
using frame::Result;
using frame::Status;
using frame::Tensor;

Status to_status(int rc, std::string_view where) {
  if (rc == FB200_OK) return Status::ok();
  ErrorCode code = ErrorCode::kInternal;
  switch (rc) {
    case FB200_INVALID_ARGUMENT: code = ErrorCode::kInvalidArgument; break;
    case FB200_NOT_FOUND: code = ErrorCode::kNotFound; break;
    case FB200_ALREADY_EXISTS: code = ErrorCode::kAlreadyExists; break;
    case FB200_UNIMPLEMENTED: code = ErrorCode::kUnimplemented; break;
    case FB200_OUT_OF_MEMORY: code = ErrorCode::kOutOfMemory; break;
    case FB200_DEVICE_ERROR: code = ErrorCode::kDeviceError; break;
    default: break;
  }
  return Status::make(code, std::string(where) + ": " + fb200_last_error());
}

namespace {

Status validate_device(Device device, std::string_view where) {
  if (device.backend != frame::kCudaBackendName) {
    return Status::make(ErrorCode::kInvalidArgument, std::string(where) + ": device backend '" +
                                                         std::string(device.backend) +
                                                         "' is not 'cuda'");
  }
  int count = 0;
  const int rc = fb200_device_count(&count);
  if (rc != FB200_OK) return to_status(rc, where);
  if (device.index < 0 || device.index >= count) {
    return Status::make(ErrorCode::kInvalidArgument,
                        std::string(where) + ": device index " + std::to_string(device.index) +
                            " is out of range [0, " + std::to_string(count) + ")");
  }
  return Status::ok();
}

class B200Allocator final : public frame::hal::Allocator {
 public:
  explicit B200Allocator(int32_t device) : device_(device) {}
  Result<void*> allocate(size_t bytes, size_t alignment) override {
    void* ptr = nullptr;
    const int rc = fb200_malloc(device_, bytes, alignment, &ptr);
    if (rc != FB200_OK) return to_status(rc, "B200Allocator::allocate");
    return ptr;
  }
  void deallocate(void* ptr) override { fb200_free(device_, ptr); }

 private:
  int32_t device_;
};

class B200Event final : public frame::hal::Event {
 public:
  B200Event(int32_t device, fb200_event event) : device_(device), event_(event) {}
  ~B200Event() override { fb200_event_destroy(device_, event_); }
  bool query() const override {
    if (!recorded_) return true;  // an event that was never recorded counts as complete
    int done = 0;
    return fb200_event_query(device_, event_, &done) == FB200_OK && done != 0;
  }
  Status synchronize() override {
    if (!recorded_) return Status::ok();
    return to_status(fb200_event_synchronize(device_, event_), "B200Event::synchronize");
  }
  fb200_event native() const { return event_; }
  void mark_recorded() { recorded_ = true; }
  bool recorded() const { return recorded_; }

 private:
  int32_t device_;
  fb200_event event_;
  bool recorded_ = false;
};

class B200Stream final : public frame::hal::Stream {
 public:
  B200Stream(int32_t device, fb200_stream stream) : device_(device), stream_(stream) {}
  ~B200Stream() override { fb200_stream_destroy(device_, stream_); }
  Status synchronize() override {
    return to_status(fb200_stream_synchronize(device_, stream_), "B200Stream::synchronize");
  }
  Status record(frame::hal::Event& event) override {
    auto& e = static_cast<B200Event&>(event);
    const int rc = fb200_event_record(device_, e.native(), stream_);
    if (rc != FB200_OK) return to_status(rc, "B200Stream::record");
    e.mark_recorded();
    return Status::ok();
  }
  Status wait(const frame::hal::Event& event) override {
    const auto& e = static_cast<const B200Event&>(event);
    if (!e.recorded()) return Status::ok();
    return to_status(fb200_stream_wait_event(device_, stream_, e.native()), "B200Stream::wait");
  }
  void* native_handle() override { return stream_; }

 private:
  int32_t device_;
  fb200_stream stream_;
};

// The plan text consumed by fb200_plan_create, produced from ops::ExecutablePlan
// (include/frame/ops/executable_plan.h:42-71).
std::string serialise_plan(const frame::ops::ExecutablePlan& p) {
  std::string text;
  auto num = [&](long long v) { text += ' '; text += std::to_string(v); };
  text += "plan slots=" + std::to_string(p.slot_count) + " arena=" +
          std::to_string(p.arena_total_bytes) + "\n";
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
      num(step.output_slots[i]);
      num(static_cast<int>(t.dtype.code()));
      num(step.output_arena_offsets[i].has_value()
              ? static_cast<long long>(*step.output_arena_offsets[i])
              : -1LL);
      num(t.shape.rank());
      for (const int64_t d : t.shape.dims()) num(d);
    }
    text += " attrs=" + std::to_string(step.attrs.size()) + "\n";
    for (const auto& kv : step.attrs) {
      text += "attr " + kv.first + " " +
              std::string(frame::ir::attr_type_name(frame::ir::attr_type_of(kv.second))) + " " +
              frame::ir::format_attr_value(kv.second) + "\n";
    }
  }
  for (const int32_t s : p.output_slots) text += "out " + std::to_string(s) + "\n";
  return text;
}

// Executable: the planner's arena is allocated once (inside the fb200 plan), every run is one
// loop of launches on the caller's stream writing straight into the caller's output tensors.
// Replaces CudaExecutable (src/backends/cuda/cuda_executable.cpp:17-128).
class B200Executable final : public frame::hal::Executable {
 public:
  ~B200Executable() override { fb200_plan_destroy(plan_); }

  static Result<std::unique_ptr<B200Executable>> compile(const frame::ir::Graph& graph,
                                                         Device device,
                                                         const frame::hal::CompileOptions& options) {
    Result<frame::ops::ExecutablePlan> plan =
        frame::ops::build_executable_plan(graph, frame::kCudaBackendName);
    if (!plan.is_ok()) return plan.status();
    auto exe = std::make_unique<B200Executable>();
    exe->device_ = device;
    for (const auto& t : plan.value().input_types) {
      exe->input_signature_.push_back(frame::hal::IoSpec{t.dtype, t.shape});
    }
    for (const auto& t : plan.value().output_types) {
      exe->output_signature_.push_back(frame::hal::IoSpec{t.dtype, t.shape});
    }
    const std::string text = serialise_plan(plan.value());
    const int rc = fb200_plan_create(text.c_str(), device.index, options.allow_tf32 ? 1 : 0,
                                     options.opt_level, &exe->plan_);
    if (rc != FB200_OK) return to_status(rc, "B200Backend::compile");
    return exe;
  }

  Status run(std::span<const Tensor> inputs, std::span<Tensor> outputs,
             frame::hal::Stream& stream) override {
    FRAME_RETURN_IF_ERROR(frame::hal::validate_io_signature(inputs, input_signature_,
                                                            "B200Executable::run: input"));
    FRAME_RETURN_IF_ERROR(frame::hal::validate_io_signature(outputs, output_signature_,
                                                            "B200Executable::run: output"));
    FRAME_RETURN_IF_ERROR(
        frame::hal::validate_tensor_devices(inputs, device_, "B200Executable::run: input"));
    FRAME_RETURN_IF_ERROR(
        frame::hal::validate_tensor_devices(outputs, device_, "B200Executable::run: output"));
    std::vector<const void*> in(inputs.size());
    std::vector<void*> out(outputs.size());
    for (size_t i = 0; i < inputs.size(); ++i) in[i] = inputs[i].raw_data();
    for (size_t i = 0; i < outputs.size(); ++i) out[i] = outputs[i].raw_data();
    return to_status(fb200_plan_run(plan_, in.data(), out.data(), stream.native_handle()),
                     "B200Executable::run");
  }

  std::vector<frame::hal::IoSpec> input_signature() const override { return input_signature_; }
  std::vector<frame::hal::IoSpec> output_signature() const override { return output_signature_; }

 private:
  Device device_{};
  fb200_plan* plan_ = nullptr;
  std::vector<frame::hal::IoSpec> input_signature_;
  std::vector<frame::hal::IoSpec> output_signature_;
};

class B200Backend final : public frame::hal::Backend {
 public:
  std::string_view name() const override { return frame::kCudaBackendName; }

  Result<int32_t> device_count() const override {
    int count = 0;
    const int rc = fb200_device_count(&count);
    if (rc != FB200_OK) return to_status(rc, "B200Backend::device_count");
    return static_cast<int32_t>(count);
  }

  Result<std::unique_ptr<frame::hal::Stream>> create_stream(Device device) override {
    FRAME_RETURN_IF_ERROR(validate_device(device, "B200Backend::create_stream"));
    fb200_stream s = nullptr;
    const int rc = fb200_stream_create(device.index, &s);
    if (rc != FB200_OK) return to_status(rc, "B200Backend::create_stream");
    return std::unique_ptr<frame::hal::Stream>(std::make_unique<B200Stream>(device.index, s));
  }

  Result<std::unique_ptr<frame::hal::Event>> create_event(Device device) override {
    FRAME_RETURN_IF_ERROR(validate_device(device, "B200Backend::create_event"));
    fb200_event e = nullptr;
    const int rc = fb200_event_create(device.index, 0, &e);
    if (rc != FB200_OK) return to_status(rc, "B200Backend::create_event");
    return std::unique_ptr<frame::hal::Event>(std::make_unique<B200Event>(device.index, e));
  }

  frame::hal::Allocator* allocator(Device device) override {
    const Status v = validate_device(device, "B200Backend::allocator");
    if (!v.is_ok()) {
      std::fprintf(stderr, "%s\n", std::string(v.message()).c_str());
      return nullptr;
    }
    const std::lock_guard<std::mutex> lock(mu_);
    while (allocators_.size() <= static_cast<size_t>(device.index)) {
      allocators_.push_back(std::make_unique<B200Allocator>(static_cast<int32_t>(allocators_.size())));
    }
    return allocators_[static_cast<size_t>(device.index)].get();
  }

  Status copy(void* dst, Device dst_device, const void* src, Device src_device, size_t bytes,
              frame::hal::Stream* stream) override {
    const bool dst_cuda = dst_device.backend == frame::kCudaBackendName;
    const bool src_cuda = src_device.backend == frame::kCudaBackendName;
    const bool dst_cpu = dst_device.backend == frame::kCpuBackendName;
    const bool src_cpu = src_device.backend == frame::kCpuBackendName;
    int kind = 0;
    int device = 0;
    if (src_cpu && dst_cuda) { kind = FB200_H2D; device = dst_device.index; }
    else if (src_cuda && dst_cpu) { kind = FB200_D2H; device = src_device.index; }
    else if (src_cuda && dst_cuda) { kind = FB200_D2D; device = dst_device.index; }
    else {
      return Status::make(ErrorCode::kInvalidArgument,
                          "B200Backend::copy: unsupported direction '" +
                              std::string(src_device.backend) + "' -> '" +
                              std::string(dst_device.backend) + "'");
    }
    if (bytes == 0) return Status::ok();
    if (dst == nullptr || src == nullptr) {
      return Status::make(ErrorCode::kInvalidArgument,
                          "B200Backend::copy: dst and src must be non-null when bytes > 0");
    }
    return to_status(fb200_memcpy(device, dst, src, bytes, kind,
                                  stream != nullptr ? stream->native_handle() : nullptr,
                                  stream == nullptr ? 1 : 0),
                     "B200Backend::copy");
  }

  Result<std::unique_ptr<frame::hal::Executable>> compile(
      const frame::ir::Graph& graph, const frame::hal::CompileOptions& options) override {
    if (graph.topological_order().empty()) {
      return Status::make(ErrorCode::kInvalidArgument, "B200Backend::compile: graph has no nodes");
    }
    Device device{};
    bool found = false;
    for (const frame::ir::Node* node : graph.topological_order()) {
      if (!node->outputs().empty()) {
        device = node->outputs()[0].type().device;
        found = true;
        break;
      }
    }
    if (!found) {
      return Status::make(ErrorCode::kInternal,
                          "B200Backend::compile: graph has node(s) but no Value carries a device");
    }
    FRAME_RETURN_IF_ERROR(validate_device(device, "B200Backend::compile"));
    Result<std::unique_ptr<B200Executable>> exe = B200Executable::compile(graph, device, options);
    if (!exe.is_ok()) return exe.status();
    return std::unique_ptr<frame::hal::Executable>(std::move(exe.value()));
  }

  Status launch(const frame::hal::KernelInvocation& invocation,
                frame::hal::Stream* stream) override {
    FRAME_RETURN_IF_ERROR(validate_device(invocation.device, "B200Backend::launch"));
    const Result<frame::ops::KernelFn> kernel =
        frame::ops::KernelRegistry::instance().find(invocation.op, name());
    if (!kernel.is_ok()) return kernel.status();
    frame::ops::KernelContext ctx{invocation.inputs, invocation.outputs, invocation.attrs,
                                  invocation.device, stream};
    return kernel.value()(ctx);
  }

 private:
  std::mutex mu_;
  std::vector<std::unique_ptr<B200Allocator>> allocators_;
};

}  // namespace
}  // namespace frame_b200

FRAME_REGISTER_BACKEND(frame::kCudaBackendName, frame_b200::B200Backend);
