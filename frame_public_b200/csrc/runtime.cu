// CUDA HAL plumbing behind the C ABI: devices, allocator, copies, streams, events, errors.
// Stands behind hal::Backend / hal::Allocator / hal::Stream / hal::Event of the reference
// (include/frame/hal/backend.h:77-109, allocator.h:13-21, stream.h:13-29, event.h:16-24) and
// replaces src/backends/cuda/cuda_backend.cpp:68-312 and cuda_allocator.cpp:26-66.
#include "common.cuh"

#include <cstring>

namespace fb200 {

static thread_local char t_error[512] = "";
std::atomic<int64_t> g_launch_count{0};

int set_error(int code, const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(t_error, sizeof(t_error), fmt, args);
  va_end(args);
  return code;
}

// cudaErrorMemoryAllocation -> OUT_OF_MEMORY, everything else -> DEVICE_ERROR for "no device"
// class errors and INTERNAL otherwise (src/backends/cuda/cuda_status.cpp:9-15 maps to
// kOutOfMemory / kInternal).
int cuda_error(cudaError_t err, const char* what) {
  int code = FB200_INTERNAL;
  if (err == cudaErrorMemoryAllocation) code = FB200_OUT_OF_MEMORY;
  if (err == cudaErrorNoDevice || err == cudaErrorInsufficientDriver ||
      err == cudaErrorInvalidDevice || err == cudaErrorNoKernelImageForDevice) {
    code = FB200_DEVICE_ERROR;
  }
  // Clear the sticky-free last error so the next call starts clean.
  (void)cudaGetLastError();
  return set_error(code, "CUDA error in %s: %s (%s)", what, cudaGetErrorName(err),
                   cudaGetErrorString(err));
}

cudaError_t scratch_alloc_async(void** ptr, size_t bytes, cudaStream_t stream) {
  static std::atomic<uint64_t> configured{0};   // one bit per device ordinal
  int device = 0;
  if (cudaGetDevice(&device) == cudaSuccess && device >= 0 && device < 64 &&
      (configured.load(std::memory_order_relaxed) & (uint64_t(1) << device)) == 0) {
    cudaMemPool_t pool = nullptr;
    if (cudaDeviceGetDefaultMemPool(&pool, device) == cudaSuccess && pool != nullptr) {
      uint64_t keep = uint64_t(1) << 30;
      (void)cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    }
    (void)cudaGetLastError();
    configured.fetch_or(uint64_t(1) << device, std::memory_order_relaxed);
  }
  return cudaMallocAsync(ptr, bytes, stream);
}

static int use_device(int device) {
  FB200_CUDA_OK(cudaSetDevice(device));
  return FB200_OK;
}

}  // namespace fb200

using namespace fb200;

extern "C" {

const char* fb200_last_error(void) { return t_error; }
const char* fb200_version(void) { return "frame_b200 0.1 (sm_100a)"; }
int64_t fb200_launch_count(void) { return g_launch_count.load(std::memory_order_relaxed); }

int fb200_device_count(int* count) {
  if (count == nullptr) return set_error(FB200_INVALID_ARGUMENT, "fb200_device_count: null count");
  *count = 0;
  FB200_CUDA_OK(cudaGetDeviceCount(count));
  return FB200_OK;
}

// PCI bus id ("0000:1b:00.0") of a CUDA device ordinal: what identifies the same physical GPU to
// NVML and nvidia-smi, whose own indices ignore CUDA_VISIBLE_DEVICES.
int fb200_device_pci_bus_id(int device, char* buf, int len) {
  if (buf == nullptr || len < 16) return set_error(FB200_INVALID_ARGUMENT, "fb200_device_pci_bus_id: buffer of at least 16 bytes");
  FB200_CUDA_OK(cudaDeviceGetPCIBusId(buf, len, device));
  return FB200_OK;
}

int fb200_malloc(int device, size_t bytes, size_t alignment, void** ptr) {
  if (ptr == nullptr) return set_error(FB200_INVALID_ARGUMENT, "fb200_malloc: null out pointer");
  *ptr = nullptr;
  if (bytes == 0) return set_error(FB200_INVALID_ARGUMENT, "fb200_malloc: bytes must be > 0");
  if (alignment == 0 || (alignment & (alignment - 1)) != 0 || alignment > 256) {
    return set_error(FB200_INVALID_ARGUMENT,
                     "fb200_malloc: alignment %zu must be a power of two <= 256", alignment);
  }
  if (int rc = use_device(device)) return rc;
  FB200_CUDA_OK(cudaMalloc(ptr, bytes));  // cudaMalloc returns >= 256-byte aligned memory
  return FB200_OK;
}

int fb200_free(int device, void* ptr) {
  if (ptr == nullptr) return FB200_OK;
  if (int rc = use_device(device)) return rc;
  FB200_CUDA_OK(cudaFree(ptr));
  return FB200_OK;
}

int fb200_host_alloc(size_t bytes, void** ptr) {
  if (ptr == nullptr || bytes == 0) {
    return set_error(FB200_INVALID_ARGUMENT, "fb200_host_alloc: null pointer or zero bytes");
  }
  FB200_CUDA_OK(cudaMallocHost(ptr, bytes));
  return FB200_OK;
}

int fb200_host_free(void* ptr) {
  if (ptr == nullptr) return FB200_OK;
  FB200_CUDA_OK(cudaFreeHost(ptr));
  return FB200_OK;
}

int fb200_memcpy(int device, void* dst, const void* src, size_t bytes, int kind,
                 fb200_stream stream, int blocking) {
  if (bytes == 0) return FB200_OK;
  if (dst == nullptr || src == nullptr) {
    return set_error(FB200_INVALID_ARGUMENT, "fb200_memcpy: null pointer with %zu bytes", bytes);
  }
  cudaMemcpyKind k;
  switch (kind) {
    case FB200_H2D: k = cudaMemcpyHostToDevice; break;
    case FB200_D2H: k = cudaMemcpyDeviceToHost; break;
    case FB200_D2D: k = cudaMemcpyDeviceToDevice; break;
    default: return set_error(FB200_INVALID_ARGUMENT, "fb200_memcpy: unknown copy kind %d", kind);
  }
  if (int rc = use_device(device)) return rc;
  if (stream == nullptr && blocking) {
    FB200_CUDA_OK(cudaMemcpy(dst, src, bytes, k));
  } else {
    FB200_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, k, as_stream(stream)));
    if (blocking) FB200_CUDA_OK(cudaStreamSynchronize(as_stream(stream)));
  }
  return FB200_OK;
}

int fb200_memset(int device, void* dst, int value, size_t bytes, fb200_stream stream) {
  if (bytes == 0) return FB200_OK;
  if (dst == nullptr) return set_error(FB200_INVALID_ARGUMENT, "fb200_memset: null pointer");
  if (int rc = use_device(device)) return rc;
  FB200_CUDA_OK(cudaMemsetAsync(dst, value, bytes, as_stream(stream)));
  return FB200_OK;
}

int fb200_stream_create(int device, fb200_stream* stream) {
  if (stream == nullptr) return set_error(FB200_INVALID_ARGUMENT, "fb200_stream_create: null out");
  if (int rc = use_device(device)) return rc;
  cudaStream_t s = nullptr;
  FB200_CUDA_OK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  *stream = s;
  return FB200_OK;
}

int fb200_stream_destroy(int device, fb200_stream stream) {
  if (stream == nullptr) return FB200_OK;
  if (int rc = use_device(device)) return rc;
  FB200_CUDA_OK(cudaStreamDestroy(as_stream(stream)));
  return FB200_OK;
}

int fb200_stream_synchronize(int device, fb200_stream stream) {
  if (int rc = use_device(device)) return rc;
  FB200_CUDA_OK(cudaStreamSynchronize(as_stream(stream)));
  return FB200_OK;
}

int fb200_event_create(int device, int timing, fb200_event* event) {
  if (event == nullptr) return set_error(FB200_INVALID_ARGUMENT, "fb200_event_create: null out");
  if (int rc = use_device(device)) return rc;
  cudaEvent_t e = nullptr;
  FB200_CUDA_OK(cudaEventCreateWithFlags(&e, timing ? cudaEventDefault : cudaEventDisableTiming));
  *event = e;
  return FB200_OK;
}

int fb200_event_destroy(int device, fb200_event event) {
  if (event == nullptr) return FB200_OK;
  if (int rc = use_device(device)) return rc;
  FB200_CUDA_OK(cudaEventDestroy(reinterpret_cast<cudaEvent_t>(event)));
  return FB200_OK;
}

int fb200_event_record(int device, fb200_event event, fb200_stream stream) {
  if (event == nullptr) return set_error(FB200_INVALID_ARGUMENT, "fb200_event_record: null event");
  if (int rc = use_device(device)) return rc;
  FB200_CUDA_OK(cudaEventRecord(reinterpret_cast<cudaEvent_t>(event), as_stream(stream)));
  return FB200_OK;
}

int fb200_stream_wait_event(int device, fb200_stream stream, fb200_event event) {
  if (event == nullptr) return set_error(FB200_INVALID_ARGUMENT, "fb200_stream_wait_event: null event");
  if (int rc = use_device(device)) return rc;
  FB200_CUDA_OK(cudaStreamWaitEvent(as_stream(stream), reinterpret_cast<cudaEvent_t>(event), 0));
  return FB200_OK;
}

int fb200_event_query(int device, fb200_event event, int* done) {
  if (event == nullptr || done == nullptr) {
    return set_error(FB200_INVALID_ARGUMENT, "fb200_event_query: null argument");
  }
  if (int rc = use_device(device)) return rc;
  cudaError_t err = cudaEventQuery(reinterpret_cast<cudaEvent_t>(event));
  if (err == cudaSuccess) { *done = 1; return FB200_OK; }
  if (err == cudaErrorNotReady) { *done = 0; (void)cudaGetLastError(); return FB200_OK; }
  return cuda_error(err, "cudaEventQuery");
}

int fb200_event_synchronize(int device, fb200_event event) {
  if (event == nullptr) return set_error(FB200_INVALID_ARGUMENT, "fb200_event_synchronize: null event");
  if (int rc = use_device(device)) return rc;
  FB200_CUDA_OK(cudaEventSynchronize(reinterpret_cast<cudaEvent_t>(event)));
  return FB200_OK;
}

int fb200_event_elapsed_ms(fb200_event start, fb200_event stop, float* ms) {
  if (start == nullptr || stop == nullptr || ms == nullptr) {
    return set_error(FB200_INVALID_ARGUMENT, "fb200_event_elapsed_ms: null argument");
  }
  FB200_CUDA_OK(cudaEventElapsedTime(ms, reinterpret_cast<cudaEvent_t>(start),
                                     reinterpret_cast<cudaEvent_t>(stop)));
  return FB200_OK;
}

}  // extern "C"
