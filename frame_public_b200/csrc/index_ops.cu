// gather along axis 0 and its adjoint scatter_add (= gather_grad_internal).
//
// Semantics: src/ops/schemas/gather.cpp:86-216 and the CPU kernels of
// src/backends/cpu/kernels/gather.cpp: x [n, f], indices [k] (int32 or int64), out [k, f] with
// out[j, :] = x[indices[j], :]; scatter_add: out [v, f] = 0, out[indices[j], :] += updates[j, :],
// repeated indices accumulate.  An index outside the table is an error that names the offending
// value (the reference's CUDA kernels look at the indices on the host before launching,
// src/backends/cuda/kernels/gather.cu); here a small reduction kernel finds the smallest and the
// largest index, the two values are read back and the stream is synchronised once — these two entry
// points are therefore not asynchronous, and the plan executor does not replay plans that contain
// them as CUDA graphs.
// gather is pure data movement (bit-exact).  scatter_add accumulates in fp32 with atomics: for
// 16-bit tensors into a stream-ordered fp32 scratch that is rounded once at the end, as the CPU
// reference rounds its float buffer once; the order of the additions is not fixed, so repeated
// indices agree with the reference within the tolerance tier only.
#include <mutex>

#include "common.cuh"

namespace fb200 {

__device__ long long g_index_range[2];   // smallest and largest index of the call in flight
static std::mutex g_index_range_mu;      // one call at a time owns g_index_range

template <typename I>
__global__ void __launch_bounds__(256)
index_range_kernel(const I* __restrict__ idx, int64_t k) {
  long long lo = 0x7fffffffffffffffLL, hi = -0x7fffffffffffffffLL - 1;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < k; i += stride) {
    const long long v = static_cast<long long>(idx[i]);
    lo = v < lo ? v : lo;
    hi = v > hi ? v : hi;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const long long ol = __shfl_xor_sync(0xffffffffu, lo, o);
    const long long oh = __shfl_xor_sync(0xffffffffu, hi, o);
    lo = ol < lo ? ol : lo;
    hi = oh > hi ? oh : hi;
  }
  if ((threadIdx.x & 31) == 0) {
    atomicMin(&g_index_range[0], lo);
    atomicMax(&g_index_range[1], hi);
  }
}

// Checks every index against [0, bound); synchronises the stream.
template <typename I>
static int check_indices(const char* op, const void* indices, int64_t k, int64_t bound, cudaStream_t s) {
  if (k == 0) return FB200_OK;
  std::lock_guard<std::mutex> lock(g_index_range_mu);
  const long long init[2] = {0x7fffffffffffffffLL, -0x7fffffffffffffffLL - 1};
  FB200_CUDA_OK(cudaMemcpyToSymbolAsync(g_index_range, init, sizeof(init), 0, cudaMemcpyHostToDevice, s));
  index_range_kernel<I><<<grid_for(k, 256, 4), 256, 0, s>>>(static_cast<const I*>(indices), k);
  if (int rc = after_launch("index_range_kernel")) return rc;
  long long range[2] = {0, 0};
  FB200_CUDA_OK(cudaMemcpyFromSymbolAsync(range, g_index_range, sizeof(range), 0, cudaMemcpyDeviceToHost, s));
  FB200_CUDA_OK(cudaStreamSynchronize(s));
  if (range[0] < 0 || range[1] >= bound) {
    const long long bad = range[0] < 0 ? range[0] : range[1];
    return set_error(FB200_INVALID_ARGUMENT, "op '%s': index %lld is out of range [0, %lld)", op, bad,
                     static_cast<long long>(bound));
  }
  return FB200_OK;
}

// One 16-byte vector (or one element) of one gathered row per thread.
template <typename V, typename I>
__global__ void __launch_bounds__(256)
gather_rows_kernel(const V* __restrict__ x, const I* __restrict__ idx, V* __restrict__ out, int64_t k,
                   int64_t row_vecs) {
  const int64_t total = k * row_vecs;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += stride) {
    const int64_t row = e / row_vecs;
    const int64_t col = e - row * row_vecs;
    out[e] = x[static_cast<int64_t>(idx[row]) * row_vecs + col];
  }
}

template <typename T, typename I>
__global__ void __launch_bounds__(256)
scatter_add_kernel(const T* __restrict__ updates, const I* __restrict__ idx, float* __restrict__ acc,
                   int64_t k, int64_t f) {
  const int64_t total = k * f;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += stride) {
    const int64_t row = e / f;
    const int64_t col = e - row * f;
    atomicAdd(acc + static_cast<int64_t>(idx[row]) * f + col, to_f32(updates[e]));
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
round_from_f32_kernel(const float* __restrict__ acc, T* __restrict__ out, int64_t n) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    out[i] = from_f32<T>(acc[i]);
  }
}

template <typename I>
static int gather_impl(const void* x, const void* indices, void* out, int64_t n, int64_t f, int64_t k,
                       int dtype, cudaStream_t s) {
  if (int rc = check_indices<I>("gather", indices, k, n, s)) return rc;
  const int64_t row_bytes = f * itemsize_of(dtype);
  if (k == 0 || f == 0) return FB200_OK;
  const I* ip = static_cast<const I*>(indices);
  if (row_bytes % 16 == 0 && aligned16(x) && aligned16(out)) {
    const int64_t rv = row_bytes / 16;
    gather_rows_kernel<uint4, I><<<grid_for(k * rv, 256, 8), 256, 0, s>>>(
        static_cast<const uint4*>(x), ip, static_cast<uint4*>(out), k, rv);
  } else if (itemsize_of(dtype) == 4) {
    gather_rows_kernel<uint32_t, I><<<grid_for(k * f, 256, 8), 256, 0, s>>>(
        static_cast<const uint32_t*>(x), ip, static_cast<uint32_t*>(out), k, f);
  } else if (itemsize_of(dtype) == 2) {
    gather_rows_kernel<uint16_t, I><<<grid_for(k * f, 256, 8), 256, 0, s>>>(
        static_cast<const uint16_t*>(x), ip, static_cast<uint16_t*>(out), k, f);
  } else if (itemsize_of(dtype) == 8) {
    gather_rows_kernel<uint64_t, I><<<grid_for(k * f, 256, 8), 256, 0, s>>>(
        static_cast<const uint64_t*>(x), ip, static_cast<uint64_t*>(out), k, f);
  } else {
    gather_rows_kernel<uint8_t, I><<<grid_for(k * f, 256, 8), 256, 0, s>>>(
        static_cast<const uint8_t*>(x), ip, static_cast<uint8_t*>(out), k, f);
  }
  return after_launch("gather_rows_kernel");
}

template <typename T, typename I>
static int scatter_impl(const void* updates, const void* indices, void* out, int64_t k, int64_t f,
                        int64_t v, cudaStream_t s) {
  if (int rc = check_indices<I>("scatter_add", indices, k, v, s)) return rc;
  const int64_t n_out = v * f;
  if (n_out == 0) return FB200_OK;
  float* acc = nullptr;
  const bool direct = sizeof(T) == 4;
  if (direct) {
    acc = static_cast<float*>(out);
  } else {
    FB200_CUDA_OK(scratch_alloc_async(reinterpret_cast<void**>(&acc), static_cast<size_t>(n_out) * 4, s));
  }
  FB200_CUDA_OK(cudaMemsetAsync(acc, 0, static_cast<size_t>(n_out) * 4, s));
  int rc = FB200_OK;
  if (k * f > 0) {
    scatter_add_kernel<T, I><<<grid_for(k * f, 256, 8), 256, 0, s>>>(
        static_cast<const T*>(updates), static_cast<const I*>(indices), acc, k, f);
    rc = after_launch("scatter_add_kernel");
  }
  if (!direct) {
    if (rc == FB200_OK) {
      round_from_f32_kernel<T><<<grid_for(n_out, 256, 8), 256, 0, s>>>(acc, static_cast<T*>(out), n_out);
      rc = after_launch("round_from_f32_kernel");
    }
    cudaFreeAsync(acc, s);
  }
  return rc;
}

}  // namespace fb200

using namespace fb200;

extern "C" int fb200_gather(const void* x, const void* indices, void* out, int64_t n, int64_t f,
                            int64_t k, int dtype, int index_dtype, fb200_stream stream) {
  if (n < 0 || f < 0 || k < 0) return set_error(FB200_INVALID_ARGUMENT, "gather: negative shape");
  if (itemsize_of(dtype) == 0) return set_error(FB200_INVALID_ARGUMENT, "gather: unknown dtype code %d", dtype);
  if (index_dtype != FB200_I32 && index_dtype != FB200_I64) {
    return set_error(FB200_INVALID_ARGUMENT, "gather: indices must be int32 or int64, got dtype code %d", index_dtype);
  }
  if (k > 0 && (indices == nullptr || (f > 0 && (x == nullptr || out == nullptr)))) {
    return set_error(FB200_INVALID_ARGUMENT, "gather: null argument");
  }
  cudaStream_t s = as_stream(stream);
  return index_dtype == FB200_I32 ? gather_impl<int32_t>(x, indices, out, n, f, k, dtype, s)
                                  : gather_impl<int64_t>(x, indices, out, n, f, k, dtype, s);
}

extern "C" int fb200_scatter_add(const void* updates, const void* indices, void* out, int64_t k,
                                 int64_t f, int64_t v, int dtype, int index_dtype,
                                 fb200_stream stream) {
  if (k < 0 || f < 0 || v < 0) return set_error(FB200_INVALID_ARGUMENT, "scatter_add: negative shape");
  if (index_dtype != FB200_I32 && index_dtype != FB200_I64) {
    return set_error(FB200_INVALID_ARGUMENT, "scatter_add: indices must be int32 or int64, got dtype code %d", index_dtype);
  }
  if ((v * f > 0 && out == nullptr) || (k > 0 && indices == nullptr) || (k * f > 0 && updates == nullptr)) {
    return set_error(FB200_INVALID_ARGUMENT, "scatter_add: null argument");
  }
  cudaStream_t s = as_stream(stream);
  const bool i32 = index_dtype == FB200_I32;
  switch (dtype) {
    case FB200_F32:
      return i32 ? scatter_impl<float, int32_t>(updates, indices, out, k, f, v, s)
                 : scatter_impl<float, int64_t>(updates, indices, out, k, f, v, s);
    case FB200_BF16:
      return i32 ? scatter_impl<__nv_bfloat16, int32_t>(updates, indices, out, k, f, v, s)
                 : scatter_impl<__nv_bfloat16, int64_t>(updates, indices, out, k, f, v, s);
    case FB200_F16:
      return i32 ? scatter_impl<__half, int32_t>(updates, indices, out, k, f, v, s)
                 : scatter_impl<__half, int64_t>(updates, indices, out, k, f, v, s);
    default:
      return set_error(FB200_INVALID_ARGUMENT, "scatter_add: dtype code %d is not float32/float16/bfloat16", dtype);
  }
}
