// Row kernels: softmax and layer_norm over the last axis of a rank-2 tensor.
//
// softmax follows src/backends/cpu/kernels/sequence.cpp:114-174 (max, exp(x-max), sum, divide)
// and replaces the cudnnSoftmaxForward call of src/backends/cuda/kernels/sequence.cpp:108-174.
// layer_norm follows sequence.cpp:182-279 (mean, then centred sum of squares, biased variance,
// r = 1/sqrt(var+eps), out = g*((x-mean)*r)+b) and replaces the three-pass shared-memory-tree
// kernel of src/backends/cuda/kernels/sequence.cu:104-155.
//
// One warp owns one row.  The row is read from HBM once with 128-bit loads and stays in
// registers; max / sum / mean / variance are warp-shuffle reductions in fp32; the result is
// written once with 128-bit stores.  HBM-bound: algorithmic bytes = 2 * rows * cols * itemsize
// (+ gamma/beta, which stay in L2).  Rows whose length or alignment does not allow 128-bit
// access use a scalar three-pass variant of the same arithmetic.
//
// Compiled with -fmad=false so that g*xhat+b rounds as the CPU reference does.
#include "common.cuh"

namespace fb200 {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

constexpr int kRowThreads = 256;                 // 8 warps = 8 rows per CTA
constexpr int kRowsPerCta = kRowThreads / 32;

// NV = 16-byte vectors per lane (compile-time so the row lives in registers).
template <typename T, int NV>
__global__ void __launch_bounds__(kRowThreads)
softmax_vec_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t rows, int64_t cols) {
  constexpr int W = 16 / sizeof(T);
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int64_t n_vec = cols / W;
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * kRowsPerCta + warp; row < rows;
       row += static_cast<int64_t>(gridDim.x) * kRowsPerCta) {
    const T* xr = x + row * cols;
    T* orow = out + row * cols;
    float v[NV][W];
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int64_t vi = lane + 32 * i;
      if (vi < n_vec) {
        load_vec<T>(xr + vi * W, v[i]);
#pragma unroll
        for (int e = 0; e < W; ++e) m = fmaxf(m, v[i][e]);
      }
    }
    m = warp_max(m);
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int64_t vi = lane + 32 * i;
      if (vi < n_vec) {
#pragma unroll
        for (int e = 0; e < W; ++e) {
          v[i][e] = expf(v[i][e] - m);
          s += v[i][e];
        }
      }
    }
    s = warp_sum(s);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int64_t vi = lane + 32 * i;
      if (vi < n_vec) {
#pragma unroll
        for (int e = 0; e < W; ++e) v[i][e] = v[i][e] / s;
        store_vec<T>(orow + vi * W, v[i]);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads)
softmax_scalar_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t rows, int64_t cols) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * kRowsPerCta + warp; row < rows;
       row += static_cast<int64_t>(gridDim.x) * kRowsPerCta) {
    const T* xr = x + row * cols;
    T* orow = out + row * cols;
    float m = -INFINITY;
    for (int64_t j = lane; j < cols; j += 32) m = fmaxf(m, to_f32(xr[j]));
    m = warp_max(m);
    float s = 0.0f;
    for (int64_t j = lane; j < cols; j += 32) s += expf(to_f32(xr[j]) - m);
    s = warp_sum(s);
    for (int64_t j = lane; j < cols; j += 32) orow[j] = from_f32<T>(expf(to_f32(xr[j]) - m) / s);
  }
}

template <typename T, int NV>
__global__ void __launch_bounds__(kRowThreads)
layer_norm_vec_kernel(const T* __restrict__ x, const T* __restrict__ res, const T* __restrict__ gamma,
                      const T* __restrict__ beta, T* __restrict__ sum_out, T* __restrict__ out, int64_t rows,
                      int64_t cols, float eps) {
  constexpr int W = 16 / sizeof(T);
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int64_t n_vec = cols / W;
  const float inv_d_den = static_cast<float>(cols);
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * kRowsPerCta + warp; row < rows;
       row += static_cast<int64_t>(gridDim.x) * kRowsPerCta) {
    const T* xr = x + row * cols;
    T* orow = out + row * cols;
    float v[NV][W];
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int64_t vi = lane + 32 * i;
      if (vi < n_vec) {
        load_vec<T>(xr + vi * W, v[i]);
        if (res != nullptr) {
          // the residual add in front of the normalisation: x + res rounded to T as the separate
          // `add` would store it, written out for the graph's other readers, normalised from registers
          float rv[W];
          load_vec<T>(res + row * cols + vi * W, rv);
#pragma unroll
          for (int e = 0; e < W; ++e) v[i][e] = round_through<T>(v[i][e] + rv[e]);
          store_vec<T>(sum_out + row * cols + vi * W, v[i]);
        }
#pragma unroll
        for (int e = 0; e < W; ++e) s += v[i][e];
      }
    }
    const float mean = warp_sum(s) / inv_d_den;
    float q = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int64_t vi = lane + 32 * i;
      if (vi < n_vec) {
#pragma unroll
        for (int e = 0; e < W; ++e) {
          const float c = v[i][e] - mean;
          q += c * c;
        }
      }
    }
    const float var = warp_sum(q) / inv_d_den;
    const float r = 1.0f / sqrtf(var + eps);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int64_t vi = lane + 32 * i;
      if (vi < n_vec) {
        float g[W], b[W];
        load_vec<T>(gamma + vi * W, g);
        load_vec<T>(beta + vi * W, b);
#pragma unroll
        for (int e = 0; e < W; ++e) {
          const float xhat = (v[i][e] - mean) * r;
          v[i][e] = g[e] * xhat + b[e];
        }
        store_vec<T>(orow + vi * W, v[i]);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads)
layer_norm_scalar_kernel(const T* __restrict__ x, const T* __restrict__ gamma,
                         const T* __restrict__ beta, T* __restrict__ out, int64_t rows,
                         int64_t cols, float eps) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const float den = static_cast<float>(cols);
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * kRowsPerCta + warp; row < rows;
       row += static_cast<int64_t>(gridDim.x) * kRowsPerCta) {
    const T* xr = x + row * cols;
    T* orow = out + row * cols;
    float s = 0.0f;
    for (int64_t j = lane; j < cols; j += 32) s += to_f32(xr[j]);
    const float mean = warp_sum(s) / den;
    float q = 0.0f;
    for (int64_t j = lane; j < cols; j += 32) {
      const float c = to_f32(xr[j]) - mean;
      q += c * c;
    }
    const float var = warp_sum(q) / den;
    const float r = 1.0f / sqrtf(var + eps);
    for (int64_t j = lane; j < cols; j += 32) {
      const float xhat = (to_f32(xr[j]) - mean) * r;
      orow[j] = from_f32<T>(to_f32(gamma[j]) * xhat + to_f32(beta[j]));
    }
  }
}

// Smallest NV in {1,2,4,8,16} with 32*NV*W >= cols, or 0 when the row does not fit in registers.
template <typename T> static int pick_nv(int64_t cols) {
  constexpr int W = 16 / sizeof(T);
  for (int nv = 1; nv <= 16; nv *= 2) {
    if (static_cast<int64_t>(32) * nv * W >= cols) return nv;
  }
  return 0;
}

template <typename T>
static int launch_softmax(const void* x, void* out, int64_t rows, int64_t cols, cudaStream_t s) {
  constexpr int W = 16 / sizeof(T);
  const T* xp = static_cast<const T*>(x);
  T* op = static_cast<T*>(out);
  const int grid = grid_for(rows * 32, kRowThreads, 8);
  const int nv = (cols % W == 0 && aligned16(x) && aligned16(out)) ? pick_nv<T>(cols) : 0;
  switch (nv) {
    case 1: softmax_vec_kernel<T, 1><<<grid, kRowThreads, 0, s>>>(xp, op, rows, cols); break;
    case 2: softmax_vec_kernel<T, 2><<<grid, kRowThreads, 0, s>>>(xp, op, rows, cols); break;
    case 4: softmax_vec_kernel<T, 4><<<grid, kRowThreads, 0, s>>>(xp, op, rows, cols); break;
    case 8: softmax_vec_kernel<T, 8><<<grid, kRowThreads, 0, s>>>(xp, op, rows, cols); break;
    case 16: softmax_vec_kernel<T, 16><<<grid, kRowThreads, 0, s>>>(xp, op, rows, cols); break;
    default: softmax_scalar_kernel<T><<<grid, kRowThreads, 0, s>>>(xp, op, rows, cols); break;
  }
  return after_launch("softmax_kernel");
}

template <typename T>
static int launch_layer_norm(const void* x, const void* gamma, const void* beta, void* out,
                             int64_t rows, int64_t cols, float eps, cudaStream_t s,
                             const void* res = nullptr, void* sum_out = nullptr) {
  constexpr int W = 16 / sizeof(T);
  const T* xp = static_cast<const T*>(x);
  const T* rp = static_cast<const T*>(res);
  T* sp = static_cast<T*>(sum_out);
  const T* gp = static_cast<const T*>(gamma);
  const T* bp = static_cast<const T*>(beta);
  T* op = static_cast<T*>(out);
  const int grid = grid_for(rows * 32, kRowThreads, 8);
  const bool al = aligned16(x) && aligned16(out) && aligned16(gamma) && aligned16(beta) &&
                  (res == nullptr || (aligned16(res) && aligned16(sum_out)));
  const int nv = (cols % W == 0 && al) ? pick_nv<T>(cols) : 0;
  if (res != nullptr && nv == 0) return FB200_UNIMPLEMENTED;   // the caller runs the two operators
  switch (nv) {
    case 1: layer_norm_vec_kernel<T, 1><<<grid, kRowThreads, 0, s>>>(xp, rp, gp, bp, sp, op, rows, cols, eps); break;
    case 2: layer_norm_vec_kernel<T, 2><<<grid, kRowThreads, 0, s>>>(xp, rp, gp, bp, sp, op, rows, cols, eps); break;
    case 4: layer_norm_vec_kernel<T, 4><<<grid, kRowThreads, 0, s>>>(xp, rp, gp, bp, sp, op, rows, cols, eps); break;
    case 8: layer_norm_vec_kernel<T, 8><<<grid, kRowThreads, 0, s>>>(xp, rp, gp, bp, sp, op, rows, cols, eps); break;
    case 16: layer_norm_vec_kernel<T, 16><<<grid, kRowThreads, 0, s>>>(xp, rp, gp, bp, sp, op, rows, cols, eps); break;
    default: layer_norm_scalar_kernel<T><<<grid, kRowThreads, 0, s>>>(xp, gp, bp, op, rows, cols, eps); break;
  }
  return after_launch("layer_norm_kernel");
}

}  // namespace fb200

using namespace fb200;

extern "C" int fb200_softmax(const void* x, void* out, int64_t rows, int64_t cols, int dtype,
                             fb200_stream stream) {
  if (rows < 0 || cols < 0) return set_error(FB200_INVALID_ARGUMENT, "softmax: negative shape");
  if (rows == 0 || cols == 0) return FB200_OK;
  if (x == nullptr || out == nullptr) return set_error(FB200_INVALID_ARGUMENT, "softmax: null argument");
  cudaStream_t s = as_stream(stream);
  switch (dtype) {
    case FB200_F32: return launch_softmax<float>(x, out, rows, cols, s);
    case FB200_BF16: return launch_softmax<__nv_bfloat16>(x, out, rows, cols, s);
    case FB200_F16: return launch_softmax<__half>(x, out, rows, cols, s);
    default:
      return set_error(FB200_INVALID_ARGUMENT,
                       "softmax: dtype code %d is not float32/float16/bfloat16", dtype);
  }
}

// layer_norm(x + res): the residual add of a transformer block and the normalisation behind it in one
// pass.  sum_out receives x + res (rounded to the dtype, exactly what a separate add stores), out
// the normalised rows.  Rows that cannot take the vector path run as the two operators.
extern "C" int fb200_add_layer_norm(const void* x, const void* res, const void* gamma, const void* beta,
                                    void* sum_out, void* out, int64_t rows, int64_t cols, double eps,
                                    int dtype, fb200_stream stream) {
  if (rows < 0 || cols < 0) return set_error(FB200_INVALID_ARGUMENT, "add_layer_norm: negative shape");
  if (rows == 0 || cols == 0) return FB200_OK;
  if (!x || !res || !gamma || !beta || !sum_out || !out) return set_error(FB200_INVALID_ARGUMENT, "add_layer_norm: null argument");
  cudaStream_t s = as_stream(stream);
  const float e = static_cast<float>(eps);
  int rc = FB200_UNIMPLEMENTED;
  switch (dtype) {
    case FB200_F32: rc = launch_layer_norm<float>(x, gamma, beta, out, rows, cols, e, s, res, sum_out); break;
    case FB200_BF16: rc = launch_layer_norm<__nv_bfloat16>(x, gamma, beta, out, rows, cols, e, s, res, sum_out); break;
    case FB200_F16: rc = launch_layer_norm<__half>(x, gamma, beta, out, rows, cols, e, s, res, sum_out); break;
    default:
      return set_error(FB200_INVALID_ARGUMENT, "add_layer_norm: dtype code %d is not float32/float16/bfloat16", dtype);
  }
  if (rc != FB200_UNIMPLEMENTED) return rc;
  const void* ins[2] = {x, res};
  const int ops[1] = {FB200_EW_ADD};
  const int arity[1] = {2};
  if (int rc2 = fb200_fused_elementwise(ins, 2, sum_out, rows * cols, dtype, ops, arity, 1, stream)) return rc2;
  return fb200_layer_norm(sum_out, gamma, beta, out, rows, cols, eps, dtype, stream);
}

extern "C" int fb200_layer_norm(const void* x, const void* gamma, const void* beta, void* out,
                                int64_t rows, int64_t cols, double eps, int dtype,
                                fb200_stream stream) {
  if (rows < 0 || cols < 0) return set_error(FB200_INVALID_ARGUMENT, "layer_norm: negative shape");
  if (rows == 0 || cols == 0) return FB200_OK;
  if (x == nullptr || gamma == nullptr || beta == nullptr || out == nullptr) {
    return set_error(FB200_INVALID_ARGUMENT, "layer_norm: null argument");
  }
  cudaStream_t s = as_stream(stream);
  const float e = static_cast<float>(eps);
  switch (dtype) {
    case FB200_F32: return launch_layer_norm<float>(x, gamma, beta, out, rows, cols, e, s);
    case FB200_BF16: return launch_layer_norm<__nv_bfloat16>(x, gamma, beta, out, rows, cols, e, s);
    case FB200_F16: return launch_layer_norm<__half>(x, gamma, beta, out, rows, cols, e, s);
    default:
      return set_error(FB200_INVALID_ARGUMENT,
                       "layer_norm: dtype code %d is not float32/float16/bfloat16", dtype);
  }
}
