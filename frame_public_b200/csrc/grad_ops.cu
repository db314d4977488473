// Gradient-side internals of pooling and convolution: max_pool2d_select_internal,
// max_pool2d_grad_internal, avg_pool2d_grad_internal, conv2d_grad_input_internal,
// conv2d_grad_filter_internal.
//
// Semantics: src/backends/cpu/kernels/pool.cpp:356-389 (max-pool gradient), :459-483 (select),
// :542-568 (avg-pool gradient) and src/backends/cpu/kernels/conv.cpp:321-353 (BackwardData),
// :424-453 (BackwardFilter).  They replace cudnnPoolingBackward / cudnnConvolutionBackwardData /
// cudnnConvolutionBackwardFilter and the hand-written kernels of src/backends/cuda/kernels/pool.cpp
// and conv.cpp.
//
// Every kernel here is written as a GATHER over its output (one thread per output element, no
// atomics) and performs the CPU reference's fp32 operations in the CPU's order; this file is
// compiled without fused multiply-add, so fp32 results are bit-identical to the reference and 16-bit
// results are the same fp32 sums rounded once.
//   * max-pool gradient: the reference scatters dy into the window's argmax, windows visited in
//     (oh, ow) order.  Seen from an input position the same additions happen, in the same order, when
//     the thread walks the windows that contain it in (oh, ow) order and adds dy where that window's
//     argmax (first maximum, strict >) is the position itself.
//   * conv BackwardFilter is one long dot product per filter element (N*OH*OW terms in (n, oh, ow)
//     order); a thread owns one filter element, a warp's lanes are neighbouring kw/kh/ci, so their
//     loads fall into the same lines.
// Bound: CUDA cores (strict order); these are training-side ops off the inference path.
#include "common.cuh"

namespace fb200 {

struct PoolGeom {
  int64_t nc, h, w, oh, ow;
  int kh, kw, sh, sw, ph, pw;
};

// First maximum of the window (oh, ow) of plane xc, in (kh, kw) order with strict >; -1 if the
// window holds no valid position (cannot happen when 2*pad <= kernel).
template <typename T>
__device__ __forceinline__ int64_t window_argmax(const T* __restrict__ xc, const PoolGeom& g, int64_t o, int64_t q) {
  bool found = false;
  float best = 0.0f;
  int64_t arg = -1;
  for (int a = 0; a < g.kh; ++a) {
    const int64_t ih = o * g.sh - g.ph + a;
    if (ih < 0 || ih >= g.h) continue;
    for (int b = 0; b < g.kw; ++b) {
      const int64_t iw = q * g.sw - g.pw + b;
      if (iw < 0 || iw >= g.w) continue;
      const float v = to_f32(xc[ih * g.w + iw]);
      if (!found || v > best) {
        found = true;
        best = v;
        arg = ih * g.w + iw;
      }
    }
  }
  return arg;
}

template <typename T>
__global__ void __launch_bounds__(256)
max_pool2d_select_kernel(const T* __restrict__ gsrc, const T* __restrict__ x, T* __restrict__ out, PoolGeom g) {
  const int64_t total = g.nc * g.oh * g.ow;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t q = i % g.ow;
    int64_t rem = i / g.ow;
    const int64_t o = rem % g.oh;
    rem /= g.oh;
    const int64_t arg = window_argmax(x + rem * g.h * g.w, g, o, q);
    out[i] = arg >= 0 ? gsrc[rem * g.h * g.w + arg] : from_f32<T>(0.0f);
  }
}

// Smallest o with o*s - p + (k-1) >= i, and largest o with o*s - p <= i, clipped to [0, n_out).
__device__ __forceinline__ void covering_range(int64_t i, int k, int s, int p, int64_t n_out, int64_t* lo, int64_t* hi) {
  const int64_t a = i + p - (k - 1);
  int64_t l = a <= 0 ? 0 : (a + s - 1) / s;
  int64_t h = (i + p) / s;
  if (h > n_out - 1) h = n_out - 1;
  *lo = l;
  *hi = h;
}

template <typename T>
__global__ void __launch_bounds__(256)
max_pool2d_grad_kernel(const T* __restrict__ dy, const T* __restrict__ x, T* __restrict__ dx, PoolGeom g) {
  const int64_t total = g.nc * g.h * g.w;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t iw = i % g.w;
    int64_t rem = i / g.w;
    const int64_t ih = rem % g.h;
    rem /= g.h;
    const T* xc = x + rem * g.h * g.w;
    const T* dyc = dy + rem * g.oh * g.ow;
    int64_t o_lo, o_hi, q_lo, q_hi;
    covering_range(ih, g.kh, g.sh, g.ph, g.oh, &o_lo, &o_hi);
    covering_range(iw, g.kw, g.sw, g.pw, g.ow, &q_lo, &q_hi);
    const int64_t me = ih * g.w + iw;
    float acc = 0.0f;
    for (int64_t o = o_lo; o <= o_hi; ++o) {
      for (int64_t q = q_lo; q <= q_hi; ++q) {
        if (window_argmax(xc, g, o, q) == me) acc += to_f32(dyc[o * g.ow + q]);
      }
    }
    dx[i] = from_f32<T>(acc);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
avg_pool2d_grad_kernel(const T* __restrict__ dy, T* __restrict__ dx, PoolGeom g) {
  const int64_t total = g.nc * g.h * g.w;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const float denom = static_cast<float>(g.kh * g.kw);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t iw = i % g.w;
    int64_t rem = i / g.w;
    const int64_t ih = rem % g.h;
    rem /= g.h;
    const T* dyc = dy + rem * g.oh * g.ow;
    float acc = 0.0f;
    // the reference's order: kh ascending (output row descending), kw ascending
    for (int a = 0; a < g.kh; ++a) {
      const int64_t num_h = ih + g.ph - a;
      if (num_h % g.sh != 0) continue;
      const int64_t o = num_h / g.sh;
      if (o < 0 || o >= g.oh) continue;
      for (int b = 0; b < g.kw; ++b) {
        const int64_t num_w = iw + g.pw - b;
        if (num_w % g.sw != 0) continue;
        const int64_t q = num_w / g.sw;
        if (q < 0 || q >= g.ow) continue;
        acc += to_f32(dyc[o * g.ow + q]);
      }
    }
    dx[i] = from_f32<T>(acc / denom);
  }
}

struct ConvGeom {
  int64_t n, cin, h, w, cout, oh, ow;
  int kh, kw, sh, sw, ph, pw, groups;
  int64_t cin_pg, cout_pg;
};

template <typename T>
__global__ void __launch_bounds__(256)
conv2d_grad_input_kernel(const T* __restrict__ dy, const T* __restrict__ wt, T* __restrict__ dx, ConvGeom g) {
  const int64_t total = g.n * g.cin * g.h * g.w;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t iw = i % g.w;
    int64_t rem = i / g.w;
    const int64_t ih = rem % g.h;
    rem /= g.h;
    const int64_t ci_full = rem % g.cin;
    const int64_t n = rem / g.cin;
    const int64_t grp = ci_full / g.cin_pg;
    const int64_t ci = ci_full - grp * g.cin_pg;
    float acc = 0.0f;
    for (int64_t co = grp * g.cout_pg; co < (grp + 1) * g.cout_pg; ++co) {
      const T* dyc = dy + (n * g.cout + co) * g.oh * g.ow;
      const T* wc = wt + (co * g.cin_pg + ci) * g.kh * g.kw;
      for (int a = 0; a < g.kh; ++a) {
        const int64_t num_h = ih + g.ph - a;
        if (num_h % g.sh != 0) continue;
        const int64_t o = num_h / g.sh;
        if (o < 0 || o >= g.oh) continue;
        for (int b = 0; b < g.kw; ++b) {
          const int64_t num_w = iw + g.pw - b;
          if (num_w % g.sw != 0) continue;
          const int64_t q = num_w / g.sw;
          if (q < 0 || q >= g.ow) continue;
          acc += to_f32(dyc[o * g.ow + q]) * to_f32(wc[a * g.kw + b]);
        }
      }
    }
    dx[i] = from_f32<T>(acc);
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
conv2d_grad_filter_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ dw, ConvGeom g) {
  const int64_t total = g.cout * g.cin_pg * g.kh * g.kw;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int b = static_cast<int>(i % g.kw);
  int64_t rem = i / g.kw;
  const int a = static_cast<int>(rem % g.kh);
  rem /= g.kh;
  const int64_t ci = rem % g.cin_pg;
  const int64_t co = rem / g.cin_pg;
  const int64_t grp = co / g.cout_pg;
  const int64_t ci_full = grp * g.cin_pg + ci;
  float acc = 0.0f;
  for (int64_t n = 0; n < g.n; ++n) {
    const T* xc = x + (n * g.cin + ci_full) * g.h * g.w;
    const T* dyc = dy + (n * g.cout + co) * g.oh * g.ow;
    for (int64_t o = 0; o < g.oh; ++o) {
      const int64_t ih = o * g.sh - g.ph + a;
      if (ih < 0 || ih >= g.h) continue;
      for (int64_t q = 0; q < g.ow; ++q) {
        const int64_t iw = q * g.sw - g.pw + b;
        if (iw < 0 || iw >= g.w) continue;
        acc += to_f32(xc[ih * g.w + iw]) * to_f32(dyc[o * g.ow + q]);
      }
    }
  }
  dw[i] = from_f32<T>(acc);
}

static int pool_geom(const char* op, int64_t n, int64_t c, int64_t h, int64_t w, int64_t kh, int64_t kw,
                     int64_t sh, int64_t sw, int64_t ph, int64_t pw, PoolGeom* g) {
  if (n < 0 || c < 0 || h < 1 || w < 1 || kh < 1 || kw < 1 || sh < 1 || sw < 1 || ph < 0 || pw < 0) {
    return set_error(FB200_INVALID_ARGUMENT, "%s: invalid geometry", op);
  }
  if (2 * ph > kh || 2 * pw > kw) return set_error(FB200_INVALID_ARGUMENT, "%s: padding*2 must not exceed kernel", op);
  if (h + 2 * ph < kh || w + 2 * pw < kw) return set_error(FB200_INVALID_ARGUMENT, "%s: non-positive output size", op);
  g->nc = n * c; g->h = h; g->w = w;
  g->oh = (h + 2 * ph - kh) / sh + 1;
  g->ow = (w + 2 * pw - kw) / sw + 1;
  g->kh = static_cast<int>(kh); g->kw = static_cast<int>(kw);
  g->sh = static_cast<int>(sh); g->sw = static_cast<int>(sw);
  g->ph = static_cast<int>(ph); g->pw = static_cast<int>(pw);
  return FB200_OK;
}

static int conv_geom(const char* op, const fb200_conv2d_params* p, ConvGeom* g) {
  if (p == nullptr) return set_error(FB200_INVALID_ARGUMENT, "%s: null params", op);
  if (p->n < 0 || p->cin < 1 || p->h < 1 || p->w < 1 || p->cout < 1 || p->kh < 1 || p->kw < 1 ||
      p->stride_h < 1 || p->stride_w < 1 || p->pad_h < 0 || p->pad_w < 0 || p->groups < 1) {
    return set_error(FB200_INVALID_ARGUMENT, "%s: invalid geometry", op);
  }
  if (p->cin % p->groups != 0 || p->cout % p->groups != 0) {
    return set_error(FB200_INVALID_ARGUMENT, "%s: channels must be divisible by groups", op);
  }
  if (p->h + 2 * p->pad_h < p->kh || p->w + 2 * p->pad_w < p->kw) {
    return set_error(FB200_INVALID_ARGUMENT, "%s: non-positive output size", op);
  }
  g->n = p->n; g->cin = p->cin; g->h = p->h; g->w = p->w; g->cout = p->cout;
  g->oh = (p->h + 2 * p->pad_h - p->kh) / p->stride_h + 1;
  g->ow = (p->w + 2 * p->pad_w - p->kw) / p->stride_w + 1;
  g->kh = static_cast<int>(p->kh); g->kw = static_cast<int>(p->kw);
  g->sh = static_cast<int>(p->stride_h); g->sw = static_cast<int>(p->stride_w);
  g->ph = static_cast<int>(p->pad_h); g->pw = static_cast<int>(p->pad_w);
  g->groups = static_cast<int>(p->groups);
  g->cin_pg = p->cin / p->groups;
  g->cout_pg = p->cout / p->groups;
  return FB200_OK;
}

}  // namespace fb200

using namespace fb200;

#define FB200_FLOAT_DISPATCH(op_name, dtype, run)                                                              \
  switch (dtype) {                                                                                             \
    case FB200_F32: run(float{}); break;                                                                       \
    case FB200_BF16: run(__nv_bfloat16{}); break;                                                              \
    case FB200_F16: run(__half{}); break;                                                                      \
    default:                                                                                                   \
      return set_error(FB200_INVALID_ARGUMENT, op_name ": dtype code %d is not float32/float16/bfloat16", dtype); \
  }

extern "C" int fb200_max_pool2d_select(const void* g, const void* x, void* out, int64_t n, int64_t c, int64_t h,
                                       int64_t w, int64_t kh, int64_t kw, int64_t stride_h, int64_t stride_w,
                                       int64_t pad_h, int64_t pad_w, int dtype, fb200_stream stream) {
  PoolGeom pg{};
  if (int rc = pool_geom("max_pool2d_select_internal", n, c, h, w, kh, kw, stride_h, stride_w, pad_h, pad_w, &pg)) return rc;
  if (pg.nc == 0) return FB200_OK;
  if (g == nullptr || x == nullptr || out == nullptr) {
    return set_error(FB200_INVALID_ARGUMENT, "max_pool2d_select_internal: null argument");
  }
  cudaStream_t s = as_stream(stream);
  const int grid = grid_for(pg.nc * pg.oh * pg.ow, 256, 8);
  auto run = [&](auto tag) {
    using T = decltype(tag);
    max_pool2d_select_kernel<T><<<grid, 256, 0, s>>>(static_cast<const T*>(g), static_cast<const T*>(x),
                                                     static_cast<T*>(out), pg);
  };
  FB200_FLOAT_DISPATCH("max_pool2d_select_internal", dtype, run)
  return after_launch("max_pool2d_select_kernel");
}

extern "C" int fb200_max_pool2d_grad(const void* dy, const void* x, void* dx, int64_t n, int64_t c, int64_t h,
                                     int64_t w, int64_t kh, int64_t kw, int64_t stride_h, int64_t stride_w,
                                     int64_t pad_h, int64_t pad_w, int dtype, fb200_stream stream) {
  PoolGeom pg{};
  if (int rc = pool_geom("max_pool2d_grad_internal", n, c, h, w, kh, kw, stride_h, stride_w, pad_h, pad_w, &pg)) return rc;
  if (pg.nc == 0) return FB200_OK;
  if (dy == nullptr || x == nullptr || dx == nullptr) {
    return set_error(FB200_INVALID_ARGUMENT, "max_pool2d_grad_internal: null argument");
  }
  cudaStream_t s = as_stream(stream);
  const int grid = grid_for(pg.nc * pg.h * pg.w, 256, 8);
  auto run = [&](auto tag) {
    using T = decltype(tag);
    max_pool2d_grad_kernel<T><<<grid, 256, 0, s>>>(static_cast<const T*>(dy), static_cast<const T*>(x),
                                                   static_cast<T*>(dx), pg);
  };
  FB200_FLOAT_DISPATCH("max_pool2d_grad_internal", dtype, run)
  return after_launch("max_pool2d_grad_kernel");
}

extern "C" int fb200_avg_pool2d_grad(const void* dy, void* dx, int64_t n, int64_t c, int64_t h, int64_t w,
                                     int64_t kh, int64_t kw, int64_t stride_h, int64_t stride_w, int64_t pad_h,
                                     int64_t pad_w, int dtype, fb200_stream stream) {
  PoolGeom pg{};
  if (int rc = pool_geom("avg_pool2d_grad_internal", n, c, h, w, kh, kw, stride_h, stride_w, pad_h, pad_w, &pg)) return rc;
  if (pg.nc == 0) return FB200_OK;
  if (dy == nullptr || dx == nullptr) return set_error(FB200_INVALID_ARGUMENT, "avg_pool2d_grad_internal: null argument");
  cudaStream_t s = as_stream(stream);
  const int grid = grid_for(pg.nc * pg.h * pg.w, 256, 8);
  auto run = [&](auto tag) {
    using T = decltype(tag);
    avg_pool2d_grad_kernel<T><<<grid, 256, 0, s>>>(static_cast<const T*>(dy), static_cast<T*>(dx), pg);
  };
  FB200_FLOAT_DISPATCH("avg_pool2d_grad_internal", dtype, run)
  return after_launch("avg_pool2d_grad_kernel");
}

extern "C" int fb200_conv2d_grad_input(const void* dy, const void* w, void* dx, const fb200_conv2d_params* p,
                                       int dtype, fb200_stream stream) {
  ConvGeom g{};
  if (int rc = conv_geom("conv2d_grad_input_internal", p, &g)) return rc;
  if (g.n == 0) return FB200_OK;
  if (dy == nullptr || w == nullptr || dx == nullptr) {
    return set_error(FB200_INVALID_ARGUMENT, "conv2d_grad_input_internal: null argument");
  }
  cudaStream_t s = as_stream(stream);
  const int grid = grid_for(g.n * g.cin * g.h * g.w, 256, 4);
  auto run = [&](auto tag) {
    using T = decltype(tag);
    conv2d_grad_input_kernel<T><<<grid, 256, 0, s>>>(static_cast<const T*>(dy), static_cast<const T*>(w),
                                                     static_cast<T*>(dx), g);
  };
  FB200_FLOAT_DISPATCH("conv2d_grad_input_internal", dtype, run)
  return after_launch("conv2d_grad_input_kernel");
}

extern "C" int fb200_conv2d_grad_filter(const void* x, const void* dy, void* dw, const fb200_conv2d_params* p,
                                        int dtype, fb200_stream stream) {
  ConvGeom g{};
  if (int rc = conv_geom("conv2d_grad_filter_internal", p, &g)) return rc;
  if (dw == nullptr || (g.n > 0 && (x == nullptr || dy == nullptr))) {
    return set_error(FB200_INVALID_ARGUMENT, "conv2d_grad_filter_internal: null argument");
  }
  cudaStream_t s = as_stream(stream);
  const int64_t total = g.cout * g.cin_pg * g.kh * g.kw;
  const int64_t blocks = (total + 127) / 128;
  if (blocks > 0x7fffffff) return set_error(FB200_INVALID_ARGUMENT, "conv2d_grad_filter_internal: filter too large");
  auto run = [&](auto tag) {
    using T = decltype(tag);
    conv2d_grad_filter_kernel<T><<<static_cast<int>(blocks), 128, 0, s>>>(
        static_cast<const T*>(x), static_cast<const T*>(dy), static_cast<T*>(dw), g);
  };
  FB200_FLOAT_DISPATCH("conv2d_grad_filter_internal", dtype, run)
  return after_launch("conv2d_grad_filter_kernel");
}

// ---- mse_loss / mse_loss_grad_internal -----------------------------------------------------------
// mse_loss(pred, target) = mean((pred - target)^2), a scalar: the CPU reference adds the squares
// one after the other in fp32 and divides by the element count
// (src/backends/cpu/kernels/loss.cpp:108-150).  Up to kMseSerialMax elements one thread repeats exactly
// that (bit-identical; a third of a millisecond at the limit); larger tensors are reduced by one
// block in double precision (the correctly rounded mean, which the serial fp32 sum itself only
// approximates), compared with the reference within the tolerance tier.
// mse_loss_grad_internal(pred, target, gy) = (2*gy/numel) * (pred - target), the coefficient formed
// first as in the reference (loss.cpp:225-255): elementwise, bit-identical.
namespace fb200 {

constexpr int64_t kMseSerialMax = 65536;

template <typename T>
__global__ void mse_loss_serial_kernel(const T* __restrict__ pred, const T* __restrict__ target, T* __restrict__ out,
                                       int64_t numel) {
  if (blockIdx.x != 0 || threadIdx.x != 0) return;
  float acc = 0.0f;
  for (int64_t i = 0; i < numel; ++i) {
    const float diff = to_f32(pred[i]) - to_f32(target[i]);
    acc += diff * diff;
  }
  out[0] = from_f32<T>(acc / static_cast<float>(numel));
}

template <typename T>
__global__ void __launch_bounds__(1024)
mse_loss_block_kernel(const T* __restrict__ pred, const T* __restrict__ target, T* __restrict__ out, int64_t numel) {
  __shared__ double part[32];
  double acc = 0.0;
  for (int64_t i = threadIdx.x; i < numel; i += blockDim.x) {
    const float diff = to_f32(pred[i]) - to_f32(target[i]);
    acc += static_cast<double>(diff * diff);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    double v = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0.0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (threadIdx.x == 0) out[0] = from_f32<T>(static_cast<float>(v / static_cast<double>(numel)));
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
mse_loss_grad_kernel(const T* __restrict__ pred, const T* __restrict__ target, const T* __restrict__ gy,
                     T* __restrict__ gpred, int64_t numel) {
  const float coefficient = 2.0f * to_f32(gy[0]) / static_cast<float>(numel);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < numel; i += stride) {
    gpred[i] = from_f32<T>(coefficient * (to_f32(pred[i]) - to_f32(target[i])));
  }
}

}  // namespace fb200

extern "C" int fb200_mse_loss(const void* pred, const void* target, void* out, int64_t numel, int dtype,
                              fb200_stream stream) {
  if (numel < 1) {
    return set_error(FB200_INVALID_ARGUMENT, "mse_loss: pred/target must have at least 1 element, got numel %lld",
                     (long long)numel);
  }
  if (pred == nullptr || target == nullptr || out == nullptr) return set_error(FB200_INVALID_ARGUMENT, "mse_loss: null argument");
  cudaStream_t s = as_stream(stream);
  auto run = [&](auto tag) {
    using T = decltype(tag);
    if (numel <= kMseSerialMax) {
      mse_loss_serial_kernel<T><<<1, 32, 0, s>>>(static_cast<const T*>(pred), static_cast<const T*>(target),
                                                 static_cast<T*>(out), numel);
    } else {
      mse_loss_block_kernel<T><<<1, 1024, 0, s>>>(static_cast<const T*>(pred), static_cast<const T*>(target),
                                                  static_cast<T*>(out), numel);
    }
  };
  FB200_FLOAT_DISPATCH("mse_loss", dtype, run)
  return after_launch("mse_loss_kernel");
}

extern "C" int fb200_mse_loss_grad(const void* pred, const void* target, const void* gy, void* gpred,
                                   int64_t numel, int dtype, fb200_stream stream) {
  if (numel < 1) {
    return set_error(FB200_INVALID_ARGUMENT,
                     "mse_loss_grad_internal: pred/target must have at least 1 element, got numel %lld", (long long)numel);
  }
  if (pred == nullptr || target == nullptr || gy == nullptr || gpred == nullptr) {
    return set_error(FB200_INVALID_ARGUMENT, "mse_loss_grad_internal: null argument");
  }
  cudaStream_t s = as_stream(stream);
  const int grid = grid_for(numel, 256, 8);
  auto run = [&](auto tag) {
    using T = decltype(tag);
    mse_loss_grad_kernel<T><<<grid, 256, 0, s>>>(static_cast<const T*>(pred), static_cast<const T*>(target),
                                                 static_cast<const T*>(gy), static_cast<T*>(gpred), numel);
  };
  FB200_FLOAT_DISPATCH("mse_loss_grad_internal", dtype, run)
  return after_launch("mse_loss_grad_kernel");
}
