// conv2d (strict-fp32 direct form), conv1d and max_pool2d.
//
// conv2d follows src/backends/cpu/kernels/conv.cpp:225-257 (NCHW cross-correlation, groups,
// stride, zero padding by skipping taps, accumulation order ci -> kh -> kw in fp32, bias last)
// and replaces cudnnConvolutionForward + cudnnAddTensor
// (src/backends/cuda/kernels/conv.cpp:385-520).  This file holds the strict-fp32 direct kernel:
// every output keeps the CPU reference's accumulation order (compiled with -fmad=false), so for
// fp32 it is bit-identical to the CPU backend.  The tensor-core implicit-GEMM form used when
// TF32 is allowed lives in conv_tcgen05.cu.
//
// conv1d follows conv.cpp:565-589; the reference CUDA backend has no conv1d kernel at all and
// drops the whole graph to its eager fallback (src/ops/schemas/conv.cpp:1021-1032).
// max_pool2d follows src/backends/cpu/kernels/pool.cpp:187-233 (valid taps only, first maximum
// wins) and replaces cudnnPoolingForward (src/backends/cuda/kernels/pool.cpp:231).
#include <cstdlib>

#include "common.cuh"
#include "epilogue.cuh"

namespace fb200 {

struct Conv2dDev {
  int64_t n, cin, h, w, cout, kh, kw, sh, sw, ph, pw, groups, oh, ow, cpg, copg;
};

// One thread: one output pixel x CO_T consecutive output channels of one group.
template <typename T, int CO_T>
__global__ void __launch_bounds__(128)
conv2d_direct_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ bias,
                     T* __restrict__ out, Conv2dDev p, EpilogueDev epi) {
  const int64_t pix_per_img = p.oh * p.ow;
  const int64_t co_tiles = (p.copg + CO_T - 1) / CO_T;
  const int64_t total = p.n * p.groups * co_tiles * pix_per_img;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += stride) {
    const int64_t pix = i % pix_per_img;
    int64_t rem = i / pix_per_img;
    const int64_t ct = rem % co_tiles;
    rem /= co_tiles;
    const int64_t g = rem % p.groups;
    const int64_t n = rem / p.groups;
    const int64_t oh = pix / p.ow;
    const int64_t ow = pix - oh * p.ow;
    const int64_t co0 = g * p.copg + ct * CO_T;
    const int64_t co_end = (ct + 1) * CO_T < p.copg ? CO_T : p.copg - ct * CO_T;
    float acc[CO_T];
#pragma unroll
    for (int c = 0; c < CO_T; ++c) acc[c] = 0.0f;
    for (int64_t ci = 0; ci < p.cpg; ++ci) {
      const T* xc = x + ((n * p.cin + g * p.cpg + ci) * p.h) * p.w;
      for (int64_t kh = 0; kh < p.kh; ++kh) {
        const int64_t ih = oh * p.sh - p.ph + kh;
        if (ih < 0 || ih >= p.h) continue;
        for (int64_t kw = 0; kw < p.kw; ++kw) {
          const int64_t iw = ow * p.sw - p.pw + kw;
          if (iw < 0 || iw >= p.w) continue;
          const float xv = to_f32(xc[ih * p.w + iw]);
#pragma unroll
          for (int c = 0; c < CO_T; ++c) {
            if (c < co_end) {
              const float wv = to_f32(w[(((co0 + c) * p.cpg + ci) * p.kh + kh) * p.kw + kw]);
              acc[c] += xv * wv;
            }
          }
        }
      }
    }
#pragma unroll
    for (int c = 0; c < CO_T; ++c) {
      if (c < co_end) {
        const int64_t co = co0 + c;
        float v = acc[c];
        if (bias != nullptr) v += to_f32(bias[co]);
        const int64_t oidx = ((n * p.cout + co) * p.oh + oh) * p.ow + ow;
        v = apply_epilogue<T>(epi, v, oidx, ow, co);
        out[oidx] = from_f32<T>(v);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
conv1d_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ bias,
              T* __restrict__ out, int64_t n, int64_t cin, int64_t l, int64_t cout, int64_t k,
              int64_t stride_, int64_t padding, int64_t groups, int64_t ol) {
  const int64_t cpg = cin / groups;
  const int64_t copg = cout / groups;
  const int64_t total = n * cout * ol;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += stride) {
    const int64_t o = i % ol;
    const int64_t rem = i / ol;
    const int64_t co = rem % cout;
    const int64_t b = rem / cout;
    const int64_t g = co / copg;
    float acc = 0.0f;
    for (int64_t ci = 0; ci < cpg; ++ci) {
      const T* xc = x + (b * cin + g * cpg + ci) * l;
      const T* wc = w + (co * cpg + ci) * k;
      for (int64_t kk = 0; kk < k; ++kk) {
        const int64_t il = o * stride_ - padding + kk;
        if (il < 0 || il >= l) continue;
        acc += to_f32(xc[il]) * to_f32(wc[kk]);
      }
    }
    if (bias != nullptr) acc += to_f32(bias[co]);
    out[i] = from_f32<T>(acc);
  }
}

// Depthwise, stride 1 (groups == Cin == Cout, one tap row per channel): the Mamba causal conv.
// One CTA walks 1024 consecutive outputs of one (batch, channel) row: no index division per
// element, taps in registers, x reads coalesced and overlapping reads served by L1.  Same order
// of operations as the generic kernel (bit-identical to the CPU reference).
template <typename T, int MAXK>
__global__ void __launch_bounds__(256)
conv1d_depthwise_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ bias,
                        T* __restrict__ out, int64_t rows, int64_t channels, int64_t l, int k,
                        int64_t padding, int64_t ol, int64_t chunks) {
  for (int64_t blk = blockIdx.x; blk < rows * chunks; blk += gridDim.x) {
    const int64_t row = blk / chunks;
    const int64_t chunk = blk - row * chunks;
    const int64_t co = row % channels;
    float taps[MAXK];
#pragma unroll
    for (int kk = 0; kk < MAXK; ++kk) taps[kk] = kk < k ? to_f32(w[co * k + kk]) : 0.0f;
    const float bv = bias != nullptr ? to_f32(bias[co]) : 0.0f;
    const T* xr = x + row * l;
    T* orow = out + row * ol;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t o = chunk * 1024 + j * 256 + threadIdx.x;
      if (o < ol) {
        float acc = 0.0f;
#pragma unroll
        for (int kk = 0; kk < MAXK; ++kk) {
          const int64_t il = o - padding + kk;
          if (kk < k && il >= 0 && il < l) acc += to_f32(xr[il]) * taps[kk];
        }
        if (bias != nullptr) acc += bv;
        orow[o] = from_f32<T>(acc);
      }
    }
  }
}

// IDX = int for tensors below 2^31 elements (no 64-bit divisions on the hot path), else int64_t.
template <typename T, typename IDX>
__global__ void __launch_bounds__(256)
max_pool2d_kernel(const T* __restrict__ x, T* __restrict__ out, IDX nc, IDX h, IDX w, IDX kh, IDX kw,
                  IDX sh, IDX sw, IDX ph, IDX pw, IDX oh, IDX ow) {
  const IDX total = nc * oh * ow;
  const IDX stride = static_cast<IDX>(gridDim.x) * blockDim.x;
  for (IDX i = static_cast<IDX>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const IDX q = i % ow;
    IDX rem = i / ow;
    const IDX o = rem % oh;
    rem /= oh;  // (n, c) plane
    const T* xc = x + static_cast<int64_t>(rem) * h * w;
    bool found = false;
    float best = 0.0f;
    T best_raw = T{};
    for (IDX a = 0; a < kh; ++a) {
      const IDX ih = o * sh - ph + a;
      if (ih < 0 || ih >= h) continue;
      for (IDX b = 0; b < kw; ++b) {
        const IDX iw = q * sw - pw + b;
        if (iw < 0 || iw >= w) continue;
        const T raw = xc[ih * w + iw];
        const float v = to_f32(raw);
        if (!found || v > best) {
          found = true;
          best = v;
          best_raw = raw;
        }
      }
    }
    out[i] = best_raw;  // the selected element itself: bit-exact, payloads included
  }
}

// Small fixed windows (3x3, 2x2): every tap is loaded from a clamped, always valid address before
// any comparison, so the loads of a window are all in flight together (with the bounds checks as
// branches in front of each load, a thread waited for up to nine memory round trips in a row and
// the kernel ran at a fifth of the copy bandwidth).  Selection order and result are unchanged.
template <typename T, int KH, int KW>
__global__ void __launch_bounds__(256)
max_pool2d_window_kernel(const T* __restrict__ x, T* __restrict__ out, int nc, int h, int w, int sh,
                         int sw, int ph, int pw, int oh, int ow) {
  const int total = nc * oh * ow;
  const int stride = static_cast<int>(gridDim.x) * blockDim.x;
  for (int i = static_cast<int>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int q = i % ow;
    int rem = i / ow;
    const int o = rem % oh;
    rem /= oh;  // (n, c) plane
    const T* xc = x + static_cast<int64_t>(rem) * h * w;
    T raw[KH][KW];
    bool ok[KH][KW];
#pragma unroll
    for (int a = 0; a < KH; ++a) {
      const int ih = o * sh - ph + a;
      const bool okh = ih >= 0 && ih < h;
      const int ihc = ih < 0 ? 0 : (ih >= h ? h - 1 : ih);
#pragma unroll
      for (int b = 0; b < KW; ++b) {
        const int iw = q * sw - pw + b;
        const int iwc = iw < 0 ? 0 : (iw >= w ? w - 1 : iw);
        ok[a][b] = okh && iw >= 0 && iw < w;
        raw[a][b] = xc[ihc * w + iwc];
      }
    }
    bool found = false;
    float best = 0.0f;
    T best_raw = T{};
#pragma unroll
    for (int a = 0; a < KH; ++a) {
#pragma unroll
      for (int b = 0; b < KW; ++b) {
        const float v = to_f32(raw[a][b]);
        if (ok[a][b] && (!found || v > best)) {
          found = true;
          best = v;
          best_raw = raw[a][b];
        }
      }
    }
    out[i] = best_raw;
  }
}

// 3x3 window, stride 2, padding 1 on rows whose length is a multiple of 4 (the stem pool of a ResNet):
// a thread produces four neighbouring outputs of one row.  They need input columns 2*ow-1 .. 2*ow+7 of
// three rows: two aligned 128-bit loads and one scalar per row, nine loads for four outputs where the
// one-output kernel issues thirty-six, and consecutive threads read consecutive 32-byte spans.
// Selection order (kh, then kw, strict >, first valid tap seeds) and result are unchanged.
template <typename T>
__global__ void __launch_bounds__(256)
max_pool2d_k3s2p1_quad_kernel(const T* __restrict__ x, T* __restrict__ out, int nc, int h, int w, int oh,
                              int ow) {
  static_assert(sizeof(T) == 4, "32-bit elements");
  const int quads = ow / 4;
  const int total = nc * oh * quads;
  const int stride = static_cast<int>(gridDim.x) * blockDim.x;
  for (int i = static_cast<int>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int qd = i % quads;
    int rem = i / quads;
    const int o = rem % oh;
    rem /= oh;
    const T* xc = x + static_cast<int64_t>(rem) * h * w;
    const int c0 = qd * 8;   // first input column covered by the aligned loads (= 2 * first ow)
    T tap[3][9];             // columns c0-1 .. c0+7
    bool row_ok[3];
#pragma unroll
    for (int a = 0; a < 3; ++a) {
      const int ih = o * 2 - 1 + a;
      row_ok[a] = ih >= 0 && ih < h;
      const int ihc = ih < 0 ? 0 : (ih >= h ? h - 1 : ih);
      const T* row = xc + static_cast<int64_t>(ihc) * w;
      const float4 lo = *reinterpret_cast<const float4*>(row + c0);
      const float4 hi = *reinterpret_cast<const float4*>(row + c0 + 4);
      tap[a][0] = row[c0 > 0 ? c0 - 1 : 0];
      tap[a][1] = lo.x; tap[a][2] = lo.y; tap[a][3] = lo.z; tap[a][4] = lo.w;
      tap[a][5] = hi.x; tap[a][6] = hi.y; tap[a][7] = hi.z; tap[a][8] = hi.w;
    }
    float4 res;
    float* resv = reinterpret_cast<float*>(&res);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      bool found = false;
      float best = 0.0f;
#pragma unroll
      for (int a = 0; a < 3; ++a) {
#pragma unroll
        for (int b = 0; b < 3; ++b) {
          const int col = c0 + 2 * j - 1 + b;          // input column of this tap
          const bool ok = row_ok[a] && col >= 0 && col < w;
          const float v = tap[a][2 * j + b];
          if (ok && (!found || v > best)) {
            found = true;
            best = v;
          }
        }
      }
      resv[j] = best;
    }
    *reinterpret_cast<float4*>(out + (static_cast<int64_t>(rem) * oh + o) * ow + qd * 4) = res;
  }
}

}  // namespace fb200

using namespace fb200;

// Implemented in conv_tcgen05.cu; returns FB200_UNIMPLEMENTED when the shape is outside what the
// tensor-core kernel covers, in which case the direct kernel below runs.
extern "C" int fb200_conv2d_tcgen05(const void* x, const void* w, const void* bias, void* out,
                                    const fb200_conv2d_params* p, int dtype,
                                    const fb200_epilogue* epilogue, fb200_stream stream);

// Implemented in conv_halo_tcgen05.cu: the halo-tile variant, tried first.
extern "C" int fb200_conv2d_planes_tcgen05(const void* x, const void* w, const void* bias, void* out,
                                           const fb200_conv2d_params* p, int dtype,
                                           const fb200_epilogue* epilogue, fb200_stream stream);
extern "C" int fb200_conv2d_halo_tcgen05(const void* x, const void* w, const void* bias, void* out,
                                         const fb200_conv2d_params* p, int dtype,
                                         const fb200_epilogue* epilogue, fb200_stream stream);
// Implemented in conv_rows_tcgen05.cu: stride 2 with few input channels (row matrices built once per
// input row).
extern "C" int fb200_conv2d_rows_tcgen05(const void* x, const void* w, const void* bias, void* out,
                                         const fb200_conv2d_params* p, int dtype,
                                         const fb200_epilogue* epilogue, fb200_stream stream);

extern "C" int fb200_conv2d_rows_pooled_tcgen05(const void* x, const void* w, const void* bias, void* pooled,
                                                const fb200_conv2d_params* p, int dtype,
                                                const fb200_epilogue* epilogue, fb200_stream stream);

extern "C" int fb200_conv2d(const void* x, const void* w, const void* bias, void* out,
                            const fb200_conv2d_params* pp, int dtype, int allow_tf32,
                            const fb200_epilogue* epilogue, fb200_stream stream) {
  if (pp == nullptr) return set_error(FB200_INVALID_ARGUMENT, "conv2d: null params");
  const fb200_conv2d_params& q = *pp;
  if (q.n < 0 || q.cin < 1 || q.h < 1 || q.w < 1 || q.cout < 1 || q.kh < 1 || q.kw < 1 ||
      q.stride_h < 1 || q.stride_w < 1 || q.pad_h < 0 || q.pad_w < 0 || q.groups < 1) {
    return set_error(FB200_INVALID_ARGUMENT, "conv2d: invalid geometry");
  }
  if (q.cin % q.groups != 0 || q.cout % q.groups != 0) {
    return set_error(FB200_INVALID_ARGUMENT,
                     "conv2d: groups %lld must divide Cin %lld and Cout %lld", (long long)q.groups,
                     (long long)q.cin, (long long)q.cout);
  }
  Conv2dDev d{};
  d.n = q.n; d.cin = q.cin; d.h = q.h; d.w = q.w; d.cout = q.cout; d.kh = q.kh; d.kw = q.kw;
  d.sh = q.stride_h; d.sw = q.stride_w; d.ph = q.pad_h; d.pw = q.pad_w; d.groups = q.groups;
  d.oh = (q.h + 2 * q.pad_h - q.kh) / q.stride_h + 1;
  d.ow = (q.w + 2 * q.pad_w - q.kw) / q.stride_w + 1;
  if (q.h + 2 * q.pad_h < q.kh || q.w + 2 * q.pad_w < q.kw || d.oh < 1 || d.ow < 1) {
    return set_error(FB200_INVALID_ARGUMENT, "conv2d: non-positive output size");
  }
  d.cpg = q.cin / q.groups;
  d.copg = q.cout / q.groups;
  if (q.n == 0) return FB200_OK;
  if (x == nullptr || w == nullptr || out == nullptr) {
    return set_error(FB200_INVALID_ARGUMENT, "conv2d: null argument");
  }
  if (allow_tf32 && dtype == FB200_F32) {
    {
      const int rc = fb200_conv2d_planes_tcgen05(x, w, bias, out, pp, dtype, epilogue, stream);
      if (rc != FB200_UNIMPLEMENTED) return rc;
    }
    {
      const int rc = fb200_conv2d_rows_tcgen05(x, w, bias, out, pp, dtype, epilogue, stream);
      if (rc != FB200_UNIMPLEMENTED) return rc;
    }
    {
      const int rc = fb200_conv2d_halo_tcgen05(x, w, bias, out, pp, dtype, epilogue, stream);
      if (rc != FB200_UNIMPLEMENTED) return rc;
    }
    const int rc = fb200_conv2d_tcgen05(x, w, bias, out, pp, dtype, epilogue, stream);
    if (rc != FB200_UNIMPLEMENTED) return rc;
  }
  EpilogueDev epi{};
  if (int rc = make_epilogue(epilogue, &epi, "conv2d")) return rc;
  cudaStream_t s = as_stream(stream);
  constexpr int CO_T = 8;
  const int64_t co_tiles = (d.copg + CO_T - 1) / CO_T;
  const int64_t total = d.n * d.groups * co_tiles * d.oh * d.ow;
  const int grid = grid_for(total, 128, 16);
  switch (dtype) {
    case FB200_F32:
      conv2d_direct_kernel<float, CO_T><<<grid, 128, 0, s>>>(
          static_cast<const float*>(x), static_cast<const float*>(w),
          static_cast<const float*>(bias), static_cast<float*>(out), d, epi);
      break;
    case FB200_BF16:
      conv2d_direct_kernel<__nv_bfloat16, CO_T><<<grid, 128, 0, s>>>(
          static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
          static_cast<const __nv_bfloat16*>(bias), static_cast<__nv_bfloat16*>(out), d, epi);
      break;
    case FB200_F16:
      conv2d_direct_kernel<__half, CO_T><<<grid, 128, 0, s>>>(
          static_cast<const __half*>(x), static_cast<const __half*>(w),
          static_cast<const __half*>(bias), static_cast<__half*>(out), d, epi);
      break;
    default:
      return set_error(FB200_INVALID_ARGUMENT,
                       "conv2d: dtype code %d is not float32/float16/bfloat16", dtype);
  }
  return after_launch("conv2d_direct_kernel");
}

extern "C" int fb200_conv1d(const void* x, const void* w, const void* bias, void* out, int64_t n,
                            int64_t cin, int64_t l, int64_t cout, int64_t k, int64_t stride,
                            int64_t padding, int64_t groups, int dtype, fb200_stream stream) {
  if (n < 0 || cin < 1 || l < 1 || cout < 1 || k < 1 || stride < 1 || padding < 0 || groups < 1) {
    return set_error(FB200_INVALID_ARGUMENT, "conv1d: invalid geometry");
  }
  if (cin % groups != 0 || cout % groups != 0) {
    return set_error(FB200_INVALID_ARGUMENT, "conv1d: groups must divide Cin and Cout");
  }
  if (l + 2 * padding < k) return set_error(FB200_INVALID_ARGUMENT, "conv1d: non-positive output size");
  const int64_t ol = (l + 2 * padding - k) / stride + 1;
  if (n == 0) return FB200_OK;
  if (x == nullptr || w == nullptr || out == nullptr) {
    return set_error(FB200_INVALID_ARGUMENT, "conv1d: null argument");
  }
  cudaStream_t s = as_stream(stream);
  if (groups == cin && cout == cin && stride == 1 && k <= 8) {
    const int64_t rows = n * cout;
    const int64_t chunks = (ol + 1023) / 1024;
    const int64_t blocks = rows * chunks;
    const int dgrid = static_cast<int>(blocks < int64_t(kNumSMs) * 16 ? blocks : int64_t(kNumSMs) * 16);
    switch (dtype) {
      case FB200_F32:
        conv1d_depthwise_kernel<float, 8><<<dgrid, 256, 0, s>>>(
            static_cast<const float*>(x), static_cast<const float*>(w), static_cast<const float*>(bias),
            static_cast<float*>(out), rows, cout, l, static_cast<int>(k), padding, ol, chunks);
        return after_launch("conv1d_depthwise_kernel");
      case FB200_BF16:
        conv1d_depthwise_kernel<__nv_bfloat16, 8><<<dgrid, 256, 0, s>>>(
            static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
            static_cast<const __nv_bfloat16*>(bias), static_cast<__nv_bfloat16*>(out), rows, cout, l,
            static_cast<int>(k), padding, ol, chunks);
        return after_launch("conv1d_depthwise_kernel");
      default:
        break;  // f16 and anything else: generic kernel below
    }
  }
  const int grid = grid_for(n * cout * ol, 256, 8);
  switch (dtype) {
    case FB200_F32:
      conv1d_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(x),
                                                static_cast<const float*>(w),
                                                static_cast<const float*>(bias),
                                                static_cast<float*>(out), n, cin, l, cout, k,
                                                stride, padding, groups, ol);
      break;
    case FB200_BF16:
      conv1d_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(
          static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
          static_cast<const __nv_bfloat16*>(bias), static_cast<__nv_bfloat16*>(out), n, cin, l,
          cout, k, stride, padding, groups, ol);
      break;
    case FB200_F16:
      conv1d_kernel<__half><<<grid, 256, 0, s>>>(static_cast<const __half*>(x),
                                                 static_cast<const __half*>(w),
                                                 static_cast<const __half*>(bias),
                                                 static_cast<__half*>(out), n, cin, l, cout, k,
                                                 stride, padding, groups, ol);
      break;
    default:
      return set_error(FB200_INVALID_ARGUMENT,
                       "conv1d: dtype code %d is not float32/float16/bfloat16", dtype);
  }
  return after_launch("conv1d_kernel");
}

extern "C" int fb200_max_pool2d(const void* x, void* out, int64_t n, int64_t c, int64_t h,
                                int64_t w, int64_t kh, int64_t kw, int64_t stride_h,
                                int64_t stride_w, int64_t pad_h, int64_t pad_w, int dtype,
                                fb200_stream stream) {
  if (n < 0 || c < 0 || h < 1 || w < 1 || kh < 1 || kw < 1 || stride_h < 1 || stride_w < 1 ||
      pad_h < 0 || pad_w < 0) {
    return set_error(FB200_INVALID_ARGUMENT, "max_pool2d: invalid geometry");
  }
  if (2 * pad_h > kh || 2 * pad_w > kw) {
    return set_error(FB200_INVALID_ARGUMENT, "max_pool2d: padding*2 must not exceed kernel");
  }
  if (h + 2 * pad_h < kh || w + 2 * pad_w < kw) {
    return set_error(FB200_INVALID_ARGUMENT, "max_pool2d: non-positive output size");
  }
  const int64_t oh = (h + 2 * pad_h - kh) / stride_h + 1;
  const int64_t ow = (w + 2 * pad_w - kw) / stride_w + 1;
  if (n == 0 || c == 0) return FB200_OK;
  if (x == nullptr || out == nullptr) return set_error(FB200_INVALID_ARGUMENT, "max_pool2d: null argument");
  cudaStream_t s = as_stream(stream);
  const int grid = grid_for(n * c * oh * ow, 256, 8);
  const bool small = n * c * h * w < (int64_t(1) << 31);
  auto run = [&](auto tag) {
    using T = decltype(tag);
    if (small && sizeof(T) == 4 && kh == 3 && kw == 3 && stride_h == 2 && stride_w == 2 && pad_h == 1 &&
        pad_w == 1 && w % 4 == 0 && ow % 4 == 0 && ow * 2 == w && aligned16(x) && aligned16(out)) {
      if constexpr (sizeof(T) == 4) {
        const int qgrid = grid_for(n * c * oh * (ow / 4), 256, 8);
        max_pool2d_k3s2p1_quad_kernel<T><<<qgrid, 256, 0, s>>>(
            static_cast<const T*>(x), static_cast<T*>(out), static_cast<int>(n * c), static_cast<int>(h),
            static_cast<int>(w), static_cast<int>(oh), static_cast<int>(ow));
      }
    } else if (small && ((kh == 3 && kw == 3) || (kh == 2 && kw == 2))) {
      const T* xp = static_cast<const T*>(x);
      T* op = static_cast<T*>(out);
      const int a[9] = {static_cast<int>(n * c), static_cast<int>(h), static_cast<int>(w),
                        static_cast<int>(stride_h), static_cast<int>(stride_w), static_cast<int>(pad_h),
                        static_cast<int>(pad_w), static_cast<int>(oh), static_cast<int>(ow)};
      if (kh == 3) {
        max_pool2d_window_kernel<T, 3, 3><<<grid, 256, 0, s>>>(xp, op, a[0], a[1], a[2], a[3], a[4], a[5], a[6], a[7], a[8]);
      } else {
        max_pool2d_window_kernel<T, 2, 2><<<grid, 256, 0, s>>>(xp, op, a[0], a[1], a[2], a[3], a[4], a[5], a[6], a[7], a[8]);
      }
    } else if (small) {
      max_pool2d_kernel<T, int><<<grid, 256, 0, s>>>(
          static_cast<const T*>(x), static_cast<T*>(out), static_cast<int>(n * c), static_cast<int>(h),
          static_cast<int>(w), static_cast<int>(kh), static_cast<int>(kw), static_cast<int>(stride_h),
          static_cast<int>(stride_w), static_cast<int>(pad_h), static_cast<int>(pad_w),
          static_cast<int>(oh), static_cast<int>(ow));
    } else {
      max_pool2d_kernel<T, int64_t><<<grid, 256, 0, s>>>(static_cast<const T*>(x), static_cast<T*>(out),
                                                         n * c, h, w, kh, kw, stride_h, stride_w, pad_h,
                                                         pad_w, oh, ow);
    }
  };
  switch (dtype) {
    case FB200_F32: run(float{}); break;
    case FB200_BF16: run(__nv_bfloat16{}); break;
    case FB200_F16: run(__half{}); break;
    default:
      return set_error(FB200_INVALID_ARGUMENT,
                       "max_pool2d: dtype code %d is not float32/float16/bfloat16", dtype);
  }
  return after_launch("max_pool2d_kernel");
}

// ---- avg_pool2d ------------------------------------------------------------------------------------
// Sum of the valid positions of the window in (kh, kw) order, divided by KH*KW whatever the padding
// (src/backends/cpu/kernels/pool.cpp:280-303): the same fp32 additions in the same order and one
// fp32 division, so results are bit-identical to the CPU reference.  As in the max-pool window
// kernel every tap is loaded from a clamped address before it is used, so the loads of a window are
// in flight together; an invalid tap contributes nothing (it is skipped, not added as zero, which
// matters for -0 and NaN only in theory but keeps the operation count identical).
namespace fb200 {

template <typename T>
__global__ void __launch_bounds__(256)
avg_pool2d_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t nc, int64_t h, int64_t w, int kh,
                  int kw, int sh, int sw, int ph, int pw, int64_t oh, int64_t ow) {
  const int64_t total = nc * oh * ow;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const float denom = static_cast<float>(kh * kw);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t q = i % ow;
    int64_t rem = i / ow;
    const int64_t o = rem % oh;
    rem /= oh;
    const T* xc = x + rem * h * w;
    float acc = 0.0f;
    for (int a = 0; a < kh; ++a) {
      const int64_t ih = o * sh - ph + a;
      if (ih < 0 || ih >= h) continue;
      for (int b = 0; b < kw; ++b) {
        const int64_t iw = q * sw - pw + b;
        if (iw < 0 || iw >= w) continue;
        acc += to_f32(xc[ih * w + iw]);
      }
    }
    out[i] = from_f32<T>(acc / denom);
  }
}

}  // namespace fb200

extern "C" int fb200_avg_pool2d(const void* x, void* out, int64_t n, int64_t c, int64_t h, int64_t w,
                                int64_t kh, int64_t kw, int64_t stride_h, int64_t stride_w,
                                int64_t pad_h, int64_t pad_w, int dtype, fb200_stream stream) {
  if (n < 0 || c < 0 || h < 1 || w < 1 || kh < 1 || kw < 1 || stride_h < 1 || stride_w < 1 ||
      pad_h < 0 || pad_w < 0) {
    return set_error(FB200_INVALID_ARGUMENT, "avg_pool2d: invalid geometry");
  }
  if (2 * pad_h > kh || 2 * pad_w > kw) {
    return set_error(FB200_INVALID_ARGUMENT, "avg_pool2d: padding*2 must not exceed kernel");
  }
  if (h + 2 * pad_h < kh || w + 2 * pad_w < kw) {
    return set_error(FB200_INVALID_ARGUMENT, "avg_pool2d: non-positive output size");
  }
  const int64_t oh = (h + 2 * pad_h - kh) / stride_h + 1;
  const int64_t ow = (w + 2 * pad_w - kw) / stride_w + 1;
  if (n == 0 || c == 0) return FB200_OK;
  if (x == nullptr || out == nullptr) return set_error(FB200_INVALID_ARGUMENT, "avg_pool2d: null argument");
  cudaStream_t s = as_stream(stream);
  const int grid = grid_for(n * c * oh * ow, 256, 8);
  auto run = [&](auto tag) {
    using T = decltype(tag);
    avg_pool2d_kernel<T><<<grid, 256, 0, s>>>(static_cast<const T*>(x), static_cast<T*>(out), n * c, h, w,
                                              static_cast<int>(kh), static_cast<int>(kw),
                                              static_cast<int>(stride_h), static_cast<int>(stride_w),
                                              static_cast<int>(pad_h), static_cast<int>(pad_w), oh, ow);
  };
  switch (dtype) {
    case FB200_F32: run(float{}); break;
    case FB200_BF16: run(__nv_bfloat16{}); break;
    case FB200_F16: run(__half{}); break;
    default:
      return set_error(FB200_INVALID_ARGUMENT, "avg_pool2d: dtype code %d is not float32/float16/bfloat16", dtype);
  }
  return after_launch("avg_pool2d_kernel");
}

// ---- depthwise conv1d along time, in the time-major layout -----------------------------------------
// The reference's Mamba block computes its causal depthwise convolution as
//   transpose [B,L,C] -> [B,C,L], conv1d(groups = C, padding = K-1), slice to L, activation,
//   transpose back (src/nn/layers.cpp:1596-1602),
// five full passes over the activation.  This kernel produces the same values straight from the
// time-major tensor (row pitch x_ld, so a column window of a wider matrix works) into a time-major
// result: out[b,t,c] = ops(bias[c] + sum_k w[c,k] * x[b, t+shift+k, c]), taps outside [0, len)
// skipped, products accumulated for k increasing and the bias added last, the sum rounded to T
// and each unary op rounded to T — the operations of conv1d_forward_compute
// (src/backends/cpu/kernels/conv.cpp:565-589) and of the elementwise chain, in their order, so
// fp32 results are bit-identical to the five-step form.
// A thread owns one 16-byte vector of channels and walks kDwRun consecutive time steps with the
// K most recent inputs in registers: every input is loaded once per run (plus K-1 halo rows);
// the loads of four steps are issued together.
namespace fb200 {

constexpr int kDwRun = 64;     // time steps per thread (a multiple of kDwUnroll)
constexpr int kDwUnroll = 4;  // outputs per group: that many loads in flight per thread
constexpr int kDwMaxK = 8;

struct DwOps { int n; int op[FB200_MAX_CHAIN]; };

template <typename T, int K>
__global__ void __launch_bounds__(128)
dwconv1d_time_major_kernel(const T* __restrict__ x, int64_t x_ld, const T* __restrict__ w,
                           const T* __restrict__ bias, T* __restrict__ out, int64_t out_ld,
                           int64_t len, int64_t out_len, int64_t channels, int64_t shift,
                           DwOps ops) {
  constexpr int V = 16 / sizeof(T);
  const int64_t c0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * V;
  if (c0 >= channels) return;
  const int64_t b = blockIdx.z;
  const int64_t t_begin = static_cast<int64_t>(blockIdx.y) * kDwRun;
  const int64_t t_end = t_begin + kDwRun < out_len ? t_begin + kDwRun : out_len;
  float taps[K][V];
#pragma unroll
  for (int kk = 0; kk < K; ++kk) {
#pragma unroll
    for (int v = 0; v < V; ++v) taps[kk][v] = to_f32(w[(c0 + v) * K + kk]);
  }
  float bv[V];
#pragma unroll
  for (int v = 0; v < V; ++v) bv[v] = bias != nullptr ? to_f32(bias[c0 + v]) : 0.0f;
  const T* xb = x + b * len * x_ld + c0;
  T* ob = out + b * out_len * out_ld + c0;
  // rows[j] = input row (t + shift + j) for the U outputs of one group: K-1 rows of history and U
  // new ones, all U loads issued before the arithmetic; rows outside [0, len) are marked invalid
  constexpr int U = kDwUnroll;
  float rows[K - 1 + U][V];
  bool valid[K - 1 + U];
  auto fetch = [&](int64_t row, float (&dst)[V], bool& ok) {
    ok = row >= 0 && row < len;
    if (ok) {
      load_vec<T>(xb + row * x_ld, dst);
    } else {
#pragma unroll
      for (int v = 0; v < V; ++v) dst[v] = 0.0f;
    }
  };
#pragma unroll
  for (int j = 0; j < K - 1; ++j) fetch(t_begin + shift + j, rows[j], valid[j]);
  // the U new rows of the next group are in flight while the current group is computed
  float ahead[U][V];
  bool ahead_valid[U];
#pragma unroll
  for (int u = 0; u < U; ++u) fetch(t_begin + u + shift + K - 1, ahead[u], ahead_valid[u]);
  for (int64_t t = t_begin; t < t_end; t += U) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int v = 0; v < V; ++v) rows[K - 1 + u][v] = ahead[u][v];
      valid[K - 1 + u] = ahead_valid[u];
    }
    if (t + U < t_end) {
#pragma unroll
      for (int u = 0; u < U; ++u) fetch(t + U + u + shift + K - 1, ahead[u], ahead_valid[u]);
    }
    float res[U * V];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float acc[V];
#pragma unroll
      for (int v = 0; v < V; ++v) acc[v] = 0.0f;
#pragma unroll
      for (int kk = 0; kk < K; ++kk) {
        if (valid[u + kk]) {
#pragma unroll
          for (int v = 0; v < V; ++v) acc[v] += rows[u + kk][v] * taps[kk][v];
        }
      }
#pragma unroll
      for (int v = 0; v < V; ++v) {
        if (bias != nullptr) acc[v] += bv[v];
        res[u * V + v] = round_through<T>(acc[v]);
      }
    }
#pragma unroll 1
    for (int o = 0; o < ops.n; ++o) ew_unary_vec<T, U * V>(ops.op[o], res);   // one switch per group
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (t + u < t_end) {
        float outv[V];
#pragma unroll
        for (int v = 0; v < V; ++v) outv[v] = res[u * V + v];
        store_vec<T>(ob + (t + u) * out_ld, outv);
      }
    }
#pragma unroll
    for (int j = 0; j < K - 1; ++j) {   // the last K-1 rows become the next group's history
#pragma unroll
      for (int v = 0; v < V; ++v) rows[j][v] = rows[j + U][v];
      valid[j] = valid[j + U];
    }
  }
}

template <typename T>
static void launch_dwconv(dim3 grid, cudaStream_t s, const void* x, int64_t x_ld, const void* w,
                          const void* bias, void* out, int64_t out_ld, int64_t len, int64_t out_len,
                          int64_t channels, int k, int64_t shift, const DwOps& ops) {
  const T* xp = static_cast<const T*>(x);
  const T* wp = static_cast<const T*>(w);
  const T* bp = static_cast<const T*>(bias);
  T* op = static_cast<T*>(out);
#define FB200_DW_CASE(KK)                                                                          \
  case KK:                                                                                         \
    dwconv1d_time_major_kernel<T, KK><<<grid, 128, 0, s>>>(xp, x_ld, wp, bp, op, out_ld, len, out_len, \
                                                           channels, shift, ops);                  \
    break;
  switch (k) {
    FB200_DW_CASE(1) FB200_DW_CASE(2) FB200_DW_CASE(3) FB200_DW_CASE(4)
    FB200_DW_CASE(5) FB200_DW_CASE(6) FB200_DW_CASE(7) FB200_DW_CASE(8)
    default: break;
  }
#undef FB200_DW_CASE
}

}  // namespace fb200

extern "C" int fb200_dwconv1d_time_major(const void* x, int64_t x_ld, const void* w, const void* bias,
                                         void* out, int64_t out_ld, int64_t batch, int64_t len,
                                         int64_t out_len, int64_t channels, int64_t k, int64_t shift,
                                         const int* unary_ops, int n_ops, int dtype,
                                         fb200_stream stream) {
  if (batch < 0 || len < 1 || out_len < 0 || channels < 1 || k < 1 || k > kDwMaxK) {
    return set_error(FB200_INVALID_ARGUMENT, "dwconv1d_time_major: invalid geometry (1 <= k <= %d)", kDwMaxK);
  }
  if (n_ops < 0 || n_ops > FB200_MAX_CHAIN || (n_ops > 0 && unary_ops == nullptr)) {
    return set_error(FB200_INVALID_ARGUMENT, "dwconv1d_time_major: bad op list");
  }
  DwOps ops{};
  ops.n = n_ops;
  for (int i = 0; i < n_ops; ++i) {
    if (!ew_is_known(unary_ops[i]) || ew_is_binary(unary_ops[i])) {
      return set_error(FB200_INVALID_ARGUMENT, "dwconv1d_time_major: op code %d is not a unary elementwise op", unary_ops[i]);
    }
    ops.op[i] = unary_ops[i];
  }
  if (dtype != FB200_F32 && dtype != FB200_BF16 && dtype != FB200_F16) {
    return set_error(FB200_INVALID_ARGUMENT, "dwconv1d_time_major: dtype code %d is not float32/float16/bfloat16", dtype);
  }
  if (batch == 0 || out_len == 0) return FB200_OK;
  if (x == nullptr || w == nullptr || out == nullptr) return set_error(FB200_INVALID_ARGUMENT, "dwconv1d_time_major: null argument");
  const int v = 16 / itemsize_of(dtype);
  if (channels % v || x_ld % v || out_ld % v || x_ld < channels || out_ld < channels || !aligned16(x) || !aligned16(out)) {
    return set_error(FB200_INVALID_ARGUMENT,
                     "dwconv1d_time_major: channels and row pitches must be multiples of %d elements and the "
                     "tensors 16-byte aligned", v);
  }
  const int64_t runs = (out_len + kDwRun - 1) / kDwRun;
  if (batch > 65535 || runs > 65535) return set_error(FB200_INVALID_ARGUMENT, "dwconv1d_time_major: batch or length too large");
  const int64_t vecs = channels / v;
  dim3 grid(static_cast<unsigned>((vecs + 127) / 128), static_cast<unsigned>(runs), static_cast<unsigned>(batch));
  cudaStream_t s = as_stream(stream);
  const int kk = static_cast<int>(k);
  if (dtype == FB200_F32) launch_dwconv<float>(grid, s, x, x_ld, w, bias, out, out_ld, len, out_len, channels, kk, shift, ops);
  else if (dtype == FB200_BF16) launch_dwconv<__nv_bfloat16>(grid, s, x, x_ld, w, bias, out, out_ld, len, out_len, channels, kk, shift, ops);
  else launch_dwconv<__half>(grid, s, x, x_ld, w, bias, out, out_ld, len, out_len, channels, kk, shift, ops);
  return after_launch("dwconv1d_time_major_kernel");
}

// conv2d -> [epilogue chain] -> max_pool2d as one call.  With allow_tf32, a 3 x 3 / stride 2 / pad 1
// pool behind a stride-2 convolution of few input channels (an image stem) runs as ONE kernel that
// never writes the convolution's result (conv_rows_tcgen05.cu); `mid` ([n, cout, oh, ow], may be
// NULL) is then left untouched.  Every other case runs the two operators one after the other
// through `mid`, which must then be given.
extern "C" int fb200_conv2d_max_pool(const void* x, const void* w, const void* bias, void* mid, void* out,
                                     const fb200_conv2d_params* pp, int64_t pool_kh, int64_t pool_kw,
                                     int64_t pool_stride_h, int64_t pool_stride_w, int64_t pool_pad_h,
                                     int64_t pool_pad_w, int dtype, int allow_tf32,
                                     const fb200_epilogue* epilogue, fb200_stream stream) {
  if (pp == nullptr) return set_error(FB200_INVALID_ARGUMENT, "conv2d_max_pool: null params");
  if (pp->n == 0) return FB200_OK;
  if (x == nullptr || w == nullptr || out == nullptr) return set_error(FB200_INVALID_ARGUMENT, "conv2d_max_pool: null argument");
  if (allow_tf32 && dtype == FB200_F32 && pool_kh == 3 && pool_kw == 3 && pool_stride_h == 2 && pool_stride_w == 2 &&
      pool_pad_h == 1 && pool_pad_w == 1 && pp->stride_h >= 1 && pp->stride_w >= 1 && pp->kh >= 1 && pp->kw >= 1) {
    const int rc = fb200_conv2d_rows_pooled_tcgen05(x, w, bias, out, pp, dtype, epilogue, stream);
    if (rc != FB200_UNIMPLEMENTED) return rc;
  }
  if (mid == nullptr) {
    return set_error(FB200_INVALID_ARGUMENT, "conv2d_max_pool: this shape runs as two kernels and needs the "
                     "intermediate buffer");
  }
  if (int rc = fb200_conv2d(x, w, bias, mid, pp, dtype, allow_tf32, epilogue, stream)) return rc;
  const int64_t oh = (pp->h + 2 * pp->pad_h - pp->kh) / pp->stride_h + 1;
  const int64_t ow = (pp->w + 2 * pp->pad_w - pp->kw) / pp->stride_w + 1;
  return fb200_max_pool2d(mid, out, pp->n, pp->cout, oh, ow, pool_kh, pool_kw, pool_stride_h, pool_stride_w,
                          pool_pad_h, pool_pad_w, dtype, stream);
}
