// Shared helpers of the sm_100a kernel set: status/error plumbing, storage <-> fp32
// conversion with one round-to-nearest-even at the store, 128-bit vector access, and launch
// geometry sized for the 148 SMs of a B200.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "../../include/frame_b200.h"

namespace fb200 {

// ---- error plumbing -------------------------------------------------------------------------
int set_error(int code, const char* fmt, ...);
int cuda_error(cudaError_t err, const char* what);
extern std::atomic<int64_t> g_launch_count;

inline cudaStream_t as_stream(fb200_stream s) { return reinterpret_cast<cudaStream_t>(s); }

#define FB200_CUDA_OK(expr)                                                 \
  do {                                                                      \
    cudaError_t fb200_err__ = (expr);                                       \
    if (fb200_err__ != cudaSuccess) return ::fb200::cuda_error(fb200_err__, #expr); \
  } while (0)

// Call after every kernel launch: counts the launch and turns a launch error into a status.
inline int after_launch(const char* kernel) {
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return cuda_error(err, kernel);
  return FB200_OK;
}

// Stream-ordered scratch for kernels that need a temporary (cudaMallocAsync on `stream`; release it
// with cudaFreeAsync on the same stream).  The first call on a device tells the device's default
// memory pool to keep up to 1 GiB of freed blocks instead of returning them to the driver at every
// synchronisation point: without that each eager call pays a driver allocation.
cudaError_t scratch_alloc_async(void** ptr, size_t bytes, cudaStream_t stream);

constexpr int kNumSMs = 148;

inline int itemsize_of(int dtype) {
  switch (dtype) {
    case FB200_F32: return 4;
    case FB200_F64: return 8;
    case FB200_F16: return 2;
    case FB200_BF16: return 2;
    case FB200_I8: return 1;
    case FB200_I16: return 2;
    case FB200_I32: return 4;
    case FB200_I64: return 8;
    case FB200_U8: return 1;
    case FB200_BOOL: return 1;
    default: return 0;
  }
}

inline bool is_float_dtype(int dtype) {
  return dtype == FB200_F32 || dtype == FB200_BF16 || dtype == FB200_F16;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Grid for a grid-stride kernel: enough CTAs to fill every SM `per_sm` times, never more than
// the work needs.
inline int grid_for(int64_t work_items, int threads, int per_sm) {
  int64_t need = (work_items + threads - 1) / threads;
  int64_t cap = static_cast<int64_t>(kNumSMs) * per_sm;
  if (need < 1) need = 1;
  return static_cast<int>(need < cap ? need : cap);
}

// ---- storage <-> fp32 ------------------------------------------------------------------------
// Storage tags: the tensor dtype as the kernels see it.
struct F32Tag { using storage = float; static constexpr int kVec = 4; };
struct BF16Tag { using storage = __nv_bfloat16; static constexpr int kVec = 8; };
struct F16Tag { using storage = __half; static constexpr int kVec = 8; };

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
// __float2bfloat16_rn: RTNE; NaN becomes the canonical quiet NaN 0x7FFF (the CPU reference keeps
// the payload's top bits) — both are NaN, and NaN never compares equal in the parity helper.
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// Value after a store to T and a load back: the rounding point between fused steps.
template <typename T> __device__ __forceinline__ float round_through(float v) {
  return to_f32(from_f32<T>(v));
}
template <> __device__ __forceinline__ float round_through<float>(float v) { return v; }

// 16-byte vector of storage elements.
template <typename T> struct alignas(16) Vec16 { T v[16 / sizeof(T)]; };

template <typename T>
__device__ __forceinline__ void load_vec(const T* p, float (&out)[16 / sizeof(T)]) {
  Vec16<T> raw = *reinterpret_cast<const Vec16<T>*>(p);
#pragma unroll
  for (int i = 0; i < int(16 / sizeof(T)); ++i) out[i] = to_f32(raw.v[i]);
}

template <typename T>
__device__ __forceinline__ void store_vec(T* p, const float (&in)[16 / sizeof(T)]) {
  Vec16<T> raw;
#pragma unroll
  for (int i = 0; i < int(16 / sizeof(T)); ++i) raw.v[i] = from_f32<T>(in[i]);
  *reinterpret_cast<Vec16<T>*>(p) = raw;
}

// ---- elementwise op semantics (fp32 math) ----------------------------------------------------
// Same formulas, in the same association, as the CPU reference lambdas; these files are
// compiled with -fmad=false so that a*b+c is a rounded multiply followed by a rounded add.
// sigmoid in the reference's two-branch stable form (1/(1+e^-x) for x >= 0, e^x/(1+e^x) below),
// evaluated branch-free with e = exp(-|x|) through ex2.approx and an approximate division: about
// 5e-7 relative, inside the fp32 tolerance tier (libm results are not bit-reproducible anyway).
__device__ __forceinline__ float ew_sigmoid(float x) {
  const float e = __expf(-fabsf(x));
  return __fdividef(x >= 0.0f ? 1.0f : e, 1.0f + e);
}

// GELU for 16-bit results: 0.5 x (1 + tanh(t)) = x / (1 + e^{-2t}), with -2 t log2(e) folded into
// x (k1 + k2 x^2): five FMA-pipe instructions and two approximations (ex2, rcp) per element against
// eleven and two for the form below.  About 1e-6 relative, far inside bf16 / f16; fp32 tensors
// keep the form below.  x -> -inf side: e = +inf, 1 / inf = 0, x * 0 = -0; NaN and +-inf as the
// reference's formula gives them.
__device__ __forceinline__ float ew_gelu16(float x) {
  constexpr float k1 = -2.0f * 0.7978845608028654f * 1.4426950408889634f;
  constexpr float k2 = k1 * 0.044715f;
  const float z = x * fmaf(k2, x * x, k1);
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(z));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return x * r;
}

// The same form on two elements at once: packed fp32 pairs take one FMA-pipe instruction per two
// elements (five per pair instead of ten); the operations and their rounding are those of ew_gelu16.
__device__ __forceinline__ float2 ew_gelu16_pair(float2 x) {
  constexpr float k1 = -2.0f * 0.7978845608028654f * 1.4426950408889634f;
  constexpr float k2 = k1 * 0.044715f;
  const float2 z = __fmul2_rn(x, __ffma2_rn(make_float2(k2, k2), __fmul2_rn(x, x), make_float2(k1, k1)));
  float2 e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.x) : "f"(z.x));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.y) : "f"(z.y));
  const float2 d = __fadd2_rn(make_float2(1.0f, 1.0f), e);
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r.x) : "f"(d.x));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r.y) : "f"(d.y));
  return __fmul2_rn(x, r);
}
// sigmoid and SiLU on two elements at once: 1 / (1 + 2^(-x log2 e)) through ex2 and rcp.  The error
// is that of the two-branch form above (the rounding of the exponent's argument dominates both:
// about 6e-8 |x| relative), inside the fp32 tolerance tier.
// Large negative x: e = +inf, 1 / inf = 0, so sigmoid = 0 and silu = x * 0 = -0; -inf and NaN as the
// reference's formula gives them.
__device__ __forceinline__ float2 ew_sigmoid16_pair(float2 x) {
  const float2 z = __fmul2_rn(x, make_float2(-1.4426950408889634f, -1.4426950408889634f));
  float2 e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.x) : "f"(z.x));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.y) : "f"(z.y));
  const float2 d = __fadd2_rn(make_float2(1.0f, 1.0f), e);
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r.x) : "f"(d.x));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r.y) : "f"(d.y));
  return r;
}
// softplus on two elements at once: the series and the logarithm of ew_unary's form with packed
// fp32 pairs (six FMA-pipe instructions for the series of both elements instead of ten), the same
// cut-over points, a NaN passing through the selects.
__device__ __forceinline__ float2 ew_softplus_pair(float2 x) {
  const float2 xc = make_float2(x.x > 20.0f ? 20.0f : x.x, x.y > 20.0f ? 20.0f : x.y);
  const float2 z = __fmul2_rn(xc, make_float2(1.4426950408889634f, 1.4426950408889634f));
  float2 e, l;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.x) : "f"(z.x));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.y) : "f"(z.y));
  const float2 ne = make_float2(-e.x, -e.y);
  float2 t = __ffma2_rn(ne, make_float2(0.2f, 0.2f), make_float2(0.25f, 0.25f));
  t = __ffma2_rn(ne, t, make_float2(0.33333334f, 0.33333334f));
  t = __ffma2_rn(ne, t, make_float2(0.5f, 0.5f));
  t = __ffma2_rn(ne, t, make_float2(1.0f, 1.0f));
  const float2 series = __fmul2_rn(e, t);
  const float2 d = __fadd2_rn(make_float2(1.0f, 1.0f), e);
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(l.x) : "f"(d.x));
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(l.y) : "f"(d.y));
  const float2 lg = __fmul2_rn(l, make_float2(0.6931471805599453f, 0.6931471805599453f));
  const float rx = e.x < 0.1f ? series.x : lg.x, ry = e.y < 0.1f ? series.y : lg.y;
  return make_float2(x.x > 20.0f ? x.x : rx, x.y > 20.0f ? x.y : ry);
}
// Two values after a store to T and a load back.  For bfloat16 the packed conversion rounds both in
// one instruction and a shift and a mask bring them back.
template <typename T> __device__ __forceinline__ float2 round_pair_through(float2 v) {
  return make_float2(round_through<T>(v.x), round_through<T>(v.y));
}
template <> __device__ __forceinline__ float2 round_pair_through<__nv_bfloat16>(float2 v) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(v.x, v.y);
  const uint32_t u = *reinterpret_cast<const uint32_t*>(&h);
  return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xFFFF0000u));
}

__device__ __forceinline__ float ew_unary(int op, float x) {
  switch (op) {
    case FB200_EW_RELU: return x < 0.0f ? 0.0f : x;  // std::max(x, 0.f): NaN and -0 pass through
    case FB200_EW_SQUARE: return x * x;
    case FB200_EW_SIGMOID: return ew_sigmoid(x);
    case FB200_EW_TANH: return tanhf(x);
    case FB200_EW_RSQRT: return 1.0f / sqrtf(x);
    case FB200_EW_GELU: {
      // 0.5*x*(1+tanh(t)) == x * e^{2t}/(e^{2t}+1): no cancellation for negative t; t is clamped
      // where tanh(t) == 1 in fp32 so that e^{2t} stays finite.
      const float inner = 0.7978845608028654f * (x + 0.044715f * (x * x * x));
      const float e2 = __expf(2.0f * fminf(inner, 15.0f));
      return x * __fdividef(e2, e2 + 1.0f);
    }
    case FB200_EW_SILU: return x * ew_sigmoid(x);
    case FB200_EW_SOFTPLUS: {
      // log1p(e^x) with the reference's cut-over to x above 20.  e = e^x through ex2.approx; for
      // small e the alternating series (error below e^6/6, 2e-7 relative at the switch point), else
      // log(1 + e) through lg2.approx, whose absolute error of 4e-7 is then below 5e-6 relative.
      // Both forms are evaluated and selected: a branch per element costs more than the five FMAs.
      const float e = __expf(x > 20.0f ? 20.0f : x);   // a NaN passes through the select
      const float series = e * (1.0f - e * (0.5f - e * (0.33333334f - e * (0.25f - e * 0.2f))));
      const float lg = __logf(1.0f + e);
      const float r = e < 0.1f ? series : lg;
      return x > 20.0f ? x : r;
    }
    case FB200_EW_EXP: return expf(x);
    case FB200_EW_HEAVISIDE: return x >= 0.0f ? 1.0f : 0.0f;
    default: return x;
  }
}

// add / mul only: the form the contraction epilogues use (a third case here cost the softplus
// epilogue of a short-K GEMM a third of its speed).
__device__ __forceinline__ float ew_binary(int op, float a, float b) {
  return op == FB200_EW_ADD ? a + b : a * b;
}
// every binary code, for the elementwise chains
__device__ __forceinline__ float ew_binary_any(int op, float a, float b) {
  return op == FB200_EW_RELU_GRAD ? (a > 0.0f ? b : 0.0f) : ew_binary(op, a, b);
}
// codes a matmul / conv2d epilogue may carry
inline bool ew_epilogue_ok(int op) { return op != FB200_EW_RELU_GRAD; }

inline bool ew_is_binary(int op) { return op == FB200_EW_ADD || op == FB200_EW_MUL || op == FB200_EW_RELU_GRAD; }
inline bool ew_commutes(int op) { return op == FB200_EW_ADD || op == FB200_EW_MUL; }
inline bool ew_is_known(int op) { return op >= FB200_EW_ADD && op <= FB200_EW_RELU_GRAD; }

}  // namespace fb200
