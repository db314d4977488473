// Epilogue chain shared by the matmul and conv2d kernels: a short list of elementwise steps
// applied to the fp32 accumulator before the single store.  Binary steps read their second
// operand from a tensor of the output's shape (FULL), a per-column vector (COL) or a
// per-row / per-channel vector (ROW).  Between steps the value is rounded to the tensor dtype,
// which is where the unfused chain of the reference would have stored it
// (src/ops/fused_elementwise_utils.cpp:122-206).
#pragma once

#include "common.cuh"

namespace fb200 {

struct EpilogueDev {
  int n_ops;
  int ops[FB200_MAX_CHAIN];
  int modes[FB200_MAX_CHAIN];
  const void* operands[FB200_MAX_CHAIN];
};

// Validates a host-side epilogue description and copies it into the by-value kernel argument.
inline int make_epilogue(const fb200_epilogue* e, EpilogueDev* out, const char* who) {
  out->n_ops = 0;
  if (e == nullptr) return FB200_OK;
  if (e->n_ops < 0 || e->n_ops > FB200_MAX_CHAIN) {
    return set_error(FB200_INVALID_ARGUMENT, "%s: epilogue length %d outside [0, %d]", who,
                     e->n_ops, FB200_MAX_CHAIN);
  }
  for (int i = 0; i < e->n_ops; ++i) {
    if (!ew_is_known(e->ops[i]) || !ew_epilogue_ok(e->ops[i])) {
      return set_error(FB200_UNIMPLEMENTED, "%s: op code %d cannot be an epilogue step", who, e->ops[i]);
    }
    if (ew_is_binary(e->ops[i])) {
      if (e->operands[i] == nullptr) {
        return set_error(FB200_INVALID_ARGUMENT, "%s: epilogue step %d is binary but has no operand",
                         who, i);
      }
      if (e->modes[i] < FB200_OPERAND_FULL || e->modes[i] > FB200_OPERAND_ROW) {
        return set_error(FB200_INVALID_ARGUMENT, "%s: epilogue step %d has unknown operand mode %d",
                         who, i, e->modes[i]);
      }
    }
    out->ops[i] = e->ops[i];
    out->modes[i] = e->modes[i];
    out->operands[i] = ew_is_binary(e->ops[i]) ? e->operands[i] : nullptr;
  }
  out->n_ops = e->n_ops;
  return FB200_OK;
}

// One binary step over W values, the result rounded through T.  Sums and products go in packed
// fp32 pairs (one FMA-pipe instruction per two elements and, for 16-bit tensors, one packed
// conversion); the arithmetic and its rounding are those of the element-wise form.
// ROUND = false leaves the fp32 result unrounded for a caller that stores it to T next (the
// store's conversion is then the one rounding).
template <typename T, int W, bool ROUND = true>
__device__ __forceinline__ void ew_binary_round_vec(int op, float* v, const float (&rhs)[W]) {
  if (W % 2 == 0 && (op == FB200_EW_ADD || op == FB200_EW_MUL)) {
#pragma unroll
    for (int e = 0; e < W; e += 2) {
      const float2 a = make_float2(v[e], v[e + 1]), b = make_float2(rhs[e], rhs[e + 1]);
      float2 y = op == FB200_EW_ADD ? __fadd2_rn(a, b) : __fmul2_rn(a, b);
      if (ROUND) y = round_pair_through<T>(y);
      v[e] = y.x;
      v[e + 1] = y.y;
    }
    return;
  }
#pragma unroll
  for (int e = 0; e < W; ++e) {
    const float y = ew_binary(op, v[e], rhs[e]);
    v[e] = ROUND ? round_through<T>(y) : y;
  }
}

// One unary step over a register vector, with the op switch hoisted out of the element loop.
template <typename T, int NV, bool ROUND = true>
__device__ __forceinline__ void ew_unary_vec(int op, float (&v)[NV]) {
  // SiLU and sigmoid (every dtype) and GELU of 16-bit tensors on packed fp32 pairs
  if (NV % 2 == 0 && (op == FB200_EW_SILU || op == FB200_EW_SIGMOID || op == FB200_EW_SOFTPLUS ||
                      (sizeof(T) == 2 && op == FB200_EW_GELU))) {
    auto pairs = [&](auto&& f) {
#pragma unroll
      for (int j = 0; j < NV; j += 2) {
        float2 y = f(make_float2(v[j], v[j + 1]));
        if (ROUND) y = round_pair_through<T>(y);
        v[j] = y.x;
        v[j + 1] = y.y;
      }
    };
    if (op == FB200_EW_GELU) {
      pairs([](float2 x) { return ew_gelu16_pair(x); });
    } else if (op == FB200_EW_SILU) {
      pairs([](float2 x) { return __fmul2_rn(x, ew_sigmoid16_pair(x)); });
    } else if (op == FB200_EW_SOFTPLUS) {
      pairs([](float2 x) { return ew_softplus_pair(x); });
    } else {
      pairs([](float2 x) { return ew_sigmoid16_pair(x); });
    }
    return;
  }
  if (sizeof(T) == 2 && op == FB200_EW_GELU) {
#pragma unroll
    for (int j = 0; j < NV; ++j) v[j] = ROUND ? round_through<T>(ew_gelu16(v[j])) : ew_gelu16(v[j]);
    return;
  }
  switch (op) {
#define FB200_UNARY_CASE(code)                                                     \
  case code:                                                                       \
    _Pragma("unroll") for (int j = 0; j < NV; ++j) v[j] = ROUND ? round_through<T>(ew_unary(code, v[j])) : ew_unary(code, v[j]); \
    break;
    FB200_UNARY_CASE(FB200_EW_RELU)
    FB200_UNARY_CASE(FB200_EW_SQUARE)
    FB200_UNARY_CASE(FB200_EW_SIGMOID)
    FB200_UNARY_CASE(FB200_EW_TANH)
    FB200_UNARY_CASE(FB200_EW_RSQRT)
    FB200_UNARY_CASE(FB200_EW_GELU)
    FB200_UNARY_CASE(FB200_EW_SILU)
    FB200_UNARY_CASE(FB200_EW_SOFTPLUS)
    FB200_UNARY_CASE(FB200_EW_EXP)
    FB200_UNARY_CASE(FB200_EW_HEAVISIDE)
#undef FB200_UNARY_CASE
    default: break;
  }
}

template <typename T>
__device__ __forceinline__ float apply_epilogue(const EpilogueDev& e, float v, int64_t full_idx,
                                                int64_t col_idx, int64_t row_idx) {
  v = round_through<T>(v);  // the contraction's own store
#pragma unroll
  for (int s = 0; s < FB200_MAX_CHAIN; ++s) {
    if (s < e.n_ops) {
      const int op = e.ops[s];
      if (e.operands[s] != nullptr) {
        const int64_t idx = e.modes[s] == FB200_OPERAND_FULL ? full_idx
                            : e.modes[s] == FB200_OPERAND_COL ? col_idx : row_idx;
        const float rhs = to_f32(static_cast<const T*>(e.operands[s])[idx]);
        v = round_through<T>(ew_binary(op, v, rhs));
      } else {
        v = round_through<T>(ew_unary(op, v));
      }
    }
  }
  return v;
}

}  // namespace fb200
