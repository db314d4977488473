// Fused elementwise groups: ONE launch per `fused_elementwise_internal` node.
//
// The reference executes a fused group by calling each sub-kernel in turn with freshly
// allocated temporaries (src/ops/fused_elementwise_utils.cpp:122-206; CUDA wrapper
// src/backends/cuda/kernels/fused_elementwise.cpp:19-36), i.e. k launches and k-1 allocations
// per group and k times the minimal HBM traffic.  Here every external operand is read once
// with 128-bit loads, the whole chain is evaluated in registers (rounding to the tensor dtype
// between steps, exactly where the unfused chain would store), and the result is written once
// with a 128-bit store.  HBM-bound: algorithmic bytes = (n_inputs + 1) * numel * itemsize.
//
// Compiled with -fmad=false: every step is a rounded multiply or a rounded add, as in the CPU
// reference built with -ffp-contract=off.
#include "common.cuh"
#include "epilogue.cuh"

namespace fb200 {

struct ChainDesc {
  int n_ops;
  int n_inputs;
  int ops[FB200_MAX_CHAIN];
  int ext[FB200_MAX_CHAIN];  // index of the external operand a binary step reads, else -1
  const void* in[FB200_MAX_CHAIN_INPUTS];
};

template <int NIN, int W>
__device__ __forceinline__ void pick(const float (&vals)[NIN][W], int idx, float (&out)[W]) {
#pragma unroll
  for (int j = 0; j < NIN; ++j) {
    if (j == idx) {
#pragma unroll
      for (int e = 0; e < W; ++e) out[e] = vals[j][e];
    }
  }
}

// One step of a chain over a register vector, its result rounded to T (ROUND) as the unfused
// chain's store would.
template <typename T, int NIN, int W, bool ROUND>
__device__ __forceinline__ void chain_vec_step(const ChainDesc& d, int s, const float (&vals)[NIN][W],
                                               float (&cur)[W]) {
  const int op = d.ops[s];
  if (d.ext[s] >= 0) {
    float rhs[W];
    pick<NIN, W>(vals, d.ext[s], rhs);
    if (op == FB200_EW_ADD || op == FB200_EW_MUL) {
      ew_binary_round_vec<T, W, ROUND>(op, cur, rhs);
    } else {
#pragma unroll
      for (int e = 0; e < W; ++e) {
        const float y = ew_binary_any(op, cur[e], rhs[e]);
        cur[e] = ROUND ? round_through<T>(y) : y;
      }
    }
  } else {
    ew_unary_vec<T, W, ROUND>(op, cur);
  }
}

// NIN = number of external inputs held in registers (compile-time for register allocation).
template <typename T, int NIN>
__global__ void __launch_bounds__(256)
fused_chain_kernel(ChainDesc d, T* __restrict__ out, int64_t n_vec, int64_t numel) {
  constexpr int W = 16 / sizeof(T);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < n_vec;
       v += stride) {
    float vals[NIN][W];
#pragma unroll
    for (int j = 0; j < NIN; ++j) {
      if (j < d.n_inputs) load_vec<T>(static_cast<const T*>(d.in[j]) + v * W, vals[j]);
    }
    float cur[W];
#pragma unroll
    for (int e = 0; e < W; ++e) cur[e] = vals[0][e];
#pragma unroll 1
    for (int s = 0; s < d.n_ops; ++s) chain_vec_step<T, NIN, W, true>(d, s, vals, cur);
    store_vec<T>(out + v * W, cur);
  }
  // Ragged tail (numel % W elements) and unaligned buffers: scalar path, first CTA only.
  if (blockIdx.x == 0) {
    for (int64_t i = n_vec * W + threadIdx.x; i < numel; i += blockDim.x) {
      float cur = to_f32(static_cast<const T*>(d.in[0])[i]);
      for (int s = 0; s < d.n_ops; ++s) {
        const int op = d.ops[s];
        if (d.ext[s] >= 0) {
          const float rhs = to_f32(static_cast<const T*>(d.in[d.ext[s]])[i]);
          cur = round_through<T>(ew_binary_any(op, cur, rhs));
        } else {
          cur = round_through<T>((sizeof(T) == 2 && op == FB200_EW_GELU) ? ew_gelu16(cur) : ew_unary(op, cur));
        }
      }
      out[i] = from_f32<T>(cur);
    }
  }
}

template <typename I>
__global__ void __launch_bounds__(256)
int_add_kernel(const I* __restrict__ a, const I* __restrict__ b, I* __restrict__ out, int64_t n) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    out[i] = a[i] + b[i];
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
bias_add_kernel(const T* __restrict__ x, const T* __restrict__ bias, T* __restrict__ out,
                int64_t rows, int64_t cols) {
  constexpr int W = 16 / sizeof(T);
  const int64_t vec_per_row = cols / W;  // host guarantees cols % W == 0 on this path
  const int64_t n_vec = rows * vec_per_row;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < n_vec;
       v += stride) {
    const int64_t c = (v % vec_per_row) * W;
    float a[W], b[W];
    load_vec<T>(x + v * W, a);
    load_vec<T>(bias + c, b);
#pragma unroll
    for (int e = 0; e < W; ++e) a[e] = a[e] + b[e];
    store_vec<T>(out + v * W, a);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
bias_add_scalar_kernel(const T* __restrict__ x, const T* __restrict__ bias, T* __restrict__ out,
                       int64_t rows, int64_t cols) {
  const int64_t n = rows * cols;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    out[i] = from_f32<T>(to_f32(x[i]) + to_f32(bias[i % cols]));
  }
}

template <typename T, int NIN>
static int launch_chain_n(const ChainDesc& d, void* out, int64_t numel, bool vec_ok,
                          cudaStream_t s) {
  constexpr int W = 16 / sizeof(T);
  const int64_t n_vec = vec_ok ? numel / W : 0;
  const int grid = grid_for(n_vec > 0 ? n_vec : numel, 256, 8);
  fused_chain_kernel<T, NIN><<<grid, 256, 0, s>>>(d, static_cast<T*>(out), n_vec, numel);
  return after_launch("fused_chain_kernel");
}

template <typename T>
static int launch_chain(const ChainDesc& d, void* out, int64_t numel, bool vec_ok, cudaStream_t s) {
  switch (d.n_inputs) {
    case 1: return launch_chain_n<T, 1>(d, out, numel, vec_ok, s);
    case 2: return launch_chain_n<T, 2>(d, out, numel, vec_ok, s);
    case 3: return launch_chain_n<T, 3>(d, out, numel, vec_ok, s);
    case 4: return launch_chain_n<T, 4>(d, out, numel, vec_ok, s);
    default: return launch_chain_n<T, FB200_MAX_CHAIN_INPUTS>(d, out, numel, vec_ok, s);
  }
}

}  // namespace fb200

using namespace fb200;

// One launch: a chain of at most FB200_MAX_CHAIN steps.
static int fused_chain_segment(const void* const* inputs, int n_inputs, void* out, int64_t numel,
                               int dtype, const int* ops, const int* arities, int n_ops,
                               fb200_stream stream) {
  if (n_ops < 1 || n_ops > FB200_MAX_CHAIN) {
    return set_error(FB200_INVALID_ARGUMENT,
                     "fused_elementwise: chain length %d outside [1, %d]", n_ops, FB200_MAX_CHAIN);
  }
  if (inputs == nullptr || ops == nullptr || arities == nullptr) {
    return set_error(FB200_INVALID_ARGUMENT, "fused_elementwise: null argument");
  }
  if (numel < 0) return set_error(FB200_INVALID_ARGUMENT, "fused_elementwise: negative numel");
  int expected_inputs = 0;
  ChainDesc d{};
  d.n_ops = n_ops;
  for (int s = 0; s < n_ops; ++s) {
    if (!ew_is_known(ops[s])) {
      return set_error(FB200_UNIMPLEMENTED, "fused_elementwise: unknown sub-op code %d", ops[s]);
    }
    const int want = ew_is_binary(ops[s]) ? 2 : 1;
    if (arities[s] != want) {
      return set_error(FB200_INVALID_ARGUMENT,
                       "fused_elementwise: sub-op %d (code %d) has arity %d, expected %d", s,
                       ops[s], arities[s], want);
    }
    d.ops[s] = ops[s];
    if (s == 0) {
      d.ext[s] = want == 2 ? 1 : -1;
      expected_inputs = want;
    } else {
      d.ext[s] = want == 2 ? expected_inputs : -1;
      expected_inputs += want - 1;
    }
  }
  // sum(arities) - (segments - 1) == number of external inputs
  if (expected_inputs != n_inputs || n_inputs > FB200_MAX_CHAIN_INPUTS) {
    return set_error(FB200_INVALID_ARGUMENT,
                     "fused_elementwise: chain needs %d external inputs, got %d", expected_inputs,
                     n_inputs);
  }
  d.n_inputs = n_inputs;
  if (numel == 0) return FB200_OK;
  if (out == nullptr) return set_error(FB200_INVALID_ARGUMENT, "fused_elementwise: null output");
  bool vec_ok = aligned16(out);
  for (int i = 0; i < n_inputs; ++i) {
    if (inputs[i] == nullptr) {
      return set_error(FB200_INVALID_ARGUMENT, "fused_elementwise: input %d is null", i);
    }
    d.in[i] = inputs[i];
    vec_ok = vec_ok && aligned16(inputs[i]);
  }
  cudaStream_t s = as_stream(stream);
  if (dtype == FB200_I32 || dtype == FB200_I64) {
    if (n_ops != 1 || ops[0] != FB200_EW_ADD) {
      return set_error(FB200_UNIMPLEMENTED,
                       "fused_elementwise: integer dtypes support a single 'add' only");
    }
    const int grid = grid_for(numel, 256, 8);
    if (dtype == FB200_I32) {
      int_add_kernel<int32_t><<<grid, 256, 0, s>>>(static_cast<const int32_t*>(inputs[0]),
                                                   static_cast<const int32_t*>(inputs[1]),
                                                   static_cast<int32_t*>(out), numel);
    } else {
      int_add_kernel<int64_t><<<grid, 256, 0, s>>>(static_cast<const int64_t*>(inputs[0]),
                                                   static_cast<const int64_t*>(inputs[1]),
                                                   static_cast<int64_t*>(out), numel);
    }
    return after_launch("int_add_kernel");
  }
  switch (dtype) {
    case FB200_F32: return launch_chain<float>(d, out, numel, vec_ok, s);
    case FB200_BF16: return launch_chain<__nv_bfloat16>(d, out, numel, vec_ok, s);
    case FB200_F16: return launch_chain<__half>(d, out, numel, vec_ok, s);
    default:
      return set_error(FB200_INVALID_ARGUMENT,
                       "fused_elementwise: dtype code %d is not float32/float16/bfloat16", dtype);
  }
}

// The reference's fusion pass builds chains of any length (src/compiler/passes/operator_fusion.cpp:
// 140-157) and its executor runs them one sub-kernel at a time.  Here a group of up to
// FB200_MAX_CHAIN steps is one launch; a longer group runs as successive launches of at most that
// many steps, each continuing from `out` as its first operand (in place: every element is read and
// written by the same thread), with the same rounding point at every step as the unfused ops.
extern "C" int fb200_fused_elementwise(const void* const* inputs, int n_inputs, void* out,
                                       int64_t numel, int dtype, const int* ops,
                                       const int* arities, int n_ops, fb200_stream stream) {
  if (n_ops < 1) return set_error(FB200_INVALID_ARGUMENT, "fused_elementwise: empty chain");
  if (inputs == nullptr || ops == nullptr || arities == nullptr) {
    return set_error(FB200_INVALID_ARGUMENT, "fused_elementwise: null argument");
  }
  if (n_ops <= FB200_MAX_CHAIN) {
    return fused_chain_segment(inputs, n_inputs, out, numel, dtype, ops, arities, n_ops, stream);
  }
  int total = 0;
  for (int s = 0; s < n_ops; ++s) {
    if (arities[s] != 1 && arities[s] != 2) {
      return set_error(FB200_INVALID_ARGUMENT, "fused_elementwise: sub-op %d has arity %d", s, arities[s]);
    }
    total += s == 0 ? arities[s] : arities[s] - 1;
  }
  if (total != n_inputs) {
    return set_error(FB200_INVALID_ARGUMENT, "fused_elementwise: chain needs %d external inputs, got %d", total, n_inputs);
  }
  int next_input = 0;
  for (int s0 = 0; s0 < n_ops; s0 += FB200_MAX_CHAIN) {
    const int count = n_ops - s0 < FB200_MAX_CHAIN ? n_ops - s0 : FB200_MAX_CHAIN;
    const void* seg[FB200_MAX_CHAIN_INPUTS];
    int n_seg = 0;
    if (s0 > 0) seg[n_seg++] = out;   // the running value
    for (int s = s0; s < s0 + count; ++s) {
      const int take = s == 0 ? arities[s] : arities[s] - 1;
      for (int t = 0; t < take; ++t) seg[n_seg++] = inputs[next_input++];
    }
    if (int rc = fused_chain_segment(seg, n_seg, out, numel, dtype, ops + s0, arities + s0, count, stream)) return rc;
  }
  return FB200_OK;
}

extern "C" int fb200_bias_add(const void* x, const void* bias, void* out, int64_t rows,
                              int64_t cols, int dtype, fb200_stream stream) {
  if (rows < 0 || cols < 0) return set_error(FB200_INVALID_ARGUMENT, "bias_add: negative shape");
  if (rows == 0 || cols == 0) return FB200_OK;
  if (x == nullptr || bias == nullptr || out == nullptr) {
    return set_error(FB200_INVALID_ARGUMENT, "bias_add: null argument");
  }
  cudaStream_t s = as_stream(stream);
  const bool al = aligned16(x) && aligned16(bias) && aligned16(out);
  auto run = [&](auto tag) -> int {
    using T = decltype(tag);
    constexpr int W = 16 / sizeof(T);
    if (al && cols % W == 0) {
      const int grid = grid_for(rows * cols / W, 256, 8);
      bias_add_kernel<T><<<grid, 256, 0, s>>>(static_cast<const T*>(x), static_cast<const T*>(bias),
                                              static_cast<T*>(out), rows, cols);
    } else {
      const int grid = grid_for(rows * cols, 256, 8);
      bias_add_scalar_kernel<T><<<grid, 256, 0, s>>>(static_cast<const T*>(x),
                                                     static_cast<const T*>(bias),
                                                     static_cast<T*>(out), rows, cols);
    }
    return after_launch("bias_add_kernel");
  };
  switch (dtype) {
    case FB200_F32: return run(float{});
    case FB200_BF16: return run(__nv_bfloat16{});
    case FB200_F16: return run(__half{});
    default: return set_error(FB200_INVALID_ARGUMENT, "bias_add: unsupported dtype code %d", dtype);
  }
}
