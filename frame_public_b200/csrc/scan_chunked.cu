// selective_scan for FEW, LONG rows: the time axis is cut into chunks that run in parallel.
//
// Semantics: src/backends/cpu/kernels/sequence.cpp:95-106 (state = a*state + b*x,
// out = c*state + d*x, state0 = 0 per row).  With fewer rows than the GPU has warps, one warp per
// row (selective_scan_steps_kernel) leaves most SMs idle; here every (row, chunk) pair gets a warp:
//   pass 1  each warp folds its chunk into one affine pair (A, B) with h_out = A*h_in + B and writes
//           it to a scratch array of rows*chunks pairs (reads a, b, x);
//   pass 2  each warp combines the pairs of the chunks before its own (a warp-shuffle scan over the
//           scratch entries) to get the state entering its chunk, then scans the chunk and writes
//           the outputs (reads all five operands).
// HBM traffic is 9 element-streams for 6 algorithmic ones (a, b, x are read twice), so the ceiling
// is two thirds of the copy bandwidth.  The association of the recurrence differs from the CPU's
// sequential order: results agree within the fp32 / bf16 tolerance tier, not bit for bit.
// The scratch (8 bytes per (row, chunk)) is global memory beyond the op's inputs and outputs; the
// regular entry point takes it from the stream-ordered allocator.
#include <mutex>

#include "common.cuh"

namespace fb200 {

struct Affine2 { float a, b; };
__device__ __forceinline__ Affine2 combine2(Affine2 first, Affine2 second) {
  return Affine2{second.a * first.a, second.a * first.b + second.b};
}

__device__ __forceinline__ Affine2 warp_inclusive_scan(Affine2 v, int lane) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float pa = __shfl_up_sync(0xffffffffu, v.a, o);
    const float pb = __shfl_up_sync(0xffffffffu, v.b, o);
    if (lane >= o) v = combine2(Affine2{pa, pb}, v);
  }
  return v;
}

constexpr int kChunkWarps = 4;
constexpr int kChunkThreads = kChunkWarps * 32;

// Pass 1: summary[row*chunks + chunk] = affine composition of the chunk's steps.
template <typename T>
__global__ void __launch_bounds__(kChunkThreads)
scan_chunk_summary_kernel(const T* __restrict__ x, const T* __restrict__ a, const T* __restrict__ b,
                          float2* __restrict__ summary, int64_t rows, int64_t steps, int64_t chunks,
                          int64_t chunk_len) {
  constexpr int W = 16 / sizeof(T);
  const int lane = threadIdx.x & 31;
  const int64_t total = rows * chunks;
  const int64_t total_warps = static_cast<int64_t>(gridDim.x) * kChunkWarps;
  for (int64_t job = static_cast<int64_t>(blockIdx.x) * kChunkWarps + (threadIdx.x >> 5); job < total;
       job += total_warps) {
    const int64_t row = job / chunks;
    const int64_t chunk = job - row * chunks;
    const int64_t t_begin = chunk * chunk_len;
    const int64_t t_end = t_begin + chunk_len < steps ? t_begin + chunk_len : steps;
    const int64_t base = row * steps;
    Affine2 carry{1.0f, 0.0f};
    // The loads of pass k + 1 are issued before pass k is folded: without that every pass paid the
    // full memory latency (a warp-wide scan needs its operands at once) and the kernel ran at a third
    // of what its traffic allows.
    float xv[W], av[W], bv[W];
    auto fetch = [&](int64_t t0, float (&fx)[W], float (&fa)[W], float (&fb)[W]) {
      const int64_t t = t0 + static_cast<int64_t>(lane) * W;
      if (t0 < t_end && t + W <= t_end) {
        load_vec<T>(x + base + t, fx);
        load_vec<T>(a + base + t, fa);
        load_vec<T>(b + base + t, fb);
      } else {
#pragma unroll
        for (int e = 0; e < W; ++e) { fx[e] = 0.0f; fa[e] = 1.0f; fb[e] = 0.0f; }   // the identity step
      }
    };
    fetch(t_begin, xv, av, bv);
    for (int64_t t0 = t_begin; t0 < t_end; t0 += 32 * W) {
      float nx[W], na[W], nb[W];
      fetch(t0 + 32 * W, nx, na, nb);
      Affine2 seg{1.0f, 0.0f};
#pragma unroll
      for (int e = 0; e < W; ++e) seg = combine2(seg, Affine2{av[e], bv[e] * xv[e]});
      const Affine2 inc = warp_inclusive_scan(seg, lane);
      const Affine2 whole{__shfl_sync(0xffffffffu, inc.a, 31), __shfl_sync(0xffffffffu, inc.b, 31)};
      carry = combine2(carry, whole);
#pragma unroll
      for (int e = 0; e < W; ++e) { xv[e] = nx[e]; av[e] = na[e]; bv[e] = nb[e]; }
    }
    if (lane == 0) summary[job] = make_float2(carry.a, carry.b);
  }
}

// Pass 2: state entering the chunk from the summaries before it, then the chunk itself.
template <typename T>
__global__ void __launch_bounds__(kChunkThreads)
scan_chunk_apply_kernel(const T* __restrict__ x, const T* __restrict__ a, const T* __restrict__ b,
                        const T* __restrict__ c, const T* __restrict__ d, T* __restrict__ out,
                        const float2* __restrict__ summary, int64_t rows, int64_t steps,
                        int64_t chunks, int64_t chunk_len) {
  constexpr int W = 16 / sizeof(T);
  const int lane = threadIdx.x & 31;
  const int64_t total = rows * chunks;
  const int64_t total_warps = static_cast<int64_t>(gridDim.x) * kChunkWarps;
  for (int64_t job = static_cast<int64_t>(blockIdx.x) * kChunkWarps + (threadIdx.x >> 5); job < total;
       job += total_warps) {
    const int64_t row = job / chunks;
    const int64_t chunk = job - row * chunks;
    // prefix over chunks [0, chunk) of this row, 32 at a time
    Affine2 prefix{1.0f, 0.0f};
    for (int64_t c0 = 0; c0 < chunk; c0 += 32) {
      Affine2 v{1.0f, 0.0f};
      if (c0 + lane < chunk) {
        const float2 s = summary[row * chunks + c0 + lane];
        v = Affine2{s.x, s.y};
      }
      const Affine2 inc = warp_inclusive_scan(v, lane);
      const Affine2 whole{__shfl_sync(0xffffffffu, inc.a, 31), __shfl_sync(0xffffffffu, inc.b, 31)};
      prefix = combine2(prefix, whole);
    }
    float carry = prefix.b;  // the row starts from state 0
    const int64_t t_begin = chunk * chunk_len;
    const int64_t t_end = t_begin + chunk_len < steps ? t_begin + chunk_len : steps;
    const int64_t base = row * steps;
    float xv[W], av[W], bv[W], cv[W], dv[W];
    auto fetch = [&](int64_t t0, float (&fx)[W], float (&fa)[W], float (&fb)[W], float (&fc)[W], float (&fd)[W]) {
      const int64_t t = t0 + static_cast<int64_t>(lane) * W;
      if (t0 < t_end && t + W <= t_end) {
        load_vec<T>(x + base + t, fx);
        load_vec<T>(a + base + t, fa);
        load_vec<T>(b + base + t, fb);
        load_vec<T>(c + base + t, fc);
        load_vec<T>(d + base + t, fd);
      } else {
#pragma unroll
        for (int e = 0; e < W; ++e) { fx[e] = 0.0f; fa[e] = 1.0f; fb[e] = 0.0f; fc[e] = 0.0f; fd[e] = 0.0f; }
      }
    };
    fetch(t_begin, xv, av, bv, cv, dv);
    for (int64_t t0 = t_begin; t0 < t_end; t0 += 32 * W) {
      const int64_t t = t0 + static_cast<int64_t>(lane) * W;
      const bool in = t + W <= t_end;
      // the next pass's loads go out before this pass is scanned (see the summary kernel)
      float nx[W], na[W], nb[W], nc[W], nd[W];
      fetch(t0 + 32 * W, nx, na, nb, nc, nd);
      Affine2 seg{1.0f, 0.0f};
#pragma unroll
      for (int e = 0; e < W; ++e) seg = combine2(seg, Affine2{av[e], bv[e] * xv[e]});
      const Affine2 inc = warp_inclusive_scan(seg, lane);
      float ea = __shfl_up_sync(0xffffffffu, inc.a, 1);
      float eb = __shfl_up_sync(0xffffffffu, inc.b, 1);
      if (lane == 0) { ea = 1.0f; eb = 0.0f; }
      float state = ea * carry + eb;
      float yv[W];
#pragma unroll
      for (int e = 0; e < W; ++e) {
        state = av[e] * state + bv[e] * xv[e];
        yv[e] = cv[e] * state + dv[e] * xv[e];
      }
      if (in) store_vec<T>(out + base + t, yv);
      const float la = __shfl_sync(0xffffffffu, inc.a, 31);
      const float lb = __shfl_sync(0xffffffffu, inc.b, 31);
      carry = la * carry + lb;
#pragma unroll
      for (int e = 0; e < W; ++e) { xv[e] = nx[e]; av[e] = na[e]; bv[e] = nb[e]; cv[e] = nc[e]; dv[e] = nd[e]; }
    }
  }
}

// Chooses the chunking for `rows` rows of `steps` steps: enough (row, chunk) warps to fill the
// GPU, chunks a multiple of one warp-wide vector pass.  Returns the number of chunks (1 = do not
// chunk).
int64_t scan_chunking(int64_t rows, int64_t steps, int elems_per_vec, int64_t* chunk_len) {
  const int64_t pass = 32 * static_cast<int64_t>(elems_per_vec);
  const int64_t want_warps = static_cast<int64_t>(kNumSMs) * 32;
  int64_t chunks = (want_warps + rows - 1) / rows;
  const int64_t max_chunks = steps / (4 * pass);   // at least four vector passes per chunk
  if (chunks > max_chunks) chunks = max_chunks;
  if (chunks < 2) { *chunk_len = steps; return 1; }
  int64_t len = (steps + chunks - 1) / chunks;
  len = (len + pass - 1) / pass * pass;
  *chunk_len = len;
  return (steps + len - 1) / len;
}

template <typename T>
int scan_chunked_launch(const void* x, const void* a, const void* b, const void* c, const void* d,
                        void* out, int64_t rows, int64_t steps, int64_t chunks, int64_t chunk_len,
                        float2* scratch, cudaStream_t s) {
  const int64_t jobs = rows * chunks;
  const int grid = grid_for(jobs * 32, kChunkThreads, 8);
  if (chunks > 1) {   // with one chunk per row the apply pass reads no summary: nothing to fold
    scan_chunk_summary_kernel<T><<<grid, kChunkThreads, 0, s>>>(
        static_cast<const T*>(x), static_cast<const T*>(a), static_cast<const T*>(b), scratch, rows, steps,
        chunks, chunk_len);
    if (int rc = after_launch("scan_chunk_summary_kernel")) return rc;
  }
  scan_chunk_apply_kernel<T><<<grid, kChunkThreads, 0, s>>>(
      static_cast<const T*>(x), static_cast<const T*>(a), static_cast<const T*>(b),
      static_cast<const T*>(c), static_cast<const T*>(d), static_cast<T*>(out), scratch, rows, steps,
      chunks, chunk_len);
  return after_launch("scan_chunk_apply_kernel");
}

template int scan_chunked_launch<float>(const void*, const void*, const void*, const void*, const void*,
                                        void*, int64_t, int64_t, int64_t, int64_t, float2*, cudaStream_t);
template int scan_chunked_launch<__nv_bfloat16>(const void*, const void*, const void*, const void*,
                                                const void*, void*, int64_t, int64_t, int64_t, int64_t,
                                                float2*, cudaStream_t);
template int scan_chunked_launch<__half>(const void*, const void*, const void*, const void*, const void*,
                                         void*, int64_t, int64_t, int64_t, int64_t, float2*, cudaStream_t);

}  // namespace fb200

// ---- the same scan without any allocation ----------------------------------------------------------
// Some callers may not allocate device memory when they run this op: a host that captures its work
// into a CUDA graph, or one that sized every device buffer up front (Frame's memory planner does
// exactly that for a compiled graph) and treats a run-time allocation as a bug.  For them the
// scratch of the two-pass scan lives in this fixed array instead of coming from the stream-ordered
// allocator.  It is part of the library image: every GPU that loads the library carries these
// 512 KiB until the process exits.
namespace fb200 {

constexpr int64_t kStaticScanPairs = 65536;  // (row, chunk) pairs the fixed scratch can hold
static __device__ __align__(256) float2 g_static_scan_scratch[kStaticScanPairs];

// In host code the name above is only a handle for the symbol, not a device address; the address
// each device gave the array is looked up once per device and kept here.
static float2* g_static_scan_ptr[64] = {nullptr};
static std::mutex g_static_scan_mu;

static int static_scan_scratch(float2** ptr) {
  int device = 0;
  FB200_CUDA_OK(cudaGetDevice(&device));
  if (device < 0 || device >= 64) return set_error(FB200_INVALID_ARGUMENT, "device index %d", device);
  std::lock_guard<std::mutex> lock(g_static_scan_mu);
  if (g_static_scan_ptr[device] == nullptr) {
    float2* p = nullptr;
    FB200_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_scan_scratch));
    g_static_scan_ptr[device] = p;
  }
  *ptr = g_static_scan_ptr[device];
  return FB200_OK;
}

}  // namespace fb200

using namespace fb200;

extern "C" int fb200_selective_scan_noalloc(const void* x, const void* a, const void* b,
                                            const void* c, const void* d, void* out, int64_t rows,
                                            int64_t steps, int dtype, fb200_stream stream) {
  if (rows < 0) return set_error(FB200_INVALID_ARGUMENT, "selective_scan_noalloc: negative rows");
  if (steps < 1) {
    return set_error(FB200_INVALID_ARGUMENT,
                     "selective_scan_noalloc: the last dimension (steps) must be >= 1, got %lld",
                     static_cast<long long>(steps));
  }
  if (rows == 0) return FB200_OK;
  if (!x || !a || !b || !c || !d || !out) {
    return set_error(FB200_INVALID_ARGUMENT, "selective_scan_noalloc: null argument");
  }
  if (dtype != FB200_F32 && dtype != FB200_BF16 && dtype != FB200_F16) {
    return set_error(FB200_INVALID_ARGUMENT,
                     "selective_scan_noalloc: dtype code %d is not float32/float16/bfloat16", dtype);
  }
  const int w = 16 / itemsize_of(dtype);
  if (steps % w != 0 || !aligned16(x) || !aligned16(a) || !aligned16(b) || !aligned16(c) ||
      !aligned16(d) || !aligned16(out)) {
    return set_error(FB200_INVALID_ARGUMENT,
                     "selective_scan_noalloc: needs 16-byte aligned operands and steps a multiple of %d", w);
  }
  if (rows > kStaticScanPairs) {
    return set_error(FB200_INVALID_ARGUMENT,
                     "selective_scan_noalloc: %lld rows exceed the fixed scratch of %lld (row, chunk) "
                     "pairs; use fb200_selective_scan",
                     static_cast<long long>(rows), static_cast<long long>(kStaticScanPairs));
  }
  int64_t chunk_len = steps;
  int64_t chunks = scan_chunking(rows, steps, w, &chunk_len);
  const int64_t pass = 32 * static_cast<int64_t>(w);
  while (rows * chunks > kStaticScanPairs) {   // fewer, longer chunks until the pairs fit
    chunk_len = (chunk_len * 2 + pass - 1) / pass * pass;
    chunks = (steps + chunk_len - 1) / chunk_len;
  }
  float2* scratch = nullptr;
  if (int rc = static_scan_scratch(&scratch)) return rc;
  cudaStream_t s = as_stream(stream);
  switch (dtype) {
    case FB200_F32: return scan_chunked_launch<float>(x, a, b, c, d, out, rows, steps, chunks, chunk_len, scratch, s);
    case FB200_BF16: return scan_chunked_launch<__nv_bfloat16>(x, a, b, c, d, out, rows, steps, chunks, chunk_len, scratch, s);
    default: return scan_chunked_launch<__half>(x, a, b, c, d, out, rows, steps, chunks, chunk_len, scratch, s);
  }
}
