// selective_scan and the fused Mamba scan.
//
// selective_scan follows src/backends/cpu/kernels/sequence.cpp:95-106: for every row (all
// leading axes flattened), time on the last axis, fp32 state starting at 0,
//     state = a*state + b*x ;  out = c*state + d*x
// and replaces the reference CUDA path, which launches three kernels PER ROW from a host loop
// and then synchronises the stream (src/backends/cuda/kernels/sequence.cu:170-217).
//
// Two single-launch kernels, both HBM-bound (algorithmic bytes = 6 * rows * steps * itemsize):
//  * rows_kernel — many rows.  A warp owns 32 rows; the five operands of a 32-step chunk are
//    read with 128-bit loads (each row segment is contiguous), transposed through padded shared
//    memory so that lane r then walks row r sequentially, conflict-free, in exactly the CPU's
//    order and association (compiled with -fmad=false: bit-identical to the CPU reference for
//    fp32), and the outputs go back through shared memory to 128-bit stores.
//  * steps_kernel — few, long rows.  A warp owns one row; each lane takes one 128-bit vector of
//    a chunk, folds it into an affine pair (A,B) with h_out = A*h_in + B, the pairs are combined
//    with a warp-shuffle inclusive scan, the carry moves to the next chunk through a register.
//    The association differs from the CPU's, so this kernel is tolerance-exact, not bit-exact.
//
// (The fused Mamba scan, a new op without a reference counterpart, lives in mamba_scan.cu.)
#include "common.cuh"

namespace fb200 {

constexpr int kScanWarps = 4;
constexpr int kScanThreads = kScanWarps * 32;
constexpr int kChunk = 32;        // steps per shared-memory tile
constexpr int kTileStride = 33;   // padded row length: conflict-free both ways
constexpr int kTileFloats = kChunk * kTileStride;

// Loads tile[i][r] = src[(row0+r)*steps + t0 + i] for r < 32, i < kChunk.
template <typename T>
__device__ __forceinline__ void load_tile(float* tile, const T* __restrict__ src, int64_t row0,
                                          int64_t rows, int64_t steps, int64_t t0, int lane,
                                          bool vec_ok) {
  constexpr int W = 16 / sizeof(T);
  constexpr int VPR = kChunk / W;        // vectors per row segment
  constexpr int RPI = 32 / VPR;          // rows covered by one warp-wide instruction
  if (vec_ok && t0 + kChunk <= steps) {
    const int v = lane % VPR;
    const int rsub = lane / VPR;
#pragma unroll
    for (int it = 0; it < 32 / RPI; ++it) {
      const int r = it * RPI + rsub;
      const int64_t row = row0 + r;
      float vals[W];
      if (row < rows) {
        load_vec<T>(src + row * steps + t0 + v * W, vals);
      } else {
#pragma unroll
        for (int e = 0; e < W; ++e) vals[e] = 0.0f;
      }
#pragma unroll
      for (int e = 0; e < W; ++e) tile[(v * W + e) * kTileStride + r] = vals[e];
    }
  } else {
    for (int r = 0; r < 32; ++r) {
      const int64_t row = row0 + r;
      const int64_t t = t0 + lane;
      float val = 0.0f;
      if (row < rows && t < steps) val = to_f32(src[row * steps + t]);
      tile[lane * kTileStride + r] = val;
    }
  }
}

template <typename T>
__device__ __forceinline__ void store_tile(const float* tile, T* __restrict__ dst, int64_t row0,
                                           int64_t rows, int64_t steps, int64_t t0, int lane,
                                           bool vec_ok) {
  constexpr int W = 16 / sizeof(T);
  constexpr int VPR = kChunk / W;
  constexpr int RPI = 32 / VPR;
  if (vec_ok && t0 + kChunk <= steps) {
    const int v = lane % VPR;
    const int rsub = lane / VPR;
#pragma unroll
    for (int it = 0; it < 32 / RPI; ++it) {
      const int r = it * RPI + rsub;
      const int64_t row = row0 + r;
      if (row < rows) {
        float vals[W];
#pragma unroll
        for (int e = 0; e < W; ++e) vals[e] = tile[(v * W + e) * kTileStride + r];
        store_vec<T>(dst + row * steps + t0 + v * W, vals);
      }
    }
  } else {
    for (int r = 0; r < 32; ++r) {
      const int64_t row = row0 + r;
      const int64_t t = t0 + lane;
      if (row < rows && t < steps) dst[row * steps + t] = from_f32<T>(tile[lane * kTileStride + r]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kScanThreads)
selective_scan_rows_kernel(const T* __restrict__ x, const T* __restrict__ a,
                           const T* __restrict__ b, const T* __restrict__ c,
                           const T* __restrict__ d, T* __restrict__ out, int64_t rows,
                           int64_t steps, int vec_ok) {
  extern __shared__ float smem[];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  float* tx = smem + warp * 6 * kTileFloats;
  float* ta = tx + kTileFloats;
  float* tb = ta + kTileFloats;
  float* tc = tb + kTileFloats;
  float* td = tc + kTileFloats;
  float* to = td + kTileFloats;
  const int64_t n_groups = (rows + 31) / 32;
  const int64_t total_warps = static_cast<int64_t>(gridDim.x) * kScanWarps;
  for (int64_t g = static_cast<int64_t>(blockIdx.x) * kScanWarps + warp; g < n_groups;
       g += total_warps) {
    const int64_t row0 = g * 32;
    float state = 0.0f;
    for (int64_t t0 = 0; t0 < steps; t0 += kChunk) {
      load_tile<T>(tx, x, row0, rows, steps, t0, lane, vec_ok);
      load_tile<T>(ta, a, row0, rows, steps, t0, lane, vec_ok);
      load_tile<T>(tb, b, row0, rows, steps, t0, lane, vec_ok);
      load_tile<T>(tc, c, row0, rows, steps, t0, lane, vec_ok);
      load_tile<T>(td, d, row0, rows, steps, t0, lane, vec_ok);
      __syncwarp();
      const int len = static_cast<int>(steps - t0 < kChunk ? steps - t0 : kChunk);
#pragma unroll 8
      for (int i = 0; i < kChunk; ++i) {
        if (i < len) {
          const float xv = tx[i * kTileStride + lane];
          state = ta[i * kTileStride + lane] * state + tb[i * kTileStride + lane] * xv;
          to[i * kTileStride + lane] =
              round_through<T>(tc[i * kTileStride + lane] * state + td[i * kTileStride + lane] * xv);
        }
      }
      __syncwarp();
      store_tile<T>(to, out, row0, rows, steps, t0, lane, vec_ok);
      __syncwarp();
    }
  }
}

// ---- many rows, aligned: double-buffered cp.async pipeline ----------------------------------------
// A warp owns 32 rows.  One chunk is 64 bytes of every row and operand (16 fp32 / 32 bf16 steps);
// the five operand tiles of chunk i+1 are in flight (cp.async, 16 bytes per request, 10 KiB per
// warp) while lane r walks row r of chunk i.  Tiles keep the global row-major order with an 80-byte
// pitch, which makes the per-lane 128-bit shared-memory reads conflict-free.  Same order and
// association of operations as the CPU reference: bit-identical for fp32.
constexpr int kSegBytes = 64;
constexpr int kPitchBytes = 80;
constexpr int kAsyncTileBytes = 32 * kPitchBytes;                 // one operand, one chunk
constexpr int kAsyncWarpBytes = (2 * 5 + 1) * kAsyncTileBytes;    // double-buffered inputs + output

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(kScanThreads)
selective_scan_rows_async_kernel(const T* __restrict__ x, const T* __restrict__ a,
                                 const T* __restrict__ b, const T* __restrict__ c,
                                 const T* __restrict__ d, T* __restrict__ out, int64_t rows,
                                 int64_t steps) {
  constexpr int W = 16 / sizeof(T);           // elements per 16-byte vector
  constexpr int CS = kSegBytes / sizeof(T);   // steps per chunk
  extern __shared__ __align__(16) uint8_t smem_bytes[];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  uint8_t* wbase = smem_bytes + warp * kAsyncWarpBytes;
  const uint32_t wbase_u32 = static_cast<uint32_t>(__cvta_generic_to_shared(wbase));
  uint8_t* otile = wbase + 10 * kAsyncTileBytes;
  const T* srcs[5] = {x, a, b, c, d};
  const int64_t n_groups = (rows + 31) / 32;
  const int64_t n_chunks = steps / CS;
  const int64_t total_warps = static_cast<int64_t>(gridDim.x) * kScanWarps;
  const int lrow = lane >> 2;   // 8 rows per warp-wide request
  const int lvec = lane & 3;    // 4 vectors per 64-byte row segment

  for (int64_t g = static_cast<int64_t>(blockIdx.x) * kScanWarps + warp; g < n_groups;
       g += total_warps) {
    const int64_t row0 = g * 32;
    auto issue = [&](int64_t chunk, int buf) {
#pragma unroll
      for (int op = 0; op < 5; ++op) {
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          const int r = it * 8 + lrow;
          const int64_t row = row0 + r;
          if (row < rows) {
            const T* src = srcs[op] + row * steps + chunk * CS + lvec * W;
            cp_async_16(wbase_u32 + (buf * 5 + op) * kAsyncTileBytes + r * kPitchBytes + lvec * 16, src);
          }
        }
      }
      cp_async_commit();
    };
    float state = 0.0f;
    issue(0, 0);
    for (int64_t ch = 0; ch < n_chunks; ++ch) {
      const int buf = static_cast<int>(ch & 1);
      if (ch + 1 < n_chunks) {
        issue(ch + 1, buf ^ 1);
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncwarp();
      const uint8_t* tin = wbase + buf * 5 * kAsyncTileBytes + lane * kPitchBytes;
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        float xv[W], av[W], bv[W], cv[W], dv[W], yv[W];
        load_vec<T>(reinterpret_cast<const T*>(tin + 0 * kAsyncTileBytes + v * 16), xv);
        load_vec<T>(reinterpret_cast<const T*>(tin + 1 * kAsyncTileBytes + v * 16), av);
        load_vec<T>(reinterpret_cast<const T*>(tin + 2 * kAsyncTileBytes + v * 16), bv);
        load_vec<T>(reinterpret_cast<const T*>(tin + 3 * kAsyncTileBytes + v * 16), cv);
        load_vec<T>(reinterpret_cast<const T*>(tin + 4 * kAsyncTileBytes + v * 16), dv);
#pragma unroll
        for (int e = 0; e < W; ++e) {
          state = av[e] * state + bv[e] * xv[e];
          yv[e] = cv[e] * state + dv[e] * xv[e];
        }
        store_vec<T>(reinterpret_cast<T*>(otile + lane * kPitchBytes + v * 16), yv);
      }
      __syncwarp();
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        const int r = it * 8 + lrow;
        const int64_t row = row0 + r;
        if (row < rows) {
          const uint4 val = *reinterpret_cast<const uint4*>(otile + r * kPitchBytes + lvec * 16);
          *reinterpret_cast<uint4*>(out + row * steps + ch * CS + lvec * W) = val;
        }
      }
      __syncwarp();
    }
  }
}

// Affine pair combine: apply (a1,b1) first, then (a2,b2): h -> a2*(a1*h+b1)+b2.
struct Affine { float a, b; };
__device__ __forceinline__ Affine combine(Affine first, Affine second) {
  return Affine{second.a * first.a, second.a * first.b + second.b};
}

template <typename T>
__global__ void __launch_bounds__(kScanThreads)
selective_scan_steps_kernel(const T* __restrict__ x, const T* __restrict__ a,
                            const T* __restrict__ b, const T* __restrict__ c,
                            const T* __restrict__ d, T* __restrict__ out, int64_t rows,
                            int64_t steps) {
  constexpr int W = 16 / sizeof(T);
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int64_t total_warps = static_cast<int64_t>(gridDim.x) * kScanWarps;
  const int64_t chunk = 32 * W;
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * kScanWarps + warp; row < rows;
       row += total_warps) {
    const int64_t base = row * steps;
    float carry = 0.0f;
    for (int64_t t0 = 0; t0 < steps; t0 += chunk) {
      const int64_t t = t0 + static_cast<int64_t>(lane) * W;
      float xv[W], av[W], bv[W], cv[W], dv[W];
      if (t + W <= steps) {
        load_vec<T>(x + base + t, xv);
        load_vec<T>(a + base + t, av);
        load_vec<T>(b + base + t, bv);
        load_vec<T>(c + base + t, cv);
        load_vec<T>(d + base + t, dv);
      } else {
#pragma unroll
        for (int e = 0; e < W; ++e) {  // identity steps past the end of the row
          xv[e] = 0.0f; av[e] = 1.0f; bv[e] = 0.0f; cv[e] = 0.0f; dv[e] = 0.0f;
        }
      }
      Affine seg{1.0f, 0.0f};
#pragma unroll
      for (int e = 0; e < W; ++e) seg = combine(seg, Affine{av[e], bv[e] * xv[e]});
      // inclusive warp scan of the affine pairs
      Affine inc = seg;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float pa = __shfl_up_sync(0xffffffffu, inc.a, o);
        const float pb = __shfl_up_sync(0xffffffffu, inc.b, o);
        if (lane >= o) inc = combine(Affine{pa, pb}, inc);
      }
      // state entering this lane's segment = exclusive prefix applied to the carry
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
      if (t + W <= steps) store_vec<T>(out + base + t, yv);
      const float la = __shfl_sync(0xffffffffu, inc.a, 31);
      const float lb = __shfl_sync(0xffffffffu, inc.b, 31);
      carry = la * carry + lb;
    }
  }
}

}  // namespace fb200

namespace fb200 {
// scan_chunked.cu
int64_t scan_chunking(int64_t rows, int64_t steps, int elems_per_vec, int64_t* chunk_len);
template <typename T>
int scan_chunked_launch(const void* x, const void* a, const void* b, const void* c, const void* d,
                        void* out, int64_t rows, int64_t steps, int64_t chunks, int64_t chunk_len,
                        float2* scratch, cudaStream_t s);
}  // namespace fb200

using namespace fb200;

template <typename T>
static int launch_scan(const void* x, const void* a, const void* b, const void* c, const void* d,
                       void* out, int64_t rows, int64_t steps, cudaStream_t s) {
  constexpr int W = 16 / sizeof(T);
  const T* xp = static_cast<const T*>(x);
  const T* ap = static_cast<const T*>(a);
  const T* bp = static_cast<const T*>(b);
  const T* cp = static_cast<const T*>(c);
  const T* dp = static_cast<const T*>(d);
  T* op = static_cast<T*>(out);
  const bool al = aligned16(x) && aligned16(a) && aligned16(b) && aligned16(c) && aligned16(d) &&
                  aligned16(out) && steps % W == 0;
  // Few long rows: parallelise along time.  Needs whole 128-bit vectors per row.
  const int64_t row_groups = (rows + 31) / 32;
  if (al && row_groups < 2 * kNumSMs && steps >= 8 * 32 * W) {
    // Fewer rows than the GPU has warps: cut the time axis into chunks (two passes and a scratch
    // array of one affine pair per (row, chunk), taken from the stream-ordered allocator).
    int64_t chunk_len = steps;
    const int64_t chunks = rows < kNumSMs * 8 ? scan_chunking(rows, steps, W, &chunk_len) : 1;
    if (chunks >= 2) {
      float2* scratch = nullptr;
      FB200_CUDA_OK(scratch_alloc_async(reinterpret_cast<void**>(&scratch),
                                    static_cast<size_t>(rows * chunks) * sizeof(float2), s));
      const int rc = scan_chunked_launch<T>(x, a, b, c, d, out, rows, steps, chunks, chunk_len, scratch, s);
      FB200_CUDA_OK(cudaFreeAsync(scratch, s));
      return rc;
    }
    const int grid = grid_for(rows * 32, kScanThreads, 8);
    selective_scan_steps_kernel<T><<<grid, kScanThreads, 0, s>>>(xp, ap, bp, cp, dp, op, rows, steps);
    return after_launch("selective_scan_steps_kernel");
  }
  if (al && steps % (kSegBytes / static_cast<int>(sizeof(T))) == 0) {
    const size_t smem_async = static_cast<size_t>(kScanWarps) * kAsyncWarpBytes;
    FB200_CUDA_OK(cudaFuncSetAttribute(selective_scan_rows_async_kernel<T>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem_async)));
    const int grid_async = grid_for(row_groups * 32, kScanThreads, 2);
    selective_scan_rows_async_kernel<T><<<grid_async, kScanThreads, smem_async, s>>>(xp, ap, bp, cp, dp,
                                                                                    op, rows, steps);
    return after_launch("selective_scan_rows_async_kernel");
  }
  const size_t smem = static_cast<size_t>(kScanWarps) * 6 * kTileFloats * sizeof(float);
  FB200_CUDA_OK(cudaFuncSetAttribute(selective_scan_rows_kernel<T>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(smem)));
  const int grid = grid_for(row_groups * 32, kScanThreads, 2);
  selective_scan_rows_kernel<T><<<grid, kScanThreads, smem, s>>>(xp, ap, bp, cp, dp, op, rows,
                                                                  steps, al ? 1 : 0);
  return after_launch("selective_scan_rows_kernel");
}

extern "C" int fb200_selective_scan(const void* x, const void* a, const void* b, const void* c,
                                    const void* d, void* out, int64_t rows, int64_t steps,
                                    int dtype, fb200_stream stream) {
  if (rows < 0) return set_error(FB200_INVALID_ARGUMENT, "selective_scan: negative rows");
  if (steps < 1) {
    return set_error(FB200_INVALID_ARGUMENT,
                     "selective_scan: the last dimension (steps) must be >= 1, got %lld",
                     static_cast<long long>(steps));
  }
  if (rows == 0) return FB200_OK;
  if (!x || !a || !b || !c || !d || !out) {
    return set_error(FB200_INVALID_ARGUMENT, "selective_scan: null argument");
  }
  cudaStream_t s = as_stream(stream);
  switch (dtype) {
    case FB200_F32: return launch_scan<float>(x, a, b, c, d, out, rows, steps, s);
    case FB200_BF16: return launch_scan<__nv_bfloat16>(x, a, b, c, d, out, rows, steps, s);
    case FB200_F16: return launch_scan<__half>(x, a, b, c, d, out, rows, steps, s);
    default:
      return set_error(FB200_INVALID_ARGUMENT,
                       "selective_scan: dtype code %d is not float32/float16/bfloat16", dtype);
  }
}

