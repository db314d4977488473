// Data-movement ops: transpose, slice, concat, and the axis-subset sum.  All are bit-exact
// (pure indexing; the sum visits the reduced positions in the CPU reference's order).
//
// Reference semantics: src/backends/cpu/kernels/shape.cpp:73 (transpose), :172 (concat),
// :276 (slice); src/backends/cpu/kernels/reduction.cpp:130 (sum).  The reference CUDA backend
// moves slices and concats with one cudaMemcpyAsync per contiguous segment
// (src/backends/cuda/kernels/shape.cpp:207,342) and transposes byte-wise with one thread per
// output element (shape.cu:65-83); here each op is one launch: pitched 128-bit copies, and a
// 32x32 shared-memory tile transpose whenever the permutation reduces to swapping the two
// innermost (merged) axes.  HBM-bound: algorithmic bytes = 2 * bytes moved.
#include "common.cuh"

namespace fb200 {

// ---- pitched copy ---------------------------------------------------------------------------
struct CopySeg {
  const char* src;
  char* dst;
  int64_t src_pitch, dst_pitch, row_bytes, rows;
};
constexpr int kMaxSegs = 16;
struct CopyBatch {
  int n;
  CopySeg seg[kMaxSegs];
};

template <typename U>
__global__ void __launch_bounds__(256) pitched_copy_kernel(CopyBatch batch) {
  for (int sidx = blockIdx.y; sidx < batch.n; sidx += gridDim.y) {
    const CopySeg sg = batch.seg[sidx];
    const int64_t units_per_row = sg.row_bytes / static_cast<int64_t>(sizeof(U));
    const int64_t total = units_per_row * sg.rows;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += stride) {
      const int64_t r = i / units_per_row;
      const int64_t u = i - r * units_per_row;
      const U* s = reinterpret_cast<const U*>(sg.src + r * sg.src_pitch) + u;
      U* d = reinterpret_cast<U*>(sg.dst + r * sg.dst_pitch) + u;
      *d = *s;
    }
  }
}

static int unit_for(const CopyBatch& b) {
  uintptr_t bits = 0;
  for (int i = 0; i < b.n; ++i) {
    const CopySeg& s = b.seg[i];
    bits |= reinterpret_cast<uintptr_t>(s.src) | reinterpret_cast<uintptr_t>(s.dst) |
            static_cast<uintptr_t>(s.src_pitch) | static_cast<uintptr_t>(s.dst_pitch) |
            static_cast<uintptr_t>(s.row_bytes);
  }
  if ((bits & 15u) == 0) return 16;
  if ((bits & 7u) == 0) return 8;
  if ((bits & 3u) == 0) return 4;
  if ((bits & 1u) == 0) return 2;
  return 1;
}

static int launch_copy(const CopyBatch& b, cudaStream_t s) {
  int64_t max_bytes = 0;
  for (int i = 0; i < b.n; ++i) {
    const int64_t t = b.seg[i].row_bytes * b.seg[i].rows;
    if (t > max_bytes) max_bytes = t;
  }
  if (max_bytes == 0) return FB200_OK;
  const int unit = unit_for(b);
  dim3 grid(static_cast<unsigned>(grid_for(max_bytes / unit, 256, 8)), static_cast<unsigned>(b.n));
  if (b.n > 1) {
    const int per = (kNumSMs * 8 + b.n - 1) / b.n;
    if (static_cast<int>(grid.x) > per) grid.x = per > 1 ? per : 1;
  }
  switch (unit) {
    case 16: pitched_copy_kernel<uint4><<<grid, 256, 0, s>>>(b); break;
    case 8: pitched_copy_kernel<uint2><<<grid, 256, 0, s>>>(b); break;
    case 4: pitched_copy_kernel<uint32_t><<<grid, 256, 0, s>>>(b); break;
    case 2: pitched_copy_kernel<uint16_t><<<grid, 256, 0, s>>>(b); break;
    default: pitched_copy_kernel<uint8_t><<<grid, 256, 0, s>>>(b); break;
  }
  return after_launch("pitched_copy_kernel");
}

// ---- transpose ------------------------------------------------------------------------------
// out[b][c][r] = in[b][r][c] for `batch` matrices of R x C elements.
template <typename U>
__global__ void __launch_bounds__(256)
transpose_tile_kernel(const U* __restrict__ in, U* __restrict__ out, int64_t batch, int64_t R,
                      int64_t C) {
  __shared__ U tile[32][33];
  const int tx = threadIdx.x & 31;
  const int ty = threadIdx.x >> 5;  // 0..7
  const int64_t tiles_c = (C + 31) / 32;
  const int64_t tiles_r = (R + 31) / 32;
  const int64_t per_mat = tiles_c * tiles_r;
  const int64_t total = per_mat * batch;
  for (int64_t tix = blockIdx.x; tix < total; tix += gridDim.x) {
    const int64_t b = tix / per_mat;
    const int64_t rem = tix - b * per_mat;
    const int64_t tr = rem / tiles_c;
    const int64_t tc = rem - tr * tiles_c;
    const U* src = in + b * R * C;
    U* dst = out + b * R * C;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t r = tr * 32 + ty + 8 * j;
      const int64_t c = tc * 32 + tx;
      if (r < R && c < C) tile[ty + 8 * j][tx] = src[r * C + c];
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t c = tc * 32 + ty + 8 * j;
      const int64_t r = tr * 32 + tx;
      if (r < R && c < C) dst[c * R + r] = tile[tx][ty + 8 * j];
    }
    __syncthreads();
  }
}

// Vectorised form for 2- and 4-byte elements whose extents allow 128-bit access on both sides:
// a 64 x 64 tile, 16-byte global loads along C, a padded shared-memory tile, 16-byte global
// stores along R.
template <typename U>
__global__ void __launch_bounds__(256)
transpose_tile64_kernel(const U* __restrict__ in, U* __restrict__ out, int64_t batch, int64_t R,
                        int64_t C) {
  constexpr int V = 16 / sizeof(U);       // elements per 16-byte vector
  constexpr int T = 64;                   // tile edge in elements
  constexpr int VPR = T / V;              // vectors per tile row
  constexpr int RPP = 256 / VPR;          // tile rows covered by one pass of the CTA
  constexpr int PAD = 4 / sizeof(U);      // one 32-bit word of padding per row
  __shared__ U tile[T][T + PAD];
  const int64_t tiles_c = (C + T - 1) / T;
  const int64_t tiles_r = (R + T - 1) / T;
  const int64_t per_mat = tiles_c * tiles_r;
  const int64_t total = per_mat * batch;
  const int vec = threadIdx.x % VPR;
  const int sub = threadIdx.x / VPR;
  for (int64_t tix = blockIdx.x; tix < total; tix += gridDim.x) {
    const int64_t b = tix / per_mat;
    const int64_t rem = tix - b * per_mat;
    const int64_t tr = rem / tiles_c;
    const int64_t tc = rem - tr * tiles_c;
    const U* src = in + b * R * C;
    U* dst = out + b * R * C;
#pragma unroll
    for (int p = 0; p < T / RPP; ++p) {
      const int lr = p * RPP + sub;
      const int64_t r = tr * T + lr;
      const int64_t c = tc * T + vec * V;
      if (r < R && c < C) {   // C % V == 0: a vector is entirely inside or outside
        const Vec16<U> v = *reinterpret_cast<const Vec16<U>*>(src + r * C + c);
#pragma unroll
        for (int e = 0; e < V; ++e) tile[lr][vec * V + e] = v.v[e];
      }
    }
    __syncthreads();
#pragma unroll
    for (int p = 0; p < T / RPP; ++p) {
      const int lc = p * RPP + sub;         // output row inside the tile = input column
      const int64_t c = tc * T + lc;
      const int64_t r = tr * T + vec * V;   // R % V == 0
      if (c < C && r < R) {
        Vec16<U> v;
#pragma unroll
        for (int e = 0; e < V; ++e) v.v[e] = tile[vec * V + e][lc];
        *reinterpret_cast<Vec16<U>*>(dst + c * R + r) = v;
      }
    }
    __syncthreads();
  }
}

struct PermDesc {
  int rank;
  int64_t out_dims[8];
  int64_t in_strides[8];  // stride (elements) in the input of output axis i
};

template <typename U>
__global__ void __launch_bounds__(256)
transpose_generic_kernel(const U* __restrict__ in, U* __restrict__ out, PermDesc d, int64_t numel) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < numel;
       i += stride) {
    int64_t rem = i, off = 0;
#pragma unroll
    for (int ax = 7; ax >= 0; --ax) {
      if (ax < d.rank) {
        const int64_t q = rem / d.out_dims[ax];
        off += (rem - q * d.out_dims[ax]) * d.in_strides[ax];
        rem = q;
      }
    }
    out[i] = in[off];
  }
}

// Launches the batched 2-D transpose out[b][c][r] = in[b][r][c].
template <typename U>
static int launch_tile_transpose(const U* ip, U* op, int64_t batch, int64_t R, int64_t C,
                                 cudaStream_t s) {
  constexpr int V = 16 / sizeof(U);
  const bool vec_ok = (sizeof(U) == 2 || sizeof(U) == 4) && R % V == 0 && C % V == 0 &&
                      aligned16(ip) && aligned16(op);
  if (vec_ok) {
    const int64_t tiles = batch * ((R + 63) / 64) * ((C + 63) / 64);
    const int grid = static_cast<int>(tiles < int64_t(kNumSMs) * 8 ? tiles : int64_t(kNumSMs) * 8);
    transpose_tile64_kernel<U><<<grid, 256, 0, s>>>(ip, op, batch, R, C);
    return after_launch("transpose_tile64_kernel");
  }
  const int64_t tiles = batch * ((R + 31) / 32) * ((C + 31) / 32);
  const int grid = static_cast<int>(tiles < int64_t(kNumSMs) * 16 ? tiles : int64_t(kNumSMs) * 16);
  transpose_tile_kernel<U><<<grid, 256, 0, s>>>(ip, op, batch, R, C);
  return after_launch("transpose_tile_kernel");
}

template <typename U>
static int launch_transpose(const void* x, void* out, int rank, const int64_t* dims,
                            const int64_t* perm, cudaStream_t s) {
  // Drop size-1 axes and merge input axes that stay adjacent and ordered in the output.
  int64_t in_strides[8];
  int64_t st = 1;
  for (int i = rank - 1; i >= 0; --i) { in_strides[i] = st; st *= dims[i]; }
  const int64_t numel = st;
  int64_t od[8], os[8];
  int n = 0;
  for (int i = 0; i < rank; ++i) {
    const int64_t ax = perm[i];
    if (dims[ax] == 1) continue;
    if (n > 0 && os[n - 1] == in_strides[ax] * dims[ax]) {
      od[n - 1] *= dims[ax];
      os[n - 1] = in_strides[ax];
    } else {
      od[n] = dims[ax];
      os[n] = in_strides[ax];
      ++n;
    }
  }
  const U* ip = static_cast<const U*>(x);
  U* op = static_cast<U*>(out);
  if (n <= 1) {  // identity permutation after merging: plain copy
    CopyBatch b{};
    b.n = 1;
    b.seg[0] = CopySeg{static_cast<const char*>(x), static_cast<char*>(out),
                       numel * int64_t(sizeof(U)), numel * int64_t(sizeof(U)),
                       numel * int64_t(sizeof(U)), 1};
    return launch_copy(b, s);
  }
  // [R,C] -> [C,R]  or  [B,R,C] -> [B,C,R]
  if (n == 2 && os[0] == 1 && os[1] == od[0]) {
    return launch_tile_transpose<U>(ip, op, 1, od[1], od[0], s);
  }
  if (n == 3 && os[1] == 1 && os[2] == od[1] && os[0] == od[1] * od[2]) {
    return launch_tile_transpose<U>(ip, op, od[0], od[2], od[1], s);
  }
  PermDesc d{};
  d.rank = n;
  for (int i = 0; i < n; ++i) { d.out_dims[i] = od[i]; d.in_strides[i] = os[i]; }
  const int grid = grid_for(numel, 256, 8);
  transpose_generic_kernel<U><<<grid, 256, 0, s>>>(ip, op, d, numel);
  return after_launch("transpose_generic_kernel");
}

// ---- sum over an axis subset ------------------------------------------------------------------
struct SumDesc {
  int n_keep, n_red;
  int64_t keep_dims[8], keep_strides[8];
  int64_t red_dims[8], red_strides[8];
  int64_t n_out, n_red_total;
};

template <typename T>
__global__ void __launch_bounds__(256)
sum_axes_kernel(const T* __restrict__ x, T* __restrict__ out, SumDesc d) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < d.n_out;
       i += stride) {
    int64_t rem = i, base = 0;
#pragma unroll
    for (int ax = 7; ax >= 0; --ax) {
      if (ax < d.n_keep) {
        const int64_t q = rem / d.keep_dims[ax];
        base += (rem - q * d.keep_dims[ax]) * d.keep_strides[ax];
        rem = q;
      }
    }
    float acc = 0.0f;
    if (d.n_red == 1) {
      for (int64_t r = 0; r < d.n_red_total; ++r) acc += to_f32(x[base + r * d.red_strides[0]]);
    } else {
      for (int64_t r = 0; r < d.n_red_total; ++r) {
        int64_t rr = r, off = base;
#pragma unroll
        for (int ax = 7; ax >= 0; --ax) {
          if (ax < d.n_red) {
            const int64_t q = rr / d.red_dims[ax];
            off += (rr - q * d.red_dims[ax]) * d.red_strides[ax];
            rr = q;
          }
        }
        acc += to_f32(x[off]);
      }
    }
    out[i] = from_f32<T>(acc);
  }
}

}  // namespace fb200

using namespace fb200;

extern "C" int fb200_transpose(const void* x, void* out, int rank, const int64_t* dims,
                               const int64_t* perm, int itemsize, fb200_stream stream) {
  if (rank < 0 || rank > 8) return set_error(FB200_INVALID_ARGUMENT, "transpose: rank %d outside [0, 8]", rank);
  if (rank > 0 && (dims == nullptr || perm == nullptr)) {
    return set_error(FB200_INVALID_ARGUMENT, "transpose: null dims/perm");
  }
  int64_t numel = 1;
  bool seen[8] = {false, false, false, false, false, false, false, false};
  for (int i = 0; i < rank; ++i) {
    if (dims[i] < 0) return set_error(FB200_INVALID_ARGUMENT, "transpose: negative dimension");
    if (perm[i] < 0 || perm[i] >= rank || seen[perm[i]]) {
      return set_error(FB200_INVALID_ARGUMENT, "transpose: perm is not a permutation of [0, %d)", rank);
    }
    seen[perm[i]] = true;
    numel *= dims[i];
  }
  if (numel == 0) return FB200_OK;
  if (x == nullptr || out == nullptr) return set_error(FB200_INVALID_ARGUMENT, "transpose: null argument");
  cudaStream_t s = as_stream(stream);
  switch (itemsize) {
    case 1: return launch_transpose<uint8_t>(x, out, rank, dims, perm, s);
    case 2: return launch_transpose<uint16_t>(x, out, rank, dims, perm, s);
    case 4: return launch_transpose<uint32_t>(x, out, rank, dims, perm, s);
    case 8: return launch_transpose<uint64_t>(x, out, rank, dims, perm, s);
    default: return set_error(FB200_INVALID_ARGUMENT, "transpose: itemsize %d not in {1,2,4,8}", itemsize);
  }
}

extern "C" int fb200_slice(const void* x, void* out, int rank, const int64_t* dims, int64_t axis,
                           int64_t start, int64_t stop, int itemsize, fb200_stream stream) {
  if (rank < 1 || rank > 8 || dims == nullptr) return set_error(FB200_INVALID_ARGUMENT, "slice: bad rank/dims");
  if (axis < 0 || axis >= rank) return set_error(FB200_INVALID_ARGUMENT, "slice: axis %lld outside [0, %d)", (long long)axis, rank);
  if (start < 0 || stop < start || stop > dims[axis]) {
    return set_error(FB200_INVALID_ARGUMENT, "slice: range [%lld, %lld) outside [0, %lld]",
                     (long long)start, (long long)stop, (long long)dims[axis]);
  }
  int64_t outer = 1, inner = 1;
  for (int i = 0; i < axis; ++i) outer *= dims[i];
  for (int i = static_cast<int>(axis) + 1; i < rank; ++i) inner *= dims[i];
  const int64_t row_bytes = (stop - start) * inner * itemsize;
  if (outer == 0 || row_bytes == 0) return FB200_OK;
  if (x == nullptr || out == nullptr) return set_error(FB200_INVALID_ARGUMENT, "slice: null argument");
  CopyBatch b{};
  b.n = 1;
  b.seg[0] = CopySeg{static_cast<const char*>(x) + start * inner * itemsize, static_cast<char*>(out),
                     dims[axis] * inner * itemsize, row_bytes, row_bytes, outer};
  return launch_copy(b, as_stream(stream));
}

extern "C" int fb200_concat(const void* const* inputs, int n_inputs, const int64_t* axis_sizes,
                            void* out, int rank, const int64_t* out_dims, int64_t axis,
                            int itemsize, fb200_stream stream) {
  if (rank < 1 || rank > 8 || out_dims == nullptr || inputs == nullptr || axis_sizes == nullptr) {
    return set_error(FB200_INVALID_ARGUMENT, "concat: bad arguments");
  }
  if (axis < 0 || axis >= rank) return set_error(FB200_INVALID_ARGUMENT, "concat: axis outside rank");
  int64_t outer = 1, inner = 1, total_axis = 0;
  for (int i = 0; i < axis; ++i) outer *= out_dims[i];
  for (int i = static_cast<int>(axis) + 1; i < rank; ++i) inner *= out_dims[i];
  for (int i = 0; i < n_inputs; ++i) total_axis += axis_sizes[i];
  if (total_axis != out_dims[axis]) {
    return set_error(FB200_INVALID_ARGUMENT, "concat: inputs cover %lld on the axis, output has %lld",
                     (long long)total_axis, (long long)out_dims[axis]);
  }
  if (outer == 0 || inner == 0 || total_axis == 0) return FB200_OK;
  if (out == nullptr) return set_error(FB200_INVALID_ARGUMENT, "concat: null output");
  const int64_t dst_pitch = total_axis * inner * itemsize;
  int64_t off = 0;
  cudaStream_t s = as_stream(stream);
  CopyBatch b{};
  for (int i = 0; i < n_inputs; ++i) {
    const int64_t row_bytes = axis_sizes[i] * inner * itemsize;
    if (row_bytes > 0) {
      if (inputs[i] == nullptr) return set_error(FB200_INVALID_ARGUMENT, "concat: input %d is null", i);
      b.seg[b.n++] = CopySeg{static_cast<const char*>(inputs[i]), static_cast<char*>(out) + off,
                             row_bytes, dst_pitch, row_bytes, outer};
    }
    off += row_bytes;
    if (b.n == kMaxSegs || (i == n_inputs - 1 && b.n > 0)) {
      if (int rc = launch_copy(b, s)) return rc;
      b.n = 0;
    }
  }
  return FB200_OK;
}

extern "C" int fb200_sum_axes(const void* x, void* out, int rank, const int64_t* dims,
                              const int64_t* axes, int n_axes, int dtype, fb200_stream stream) {
  if (rank < 0 || rank > 8 || n_axes < 0 || n_axes > rank) {
    return set_error(FB200_INVALID_ARGUMENT, "sum: bad rank/axes");
  }
  bool red[8] = {false, false, false, false, false, false, false, false};
  for (int i = 0; i < n_axes; ++i) {
    int64_t ax = axes[i] < 0 ? axes[i] + rank : axes[i];
    if (ax < 0 || ax >= rank || red[ax]) return set_error(FB200_INVALID_ARGUMENT, "sum: bad axis %lld", (long long)axes[i]);
    red[ax] = true;
  }
  int64_t strides[8];
  int64_t st = 1;
  for (int i = rank - 1; i >= 0; --i) { strides[i] = st; st *= dims[i]; }
  SumDesc d{};
  d.n_out = 1;
  d.n_red_total = 1;
  for (int i = 0; i < rank; ++i) {
    if (red[i]) {
      d.red_dims[d.n_red] = dims[i]; d.red_strides[d.n_red] = strides[i]; ++d.n_red;
      d.n_red_total *= dims[i];
    } else {
      d.keep_dims[d.n_keep] = dims[i]; d.keep_strides[d.n_keep] = strides[i]; ++d.n_keep;
      d.n_out *= dims[i];
    }
  }
  // merge adjacent reduced axes that are contiguous with each other
  if (d.n_red > 1) {
    int m = 0;
    for (int i = 1; i < d.n_red; ++i) {
      if (d.red_strides[m] == d.red_strides[i] * d.red_dims[i]) {
        d.red_dims[m] *= d.red_dims[i];
        d.red_strides[m] = d.red_strides[i];
      } else {
        ++m;
        d.red_dims[m] = d.red_dims[i];
        d.red_strides[m] = d.red_strides[i];
      }
    }
    d.n_red = m + 1;
  }
  if (d.n_out == 0) return FB200_OK;
  if (x == nullptr && d.n_red_total > 0) return set_error(FB200_INVALID_ARGUMENT, "sum: null input");
  if (out == nullptr) return set_error(FB200_INVALID_ARGUMENT, "sum: null output");
  cudaStream_t s = as_stream(stream);
  const int grid = grid_for(d.n_out, 256, 8);
  switch (dtype) {
    case FB200_F32:
      sum_axes_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(x), static_cast<float*>(out), d);
      break;
    case FB200_BF16:
      sum_axes_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x),
                                                          static_cast<__nv_bfloat16*>(out), d);
      break;
    case FB200_F16:
      sum_axes_kernel<__half><<<grid, 256, 0, s>>>(static_cast<const __half*>(x), static_cast<__half*>(out), d);
      break;
    default: return set_error(FB200_INVALID_ARGUMENT, "sum: unsupported dtype code %d", dtype);
  }
  return after_launch("sum_axes_kernel");
}
