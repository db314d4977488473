// attention_fan — one launch for a whole fan of per-head `matmul -> softmax -> matmul` chains.
//
// The reference expresses multi-head attention per (batch, head) as separate graph nodes
// (src/nn/layers.cpp:950-1170: slice q/k/v, transpose k, matmul, softmax, matmul, concat) and
// its executable runs each node as its own kernel (src/backends/cuda/cuda_executable.cpp:84-118):
// for 8 x 16 heads that is about 900 launches of tiny kernels.  This kernel computes, for every
// head h of a table,
//     S = Q_h K_h^T   (fp32 accumulate, rounded once to T: the first matmul's store; then, when a
//                     scale other than 1 is given, multiplied by it and rounded to T again: the
//                     `mul` by a constant of the reference's own attention)
//     P = softmax(S)  (row max, exp(x - max), sum, e * (1 / sum) in fp32; rounded once to T)
//     O = P V_h       (fp32 accumulate, rounded once to T)
// i.e. the same three operators with the same rounding points (matmul:
// src/backends/cpu/kernels/matmul.cpp:92-131, softmax: src/backends/cpu/kernels/sequence.cpp:114-174);
// only the order of the fp32 additions differs, as in every tensor-core path.
//
// Q_h, K_h, V_h are [sq, 64] / [sk, 64] / [sk, 64] windows of row-major matrices (the fused QKV
// projection), addressed by TMA through (row, column) coordinates, so no slice or transpose is
// materialised; O_h is written at an element offset of an output matrix with its own row pitch,
// so a concat can be skipped too.
//
// One CTA (256 threads) per (head, block of 128 query rows):
//   thread 0   TMA loads of Q (16 KiB), K and V (sk x 128 B each, 128-byte swizzle);
//              tcgen05.mma S[128, sk] = Q K^T into TMEM (N <= 256 per instruction);
//   all        two threads per query row (= TMEM lane), each on half of the keys: three sweeps
//              with tcgen05.ld (max; exp and sum, written back with tcgen05.st; normalise), P
//              written to shared memory as the K-major, 128-byte-swizzled A operand (over K's
//              bytes);
//   thread 0   tcgen05.mma O[128, 64] = P V (V is the MN-major B operand straight from TMA);
//   all        tcgen05.ld O, convert, 128-byte row stores.
// Shared memory: 16 KiB + sk*256 + sk*128 (208 KiB at sk = 512); TMEM: sk columns (power of two).
// Algorithmic work per head: 4*sq*sk*64 FLOP; bytes (sq + 2*sk + sq) * 64 * itemsize.
#include <cuda.h>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace fb200 {

int make_tmap_2d(CUtensorMap* map, const void* ptr, int dtype, int64_t rows, int64_t cols,
                 int box_rows, bool swizzle_32b_units);
int device_status_word(int** dev_ptr);

using namespace sm100;

constexpr int kAttnThreads = 256;
constexpr int kAttnBlockM = 128;
constexpr int kAttnHeadDim = 64;
constexpr int kAttnMaxKeys = 512;
constexpr int kAttnKvBoxRows = 64;

enum AttnFault : int {
  kFaultAttnLoad = 301,     // Q/K tiles never arrived
  kFaultAttnScores = 302,   // the first tcgen05.mma batch never completed
  kFaultAttnValues = 303,   // V tile never arrived
  kFaultAttnOutput = 304,   // the second tcgen05.mma batch never completed
  kFaultAttnBadHead = 305,  // a column coordinate or output offset is not a multiple of 8 elements
};

__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0],"
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16,"
      " %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
        "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
        "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  const __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// Value of an fp32 score after the first matmul's store to T and the softmax's load of it.  The
// conversion instructions run on the quarter-rate XU pipe, which exp2 already saturates, so the
// bfloat16 round-to-nearest-even is done with integer arithmetic instead (finite inputs; a NaN
// stays a NaN).
template <typename T> __device__ __forceinline__ float stored_score(float v) { return round_through<T>(v); }
template <> __device__ __forceinline__ float stored_score<__nv_bfloat16>(float v) {
  const uint32_t b = __float_as_uint(v);
  return __uint_as_float((b + 0x7FFFu + ((b >> 16) & 1u)) & 0xFFFF0000u);
}

template <typename T>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_fan_kernel(const __grid_constant__ CUtensorMap tmap_q,
                     const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v,
                     const fb200_attention_head* __restrict__ heads, T* __restrict__ o_base,
                     int64_t o_ld, int sq, int sk, int q_blocks, uint32_t tmem_cols, uint32_t fmt,
                     float scale, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;  // swizzle atoms need 1024-byte alignment
  uint8_t* base_ptr = smem_raw + (base - raw_addr);
  const uint32_t q_s = base;
  const uint32_t kp_off = kAttnBlockM * 128;                       // K, later P
  const uint32_t v_off = kp_off + static_cast<uint32_t>(sk) * 256u;
  const uint32_t bar_off = v_off + static_cast<uint32_t>(sk) * 128u;
  const uint32_t kp_s = base + kp_off, v_s = base + v_off, bars = base + bar_off;
  const uint32_t bar_qk = bars, bar_v = bars + 8, bar_s = bars + 16, bar_o = bars + 24;
  const uint32_t tmem_slot = bars + 32;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(base_ptr + bar_off + 32);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int head = blockIdx.x / q_blocks;
  const int qb = blockIdx.x - head * q_blocks;
  const fb200_attention_head h = heads[head];

  if (tid == 0) {
    mbar_init(bar_qk, 1);
    mbar_init(bar_v, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(tmem_slot, tmem_cols);
    tmem_relinquish();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;

  // A TMA copy whose innermost coordinate is not 16-byte aligned is an illegal instruction, so a
  // bad table entry is refused here, before any copy is issued.
  const bool head_ok = ((h.q_col | h.k_col | h.v_col) & 7) == 0 && (h.o_offset & 7) == 0;
  if (!head_ok && tid == 0) *reinterpret_cast<volatile int*>(status) = kFaultAttnBadHead;

  if (tid == 0 && head_ok) {
    mbar_arrive_expect_tx(bar_qk, kAttnBlockM * 128u + static_cast<uint32_t>(sk) * 128u);
    tma_load_2d(q_s, &tmap_q, bar_qk, h.q_col, h.q_row + qb * kAttnBlockM);
    for (int r = 0; r < sk; r += kAttnKvBoxRows) {
      tma_load_2d(kp_s + static_cast<uint32_t>(r) * 128u, &tmap_k, bar_qk, h.k_col, h.k_row + r);
    }
    mbar_arrive_expect_tx(bar_v, static_cast<uint32_t>(sk) * 128u);
    for (int r = 0; r < sk; r += kAttnKvBoxRows) {
      tma_load_2d(v_s + static_cast<uint32_t>(r) * 128u, &tmap_v, bar_v, h.v_col, h.v_row + r);
    }
    if (mbar_wait(bar_qk, 0, status, kFaultAttnLoad)) {
      tcgen05_fence_after_sync();
      // S[128, sk] = Q[128, 64] K[sk, 64]^T: both operands K-major, four 32-byte K steps.
      for (int n0 = 0; n0 < sk; n0 += 256) {
        const int n = sk - n0 < 256 ? sk - n0 : 256;
        const uint32_t idesc = make_instr_desc(fmt, 0, 0, kAttnBlockM, static_cast<uint32_t>(n));
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const uint64_t a_desc = make_smem_desc_sw128(q_s + ks * 32, 16, 1024);
          const uint64_t b_desc =
              make_smem_desc_sw128(kp_s + static_cast<uint32_t>(n0) * 128u + ks * 32, 16, 1024);
          mma_f16(tmem_base + static_cast<uint32_t>(n0), a_desc, b_desc, idesc, ks > 0 ? 1u : 0u);
        }
      }
      mma_commit(bar_s);
    }
  }
  __syncwarp();
  bool ok = head_ok && mbar_wait(bar_s, 0, status, kFaultAttnScores);
  ok = __all_sync(0xffffffffu, ok);

  // Two threads per query row: warp w works on TMEM lanes 32*(w & 3) .. +31 (the only lanes it may
  // touch) and on the key columns of half w >> 2; row maximum and row sum are exchanged through
  // shared memory.  Each sweep keeps the next 32-column tcgen05.ld in flight while the current one
  // is processed.
  const int quad = warp & 3, half = warp >> 2;
  const int row_in_tile = quad * 32 + (tid & 31);
  const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
  const int c_begin = half * (sk / 2), c_end = c_begin + sk / 2;
  float* red_max = reinterpret_cast<float*>(base_ptr + bar_off + 64);   // [2][128]
  float* red_sum = red_max + 2 * kAttnBlockM;
  auto sweep = [&](auto&& body) {
    uint32_t ra[32], rb[32];
    tmem_ld_32x32b_x32(lane_addr + static_cast<uint32_t>(c_begin), ra);
    for (int c = c_begin; c < c_end; c += 64) {
      tmem_ld_wait();
      const bool two = c + 32 < c_end;
      if (two) tmem_ld_32x32b_x32(lane_addr + static_cast<uint32_t>(c + 32), rb);
      body(c, ra);
      if (two) {
        tmem_ld_wait();
        if (c + 64 < c_end) tmem_ld_32x32b_x32(lane_addr + static_cast<uint32_t>(c + 64), ra);
        body(c + 32, rb);
      }
    }
  };
  const bool scaled = scale != 1.0f;
  float mx = -INFINITY;
  if (ok) {
    tcgen05_fence_after_sync();
    sweep([&](int, uint32_t (&r)[32]) {
#pragma unroll
      for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
    });
    mx = stored_score<T>(mx);   // rounding is monotonic: max of the rounded = rounded max
    // an optional `mul` by a constant between the matmul and the softmax (the reference's own
    // attention scales there): its result is rounded to T again; a positive scale keeps the maximum
    if (scaled) mx = stored_score<T>(mx * scale);
  }
  red_max[half * kAttnBlockM + row_in_tile] = mx;
  __syncthreads();
  mx = fmaxf(red_max[row_in_tile], red_max[kAttnBlockM + row_in_tile]);
  float sum = 0.0f;
  if (ok) {
    const float mx2 = mx * 1.4426950408889634f;
    sweep([&](int c, uint32_t (&r)[32]) {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        float sc = stored_score<T>(__uint_as_float(r[i]));
        if (scaled) sc = stored_score<T>(sc * scale);
        const float e = ex2_approx(fmaf(sc, 1.4426950408889634f, -mx2));
        sum += e;
        r[i] = __float_as_uint(e);
      }
      tmem_st_32x32b_x32(lane_addr + static_cast<uint32_t>(c), r);
    });
    tmem_st_wait();
  }
  red_sum[half * kAttnBlockM + row_in_tile] = sum;
  __syncthreads();
  sum = red_sum[row_in_tile] + red_sum[kAttnBlockM + row_in_tile];
  if (ok) {
    // P in the A-operand layout: blocks of 64 keys (128 bytes per row, 16 KiB per block), the
    // 16-byte unit index XORed with (row & 7).
    uint8_t* p_row = base_ptr + kp_off + static_cast<uint32_t>(row_in_tile) * 128u;
    const uint32_t swz = static_cast<uint32_t>(row_in_tile & 7);
    const float inv = 1.0f / sum;
    sweep([&](int c, uint32_t (&r)[32]) {
      uint8_t* blk = p_row + static_cast<uint32_t>(c >> 6) * 16384u;
      const uint32_t unit0 = static_cast<uint32_t>((c >> 3) & 7);   // 0 or 4
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        uint4 v;
        v.x = pack2<T>(__uint_as_float(r[8 * u + 0]) * inv, __uint_as_float(r[8 * u + 1]) * inv);
        v.y = pack2<T>(__uint_as_float(r[8 * u + 2]) * inv, __uint_as_float(r[8 * u + 3]) * inv);
        v.z = pack2<T>(__uint_as_float(r[8 * u + 4]) * inv, __uint_as_float(r[8 * u + 5]) * inv);
        v.w = pack2<T>(__uint_as_float(r[8 * u + 6]) * inv, __uint_as_float(r[8 * u + 7]) * inv);
        *reinterpret_cast<uint4*>(blk + (((unit0 + u) ^ swz) << 4)) = v;
      }
    });
    fence_proxy_async_smem();   // P must be visible to the tensor core's reads
  }
  tcgen05_fence_before_sync();
  __syncthreads();

  if (tid == 0 && ok) {
    if (mbar_wait(bar_v, 0, status, kFaultAttnValues)) {
      tcgen05_fence_after_sync();
      // O[128, 64] = P[128, sk] V[sk, 64]: A K-major (blocks of 64 keys), B MN-major as loaded.
      const uint32_t idesc = make_instr_desc(fmt, 0, 1, kAttnBlockM, kAttnHeadDim);
      const int k_steps = sk / 16;
      for (int kk = 0; kk < k_steps; ++kk) {
        const uint64_t a_desc = make_smem_desc_sw128(
            kp_s + static_cast<uint32_t>(kk >> 2) * 16384u + static_cast<uint32_t>(kk & 3) * 32u, 16, 1024);
        const uint64_t b_desc = make_smem_desc(v_s + static_cast<uint32_t>(kk) * 2048u,
                                               static_cast<uint32_t>(sk) * 128u, 1024, kLayoutSw128);
        mma_f16(tmem_base, a_desc, b_desc, idesc, kk > 0 ? 1u : 0u);
      }
      mma_commit(bar_o);
    }
  }
  __syncwarp();
  ok = ok && mbar_wait(bar_o, 0, status, kFaultAttnOutput);
  ok = __all_sync(0xffffffffu, ok);
  if (ok) {
    tcgen05_fence_after_sync();
    const int row = qb * kAttnBlockM + row_in_tile;
    const int c = half * 32;   // each half of the warps stores 32 of the 64 columns
    T* dst = o_base + h.o_offset + static_cast<int64_t>(row) * o_ld + c;
    uint32_t r[32];
    tmem_ld_32x32b_x32(lane_addr + static_cast<uint32_t>(c), r);
    tmem_ld_wait();
    if (row < sq) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        uint4 v;
        v.x = pack2<T>(__uint_as_float(r[8 * u + 0]), __uint_as_float(r[8 * u + 1]));
        v.y = pack2<T>(__uint_as_float(r[8 * u + 2]), __uint_as_float(r[8 * u + 3]));
        v.z = pack2<T>(__uint_as_float(r[8 * u + 4]), __uint_as_float(r[8 * u + 5]));
        v.w = pack2<T>(__uint_as_float(r[8 * u + 6]), __uint_as_float(r[8 * u + 7]));
        *reinterpret_cast<uint4*>(dst + 8 * u) = v;
      }
    }
  }
  // Common exit: reached by every thread on success and after any bounded wait gave up.
  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

}  // namespace fb200

using namespace fb200;

extern "C" int fb200_attention_fan_supported(int64_t sq, int64_t sk, int64_t head_dim, int dtype) {
  return (dtype == FB200_BF16 || dtype == FB200_F16) && head_dim == kAttnHeadDim && sq >= 1 &&
         sk >= 64 && sk <= kAttnMaxKeys && sk % 64 == 0;
}

extern "C" int fb200_attention_fan(const void* q_base, int64_t q_rows, int64_t q_ld,
                                   const void* k_base, int64_t k_rows, int64_t k_ld,
                                   const void* v_base, int64_t v_rows, int64_t v_ld, void* o_base,
                                   int64_t o_ld, const fb200_attention_head* heads_dev,
                                   int64_t n_heads, int64_t sq, int64_t sk, int64_t head_dim,
                                   float scale, int dtype, fb200_stream stream) {
  if (n_heads < 0 || sq < 0) return set_error(FB200_INVALID_ARGUMENT, "attention_fan: negative size");
  if (!fb200_attention_fan_supported(sq > 0 ? sq : 1, sk, head_dim, dtype)) {
    return set_error(FB200_UNIMPLEMENTED,
                     "attention_fan: needs bfloat16/float16, head_dim 64 and 64 <= keys <= 512 in "
                     "multiples of 64 (got dtype %d, head_dim %lld, keys %lld)",
                     dtype, static_cast<long long>(head_dim), static_cast<long long>(sk));
  }
  if (!(scale > 0.0f)) return set_error(FB200_INVALID_ARGUMENT, "attention_fan: the score scale must be positive");
  if (n_heads == 0 || sq == 0) return FB200_OK;
  if (!q_base || !k_base || !v_base || !o_base || !heads_dev) {
    return set_error(FB200_INVALID_ARGUMENT, "attention_fan: null argument");
  }
  if (!aligned16(q_base) || !aligned16(k_base) || !aligned16(v_base) || !aligned16(o_base) ||
      q_ld % 8 || k_ld % 8 || v_ld % 8 || o_ld % 8 || q_ld < 64 || k_ld < 64 || v_ld < 64 || o_ld < 64) {
    return set_error(FB200_INVALID_ARGUMENT,
                     "attention_fan: bases must be 16-byte aligned and row pitches multiples of 8 elements");
  }
  const int64_t q_blocks = (sq + kAttnBlockM - 1) / kAttnBlockM;
  if (n_heads * q_blocks > 0x7fffffff) return set_error(FB200_INVALID_ARGUMENT, "attention_fan: too many tiles");
  CUtensorMap tq, tk, tv;
  if (int rc = make_tmap_2d(&tq, q_base, dtype, q_rows, q_ld, kAttnBlockM, false)) return rc;
  if (int rc = make_tmap_2d(&tk, k_base, dtype, k_rows, k_ld, kAttnKvBoxRows, false)) return rc;
  if (int rc = make_tmap_2d(&tv, v_base, dtype, v_rows, v_ld, kAttnKvBoxRows, false)) return rc;
  int* status = nullptr;
  if (int rc = device_status_word(&status)) return rc;
  uint32_t tmem_cols = 64;
  while (tmem_cols < static_cast<uint32_t>(sk)) tmem_cols *= 2;
  const size_t smem = kAttnBlockM * 128 + static_cast<size_t>(sk) * 384 + 1024 /*align*/ + 64 /*barriers*/ +
                      4 * kAttnBlockM * sizeof(float) /*row max and sum exchange*/;
  const int grid = static_cast<int>(n_heads * q_blocks);
  cudaStream_t s = as_stream(stream);
  if (dtype == FB200_BF16) {
    auto kernel = attention_fan_kernel<__nv_bfloat16>;
    FB200_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    kernel<<<grid, kAttnThreads, smem, s>>>(tq, tk, tv, heads_dev, static_cast<__nv_bfloat16*>(o_base), o_ld,
                                            static_cast<int>(sq), static_cast<int>(sk),
                                            static_cast<int>(q_blocks), tmem_cols, kFmtBF16, scale, status);
  } else {
    auto kernel = attention_fan_kernel<__half>;
    FB200_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    kernel<<<grid, kAttnThreads, smem, s>>>(tq, tk, tv, heads_dev, static_cast<__half*>(o_base), o_ld,
                                            static_cast<int>(sq), static_cast<int>(sk),
                                            static_cast<int>(q_blocks), tmem_cols, kFmtF16, scale, status);
  }
  return after_launch("attention_fan_kernel");
}
