// attention_fan — one launch for a whole fan of per-head `matmul -> softmax -> matmul` chains.
//
// The reference expresses multi-head attention per (batch, head) as separate graph nodes
// (src/nn/layers.cpp:950-1170: slice q/k/v, transpose k, matmul, softmax, matmul, concat) and
// its executable runs each node as its own kernel (src/backends/cuda/cuda_executable.cpp:84-118):
// for 8 x 16 heads that is about 900 launches of tiny kernels.  This kernel computes, for every
// head h of a table,
//     S = Q_h K_h^T   (fp32 accumulate, rounded once to T: the first matmul's store; then, when a
//                     scale other than 1 is given, multiplied by it and rounded to T again: the
//                     `mul` by a constant of the reference's own attention; a power-of-two scale
//                     of bfloat16 scores is exact and folds into the exponent's multiplier)
//     e = exp(S - rowmax(S)), l = sum(e) in fp32
//     O = (round_T(e) V_h) / l   (fp32 accumulate, divided in fp32, rounded once to T)
// The reference's operators (matmul: src/backends/cpu/kernels/matmul.cpp:92-131, softmax:
// src/backends/cpu/kernels/sequence.cpp:114-174) round P = e / l to T and then multiply by V; here
// e is rounded to T and the division by l is applied to the fp32 result of the second product, as
// fused attention kernels do, which saves a third sweep over the scores.  Both forms carry one
// rounding to T per probability; they differ by a fraction of that rounding step (about 2^-9
// relative per probability, averaged over the keys), far inside the tolerance of a chain of three
// 16-bit operators.  The rounding of S and of O and the order of the row maximum, the exponentials
// and their fp32 sum are the reference's; the order of the fp32 additions inside the products
// differs, as in every tensor-core path.
//
// Q_h, K_h, V_h are [sq, 64] / [sk, 64] / [sk, 64] windows of row-major matrices (the fused QKV
// projection), addressed by TMA through (row, column) coordinates, so no slice or transpose is
// materialised; O_h is written at an element offset of an output matrix with its own row pitch,
// so a concat can be skipped too.
//
// One CTA per (head, run of 128-row query blocks); K and V of the head are loaded once and stay in
// shared memory while the CTA walks its query blocks:
//   warp 16    one elected lane of warp-uniform code: TMA loads (K, V once; Q per block, the next
//              one as soon as QK^T has read the current one); tcgen05.mma S[128, sk] = Q K^T into
//              TMEM (N <= 256 per instruction); then, per 64 keys of P that the softmax warps hand
//              over, tcgen05.mma O[128, 64] += P V (V is the MN-major B operand straight from TMA);
//   warps 0-15 four threads per query row (= TMEM lane): a sweep with tcgen05.ld over a quarter of
//              the keys for the row maximum; then one sweep for exp, the row sum and P (16 of every
//              64 keys per thread), P going in blocks of 64 keys into a ring of four K-major,
//              128-byte-swizzled A-operand blocks, so that P V of a block runs while the next one is
//              computed; tcgen05.ld of O, times 1 / l, row stores.
// S fills TMEM (sk columns), so O accumulates over S's first 64 columns, which the first block of
// P has consumed before the first P V instruction is issued.  The next query block's scores are
// issued in two parts: key columns from 64 up as soon as the last block of P has been handed over
// (all of S has been read by then), the first 64 columns once every thread has read O.
// Shared memory: Q 16 KiB + K, V sk*128 B each + P ring 64 KiB (212 KiB at sk = 512); TMEM: sk
// columns (power of two).
// Algorithmic work per head: 4*sq*sk*64 FLOP; bytes (sq + 2*sk + sq) * 64 * itemsize.
#include <cuda.h>

#include <cmath>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace fb200 {

int make_tmap_2d(CUtensorMap* map, const void* ptr, int dtype, int64_t rows, int64_t cols,
                 int box_rows, bool swizzle_32b_units);
int device_status_word(int** dev_ptr);

using namespace sm100;

constexpr int kAttnParts = 4;           // threads per query row, each on 1/4 of the keys
constexpr int kAttnSoftmaxThreads = 128 * kAttnParts;
constexpr int kAttnCtrlWarp = kAttnSoftmaxThreads / 32;
constexpr int kAttnThreads = kAttnSoftmaxThreads + 32;
constexpr int kAttnPRing = 4;          // 64-key blocks of P between the softmax warps and P V
constexpr int kAttnPBlockBytes = 128 * 128;
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
  kFaultAttnProbs = 306,    // a block of P never arrived, or its ring slot was never released
  kFaultAttnDrain = 307,    // the softmax warps never finished reading O
};

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

// Values of two fp32 scores after the first matmul's store to T and the softmax's load of them.
// The packed conversion rounds both to nearest even in one instruction; unpacking a bfloat16 pair
// is a shift and a mask, so a score costs 1.5 instructions here.
template <typename T> __device__ __forceinline__ float stored_score(float v) { return round_through<T>(v); }
template <typename T> __device__ __forceinline__ void stored_pair(float& a, float& b) {
  a = round_through<T>(a);
  b = round_through<T>(b);
}
template <> __device__ __forceinline__ void stored_pair<__nv_bfloat16>(float& a, float& b) {
  const uint32_t u = pack2<__nv_bfloat16>(a, b);
  a = __uint_as_float(u << 16);
  b = __uint_as_float(u & 0xFFFF0000u);
}

template <typename T, bool RESCALE>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_fan_kernel(const __grid_constant__ CUtensorMap tmap_q,
                     const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v,
                     const fb200_attention_head* __restrict__ heads, T* __restrict__ o_base,
                     int64_t o_ld, int sq, int sk, int q_blocks, int blocks_per_cta, int groups,
                     uint32_t tmem_cols, uint32_t fmt, float scale, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;  // swizzle atoms need 1024-byte alignment
  uint8_t* base_ptr = smem_raw + (base - raw_addr);
  const uint32_t q_s = base;
  const uint32_t k_off = kAttnBlockM * 128;
  const uint32_t v_off = k_off + static_cast<uint32_t>(sk) * 128u;
  const uint32_t p_off = v_off + static_cast<uint32_t>(sk) * 128u;
  const uint32_t bar_off = p_off + kAttnPRing * kAttnPBlockBytes;
  const uint32_t k_s = base + k_off, v_s = base + v_off, p_s = base + p_off, bars = base + bar_off;
  const uint32_t bar_q = bars, bar_k = bars + 8, bar_v = bars + 16, bar_s = bars + 24, bar_o = bars + 32;
  const uint32_t bar_oread = bars + 40, p_full = bars + 48, p_free = bars + 48 + 8 * kAttnPRing;
  const uint32_t bar_su = bars + 48 + 16 * kAttnPRing;
  const uint32_t tmem_slot = bar_su + 8;
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(base_ptr + bar_off + 56 + 16 * kAttnPRing);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int head = blockIdx.x / groups;
  const int blk_begin = (blockIdx.x - head * groups) * blocks_per_cta;
  const int nb = q_blocks - blk_begin < blocks_per_cta ? q_blocks - blk_begin : blocks_per_cta;
  const int n_chunks = sk >> 6;   // 64-key blocks of P per query block
  const fb200_attention_head h = heads[head];

  // A TMA copy whose innermost coordinate is not 16-byte aligned is an illegal instruction, so a
  // bad table entry is refused here, before any copy is issued.
  const bool head_ok = ((h.q_col | h.k_col | h.v_col) & 7) == 0 && (h.o_offset & 7) == 0;
  if (!head_ok && tid == 0) *reinterpret_cast<volatile int*>(status) = kFaultAttnBadHead;

  // The control warp sets the barriers up and sends the first copies on their way before the CTA
  // meets: K, Q and V travel while warp 0 allocates TMEM.
  if (warp == kAttnCtrlWarp) {
    if ((tid & 31) == 0) {
      mbar_init(bar_q, 1);
      mbar_init(bar_k, 1);
      mbar_init(bar_v, 1);
      mbar_init(bar_s, 1);
      mbar_init(bar_su, 1);
      mbar_init(bar_o, 1);
      mbar_init(bar_oread, kAttnSoftmaxThreads / 32);
      for (int i = 0; i < kAttnPRing; ++i) {
        mbar_init(p_full + 8 * i, kAttnSoftmaxThreads / 32);
        mbar_init(p_free + 8 * i, 1);
      }
      mbar_fence_init();
      tma_prefetch_desc(&tmap_q);
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_v);
    }
    __syncwarp();
    if (head_ok) {
      mbar_arrive_expect_tx_elect(bar_k, static_cast<uint32_t>(sk) * 128u);
      for (int r = 0; r < sk; r += kAttnKvBoxRows) {
        tma_load_2d_elect(k_s + static_cast<uint32_t>(r) * 128u, &tmap_k, bar_k, h.k_col, h.k_row + r);
      }
      mbar_arrive_expect_tx_elect(bar_q, kAttnBlockM * 128u);
      tma_load_2d_elect(q_s, &tmap_q, bar_q, h.q_col, h.q_row + blk_begin * kAttnBlockM);
      mbar_arrive_expect_tx_elect(bar_v, static_cast<uint32_t>(sk) * 128u);
      for (int r = 0; r < sk; r += kAttnKvBoxRows) {
        tma_load_2d_elect(v_s + static_cast<uint32_t>(r) * 128u, &tmap_v, bar_v, h.v_col, h.v_row + r);
      }
    }
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

  if (warp == kAttnCtrlWarp) {
    // ---- control warp: every copy and every tensor-core instruction, issued by one elected lane
    // of warp-uniform code (descriptors then stay in uniform registers, which is what keeps the
    // issue of the small P V instructions cheap) ------------------------------------------------------
    if (head_ok) {
      // Descriptors differ only in the start address (bits 0-13, in 16-byte units), so a step is an add.
      const uint32_t idesc_pv = make_instr_desc(fmt, 0, 1, kAttnBlockM, kAttnHeadDim);
      const uint64_t q_desc = make_smem_desc_sw128(q_s, 16, 1024);
      const uint64_t k_desc = make_smem_desc_sw128(k_s, 16, 1024);
      const uint64_t p_desc = make_smem_desc_sw128(p_s, 16, 1024);
      const uint64_t v_desc = make_smem_desc(v_s, static_cast<uint32_t>(sk) * 128u, 1024, kLayoutSw128);
      // S[128, sk] = Q[128, 64] K[sk, 64]^T over key columns [n0, n0 + nn): both operands K-major,
      // four 32-byte K steps.
      auto scores = [&](int n0, int nn) {
        if (nn <= 0) return;
        const uint32_t idesc = make_instr_desc(fmt, 0, 0, kAttnBlockM, static_cast<uint32_t>(nn));
        const uint64_t kb_desc = k_desc + static_cast<uint64_t>(n0 * 8);   // n0 rows of 128 bytes
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          mma_f16_elect(tmem_base + static_cast<uint32_t>(n0), q_desc + ks * 2, kb_desc + ks * 2, idesc,
                        ks > 0 ? 1u : 0u);
        }
      };
      // O lies over S's first 64 columns, so the next block's scores are issued in two parts: the
      // columns from 64 up as soon as every softmax warp has handed over its last block of P (it
      // has then read all of S), the first 64 once O has been read.
      auto scores_upper = [&] {
        scores(64, (sk < 256 ? sk : 256) - 64);
        scores(256, sk - 256);
        mma_commit_elect(bar_su);   // the row-maximum sweep starts on these columns
      };
      bool live = mbar_wait_warp(bar_k, 0, status, kFaultAttnLoad) &&
                  mbar_wait_warp(bar_q, 0, status, kFaultAttnLoad);
      if (live) {
        tcgen05_fence_after_sync();
        scores_upper();
        scores(0, 64);
        mma_commit_elect(bar_s);
      }
      uint32_t n = 0;   // blocks of P consumed so far: ring slot n % 4, use n / 4
      for (int b = 0; live && b < nb; ++b) {
        const uint32_t ph = static_cast<uint32_t>(b & 1);
        live = mbar_wait_warp(bar_s, ph, status, kFaultAttnScores);
        if (!live) break;
        if (b + 1 < nb) {   // Q's bytes are free again: the next block's rows travel under the softmax
          mbar_arrive_expect_tx_elect(bar_q, kAttnBlockM * 128u);
          tma_load_2d_elect(q_s, &tmap_q, bar_q, h.q_col, h.q_row + (blk_begin + b + 1) * kAttnBlockM);
        }
        if (b == 0) live = mbar_wait_warp(bar_v, 0, status, kFaultAttnValues);
        // O[128, 64] += P[128, 64 keys] V[64 keys, 64]: A K-major, B MN-major as loaded.
        uint64_t vb_desc = v_desc;
        for (int c = 0; live && c < n_chunks; ++c, ++n) {
          const uint32_t slot = n & (kAttnPRing - 1), use = n / kAttnPRing;
          live = mbar_wait_warp(p_full + 8 * slot, use & 1u, status, kFaultAttnProbs);
          if (!live) break;
          tcgen05_fence_after_sync();
          const uint64_t pa_desc = p_desc + static_cast<uint64_t>(slot * (kAttnPBlockBytes / 16));
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            mma_f16_elect(tmem_base, pa_desc + ks * 2, vb_desc + ks * 128, idesc_pv, (c > 0 || ks > 0) ? 1u : 0u);
          }
          vb_desc += 4 * 128;   // 64 keys = four 2048-byte steps
          mma_commit_elect(p_free + 8 * slot);
        }
        if (!live) break;
        mma_commit_elect(bar_o);
        if (b + 1 < nb) {
          live = mbar_wait_warp(bar_q, static_cast<uint32_t>((b + 1) & 1), status, kFaultAttnLoad);
          if (!live) break;
          scores_upper();
          // every softmax thread has read O of this block
          live = mbar_wait_warp(bar_oread, ph, status, kFaultAttnDrain);
          if (!live) break;
          tcgen05_fence_after_sync();
          scores(0, 64);
          mma_commit_elect(bar_s);
        }
      }
    }
    __syncwarp();
  } else {
    // ---- softmax warps: four threads per query row -----------------------------------------------
    // Warp w works on TMEM lanes 32*(w & 3) .. +31 (the only lanes it may touch), on 16 of every 64
    // keys (a quarter of each block of P).  Row maximum and row sum are exchanged through shared
    // memory.  Each sweep keeps the next 16-column tcgen05.ld in flight while the current one is
    // processed.
    const int quad = warp & 3, part = warp >> 2;
    const int row_in_tile = quad * 32 + (tid & 31);
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    float* red_max = reinterpret_cast<float*>(base_ptr + bar_off + 128);   // [parts][128]
    float* red_sum = red_max + kAttnParts * kAttnBlockM;
    auto softmax_sync = [] { asm volatile("bar.sync 1, %0;" ::"n"(kAttnSoftmaxThreads) : "memory"); };
    const uint32_t col0 = lane_addr + static_cast<uint32_t>(part * 16);   // this thread's 16 of every 64 keys
    // RESCALE: the scaled scores are rounded to T again (the reference's `mul` stores them).  Without
    // it the scale is 1 or a power of two, the product is exact, and the factor folds into the exp.
    const float exp_mul = RESCALE ? 1.4426950408889634f : scale * 1.4426950408889634f;
    uint8_t* p_row = base_ptr + p_off + static_cast<uint32_t>(row_in_tile) * 128u;
    const uint32_t swz = static_cast<uint32_t>(row_in_tile & 7);
    const uint32_t unit0 = static_cast<uint32_t>(part * 2);   // this thread's 16-byte units of a P row
    bool ok = head_ok;   // warp-uniform throughout: every wait below is taken by the warp as one
    uint32_t n = 0;      // blocks of P produced so far
    for (int b = 0; b < nb; ++b) {
      const uint32_t ph = static_cast<uint32_t>(b & 1);
      // Row maximum: the key columns from 64 up as soon as they are there, the first 64 (which wait
      // for the previous block's O to be read) after them.
      float mx = -INFINITY;
      auto max16 = [&](const uint32_t (&r)[16]) {
#pragma unroll
        for (int i = 0; i < 16; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
      };
      ok = ok && mbar_wait_warp(bar_su, ph, status, kFaultAttnScores);
      if (ok && n_chunks > 1) {
        tcgen05_fence_after_sync();
        uint32_t ra[16], rb[16];
        tmem_ld_32x32b_x16(col0 + 64u, ra);
        for (int c = 1; c < n_chunks; c += 2) {
          tmem_ld_wait(ra);
          const bool two = c + 1 < n_chunks;
          if (two) tmem_ld_32x32b_x16(col0 + static_cast<uint32_t>((c + 1) * 64), rb);
          max16(ra);
          if (two) {
            tmem_ld_wait(rb);
            if (c + 2 < n_chunks) tmem_ld_32x32b_x16(col0 + static_cast<uint32_t>((c + 2) * 64), ra);
            max16(rb);
          }
        }
      }
      ok = ok && mbar_wait_warp(bar_s, ph, status, kFaultAttnScores);
      if (ok) {
        tcgen05_fence_after_sync();
        uint32_t r0[16];
        tmem_ld_32x32b_x16(col0, r0);
        tmem_ld_wait(r0);
        max16(r0);
        mx = stored_score<T>(mx);   // rounding is monotonic: max of the rounded = rounded max
        // an optional `mul` by a constant between the matmul and the softmax (the reference's own
        // attention scales there): its result is rounded to T again; a positive scale keeps the maximum
        mx = RESCALE ? stored_score<T>(mx * scale) : mx * scale;
      }
      red_max[part * kAttnBlockM + row_in_tile] = mx;
      softmax_sync();
#pragma unroll
      for (int i = 0; i < kAttnParts; ++i) mx = fmaxf(mx, red_max[i * kAttnBlockM + row_in_tile]);
      float sum = 0.0f;
      if (ok) {
        // exp, row sum and P in one sweep: P = e rounded to T, in the A-operand layout (a block of 64
        // keys is 128 rows of 128 bytes, the 16-byte unit index XORed with (row & 7)); this thread
        // converts keys 16*part .. +15 of every block.  The division by the row sum is applied to O.
        const float mx2 = mx * 1.4426950408889634f;
        const float2 mul2 = make_float2(exp_mul, exp_mul), nmx2 = make_float2(-mx2, -mx2);
        float2 sum2 = make_float2(0.0f, 0.0f);
        auto emit = [&](int c, uint32_t (&r)[16]) {
          // the ring slot's release is polled before the arithmetic, so the answer is there after it
          const uint32_t slot = (n + c) & (kAttnPRing - 1), use = (n + c) / kAttnPRing;
          const bool slot_free = use == 0 || mbar_try_wait(p_free + 8 * slot, (use - 1) & 1u);
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            float s0 = __uint_as_float(r[i]), s1 = __uint_as_float(r[i + 1]);
            stored_pair<T>(s0, s1);
            if constexpr (RESCALE) {
              s0 *= scale;
              s1 *= scale;
              stored_pair<T>(s0, s1);
            }
            // packed fp32 pairs: one FMA-pipe instruction per two scores for the exponent and the sum
            const float2 x = __ffma2_rn(make_float2(s0, s1), mul2, nmx2);
            const float e0 = ex2_approx(x.x), e1 = ex2_approx(x.y);
            sum2 = __fadd2_rn(sum2, make_float2(e0, e1));
            r[i >> 1] = pack2<T>(e0, e1);
          }
          if (!__all_sync(0xffffffffu, slot_free)) ok = mbar_wait_warp(p_free + 8 * slot, (use - 1) & 1u, status, kFaultAttnProbs);
          if (!ok) return;
          uint8_t* blk = p_row + slot * kAttnPBlockBytes;
          *reinterpret_cast<uint4*>(blk + (((unit0 + 0) ^ swz) << 4)) = make_uint4(r[0], r[1], r[2], r[3]);
          *reinterpret_cast<uint4*>(blk + (((unit0 + 1) ^ swz) << 4)) = make_uint4(r[4], r[5], r[6], r[7]);
          fence_proxy_async_smem();      // P must be visible to the tensor core's reads
          tcgen05_fence_before_sync();   // and the loads of these columns ordered before O is written
          __syncwarp();
          if ((tid & 31) == 0) mbar_arrive(p_full + 8 * slot);
        };
        uint32_t ra[16], rb[16];
        tmem_ld_32x32b_x16(col0, ra);
        for (int c = 0; c < n_chunks; c += 2) {
          tmem_ld_wait(ra);
          const bool two = c + 1 < n_chunks;
          if (two) tmem_ld_32x32b_x16(col0 + static_cast<uint32_t>((c + 1) * 64), rb);
          emit(c, ra);
          if (two) {
            tmem_ld_wait(rb);
            if (c + 2 < n_chunks) tmem_ld_32x32b_x16(col0 + static_cast<uint32_t>((c + 2) * 64), ra);
            emit(c + 1, rb);
          }
        }
        sum = sum2.x + sum2.y;
      }
      red_sum[part * kAttnBlockM + row_in_tile] = sum;
      softmax_sync();
      sum = 0.0f;   // the same order in every thread of a row
#pragma unroll
      for (int i = 0; i < kAttnParts; ++i) sum += red_sum[i * kAttnBlockM + row_in_tile];
      const float inv = 1.0f / sum;
      n += static_cast<uint32_t>(n_chunks);
      ok = ok && mbar_wait_warp(bar_o, ph, status, kFaultAttnOutput);
      if (ok) {
        tcgen05_fence_after_sync();
        const int row = (blk_begin + b) * kAttnBlockM + row_in_tile;
        const int c = part * 16;   // each quarter of the warps stores 16 of the 64 columns
        T* dst = o_base + h.o_offset + static_cast<int64_t>(row) * o_ld + c;
        uint32_t r[16];
        tmem_ld_32x32b_x16(lane_addr + static_cast<uint32_t>(c), r);
        tmem_ld_wait(r);
        tcgen05_fence_before_sync();
        __syncwarp();
        if ((tid & 31) == 0) mbar_arrive(bar_oread);   // the next block's scores may overwrite O now
        if (row < sq) {
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            uint4 v;
            v.x = pack2<T>(__uint_as_float(r[8 * u + 0]) * inv, __uint_as_float(r[8 * u + 1]) * inv);
            v.y = pack2<T>(__uint_as_float(r[8 * u + 2]) * inv, __uint_as_float(r[8 * u + 3]) * inv);
            v.z = pack2<T>(__uint_as_float(r[8 * u + 4]) * inv, __uint_as_float(r[8 * u + 5]) * inv);
            v.w = pack2<T>(__uint_as_float(r[8 * u + 6]) * inv, __uint_as_float(r[8 * u + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + 8 * u) = v;
          }
        }
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
  // Query blocks per CTA: the run length that minimises (waves of CTAs) x (loading K and V once +
  // one softmax per block), the load counted as 0.8 of a block; longer runs win ties (less traffic).
  int64_t per_cta = 1;
  double best = 0.0;
  for (int64_t g = 1; g <= q_blocks; ++g) {
    const int64_t ctas = n_heads * ((q_blocks + g - 1) / g);
    const double cost = static_cast<double>((ctas + kNumSMs - 1) / kNumSMs) * (0.8 + static_cast<double>(g));
    if (g == 1 || cost <= best) { best = cost; per_cta = g; }
  }
  const int64_t groups = (q_blocks + per_cta - 1) / per_cta;
  if (n_heads * groups > 0x7fffffff) return set_error(FB200_INVALID_ARGUMENT, "attention_fan: too many tiles");
  CUtensorMap tq, tk, tv;
  if (int rc = make_tmap_2d(&tq, q_base, dtype, q_rows, q_ld, kAttnBlockM, false)) return rc;
  if (int rc = make_tmap_2d(&tk, k_base, dtype, k_rows, k_ld, kAttnKvBoxRows, false)) return rc;
  if (int rc = make_tmap_2d(&tv, v_base, dtype, v_rows, v_ld, kAttnKvBoxRows, false)) return rc;
  int* status = nullptr;
  if (int rc = device_status_word(&status)) return rc;
  uint32_t tmem_cols = 64;
  while (tmem_cols < static_cast<uint32_t>(sk)) tmem_cols *= 2;
  const size_t smem = 1024 /*align*/ + kAttnBlockM * 128 + static_cast<size_t>(sk) * 256 +
                      kAttnPRing * kAttnPBlockBytes + 128 /*barriers*/ +
                      2 * kAttnParts * kAttnBlockM * sizeof(float) /*row max and sum exchange*/;
  const int grid = static_cast<int>(n_heads * groups);
  cudaStream_t s = as_stream(stream);
  // A power-of-two scale multiplies a bfloat16 score exactly, so rounding it again changes nothing.
  int scale_exp = 0;
  const bool exact_scale = scale == 1.0f || (dtype == FB200_BF16 && std::frexp(scale, &scale_exp) == 0.5f &&
                                             scale_exp >= -15 && scale_exp <= 17);
  auto launch = [&](auto kernel, auto* out, uint32_t fmt) -> int {
    FB200_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    kernel<<<grid, kAttnThreads, smem, s>>>(tq, tk, tv, heads_dev, out, o_ld, static_cast<int>(sq),
                                            static_cast<int>(sk), static_cast<int>(q_blocks),
                                            static_cast<int>(per_cta), static_cast<int>(groups), tmem_cols, fmt,
                                            scale, status);
    return FB200_OK;
  };
  int rc = FB200_OK;
  if (dtype == FB200_BF16) {
    auto* out = static_cast<__nv_bfloat16*>(o_base);
    rc = exact_scale ? launch(attention_fan_kernel<__nv_bfloat16, false>, out, kFmtBF16)
                     : launch(attention_fan_kernel<__nv_bfloat16, true>, out, kFmtBF16);
  } else {
    auto* out = static_cast<__half*>(o_base);
    rc = exact_scale ? launch(attention_fan_kernel<__half, false>, out, kFmtF16)
                     : launch(attention_fan_kernel<__half, true>, out, kFmtF16);
  }
  if (rc != FB200_OK) return rc;
  return after_launch("attention_fan_kernel");
}
