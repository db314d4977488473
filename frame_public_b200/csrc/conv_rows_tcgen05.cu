// conv2d with stride 2 and few input channels (an image stem: 3 -> 64 channels, 7 x 7, stride 2) as
// an implicit GEMM on the tensor cores whose A operand is built ONCE PER INPUT ROW instead of once
// per output tile (fp32 tensors, TF32 math, fp32 accumulation).
//
// Semantics: src/backends/cpu/kernels/conv.cpp:225-257 (NCHW cross-correlation, zero padding, bias
// per output channel added last); used when CompileOptions::allow_tf32 permits reduced precision
// (include/frame/hal/backend.h:51-63).  Replaces cudnnConvolutionForward + cudnnAddTensor of
// src/backends/cuda/kernels/conv.cpp:385-520 and the activation launch after it.
//
// GEMM view of one output row oy of one image: D[px, co] = sum_ky sum_(kx, c) A_ky[px, (kx, c)] *
// W_ky[co, (kx, c)], with A_ky[px, (kx, c)] = in[c][2 oy + ky - pad][2 px + kx - pad].  For a fixed
// INPUT row r the matrix P_r[(kx, c)][px] = in[c][r][2 px + kx - pad] does not depend on which output
// row reads it: output row oy uses P_r for r = 2 oy - pad + ky, ky = 0 .. KH-1, and its neighbour
// oy + 1 shares all but two of those rows.  A CTA therefore walks a contiguous run of output rows and
// keeps a ring of row matrices in shared memory, in exactly the layout tcgen05 wants for an MN-major
// 32-bit A operand (32-pixel spans of 128 bytes per k-row, 32-byte units XOR-swizzled by k & 3):
//   * per new output row only TWO input rows are turned into row matrices: every input element is
//     loaded once (8-byte loads straight from global memory, issued one output row ahead) and stored
//     to the up to four (kx, px) positions that read it, consecutive lanes to consecutive pixels, at
//     byte offsets worked out once per thread.  The halo kernel this replaces for such shapes
//     gathered 128 x 160 operand elements per output row through a table (17 instructions per
//     element, shared-memory wavefronts on 47 % of all cycles);
//   * a filter row ky is a descriptor whose start address is the ring slot of input row
//     2 oy - pad + ky; rows above or below the image point at a slot that stays zero;
//   * K per filter row is KW * Cin padded to a multiple of 8 (21 -> 24 for the stem): KH * 3 = 21
//     tcgen05.mma (M = 128 pixels, N = Cout) per output row, issued from straight-line code;
//   * the weights of all filter rows stay resident (K-major, 128-byte swizzle).
// 672 threads: warps 0-3 build row matrices, warp 4 issues the MMAs, warps 5-20 are TWO epilogue
// groups of eight warps, one per TMEM accumulator, so that the stores of output row i run under the
// TMEM loads and the arithmetic of row i + 1.  Results are stored straight from registers: lane =
// pixel, one 128-byte run per channel and warp.  (A shared-memory tile handed to a 4-D TMA store per
// row costs the same per row and cannot overlap without a second tile, for which there is no room.)
// Positions of a ring slot that no input element maps to (left and right padding, the k-rows past
// KW * Cin, pixels past OW) are zeroed once and never written.  Every wait is bounded.
//
// What bounds it (per-role cycle counters, 32 x 3 x 224 x 224 -> 64 channels, 24 output rows per CTA):
// the launch writes 103 MB, and while the epilogue's stores queue in the SM's load/store path (about
// 2 K cycles per output row when the memory system takes 3.9 TB/s of writes) the builders' shared
// memory stores and global loads wait in the same queue: 42 stores take 1.8 K cycles and a load
// takes 5 K cycles to come back, hence the cp.async prefetch two rows ahead.  The MMAs themselves
// need 1.7 K cycles per output row (82 per instruction).  Measured: 73 us against 95 us for the
// halo kernel on this shape (floor: 103 MB of writes = 27 us).
// FLOPs per launch = 2 * N*OH*OW * Cout * Cin*KH*KW; bytes = input + output once.
#include <cuda.h>

#include "common.cuh"
#include "epilogue.cuh"
#include "sm100_ptx.cuh"

namespace fb200 {

int device_status_word(int** dev_ptr);  // gemm_tcgen05.cu

using namespace sm100;

constexpr int kRowsBuilders = 128;                    // warps 0-3 (eight warps with two tasks each measured the same)
constexpr int kRowsMmaWarp = 4;
constexpr int kRowsFirstEpiWarp = 5;                  // warps 5-12: accumulator 0, warps 13-20: accumulator 1
constexpr int kRowsThreads = (kRowsFirstEpiWarp + 16) * 32;
constexpr int kRowsTasks = 3;                         // element pairs per builder thread and input row
constexpr int kRowsMaxKh = 8;
constexpr int kRowsMaxKw = 8;
constexpr int kRowsPfStages = 3;                      // output rows the input-row prefetch runs ahead, plus one

enum RowsFault : int {
  kFaultRowsFreed = 231,     // builders: the MMAs two output rows back never completed
  kFaultRowsBuilt = 232,     // MMA: the row matrices of this output row never arrived
  kFaultRowsTmem = 233,      // MMA: accumulator never drained
  kFaultRowsEpilogue = 234,  // epilogue: accumulator never completed
  kFaultRowsPoolRow = 235,   // pooling epilogue: the other group's row never arrived / was never consumed
};

struct RowsGeom {
  int n, cin, h, w, cout, kh, kw, ph, pw, oh, ow;
  int kp;          // KW * Cin padded to a multiple of 8: k extent of one filter row
  int npad;        // Cout padded to a multiple of 32
  int n_slots;     // ring slots (KH + 2: the KH rows an output row reads and the two being built); slot n_slots is the zero slot
  int slot_bytes;  // 4 spans x kp k-rows x 128 bytes
  int w_bytes;     // KH x npad x 128
  int tmem_cols;
  int64_t total_rows;   // n * oh
  int poh, pow;         // fused 3 x 3 / stride 2 / pad 1 max-pool: pooled rows and columns (else 0)
};

// Byte offset of element (k, px) inside a row matrix.
__device__ __forceinline__ uint32_t rows_elem_off(int k, int px, int kp) {
  return static_cast<uint32_t>((px >> 5) * kp * 128 + k * 128 + ((((px >> 3) & 3) ^ (k & 3)) << 5) + (px & 7) * 4);
}

// KH and KSTEPS (= kp / 8) are compile-time so that the MMA warp's loop over an output row's filter
// rows is straight-line code: KH descriptors, then KH * KSTEPS instructions with immediate offsets
// (with run-time loops the issue took 167 cycles per tcgen05.mma instead of 63).
// POOL: the epilogue max-pools the finished rows (3 x 3 windows, stride 2, padding 1) and stores only
// the pooled tensor.  A CTA then owns a run of POOLED rows and computes the conv rows they cover
// (2 p - 1 .. 2 p + 1; the first of them is also computed by the CTA before: one row in 25 twice).
// Conv rows alternate between the two epilogue groups, so one group always has the odd rows and the
// other the even ones: a thread of the odd group keeps its previous row's column maxima in
// registers, the even row in between crosses through one of two 14 KB shared-memory buffers.
template <int KH, int KSTEPS, bool POOL>
__global__ void __launch_bounds__(kRowsThreads, 1)
conv2d_rows_tcgen05_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                           float* __restrict__ out, RowsGeom g, uint32_t idesc, EpilogueDev epi, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw_addr);
  // layout: ring slots + zero slot | weights | barriers, bias | input-row prefetch slices
  const uint32_t w_off = static_cast<uint32_t>((g.n_slots + 1) * g.slot_bytes);
  const uint32_t bar_off = w_off + static_cast<uint32_t>(g.w_bytes);
  const uint32_t bars = base + bar_off;
  auto built_bar = [&](int p) { return bars + 8u * p; };
  auto freed_bar = [&](int p) { return bars + 8u * (2 + p); };
  auto tmem_full = [&](int a) { return bars + 8u * (4 + a); };
  auto tmem_empty = [&](int a) { return bars + 8u * (6 + a); };
  const uint32_t tmem_slot = bars + 64;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(base_ptr + bar_off + 64);
  float* bias_s = reinterpret_cast<float*>(base_ptr + bar_off + 128);   // [256]
  const uint32_t pf_off = bar_off + 128 + 1024;   // input-row prefetch: [stages][2 rows][tasks][128 threads] x 8 bytes
  const uint32_t edge_off = pf_off + kRowsPfStages * 2 * kRowsTasks * kRowsBuilders * 8;   // POOL: [16 warps][32] floats
  const uint32_t even_off = edge_off + 16 * 32 * 4;                                          // POOL: two buffers of [npad][pow] floats
  auto even_ready = [&](int b) { return bars + 8u * (9 + b); };
  auto even_free = [&](int b) { return bars + 8u * (11 + b); };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  int64_t row_begin, row_end;
  if (POOL) {
    // pooled rows [p0, p1) of the list (image, pooled row) -> the conv rows they cover
    const int64_t p_total = static_cast<int64_t>(g.n) * g.poh;
    const int64_t p0 = p_total * blockIdx.x / gridDim.x, p1 = p_total * (blockIdx.x + 1) / gridDim.x;
    if (p1 > p0) {
      const int64_t img_a = p0 / g.poh, img_b = (p1 - 1) / g.poh;
      const int pa = static_cast<int>(p0 - img_a * g.poh), pb = static_cast<int>(p1 - 1 - img_b * g.poh);
      row_begin = img_a * g.oh + (2 * pa - 1 > 0 ? 2 * pa - 1 : 0);
      row_end = img_b * g.oh + (2 * pb + 1 < g.oh - 1 ? 2 * pb + 1 : g.oh - 1) + 1;
    } else {
      row_begin = row_end = 0;
    }
  } else {
    row_begin = g.total_rows * blockIdx.x / gridDim.x;
    row_end = g.total_rows * (blockIdx.x + 1) / gridDim.x;
  }
  const int n_items = static_cast<int>(row_end - row_begin);

  if (threadIdx.x == 0) {
    for (int p = 0; p < 2; ++p) {
      mbar_init(built_bar(p), kRowsBuilders / 32);   // one arrival per builder warp
      mbar_init(freed_bar(p), 1);
      mbar_init(tmem_full(p), 1);
      mbar_init(tmem_empty(p), 8);                   // the eight warps of the accumulator's group
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(even_ready(b), 8);
      mbar_init(even_free(b), 8);
    }
    mbar_fence_init();
  }
  // The weights' loads go out first (16 per thread in flight) and land while the ring and the
  // weight block are zeroed (the positions nothing maps to stay zero for good).
  const int khkw = g.kh * g.kw;
  const int per_co = g.cin * khkw;
  const int w_total = g.cout * per_co;
  float wv[16];
#pragma unroll
  for (int u = 0; u < 16; ++u) {
    const int e = threadIdx.x + u * kRowsThreads;
    wv[u] = __ldg(w + (e < w_total ? e : 0));
  }
  {
    const uint32_t zero_bytes = w_off + static_cast<uint32_t>(g.w_bytes);
    uint4* z = reinterpret_cast<uint4*>(base_ptr);
    for (uint32_t i = threadIdx.x; i < zero_bytes / 16; i += kRowsThreads) z[i] = make_uint4(0, 0, 0, 0);
  }
  for (int c = threadIdx.x; c < 256; c += kRowsThreads) {
    bias_s[c] = (bias != nullptr && c < g.cout) ? __ldg(bias + c) : 0.0f;
  }
  if (warp == kRowsMmaWarp) {
    __syncwarp();
    tmem_alloc(tmem_slot, static_cast<uint32_t>(g.tmem_cols));
    tmem_relinquish();
  }
  __syncthreads();
  // weights: w[co][c][ky][kx] -> block ky, row co, k = kx * Cin + c (K-major, 16-byte units XORed
  // with co & 7)
  auto put_weight = [&](int e, float val) {
    const int co = e / per_co, rem = e - co * per_co;
    const int c = rem / khkw, tap = rem - c * khkw;
    const int ky = tap / g.kw, kx = tap - ky * g.kw;
    const int k = kx * g.cin + c;
    const uint32_t off = w_off + static_cast<uint32_t>(ky * g.npad * 128 + (co >> 3) * 1024 + (co & 7) * 128 +
                                                       (((k >> 2) ^ (co & 7)) << 4) + (k & 3) * 4);
    *reinterpret_cast<float*>(base_ptr + off) = val;
  };
#pragma unroll
  for (int u = 0; u < 16; ++u) {
    const int e = threadIdx.x + u * kRowsThreads;
    if (e < w_total) put_weight(e, wv[u]);
  }
  for (int e = threadIdx.x + 16 * kRowsThreads; e < w_total; e += kRowsThreads) put_weight(e, __ldg(w + e));
  fence_proxy_async_smem();
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;

  // Output rows are walked in order: (img, oy) advance by increments (a 64-bit division per row and
  // role costs more than the row's stores); the ring starts afresh at the CTA's first row and at
  // the first row of every image.
  const int img0 = static_cast<int>(row_begin / g.oh);
  const int oy0 = static_cast<int>(row_begin - static_cast<int64_t>(img0) * g.oh);

  if (warp < kRowsMmaWarp) {
    // ---- builders -------------------------------------------------------------------------------
    // A task is one pair of neighbouring input elements (c, 2 j), (c, 2 j + 1) of a row: thread t
    // owns tasks t, t + 128, t + 256 of every row (Cin * W / 2 tasks per row).  Where a pair goes
    // inside a row matrix does not depend on the row: filter column kx reads element
    // e = (kx + pad) & 1 of the pair, at pixel j + (e + pad - kx) / 2.  The byte offsets are worked
    // out once per thread (bit 0: which element; -1: outside the row), so that a row costs its
    // loads, its stores and one addition per store.
    const int tid = threadIdx.x;
    const int wh = g.w / 2;
    const int tasks_per_row = g.cin * wh;
    int st_off[kRowsTasks][kRowsMaxKw];
    int ld_off[kRowsTasks];
    bool t_ok[kRowsTasks];
#pragma unroll
    for (int t = 0; t < kRowsTasks; ++t) {
      const int q = tid + t * kRowsBuilders;
      t_ok[t] = q < tasks_per_row;
      const int c = t_ok[t] ? q / wh : 0;
      const int j = t_ok[t] ? q - c * wh : 0;
      ld_off[t] = c * g.h * g.w + 2 * j;   // 0 for a thread without this task: a valid address
#pragma unroll
      for (int kx = 0; kx < kRowsMaxKw; ++kx) {
        const int e = (kx + g.pw) & 1;
        const int px = j + ((e + g.pw - kx) >> 1);   // e + pad - kx is even: exact
        st_off[t][kx] = (t_ok[t] && kx < g.kw && px >= 0 && px < g.ow)
                            ? static_cast<int>(rows_elem_off(kx * g.cin + c, px, g.kp)) | e : -1;
      }
    }
    auto scatter = [&](int slot, int t, float2 v) {
      const uint32_t sb = base + static_cast<uint32_t>(slot) * static_cast<uint32_t>(g.slot_bytes);
#pragma unroll
      for (int kx = 0; kx < kRowsMaxKw; ++kx) {
        const int o = st_off[t][kx];
        if (o >= 0) {
          asm volatile("st.shared.f32 [%0], %1;" ::"r"(sb + static_cast<uint32_t>(o & ~3)), "f"((o & 1) ? v.y : v.x) : "memory");
        }
      }
    };
    auto load_pair = [&](int64_t img_off, int r, int t) {
      return __ldg(reinterpret_cast<const float2*>(x + img_off + r * g.w + ld_off[t]));
    };
    const int64_t img_elems = static_cast<int64_t>(g.cin) * g.h * g.w;
    int img = img0, oy = oy0;
    // The two new input rows of an output row are fetched TWO output rows ahead with cp.async into
    // a slice of shared memory that only this thread reads back (no barrier: cp.async.wait_group
    // covers it).  Register prefetching one row ahead was not enough: with the epilogue's stores
    // saturating the memory system a load takes about 5 K cycles to come back.  The copies are
    // unconditional, from a clamped row and (for a thread without a task) from offset 0; rows outside
    // the image are simply not scattered, and an output row whose ring starts afresh loads all of
    // its input rows itself.
    const uint32_t pf_mine = base + pf_off + static_cast<uint32_t>(tid) * 8u;
    auto pf_addr = [&](int stage, int rr, int t) {
      return pf_mine + static_cast<uint32_t>(((stage * 2 + rr) * kRowsTasks + t) * (kRowsBuilders * 8));
    };
    int pc_img = img0, pc_oy = oy0;   // cursor of the output row whose input rows are fetched next
    auto advance_cursor = [&]() { if (++pc_oy == g.oh) { pc_oy = 0; ++pc_img; } };
    auto fetch = [&](int item) {      // item = index of the cursor's output row; always commits a group
      if (item < n_items) {
        const int r_hi = 2 * pc_oy - g.ph + g.kh - 1;
        const int64_t img_off = static_cast<int64_t>(pc_img) * img_elems;
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
          int r = r_hi - 1 + rr;
          r = r < 0 ? 0 : (r >= g.h ? g.h - 1 : r);
#pragma unroll
          for (int t = 0; t < kRowsTasks; ++t) {
            const float* src = x + img_off + r * g.w + ld_off[t];
            asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(pf_addr(item % kRowsPfStages, rr, t)), "l"(src) : "memory");
          }
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    advance_cursor();   // item 0 starts the ring afresh and loads its rows itself
    fetch(1);
    advance_cursor();
    bool ok = true;
    int slot_hi = 0;   // ring slot of the newest row of the output row being built
    for (int i = 0; i < n_items && ok; ++i) {
      const bool fresh = i == 0 || oy == 0;
      fetch(i + 2);
      advance_cursor();
      asm volatile("cp.async.wait_group 2;" ::: "memory");   // the group of item i has landed
      float2 cur[2][kRowsTasks];
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
#pragma unroll
        for (int t = 0; t < kRowsTasks; ++t) {
          asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(cur[rr][t].x), "=f"(cur[rr][t].y) : "r"(pf_addr(i % kRowsPfStages, rr, t)) : "memory");
        }
      }
      // The slots written now were last read by the MMAs of item i - 2 (i - 1 when the ring starts
      // afresh: all of its slots are rewritten).
      if (i >= 2) ok = mbar_wait(freed_bar(i & 1), static_cast<uint32_t>((i >> 1) - 1) & 1u, status, kFaultRowsFreed);
      if (ok && fresh && i >= 1) {
        ok = mbar_wait(freed_bar((i - 1) & 1), static_cast<uint32_t>((i - 1) >> 1) & 1u, status, kFaultRowsFreed);
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const int r_lo = 2 * oy - g.ph, r_hi = r_lo + g.kh - 1;
      if (fresh) {
        // all KH rows, four at a time with their loads in flight together
        const int64_t img_off = static_cast<int64_t>(img) * img_elems;
        int slot = (2 * oy) % g.n_slots;   // slot of row r is (r + pad) mod n_slots
        for (int r0 = r_lo; r0 <= r_hi; r0 += 4) {
          float2 v[4][kRowsTasks];
#pragma unroll
          for (int rr = 0; rr < 4; ++rr) {
            int r = r0 + rr;
            r = r < 0 ? 0 : (r >= g.h ? g.h - 1 : r);
#pragma unroll
            for (int t = 0; t < kRowsTasks; ++t) v[rr][t] = load_pair(img_off, r, t);
          }
#pragma unroll
          for (int rr = 0; rr < 4; ++rr) {
            const int r = r0 + rr;
            if (r <= r_hi) {
              if (r >= 0 && r < g.h) {
#pragma unroll
                for (int t = 0; t < kRowsTasks; ++t) scatter(slot, t, v[rr][t]);
              }
              slot_hi = slot;
              if (++slot == g.n_slots) slot = 0;
            }
          }
        }
      } else {
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
          if (++slot_hi == g.n_slots) slot_hi = 0;
          const int r = r_hi - 1 + rr;
          if (r >= 0 && r < g.h) {
#pragma unroll
            for (int t = 0; t < kRowsTasks; ++t) scatter(slot_hi, t, cur[rr][t]);
          }
        }
      }
      fence_proxy_async_smem();   // generic-proxy writes -> visible to the tensor core's reads
      __syncwarp();
      if (lane == 0) mbar_arrive(built_bar(i & 1));
      if (++oy == g.oh) { oy = 0; ++img; }
    }
  } else if (warp == kRowsMmaWarp) {
    // ---- MMA issue: the whole warp runs the loop, one elected lane issues ---------------------------
    // A: MN-major, 32-pixel spans kp * 128 bytes apart (LBO), 4-row k groups 512 bytes apart (SBO);
    // one MMA (K = 8) covers two groups = 1024 bytes.  B: K-major, 8-row groups 1024 bytes apart; a K
    // step is 32 bytes inside the row.
    const uint64_t a_desc0 = make_smem_desc(base, static_cast<uint32_t>(g.kp) * 128u, 512, kLayoutSw128Base32);
    const uint64_t b_desc0 = make_smem_desc(base + w_off, 16, 1024, kLayoutSw128);
    const uint32_t slot_units = static_cast<uint32_t>(g.slot_bytes) >> 4;
    const uint32_t wrow_units = static_cast<uint32_t>(g.npad * 128) >> 4;
    bool ok = true;
    int oy = oy0;
    int slot_lo = (2 * oy0) % g.n_slots;   // slot of the row that filter row 0 reads
    for (int i = 0; i < n_items && ok; ++i) {
      const int acc = i & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(tmem_empty(acc), (static_cast<uint32_t>(i >> 1) & 1u) ^ 1u, status, kFaultRowsTmem));
      if (!ok) break;
      ok = __all_sync(0xffffffffu, mbar_wait(built_bar(acc), static_cast<uint32_t>(i >> 1) & 1u, status, kFaultRowsBuilt));
      if (!ok) break;
      tcgen05_fence_after_sync();
      const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * g.npad);
      uint64_t a_desc[KH];
      {
        int slot = slot_lo;
        int r = 2 * oy - g.ph;
#pragma unroll
        for (int ky = 0; ky < KH; ++ky) {
          const int use = (r < 0 || r >= g.h) ? g.n_slots : slot;   // rows outside the image: the zero slot
          a_desc[ky] = a_desc0 + static_cast<uint64_t>(static_cast<uint32_t>(use) * slot_units);
          ++r;
          if (++slot == g.n_slots) slot = 0;
        }
      }
#pragma unroll
      for (int ky = 0; ky < KH; ++ky) {
        const uint64_t b_desc = b_desc0 + static_cast<uint64_t>(static_cast<uint32_t>(ky) * wrow_units);
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
          mma_tf32_elect(d_tmem, a_desc[ky] + static_cast<uint64_t>(ks * 64), b_desc + static_cast<uint64_t>(ks * 2), idesc,
                         (ky > 0 || ks > 0) ? 1u : 0u);
        }
      }
      mma_commit_elect(tmem_full(acc));
      mma_commit_elect(freed_bar(acc));
      if (++oy == g.oh) {
        oy = 0;
        slot_lo = 0;
      } else {
        slot_lo += 2;
        if (slot_lo >= g.n_slots) slot_lo -= g.n_slots;
      }
    }
  } else {
    // ---- epilogue: group (warp - 5) / 8 drains accumulator `group`, i.e. every second output row.
    // TMEM lane = pixel of the row; a warp may only touch lanes 32 * (warp % 4) .. + 31, and the two
    // warps of a lane quarter split the 32-channel chunks. --------------------------------------------
    const int ew = warp - kRowsFirstEpiWarp;
    const int group = ew >> 3;
    const int half = (ew >> 2) & 1;
    const int quarter = warp & 3;
    const int chunks = g.npad / 32;
    const int c_begin = half * ((chunks + 1) / 2) * 32;
    const int c_end = half == 0 ? ((chunks + 1) / 2) * 32 : g.npad;
    const int px = quarter * 32 + lane;
    const bool valid = px < g.ow;
    const int64_t ohow = static_cast<int64_t>(g.oh) * g.ow;
    bool ok = true;
    int img = img0, oy = oy0 + group;
    if (oy >= g.oh) { oy -= g.oh; ++img; }
    if constexpr (POOL) {
      // ---- pooling epilogue ------------------------------------------------------------------------
      // This group's rows all have the parity of its first row (OH is even, so the alternation carries
      // over from the last row of an image to the first row of the next).  A warp works on its 32
      // channels in two passes of 16, to keep the previous odd row's column maxima (32 values per
      // thread) in registers beside the pass's own values.
      float prev_odd[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) prev_odd[j] = -INFINITY;
      int even_rows = 0;           // even group: rows published; odd group: rows consumed
      // edges: [pass][group, half, quarter][16]; even rows: two buffers, so that the even group can
      // publish its next row while the odd group still reads the one before
      float* edge_base = reinterpret_cast<float*>(base_ptr + edge_off) + ((group * 2 + half) * 4 + quarter) * 16;
      float* even_base = reinterpret_cast<float*>(base_ptr + even_off);
      const int even_buf_elems = g.npad * g.pow;
      const int c0 = c_begin;      // one 32-channel chunk per warp (npad == 64)
      const bool out_px = (px & 1) == 0 && (px >> 1) < g.pow;
      const int q = px >> 1;
      const int bar_id = 2 + group * 2 + half;   // the four warps (lane quarters) of this group and half
      for (int i = group; i < n_items && ok; i += 2) {
        const int acc = group;
        if (!mbar_wait(tmem_full(acc), static_cast<uint32_t>(i >> 1) & 1u, status, kFaultRowsEpilogue)) { ok = false; break; }
        tcgen05_fence_after_sync();
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * g.npad + c0);
        const bool even_row = (oy & 1) == 0;
        const bool emits = !even_row && i != 0;   // a run's leading odd row only feeds the next pooled row
        if (!even_row && oy == 1) {
#pragma unroll
          for (int j = 0; j < 32; ++j) prev_odd[j] = -INFINITY;   // row -1 of an image is padding
        }
        // the k-th even row of the run goes through buffer k & 1; its barriers complete once per use
        const int eb = even_rows & 1;
        if (even_row && even_rows >= 2) {
          ok = mbar_wait_warp(even_free(eb), static_cast<uint32_t>((even_rows >> 1) - 1) & 1u, status, kFaultRowsPoolRow);
        } else if (emits) {
          ok = mbar_wait_warp(even_ready(eb), static_cast<uint32_t>(even_rows >> 1) & 1u, status, kFaultRowsPoolRow);
        }
        if (!ok) break;
        float* even_s = even_base + eb * even_buf_elems;
        const int p = oy >> 1;   // pooled row completed by an odd row
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          uint32_t r[16];
          tmem_ld_32x32b_x16(t_row + static_cast<uint32_t>(hh * 16), r);
          tmem_ld_wait();
          if (hh == 1) {
            // the accumulator is in registers: the MMAs of the row after next may have it
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(tmem_empty(acc));
          }
          float v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]) + bias_s[c0 + hh * 16 + j];
#pragma unroll 1
          for (int s = 0; s < epi.n_ops; ++s) ew_unary_vec<float, 16>(epi.ops[s], v);   // unary steps only
          // Column maxima over px - 1, px, px + 1 (needed at even px).  Neighbours are the lanes next
          // door; lane 0 takes its left neighbour from the warp of the quarter before.
          if (!valid) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = -INFINITY;
          }
          // (one edge buffer per pass: when a pass's buffer is rewritten for the next row, the other
          // pass's barrier lies in between, so one barrier per pass is enough)
          float* edge_s = edge_base + hh * (16 * 16);
          if (lane == 31) {
#pragma unroll
            for (int j = 0; j < 16; ++j) edge_s[j] = v[j];
          }
          asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float l = __shfl_up_sync(0xffffffffu, v[j], 1);
            const float r1 = __shfl_down_sync(0xffffffffu, v[j], 1);
            if (lane == 0) l = quarter == 0 ? -INFINITY : (edge_s - 16)[j];   // pixel -1 is padding
            v[j] = fmaxf(fmaxf(l, v[j]), r1);
          }
          if (even_row) {
            if (out_px) {
#pragma unroll
              for (int j = 0; j < 16; ++j) even_s[(c0 + hh * 16 + j) * g.pow + q] = v[j];
            }
          } else {
            if (emits && out_px) {
              // the pooled value replaces the even row's entry (this thread is its only reader)
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                float* e = even_s + (c0 + hh * 16 + j) * g.pow + q;
                *e = fmaxf(fmaxf(prev_odd[hh * 16 + j], *e), v[j]);
              }
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) prev_odd[hh * 16 + j] = v[j];
          }
        }
        __syncwarp();
        if (emits) {
          // The pooled row [Cout][POW] is complete in the buffer once the group's eight warps are
          // here: it leaves with 16-byte stores, consecutive threads along a channel's row (32
          // four-byte stores per thread from the lane = pixel layout took 7 K cycles per row).
          asm volatile("bar.sync %0, 256;" ::"r"(6 + group) : "memory");
          const int row_f4 = g.pow / 4;
          const int total_f4 = g.cout * row_f4;
          float* orow = out + (static_cast<int64_t>(img) * g.cout * g.poh + p) * g.pow;   // + ch * poh * pow
          for (int idx = (ew & 7) * 32 + lane; idx < total_f4; idx += 256) {
            const int ch = idx / row_f4, qq = idx - ch * row_f4;
            const float4 v4 = *reinterpret_cast<const float4*>(even_s + ch * g.pow + qq * 4);
            *reinterpret_cast<float4*>(orow + static_cast<int64_t>(ch) * g.poh * g.pow + qq * 4) = v4;
          }
          __syncwarp();
        }
        if (lane == 0) {
          if (even_row) mbar_arrive(even_ready(eb));
          else if (emits) mbar_arrive(even_free(eb));
        }
        if (even_row || emits) ++even_rows;
        oy += 2;
        while (oy >= g.oh) { oy -= g.oh; ++img; }
      }
    } else
    for (int i = group; i < n_items && ok; i += 2) {
      const int acc = group;
      if (!mbar_wait(tmem_full(acc), static_cast<uint32_t>(i >> 1) & 1u, status, kFaultRowsEpilogue)) { ok = false; break; }
      tcgen05_fence_after_sync();
      const int64_t pix = static_cast<int64_t>(oy) * g.ow + px;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * g.npad);
#pragma unroll 1
      for (int c0 = c_begin; c0 < c_end; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + static_cast<uint32_t>(c0), r);
        tmem_ld_wait();
        if (c0 + 32 >= c_end) {
          // the warp's share of the accumulator is in registers: the MMAs of the row after next may
          // have it while the arithmetic and the stores run
          tcgen05_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(tmem_empty(acc));
        }
        if (valid) {
          float v[32];
          const int64_t obase = (static_cast<int64_t>(img) * g.cout + c0) * ohow + pix;   // + j * ohow per channel
          const int nch = g.cout - c0 < 32 ? g.cout - c0 : 32;
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) + bias_s[c0 + j];
#pragma unroll 1
          for (int s = 0; s < epi.n_ops; ++s) {
            const int op = epi.ops[s];
            const float* opnd = static_cast<const float*>(epi.operands[s]);
            if (opnd != nullptr) {
              const int mode = epi.modes[s];
              float rhs[32];
              if (mode == FB200_OPERAND_FULL) {
                const float* src = opnd + obase;
#pragma unroll
                for (int j = 0; j < 32; ++j) rhs[j] = j < nch ? __ldg(src + j * ohow) : 0.0f;
              } else if (mode == FB200_OPERAND_ROW) {
#pragma unroll
                for (int j = 0; j < 32; ++j) rhs[j] = j < nch ? __ldg(opnd + c0 + j) : 0.0f;
              } else {
                const float colv = __ldg(opnd + px);
#pragma unroll
                for (int j = 0; j < 32; ++j) rhs[j] = colv;
              }
              if (op == FB200_EW_ADD) {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = v[j] + rhs[j];
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = v[j] * rhs[j];
              }
            } else {
              ew_unary_vec<float, 32>(op, v);
            }
          }
          float* dst = out + obase;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (j < nch) dst[j * ohow] = v[j];
          }
        }
      }
      if (c_begin >= c_end) {   // a warp without a chunk (Cout <= 32) still owes its arrival
        __syncwarp();
        if (lane == 0) mbar_arrive(tmem_empty(acc));
      }
      oy += 2;
      while (oy >= g.oh) { oy -= g.oh; ++img; }
    }
  }

  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == kRowsMmaWarp) {
    __syncwarp();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(g.tmem_cols));
  }
}

}  // namespace fb200

using namespace fb200;

// Launches the row-matrix kernel, or returns FB200_UNIMPLEMENTED for shapes outside its reach.
// pooled != nullptr: the 3 x 3 / stride 2 / pad 1 max-pool of the result is stored there instead
// of the result itself ([n, cout, poh, pow]).
static int rows_launch(const void* x, const void* w, const void* bias, void* out, void* pooled,
                       const fb200_conv2d_params* p, int dtype, const fb200_epilogue* epilogue,
                       fb200_stream stream) {
  if (dtype != FB200_F32 || p->groups != 1 || p->cout > 256 || p->cout < 1) return FB200_UNIMPLEMENTED;
  if (p->stride_h != 2 || p->stride_w != 2) return FB200_UNIMPLEMENTED;
  if (p->kh < 1 || p->kh > kRowsMaxKh || p->kw < 1 || p->kw > kRowsMaxKw || p->kw * p->cin > 32) return FB200_UNIMPLEMENTED;
  if (p->pad_h < 0 || p->pad_w < 0 || p->pad_h >= p->kh || p->pad_w >= p->kw) return FB200_UNIMPLEMENTED;
  if (p->n * p->cin * p->h * p->w >= (int64_t(1) << 31)) return FB200_UNIMPLEMENTED;
  RowsGeom g{};
  g.n = static_cast<int>(p->n); g.cin = static_cast<int>(p->cin); g.h = static_cast<int>(p->h);
  g.w = static_cast<int>(p->w); g.cout = static_cast<int>(p->cout); g.kh = static_cast<int>(p->kh);
  g.kw = static_cast<int>(p->kw); g.ph = static_cast<int>(p->pad_h); g.pw = static_cast<int>(p->pad_w);
  g.oh = (g.h + 2 * g.ph - g.kh) / 2 + 1;
  g.ow = (g.w + 2 * g.pw - g.kw) / 2 + 1;
  // 8-byte loads of element pairs; one output row of at most 128 pixels per tile
  if (g.oh < 1 || g.ow < 1 || g.ow > 128 || g.w % 2 != 0) return FB200_UNIMPLEMENTED;
  if ((reinterpret_cast<uintptr_t>(x) & 7u) != 0) return FB200_UNIMPLEMENTED;
  if (g.cin * (g.w / 2) > kRowsTasks * kRowsBuilders) return FB200_UNIMPLEMENTED;
  g.kp = (g.kw * g.cin + 7) / 8 * 8;
  g.npad = (g.cout + 31) / 32 * 32;
  if (2 * g.npad > 512) return FB200_UNIMPLEMENTED;
  if (pooled != nullptr) {
    // both halves of an epilogue group must have a chunk, rows must alternate in parity across images
    if (g.npad != 64 || g.oh % 2 != 0 || g.oh < 2 || g.ow < 2) return FB200_UNIMPLEMENTED;
    if ((((g.ow + 2 - 3) / 2 + 1) % 4) != 0 || !aligned16(pooled)) return FB200_UNIMPLEMENTED;   // 16-byte stores of pooled rows
    g.poh = (g.oh + 2 - 3) / 2 + 1;
    g.pow = (g.ow + 2 - 3) / 2 + 1;
  }
  g.tmem_cols = 32;
  while (g.tmem_cols < 2 * g.npad) g.tmem_cols *= 2;
  g.n_slots = g.kh + 2;
  g.slot_bytes = 4 * g.kp * 128;
  g.w_bytes = g.kh * g.npad * 128;
  g.total_rows = static_cast<int64_t>(g.n) * g.oh;
  const size_t smem = 1024 /*align*/ + static_cast<size_t>(g.n_slots + 1) * g.slot_bytes + g.w_bytes + 128 /*barriers*/ +
                      1024 /*bias*/ + kRowsPfStages * 2 * kRowsTasks * kRowsBuilders * 8 /*prefetch*/ +
                      (pooled != nullptr ? 16 * 32 * 4 + 2 * g.npad * g.pow * 4 : 0) + 128;
  if (smem > 227 * 1024) return FB200_UNIMPLEMENTED;
  EpilogueDev epi{};
  if (int rc = make_epilogue(epilogue, &epi, "conv2d")) return rc;
  if (pooled != nullptr) {
    // chain operands are indexed in the conv result's shape, which is never materialised here:
    // unary steps only
    for (int i = 0; i < epi.n_ops; ++i) if (epi.operands[i] != nullptr) return FB200_UNIMPLEMENTED;
  }
  int* status = nullptr;
  if (int rc = device_status_word(&status)) return rc;
  const uint32_t idesc = make_instr_desc(kFmtTF32, /*a MN-major*/ 1, /*b MN-major*/ 0, 128, static_cast<uint32_t>(g.npad));
  const int64_t units = pooled != nullptr ? static_cast<int64_t>(g.n) * g.poh : g.total_rows;
  const int grid = static_cast<int>(units < kNumSMs ? units : kNumSMs);
  auto launch = [&](auto kernel) -> int {
    FB200_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    kernel<<<grid, kRowsThreads, smem, as_stream(stream)>>>(
        static_cast<const float*>(x), static_cast<const float*>(w), static_cast<const float*>(bias),
        static_cast<float*>(pooled != nullptr ? pooled : out), g, idesc, epi, status);
    return FB200_OK;
  };
  int rc = FB200_UNIMPLEMENTED;
  const int ksteps = g.kp / 8;
  if (pooled != nullptr) {
    if (g.kh == 7 && ksteps == 3) rc = launch(conv2d_rows_tcgen05_kernel<7, 3, true>);
    if (g.kh == 3 && ksteps == 2) rc = launch(conv2d_rows_tcgen05_kernel<3, 2, true>);
  } else {
#define FB200_ROWS_CASE(kh_, ks_) if (g.kh == kh_ && ksteps == ks_) rc = launch(conv2d_rows_tcgen05_kernel<kh_, ks_, false>);
    FB200_ROWS_CASE(7, 3)   // 7 x 7 over 3 channels (21 -> 24)
    FB200_ROWS_CASE(7, 1)   // 7 x 7 over 1 channel
    FB200_ROWS_CASE(5, 2)   // 5 x 5 over 3 channels (15 -> 16)
    FB200_ROWS_CASE(5, 1)   // 5 x 5 over 1 channel
    FB200_ROWS_CASE(3, 2)   // 3 x 3 over 3-5 channels
    FB200_ROWS_CASE(3, 1)   // 3 x 3 over 1-2 channels
    FB200_ROWS_CASE(3, 3)   // 3 x 3 over 6-8 channels
    FB200_ROWS_CASE(3, 4)   // 3 x 3 over 9-10 channels
    FB200_ROWS_CASE(4, 2)   // 4 x 4 over 3-4 channels
#undef FB200_ROWS_CASE
  }
  if (rc != FB200_OK) return rc;
  return after_launch("conv2d_rows_tcgen05_kernel");
}

// Returns FB200_UNIMPLEMENTED for shapes outside this kernel's reach (the caller then tries the halo
// kernel, the gather kernel and the direct kernel).
extern "C" int fb200_conv2d_rows_tcgen05(const void* x, const void* w, const void* bias, void* out,
                                         const fb200_conv2d_params* p, int dtype,
                                         const fb200_epilogue* epilogue, fb200_stream stream) {
  return rows_launch(x, w, bias, out, nullptr, p, dtype, epilogue, stream);
}

// conv2d -> [unary chain] -> max_pool2d(3 x 3, stride 2, padding 1) in one launch when the shape
// allows (FB200_UNIMPLEMENTED otherwise; fb200_conv2d_max_pool then runs the two kernels).
extern "C" int fb200_conv2d_rows_pooled_tcgen05(const void* x, const void* w, const void* bias, void* pooled,
                                                const fb200_conv2d_params* p, int dtype,
                                                const fb200_epilogue* epilogue, fb200_stream stream) {
  if (pooled == nullptr) return FB200_UNIMPLEMENTED;
  return rows_launch(x, w, bias, nullptr, pooled, p, dtype, epilogue, stream);
}
