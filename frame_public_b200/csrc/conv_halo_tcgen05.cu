// conv2d as an implicit GEMM on the tensor cores, with the input staged as halo tiles in shared
// memory (fp32 tensors, TF32 math, fp32 accumulation).
//
// Semantics: src/backends/cpu/kernels/conv.cpp:225-257 (NCHW cross-correlation, zero padding, bias
// per output channel added last); used when CompileOptions::allow_tf32 permits reduced precision
// (include/frame/hal/backend.h:51-63).  Replaces cudnnConvolutionForward + cudnnAddTensor of
// src/backends/cuda/kernels/conv.cpp:385-520 and the activation / residual launches after it.
//
// GEMM view: D[pixel, co] = sum_k A[pixel, k] * W[co, k].  A tile is 128 pixels = whole output rows
// of one image (rows = 128 / OW of them), so everything it reads from one input channel is a
// rectangle: ((rows-1)*stride + KH) x ((OW-1)*stride + KW) elements.  Where the first
// tensor-core convolution here gathered every im2col element from global memory (one L2 round trip
// per k-block, 9x re-reads for a 3x3 window: 40-48 TFLOP/s), this kernel
//   * fetches that rectangle for a block of channels with ONE 4-D TMA copy (zero fill outside the
//     image does the padding; the copy starts at a column that is a multiple of 4 so that its
//     address is 16-byte aligned, the few extra columns are skipped by the gather), double
//     buffered across tiles;
//   * builds the 128 x 32 A operand of each k-block from shared memory (256 producer threads, one
//     LDS + one STS per element) in the 128-byte swizzle with 32-byte units that tcgen05 needs for
//     MN-major 32-bit operands;
//   * keeps the weights of the current channel block resident in shared memory (K-major,
//     128-byte swizzle), written once per pass instead of once per tile and k-block;
//   * orders k as (tap, channel) inside a channel block, so a pass over one channel block touches
//     one halo tile and one weight block; with several channel blocks the CTA sweeps all its tiles
//     (up to 512/N accumulators live in TMEM at once) per block before moving to the next.
// warp 8 issues tcgen05.mma kind::tf32 (M = 128, N = Cout padded to 32, K = 8 per instruction);
// warps 9-12 run the epilogue (bias, chain, coalesced NCHW stores) of finished tiles.
// Every wait is bounded; a wait that gives up records a status code and the CTA exits cleanly.
// Measured with per-role cycle counters (Cout = 64): the single issuing thread spends about 130
// cycles per tcgen05.mma although an M128 x N64 x K8 TF32 instruction is 32 cycles of tensor work,
// i.e. with N = 64 the instruction rate, not the FLOP rate, bounds the mainloop, and TMEM reads of
// the epilogue queue behind the MMAs.  (A transposed formulation, M = Cout, N = 256 pixels, would
// halve the instruction count; not built.)
// Bound: tensor pipe / shared-memory gather.  FLOPs per launch = 2 * N*OH*OW * Cout * Cin*KH*KW.
#include <cuda.h>

#include "common.cuh"
#include "epilogue.cuh"
#include "sm100_ptx.cuh"

namespace fb200 {

int device_status_word(int** dev_ptr);  // gemm_tcgen05.cu
int make_tmap_nchw_f32(CUtensorMap* map, const void* ptr, int64_t n, int64_t c, int64_t h, int64_t w,
                       int box_c, int box_h, int box_w);

using namespace sm100;

constexpr int kHaloTileM = 128;
constexpr int kHaloBlockK = 32;
constexpr int kHaloProducers = 256;
constexpr int kHaloThreads = 416;   // 8 producer warps, 1 MMA warp, 4 epilogue warps
constexpr int kHaloMmaWarp = 8;
constexpr int kHaloAStage = kHaloTileM * 128;   // 16 KiB: 128 pixels x one 32-wide k-block
constexpr int kHaloSub = 2;                     // k-blocks per ring stage: one handshake per 64 k
constexpr int kHaloStageBytes = kHaloSub * kHaloAStage;
constexpr int kHaloMaxAcc = 8;
constexpr int kHaloMaxBufs = 4;                 // halo tiles in flight

enum HaloFault : int {
  kFaultHaloEmpty = 211,      // producers: A stage never freed
  kFaultHaloLoad = 212,       // producers: halo tile never arrived
  kFaultHaloReuse = 213,      // loader: halo buffer never released
  kFaultHaloWeights = 214,    // producers: weight block still in use
  kFaultHaloMmaFull = 215,    // MMA: A stage never filled
  kFaultHaloMmaTmem = 216,    // MMA: accumulator never drained
  kFaultHaloEpilogue = 217,   // epilogue: accumulator never completed
};

struct HaloGeom {
  int n, cin, h, w, cout, kh, kw, sh, sw, ph, pw, oh, ow;
  int rows, tiles_per_img;
  int64_t n_tiles;
  int cb, n_cb;          // channels per block, blocks
  int ih_t, iwp;         // halo tile: rows, padded width (elements)
  int x0a, xoff;         // first column fetched (multiple of 4, <= -pw); -pw - x0a
  int kcb, kblocks;      // k extent of one channel block, its 32-wide blocks
  int npad, tmem_cols, acc_per_round, stages;
  int halo_bytes, w_bytes, n_halo;
  int out_stage_bytes;   // > 0: results leave through a shared-memory tile and a TMA store
};

// Flat walk over (round, channel block, tile) shared by all roles.
struct HaloItem {
  int round, cb, ti, acc;
  bool first_of_pass, last_of_pass;
};
__device__ __forceinline__ HaloItem halo_decode(int idx, int my_tiles, int apr, int n_cb) {
  HaloItem it;
  const int per_round = apr * n_cb;
  it.round = idx / per_round;
  const int rem = idx - it.round * per_round;
  const int left = my_tiles - it.round * apr;
  const int in_round = left < apr ? left : apr;
  it.cb = rem / in_round;
  it.acc = rem - it.cb * in_round;
  it.ti = it.round * apr + it.acc;
  it.first_of_pass = it.acc == 0;
  it.last_of_pass = it.acc == in_round - 1;
  return it;
}

__global__ void __launch_bounds__(kHaloThreads, 1)
conv2d_halo_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_x,
                           const __grid_constant__ CUtensorMap tmap_out, const float* __restrict__ w,
                           const float* __restrict__ bias, float* __restrict__ out, HaloGeom g,
                           uint32_t idesc, EpilogueDev epi, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw_addr);
  const uint32_t w_off = static_cast<uint32_t>(g.stages) * kHaloStageBytes;
  const uint32_t halo_off = w_off + static_cast<uint32_t>(g.w_bytes);
  const uint32_t bar_off = halo_off + static_cast<uint32_t>(g.n_halo) * static_cast<uint32_t>(g.halo_bytes);
  const uint32_t bars = base + bar_off;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (g.stages + s); };
  const uint32_t misc = bars + 8u * (2 * g.stages);
  auto halo_full = [&](int b) { return misc + 8u * b; };
  auto halo_empty = [&](int b) { return misc + 8u * (kHaloMaxBufs + b); };
  const uint32_t w_free = misc + 8u * (2 * kHaloMaxBufs);
  auto tmem_full = [&](int a) { return misc + 8u * (2 * kHaloMaxBufs + 1 + a); };
  auto tmem_empty = [&](int a) { return misc + 8u * (2 * kHaloMaxBufs + 1 + kHaloMaxAcc + a); };
  const uint32_t slot_off = bar_off + 8u * (2 * g.stages + 2 * kHaloMaxBufs + 1 + 2 * kHaloMaxAcc);
  const uint32_t tmem_slot = base + slot_off;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(base_ptr + slot_off);
  float* bias_s = reinterpret_cast<float*>(base_ptr + slot_off + 16);          // [256]
  int* ktab = reinterpret_cast<int*>(base_ptr + slot_off + 16 + 1024);
  // staging tile of the TMA store: [cout][rows][ow] floats, 128-byte aligned, after the k-table
  const uint32_t ostage_off = (slot_off + 16 + 1024 + static_cast<uint32_t>(g.kblocks) * kHaloBlockK * 4 + 127u) & ~127u;
  float* ostage = reinterpret_cast<float*>(base_ptr + ostage_off);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int my_tiles = blockIdx.x < g.n_tiles
                           ? static_cast<int>((g.n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0;
  const int total_items = my_tiles * g.n_cb;
  const int apr = g.acc_per_round;
  const int n_stage_blocks = (g.kblocks + kHaloSub - 1) / kHaloSub;   // handshakes per (tile, block)

  if (threadIdx.x == 0) {
    for (int s = 0; s < g.stages; ++s) {
      mbar_init(full_bar(s), kHaloProducers / 32);   // one arrival per producer warp
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < kHaloMaxBufs; ++b) {
      mbar_init(halo_full(b), 1);
      mbar_init(halo_empty(b), kHaloProducers / 32);
    }
    mbar_init(w_free, 1);
    for (int a = 0; a < kHaloMaxAcc; ++a) {
      mbar_init(tmem_full(a), 1);
      mbar_init(tmem_empty(a), 4);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmap_x);
  }
  // k -> offset of (channel in block, ky, kx) inside the halo tile; -1 for the padding rows of the
  // last k-block.  k = tap * cb + channel.
  for (int k = threadIdx.x; k < g.kblocks * kHaloBlockK; k += kHaloThreads) {
    int e = -1;
    if (k < g.kcb) {
      const int tap = k / g.cb, cil = k - tap * g.cb;
      const int ky = tap / g.kw, kx = tap - ky * g.kw;
      e = (cil * g.ih_t + ky) * g.iwp + kx + g.xoff;
    }
    ktab[k] = e;
  }
  for (int c = threadIdx.x; c < 256; c += kHaloThreads) {
    bias_s[c] = (bias != nullptr && c < g.cout) ? __ldg(bias + c) : 0.0f;
  }
  if (warp == kHaloMmaWarp) {
    __syncwarp();
    tmem_alloc(tmem_slot, static_cast<uint32_t>(g.tmem_cols));
    tmem_relinquish();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;

  auto tile_of = [&](int ti, int* img, int* oy0) {
    const int64_t tile = blockIdx.x + static_cast<int64_t>(ti) * gridDim.x;
    *img = static_cast<int>(tile / g.tiles_per_img);
    *oy0 = static_cast<int>(tile - static_cast<int64_t>(*img) * g.tiles_per_img) * g.rows;
  };

  if (warp < kHaloMmaWarp) {
    // ---- producers: 256 threads = 128 pixels x 2 halves of the 32 k-rows of a sub-block -----------
    const int tid = threadIdx.x;
    const int ptid = tid & 127;
    const int khalf = tid >> 7;
    const uint32_t a_thread_off = static_cast<uint32_t>((ptid >> 5) * (kHaloBlockK * 128) + (ptid & 7) * 4);
    const uint32_t a_unit = static_cast<uint32_t>((ptid & 31) >> 3);
    const bool pix_ok = ptid < g.rows * g.ow;
    const int pr = pix_ok ? ptid / g.ow : 0;
    const int px = pix_ok ? ptid - pr * g.ow : 0;
    const int pbase = pr * g.sh * g.iwp + px * g.sw;
    const int64_t K = static_cast<int64_t>(g.cin) * g.kh * g.kw;
    const int khkw = g.kh * g.kw;
    auto issue_halo = [&](const HaloItem& it, int buf) {
      int img, oy0;
      tile_of(it.ti, &img, &oy0);
      mbar_arrive_expect_tx(halo_full(buf), static_cast<uint32_t>(g.cb * g.ih_t * g.iwp * 4));
      tma_load_4d(base + halo_off + static_cast<uint32_t>(buf * g.halo_bytes), &tmap_x, halo_full(buf),
                  g.x0a, oy0 * g.sh - g.ph, it.cb * g.cb, img);
    };
    int stage = 0;
    uint32_t phase = 0;
    int passes = 0;
    bool ok = true;
    // halo tiles are fetched n_halo - 1 items ahead of the one being gathered
    const int nb = g.n_halo;
    if (tid == 0) {
      for (int i = 0; i < nb - 1 && i < total_items; ++i) issue_halo(halo_decode(i, my_tiles, apr, g.n_cb), i);
    }
    for (int idx = 0; idx < total_items && ok; ++idx) {
      const HaloItem it = halo_decode(idx, my_tiles, apr, g.n_cb);
      const int buf = idx % nb;
      if (tid == 0 && idx + nb - 1 < total_items) {
        // the buffer of item idx + nb - 1 was last used by item idx - 1: every producer must have
        // left it
        const int nbuf = (idx + nb - 1) % nb;
        if (idx >= 1 && !mbar_wait(halo_empty(nbuf), ((idx - 1) / nb) & 1, status, kFaultHaloReuse)) {
          ok = false;
        } else {
          issue_halo(halo_decode(idx + nb - 1, my_tiles, apr, g.n_cb), nbuf);
        }
      }
      if (it.first_of_pass && (g.n_cb > 1 || idx == 0)) {
        // weight block of this channel block: [kblocks][npad rows x 32 k], K-major, 16-byte swizzle
        if (passes >= 1 && !mbar_wait(w_free, (passes - 1) & 1, status, kFaultHaloWeights)) ok = false;
        // A row of w restricted to this channel block is cb*KH*KW contiguous floats.  Each warp
        // takes every eighth row and reads them with coalesced loads, 32 in flight per lane (four
        // steps along the row for up to eight rows), then scatters them into the k-blocks.
        const int row_len = g.cb * khkw;
        const int wwarp = tid >> 5;
        if (ok && (g.kcb != g.kblocks * kHaloBlockK || g.cout != g.npad)) {
          // zeros for the padding only (rows past Cout, k past the block's extent): disjoint from
          // what the loads below write, so no barrier is needed between the two
          const int total_w = g.kblocks * kHaloBlockK * g.npad;
          for (int e = tid; e < total_w; e += kHaloProducers) {
            const int k = e / g.npad, co = e - k * g.npad;
            if (co >= g.cout || k >= g.kcb) {
              const uint32_t kk = static_cast<uint32_t>(k & 31);
              const uint32_t addr = base + w_off + static_cast<uint32_t>((k >> 5) * g.npad * 128) +
                                    static_cast<uint32_t>((co >> 3) * 1024 + (co & 7) * 128) +
                                    (((kk >> 2) ^ static_cast<uint32_t>(co & 7)) << 4) + (kk & 3u) * 4u;
              asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(0.0f) : "memory");
            }
          }
        }
        for (int co0 = wwarp; ok && co0 < g.cout; co0 += 8 * (kHaloProducers / 32)) {
          for (int j0 = lane; j0 < row_len; j0 += 4 * 32) {
            float wv[8][4];
#pragma unroll
            for (int r = 0; r < 8; ++r) {
              const int co = co0 + r * (kHaloProducers / 32);
              const float* wrow = w + co * K + static_cast<int64_t>(it.cb) * row_len;
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const int j = j0 + q * 32;
                wv[r][q] = (co < g.cout && j < row_len) ? __ldg(wrow + j) : 0.0f;
              }
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int j = j0 + q * 32;
              if (j < row_len) {
                const int cil = j / khkw, tap = j - cil * khkw;
                const int k = tap * g.cb + cil;
                const uint32_t kk = static_cast<uint32_t>(k & 31);
                const uint32_t kb_off = base + w_off + static_cast<uint32_t>((k >> 5) * g.npad * 128) + (kk & 3u) * 4u;
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                  const int co = co0 + r * (kHaloProducers / 32);
                  if (co < g.cout) {
                    const uint32_t addr = kb_off + static_cast<uint32_t>((co >> 3) * 1024 + (co & 7) * 128) +
                                          (((kk >> 2) ^ static_cast<uint32_t>(co & 7)) << 4);
                    asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(wv[r][q]) : "memory");
                  }
                }
              }
            }
          }
        }
        ++passes;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (!mbar_wait(halo_full(buf), (idx / nb) & 1, status, kFaultHaloLoad)) { ok = false; break; }
      const float* halo = reinterpret_cast<const float*>(base_ptr + halo_off + buf * g.halo_bytes) + pbase;
      for (int sb = 0; sb < n_stage_blocks; ++sb) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, status, kFaultHaloEmpty)) { ok = false; break; }
        const int nsub = g.kblocks - sb * kHaloSub < kHaloSub ? g.kblocks - sb * kHaloSub : kHaloSub;
        for (int sub = 0; sub < nsub; ++sub) {
          const uint32_t a_sub = base + static_cast<uint32_t>(stage) * kHaloStageBytes + sub * kHaloAStage;
          const int* tab = ktab + (sb * kHaloSub + sub) * kHaloBlockK + khalf * 16;
          float v[16];
#pragma unroll
          for (int u = 0; u < 16; ++u) {
            const int e = tab[u];
            v[u] = e >= 0 ? halo[e] : 0.0f;
          }
#pragma unroll
          for (int u = 0; u < 16; ++u) {
            const uint32_t kk = static_cast<uint32_t>(khalf * 16 + u);
            const uint32_t addr = a_sub + a_thread_off + kk * 128u + ((a_unit ^ (kk & 3u)) << 5);
            asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v[u]) : "memory");
          }
        }
        fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor-core (async) proxy
        __syncwarp();
        // one arrival per warp: 256 single-thread arrivals on one mbarrier serialise
        if (lane == 0) mbar_arrive(full_bar(stage));
        if (++stage == g.stages) { stage = 0; phase ^= 1u; }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(halo_empty(buf));
    }
  } else if (warp == kHaloMmaWarp) {
    // The whole warp runs this loop and one elected lane issues (warp-uniform code keeps the
    // descriptors in uniform registers: the single-lane branch this replaces fed the tensor pipe
    // about a third slower).
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    // A: MN-major, 32-pixel spans 4096 bytes apart (LBO), 4-row k groups 512 bytes apart (SBO);
    // one MMA (K = 8) covers two groups = 1024 bytes.  B: K-major, 8-row groups 1024 bytes apart;
    // a K step is 32 bytes inside the row.  The descriptors differ only in their address field
    // (bytes >> 4), so they are built once and advanced by additions.
    const uint64_t a_desc0 = make_smem_desc(base, kHaloBlockK * 128, 512, kLayoutSw128Base32);
    const uint64_t b_desc0 = make_smem_desc(base + w_off, 16, 1024, kLayoutSw128);
    for (int idx = 0; idx < total_items && ok; ++idx) {
      const HaloItem it = halo_decode(idx, my_tiles, apr, g.n_cb);
      if (it.cb == 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(tmem_empty(it.acc), (static_cast<uint32_t>(it.round) & 1u) ^ 1u, status, kFaultHaloMmaTmem));
        if (!ok) break;
        tcgen05_fence_after_sync();
      }
      const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(it.acc * g.npad);
      for (int sb = 0; sb < n_stage_blocks; ++sb) {
        ok = __all_sync(0xffffffffu, mbar_wait(full_bar(stage), phase, status, kFaultHaloMmaFull));
        if (!ok) break;
        tcgen05_fence_after_sync();
        const int nsub = g.kblocks - sb * kHaloSub < kHaloSub ? g.kblocks - sb * kHaloSub : kHaloSub;
        for (int sub = 0; sub < nsub; ++sub) {
          const int kb = sb * kHaloSub + sub;
          const uint64_t a_desc = a_desc0 + static_cast<uint64_t>((stage * kHaloStageBytes + sub * kHaloAStage) >> 4);
          const uint64_t b_desc = b_desc0 + static_cast<uint64_t>((kb * g.npad * 128) >> 4);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            mma_tf32_elect(d_tmem, a_desc + static_cast<uint64_t>(ks * 64), b_desc + static_cast<uint64_t>(ks * 2), idesc,
                           (it.cb > 0 || kb > 0 || ks > 0) ? 1u : 0u);
          }
        }
        mma_commit_elect(empty_bar(stage));
        if (++stage == g.stages) { stage = 0; phase ^= 1u; }
      }
      if (!ok) break;
      if (it.last_of_pass) mma_commit_elect(w_free);
      if (it.cb == g.n_cb - 1) mma_commit_elect(tmem_full(it.acc));
    }
  } else {
    // ---- epilogue warps 9..12: TMEM lane = pixel of the tile ------------------------------------
    // All tiles of a round finish during its last channel-block pass, so what this role costs per
    // tile is the tail of the kernel: operands are fetched with 32 independent loads before they are
    // used, the bias comes from shared memory, addresses advance by additions.
    const int quarter = warp & 3;
    const int m = quarter * 32 + lane;
    const bool pix_ok = m < g.rows * g.ow;
    const int pr = pix_ok ? m / g.ow : 0;
    const int px = pix_ok ? m - pr * g.ow : 0;
    const int64_t ohow = static_cast<int64_t>(g.oh) * g.ow;
    const bool use_tma_store = g.out_stage_bytes > 0;
    const int tile_px = g.rows * g.ow;
    bool ok = true;
    for (int ti = 0; ti < my_tiles && ok; ++ti) {
      const int acc = ti % apr, round = ti / apr;
      if (!mbar_wait(tmem_full(acc), static_cast<uint32_t>(round) & 1u, status, kFaultHaloEpilogue)) { ok = false; break; }
      tcgen05_fence_after_sync();
      int img, oy0;
      tile_of(ti, &img, &oy0);
      const int oy = oy0 + pr;
      const bool valid = pix_ok && oy < g.oh;
      const int64_t pix = static_cast<int64_t>(oy) * g.ow + px;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(acc * g.npad);
#pragma unroll 1
      for (int c0 = 0; c0 < g.npad; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + static_cast<uint32_t>(c0), r);
        tmem_ld_wait();
        if (valid) {
          float v[32];
          const int64_t obase = (static_cast<int64_t>(img) * g.cout + c0) * ohow + pix;   // + j*ohow per channel
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
          if (use_tma_store) {
            float* dst = ostage + static_cast<size_t>(c0) * tile_px + m;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (j < nch) dst[j * tile_px] = v[j];
            }
          } else {
            float* dst = out + obase;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (j < nch) dst[j * ohow] = v[j];
            }
          }
        }
      }
      tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty(acc));
      if (use_tma_store) {
        // the tile is complete in shared memory: one thread hands it to the TMA, which writes the
        // cout x rows runs of ow floats (rows past the image are clipped by the tensor map)
        fence_proxy_async_smem();
        asm volatile("bar.sync 2, 128;" ::: "memory");   // the four epilogue warps
        if (warp == kHaloMmaWarp + 1 && lane == 0) {
          tma_store_4d(&tmap_out, base + ostage_off, 0, oy0, 0, img);
          tma_store_commit();
          tma_store_wait_read<0>();   // the staging tile may be overwritten by the next tile
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
      }
    }
    if (use_tma_store && warp == kHaloMmaWarp + 1 && lane == 0) tma_store_wait_all();
  }

  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == kHaloMmaWarp) {
    __syncwarp();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(g.tmem_cols));
  }
}

}  // namespace fb200

using namespace fb200;

// Returns FB200_UNIMPLEMENTED for shapes outside the halo kernel's reach (the caller then tries
// the gather kernel and the direct kernel).
extern "C" int fb200_conv2d_halo_tcgen05(const void* x, const void* w, const void* bias, void* out,
                                         const fb200_conv2d_params* p, int dtype,
                                         const fb200_epilogue* epilogue, fb200_stream stream) {
  if (dtype != FB200_F32 || p->groups != 1 || p->cout > 256 || p->cout < 1) return FB200_UNIMPLEMENTED;
  HaloGeom g{};
  g.n = static_cast<int>(p->n); g.cin = static_cast<int>(p->cin); g.h = static_cast<int>(p->h);
  g.w = static_cast<int>(p->w); g.cout = static_cast<int>(p->cout); g.kh = static_cast<int>(p->kh);
  g.kw = static_cast<int>(p->kw); g.sh = static_cast<int>(p->stride_h); g.sw = static_cast<int>(p->stride_w);
  g.ph = static_cast<int>(p->pad_h); g.pw = static_cast<int>(p->pad_w);
  if (p->n * p->cin * p->h * p->w >= (int64_t(1) << 31) || p->n > 65535 * 64) return FB200_UNIMPLEMENTED;
  g.oh = (g.h + 2 * g.ph - g.kh) / g.sh + 1;
  g.ow = (g.w + 2 * g.pw - g.kw) / g.sw + 1;
  if (g.oh < 1 || g.ow < 1 || g.ow > kHaloTileM || g.w % 4 != 0 || !aligned16(x)) return FB200_UNIMPLEMENTED;
  g.rows = kHaloTileM / g.ow;
  if (g.rows > g.oh) g.rows = g.oh;
  g.tiles_per_img = (g.oh + g.rows - 1) / g.rows;
  g.n_tiles = static_cast<int64_t>(g.n) * g.tiles_per_img;
  if (g.n_tiles <= 0) return FB200_UNIMPLEMENTED;
  g.ih_t = (g.rows - 1) * g.sh + g.kh;
  g.x0a = -((g.pw + 3) / 4) * 4;
  g.xoff = -g.pw - g.x0a;
  g.iwp = ((g.ow - 1) * g.sw + g.kw + g.xoff + 3) / 4 * 4;
  if (g.iwp > 256 || g.ih_t > 256) return FB200_UNIMPLEMENTED;
  // channel block: 32 channels when that divides Cin, else all of Cin; the halo tile of a block
  // must fit twice next to the weights and the operand ring
  g.cb = (g.cin % 32 == 0) ? 32 : g.cin;
  if (g.cb > 256) return FB200_UNIMPLEMENTED;
  g.n_cb = g.cin / g.cb;
  g.kcb = g.cb * g.kh * g.kw;
  g.kblocks = (g.kcb + kHaloBlockK - 1) / kHaloBlockK;
  g.npad = (g.cout + 31) / 32 * 32;
  g.acc_per_round = 512 / g.npad < kHaloMaxAcc ? 512 / g.npad : kHaloMaxAcc;
  g.tmem_cols = 32;
  while (g.tmem_cols < g.acc_per_round * g.npad) g.tmem_cols *= 2;
  g.halo_bytes = (g.cb * g.ih_t * g.iwp * 4 + 1023) / 1024 * 1024;
  g.w_bytes = g.kblocks * g.npad * 128;
  // shared memory: weights, two ring stages (the ring is not latency-bound: each handshake costs
  // about as much as the MMAs it covers), and as many halo buffers as fit, up to four, because the
  // strided 4-D copy of a halo tile takes longer than gathering one
  const int64_t fixed = static_cast<int64_t>(g.w_bytes) + 1024 /*align*/ + 512 /*barriers*/ + 1024 /*bias*/ +
                        static_cast<int64_t>(g.kblocks) * kHaloBlockK * 4;
  g.stages = 2;
  const int64_t room = 227 * 1024 - fixed - static_cast<int64_t>(g.stages) * kHaloStageBytes;
  // results through a shared-memory tile and one TMA store per tile when there is room for the tile
  // next to two halo buffers (scattered per-channel warp stores were the longest part of the
  // epilogue); needs 16-byte aligned rows
  int64_t room_left = room;
  g.out_stage_bytes = 0;
  const int64_t stage_need = (static_cast<int64_t>(g.cout) * g.rows * g.ow * 4 + 127) / 128 * 128 + 128;
  if (g.ow % 4 == 0 && aligned16(out) && room - stage_need >= 2 * static_cast<int64_t>(g.halo_bytes)) {
    g.out_stage_bytes = static_cast<int>(stage_need);
    room_left = room - stage_need;
  }
  g.n_halo = static_cast<int>(room_left / g.halo_bytes);
  if (g.n_halo > kHaloMaxBufs) g.n_halo = kHaloMaxBufs;
  if (g.n_halo < 2) return FB200_UNIMPLEMENTED;
  EpilogueDev epi{};
  if (int rc = make_epilogue(epilogue, &epi, "conv2d")) return rc;
  CUtensorMap tx;
  if (int rc = make_tmap_nchw_f32(&tx, x, g.n, g.cin, g.h, g.w, g.cb, g.ih_t, g.iwp)) return rc;
  CUtensorMap tout = tx;   // placeholder when the direct-store epilogue is used
  if (g.out_stage_bytes > 0) {
    if (int rc = make_tmap_nchw_f32(&tout, out, g.n, g.cout, g.oh, g.ow, g.cout, g.rows, g.ow)) return rc;
  }
  int* status = nullptr;
  if (int rc = device_status_word(&status)) return rc;
  const size_t smem = static_cast<size_t>(g.stages) * kHaloStageBytes + static_cast<size_t>(fixed) +
                      static_cast<size_t>(g.n_halo) * g.halo_bytes + static_cast<size_t>(g.out_stage_bytes);
  FB200_CUDA_OK(cudaFuncSetAttribute(conv2d_halo_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(smem)));
  const uint32_t idesc = make_instr_desc(kFmtTF32, /*a MN-major*/ 1, /*b MN-major*/ 0, kHaloTileM,
                                         static_cast<uint32_t>(g.npad));
  const int grid = static_cast<int>(g.n_tiles < kNumSMs ? g.n_tiles : kNumSMs);
  conv2d_halo_tcgen05_kernel<<<grid, kHaloThreads, smem, as_stream(stream)>>>(
      tx, tout, static_cast<const float*>(w), static_cast<const float*>(bias), static_cast<float*>(out), g, idesc,
      epi, status);
  return after_launch("conv2d_halo_tcgen05_kernel");
}

