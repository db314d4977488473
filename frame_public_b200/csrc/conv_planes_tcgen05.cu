// conv2d (stride 1) as an implicit GEMM on the tensor cores whose A operand is never gathered per
// k-block: the tcgen05 descriptors point straight at column-shifted copies of the input rows.
//
// Semantics: src/backends/cpu/kernels/conv.cpp:225-257 (NCHW cross-correlation, zero padding, bias
// per output channel added last); fp32 tensors, TF32 math, fp32 accumulation, taken when
// CompileOptions::allow_tf32 permits reduced precision (include/frame/hal/backend.h:51-63).
// Replaces cudnnConvolutionForward + cudnnAddTensor of src/backends/cuda/kernels/conv.cpp:385-520
// and the activation / residual launches behind it.
//
// GEMM view: D[pixel, co] = sum over (tap, ci) of X_tap[pixel, ci] * W[co, ci, tap].  A tile is R
// output rows of one image, each padded to OWP = 32, 64 or 128 pixels (M = 128 = R * OWP).  For a
// block of CB input channels the producers write, once per tile, KW "planes": plane kx holds, for
// every channel and every input row the tile touches, the OW pixels x[ci, row, ow + kx - pad],
// laid out exactly as tcgen05 wants an MN-major TF32 operand (32-pixel spans of 128 bytes per
// channel, four channels per 512-byte group, 32-byte units XOR-swizzled by the channel; consecutive
// spans CB * 128 bytes apart).  A tap (ky, kx) of the filter is then nothing but plane kx read from
// `ky` rows further down: a descriptor whose start address is moved by ky * (OWP / 32) spans.  The
// im2col matrix of the halo kernel (KH * KW shifted copies, one shared-memory load and store per
// element and k-block, a ring handshake per 64 k) shrinks to KW copies made with 128-bit loads and
// stores, and one handshake per (tile, channel block).
//
// Roles (448 threads): warp 13 fetches halo tiles by 4-D TMA (zero fill = padding) and the packed
// weights of each channel block by one bulk copy (K-major, 128-byte swizzle); warps 0-7 build the planes;
// warp 8 issues tcgen05.mma kind::tf32 (M = 128, N = Cout padded to 32, K = 8 channels of one tap);
// warps 9-12 run the epilogue (bias, chain, results through a shared-memory tile and one 4-D TMA
// store per tile, or direct stores).  With several channel blocks the CTA sweeps all its tiles per
// block, up to 512 / N accumulators live in TMEM.  Every wait is bounded; a wait that gives up
// records a status code and the CTA exits cleanly.
// Bound: tensor pipe (at Cout = 64 its instruction rate: an M128 x N64 x K8 instruction takes about
// 92 cycles for 32 of tensor work).  FLOPs per launch = 2 * N*OH*OW * Cout * Cin*KH*KW.
#include <cuda.h>

#include "common.cuh"
#include "epilogue.cuh"
#include "sm100_ptx.cuh"

namespace fb200 {

int device_status_word(int** dev_ptr);  // gemm_tcgen05.cu
int make_tmap_nchw_f32(CUtensorMap* map, const void* ptr, int64_t n, int64_t c, int64_t h, int64_t w,
                       int box_c, int box_h, int box_w);

using namespace sm100;

constexpr int kPlTileM = 128;
constexpr int kPlProducers = 256;
constexpr int kPlThreads = 576;   // 8 producer warps, 1 MMA warp, 4 + 4 epilogue warps (9-12, 14-17), 1 loader warp
constexpr int kPlMmaWarp = 8;
constexpr int kPlLoaderWarp = 13;
constexpr int kPlMaxAcc = 8;
constexpr int kPlMaxBufs = 4;     // halo tiles in flight
constexpr int kPlSets = 2;        // plane sets: one being built while the other is multiplied (a third measured no faster)

enum PlanesFault : int {
  kFaultPlLoad = 221,       // producers: halo tile never arrived
  kFaultPlReuse = 222,      // loader: halo buffer never released
  kFaultPlWeights = 223,    // producers: weight block still in use
  kFaultPlSetBusy = 224,    // producers: plane set never released
  kFaultPlMmaSet = 225,     // MMA: plane set never filled
  kFaultPlMmaTmem = 226,    // MMA: accumulator never drained
  kFaultPlEpilogue = 227,   // epilogue: accumulator never completed
};

struct PlanesGeom {
  int n, cin, h, w, cout, kh, kw, ph, pw, oh, ow;
  int owp, rows, spr;      // padded row length (pixels), output rows per tile, 32-pixel spans per row
  int tiles_per_img;
  int64_t n_tiles;
  int cb, n_cb;            // channels per block, blocks
  int ih_t, iwp;           // halo tile: rows, padded width (elements)
  int x0a;                 // first column fetched (multiple of 4, <= -pw)
  int kcb, kblocks;        // k extent of one channel block (taps x cb), its 32-wide blocks
  int npad, tmem_cols, acc_per_round;
  int halo_bytes, w_bytes, n_halo;
  int lbo;                 // bytes between consecutive 32-pixel spans of a plane (cb * 128)
  int plane_bytes, set_bytes;
  int out_stage_bytes;     // > 0: results leave through a shared-memory tile and a TMA store
};

// The walk over (round, channel block, tile of the round) that all roles share, advanced by
// increments only: every role runs this bookkeeping in a single warp (or thread) between two
// handshakes, where a pair of integer divisions per item cost more than the MMAs of the item.
struct PlWalk {
  int my_tiles, apr, n_cb;
  int idx;        // items so far
  int round, cb, acc, in_round;
  __device__ __forceinline__ void start(int tiles, int acc_per_round, int blocks) {
    my_tiles = tiles; apr = acc_per_round; n_cb = blocks;
    idx = 0; round = 0; cb = 0; acc = 0;
    in_round = tiles < acc_per_round ? tiles : acc_per_round;
  }
  __device__ __forceinline__ bool done() const { return idx >= my_tiles * n_cb; }
  __device__ __forceinline__ int ti() const { return round * apr + acc; }
  __device__ __forceinline__ bool first_of_pass() const { return acc == 0; }
  __device__ __forceinline__ bool last_of_pass() const { return acc == in_round - 1; }
  __device__ __forceinline__ void next() {
    ++idx;
    if (++acc == in_round) {
      acc = 0;
      if (++cb == n_cb) {
        cb = 0;
        ++round;
        const int left = my_tiles - round * apr;
        in_round = left < apr ? left : apr;
      }
    }
  }
};

// 1-D bulk copy global -> shared memory, completion counted in bytes on an mbarrier.  Both addresses
// 16-byte aligned, the size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_load_1d(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               :
               : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(bar)
               : "memory");
}

// The filter, once per launch, in the exact image the main kernel keeps in shared memory for each
// channel block: [channel block][k-block of 32][npad rows x 32 k], K-major rows of 128 bytes whose
// 16-byte pieces are XOR-swizzled by the row, k = tap * cb + channel, zeros for the padding (rows
// past Cout, k past taps * cb).  A channel block then arrives by ONE bulk copy instead of being
// scattered element by element by the producer warps at every pass.
__global__ void __launch_bounds__(256)
conv_pack_weights_kernel(const float* __restrict__ w, float* __restrict__ packed, int cin, int cout, int khkw,
                         int cb, int n_cb, int kblocks, int npad) {
  const int per_block = kblocks * 32 * npad;
  const int total = n_cb * per_block;
  for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < total; e += gridDim.x * blockDim.x) {
    const int blk = e / per_block;
    const int r = e - blk * per_block;
    const int k = r / npad, co = r - k * npad;
    float v = 0.0f;
    if (co < cout && k < cb * khkw) {
      const int tap = k / cb, cil = k - tap * cb;
      v = w[(static_cast<int64_t>(co) * cin + blk * cb + cil) * khkw + tap];
    }
    const int kk = k & 31;
    const int dst = (k >> 5) * npad * 32 + (co >> 3) * 256 + (co & 7) * 32 + (((kk >> 2) ^ (co & 7)) << 2) + (kk & 3);
    packed[static_cast<int64_t>(blk) * per_block + dst] = v;
  }
}

// KW: filter width; XOFF: position of the window's first column inside the first 16-byte vector of a
// halo row (the halo copy starts at a column that is a multiple of 4 so that TMA may address it).
// KH: filter height; GROUPS: eight-channel groups per channel block (cb / 8).  With all four fixed the
// MMA warp's loop over the taps of an item unrolls into straight-line code with immediate offsets:
// a single warp issues it, one dependent instruction every few cycles, and anything recomputed per
// MMA shows up directly in the issue rate.
template <int KH, int KW, int XOFF, int GROUPS>
__global__ void __launch_bounds__(kPlThreads, 1)
conv2d_planes_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_x,
                             const __grid_constant__ CUtensorMap tmap_out, const float* __restrict__ w_packed,
                             const float* __restrict__ bias, float* __restrict__ out, PlanesGeom g,
                             uint32_t idesc, EpilogueDev epi, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw_addr);
  // layout: plane sets | weights | halo buffers | barriers, TMEM slot, bias | output staging tile
  const uint32_t w_off = static_cast<uint32_t>(kPlSets) * static_cast<uint32_t>(g.set_bytes);
  const uint32_t halo_off = w_off + static_cast<uint32_t>(g.w_bytes);
  const uint32_t bar_off = halo_off + static_cast<uint32_t>(g.n_halo) * static_cast<uint32_t>(g.halo_bytes);
  const uint32_t bars = base + bar_off;
  auto set_full = [&](int s) { return bars + 8u * s; };
  auto set_empty = [&](int s) { return bars + 8u * (kPlSets + s); };
  const uint32_t misc = bars + 8u * (2 * kPlSets);
  auto halo_full = [&](int b) { return misc + 8u * b; };
  auto halo_empty = [&](int b) { return misc + 8u * (kPlMaxBufs + b); };
  const uint32_t w_free = misc + 8u * (2 * kPlMaxBufs);
  const uint32_t w_full = misc + 8u * (2 * kPlMaxBufs + 1);
  auto tmem_full = [&](int a) { return misc + 8u * (2 * kPlMaxBufs + 2 + a); };
  auto tmem_empty = [&](int a) { return misc + 8u * (2 * kPlMaxBufs + 2 + kPlMaxAcc + a); };
  const uint32_t slot_off = bar_off + 8u * (2 * kPlSets + 2 * kPlMaxBufs + 2 + 2 * kPlMaxAcc);
  const uint32_t tmem_slot = base + slot_off;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(base_ptr + slot_off);
  float* bias_s = reinterpret_cast<float*>(base_ptr + slot_off + 16);          // [256]
  int2* pair_tab = reinterpret_cast<int2*>(base_ptr + slot_off + 16 + 1024);          // [ih_t * ow / 4]
  const uint32_t ostage_off = (slot_off + 16 + 1024 + static_cast<uint32_t>(g.ih_t * (g.ow / 4)) * 8u + 127u) & ~127u;
  float* ostage = reinterpret_cast<float*>(base_ptr + ostage_off);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int my_tiles = blockIdx.x < g.n_tiles
                           ? static_cast<int>((g.n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0;
  const int apr = g.acc_per_round;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPlSets; ++s) {
      mbar_init(set_full(s), kPlProducers / 32);   // one arrival per producer warp
      mbar_init(set_empty(s), 1);
    }
    for (int b = 0; b < kPlMaxBufs; ++b) {
      mbar_init(halo_full(b), 1);
      mbar_init(halo_empty(b), kPlProducers / 32);
    }
    mbar_init(w_free, 1);
    mbar_init(w_full, 1);
    for (int a = 0; a < kPlMaxAcc; ++a) {
      mbar_init(tmem_full(a), 1);
      mbar_init(tmem_empty(a), 8);   // two epilogue warps per TMEM lane quarter, each on half of the channels
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmap_x);
  }
  for (int c = threadIdx.x; c < 256; c += kPlThreads) {
    bias_s[c] = (bias != nullptr && c < g.cout) ? __ldg(bias + c) : 0.0f;
  }
  if (warp == kPlMmaWarp) {
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

  if (warp < kPlMmaWarp) {
    // ---- producers ---------------------------------------------------------------------------------
    const int tid = threadIdx.x;
    bool ok = true;
    const int nb = g.n_halo;
    const int G = g.ow / 4;                      // 4-pixel groups per row
    const int pairs = g.ih_t * G;                // (halo row, group) pairs of one channel
    const int units = g.cb * pairs;              // (channel, halo row, group) triples per item
    // per pair: where its 16 bytes come from inside a channel of the halo tile (float4 index) and
    // where they go inside a plane (byte offset of the span row + half of the 32-byte unit; the
    // unit's index before the channel's swizzle in the low bits)
    for (int pq = tid; pq < pairs; pq += kPlProducers) {
      const int i = pq / G, gq = pq - i * G;
      const int px = 4 * gq;
      pair_tab[pq] = make_int2(i * (g.iwp / 4) + gq,
                               (((i * g.spr + (px >> 5)) * g.lbo + (px & 7) * 4) << 2) | ((px & 31) >> 3));
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");   // the eight producer warps
    const int step_c = kPlProducers / pairs, step_p = kPlProducers - step_c * pairs;
    const int c_first = tid / pairs, p_first = tid - c_first * pairs;
    PlWalk it;
    it.start(my_tiles, apr, g.n_cb);
    int buf = 0, set = 0;
    uint32_t halo_phase = 0, set_phase = 0;   // parities of the current use of `buf` / `set`
    for (; !it.done() && ok; it.next()) {
      const int idx = it.idx;
      // the plane set of this item was last read by the MMAs of item idx - kPlSets
      if (idx >= kPlSets && !mbar_wait(set_empty(set), set_phase ^ 1u, status, kFaultPlSetBusy)) { ok = false; break; }
      if (!mbar_wait(halo_full(buf), halo_phase, status, kFaultPlLoad)) { ok = false; break; }
      // ---- planes: KW column-shifted copies of every (channel, halo row) of the tile -----------------
      const float4* halo4 = reinterpret_cast<const float4*>(base_ptr + halo_off + buf * g.halo_bytes);
      const uint32_t set_base = base + static_cast<uint32_t>(set * g.set_bytes);
      constexpr int NV = (XOFF + KW + 2) / 4 + 1;   // 16-byte vectors that cover the KW windows of 4 pixels
      const int iwp4 = g.iwp / 4;
      const int ch4 = g.ih_t * iwp4;   // float4 per channel of the halo tile
      // Two units per trip: the table entries and the halo vectors of both are in flight together
      // (two warps per scheduler cannot hide the shared-memory round trips of a single chain).
      int c = c_first, pq = p_first;
      auto advance = [&]() {
        c += step_c;
        pq += step_p;
        if (pq >= pairs) { pq -= pairs; ++c; }
      };
      auto store_unit = [&](int cc, const int2 e, const float (&f)[NV * 4]) {
        // the channel's row inside its 4-channel group, and the 32-byte unit swizzled by the channel
        const uint32_t dst = set_base + static_cast<uint32_t>(e.y >> 2) + static_cast<uint32_t>(cc * 128) +
                             (((static_cast<uint32_t>(e.y) & 3u) ^ static_cast<uint32_t>(cc & 3)) << 5);
#pragma unroll
        for (int kx = 0; kx < KW; ++kx) {
          asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst + static_cast<uint32_t>(kx * g.plane_bytes)),
                       "f"(f[XOFF + kx]), "f"(f[XOFF + kx + 1]), "f"(f[XOFF + kx + 2]), "f"(f[XOFF + kx + 3]) : "memory");
        }
      };
      int u = tid;
      for (; u + kPlProducers < units; u += 2 * kPlProducers) {
        const int c0 = c;
        const int2 e0 = pair_tab[pq];
        advance();
        const int c1 = c;
        const int2 e1 = pair_tab[pq];
        advance();
        const float4* s0 = halo4 + c0 * ch4 + e0.x;
        const float4* s1 = halo4 + c1 * ch4 + e1.x;
        float f0[NV * 4], f1[NV * 4];
#pragma unroll
        for (int v = 0; v < NV; ++v) {
          const float4 q0 = s0[v], q1 = s1[v];
          f0[4 * v] = q0.x; f0[4 * v + 1] = q0.y; f0[4 * v + 2] = q0.z; f0[4 * v + 3] = q0.w;
          f1[4 * v] = q1.x; f1[4 * v + 1] = q1.y; f1[4 * v + 2] = q1.z; f1[4 * v + 3] = q1.w;
        }
        store_unit(c0, e0, f0);
        store_unit(c1, e1, f1);
      }
      if (u < units) {
        const int2 e = pair_tab[pq];
        const float4* src = halo4 + c * ch4 + e.x;
        float f[NV * 4];
#pragma unroll
        for (int v = 0; v < NV; ++v) {
          const float4 q = src[v];
          f[4 * v] = q.x; f[4 * v + 1] = q.y; f[4 * v + 2] = q.z; f[4 * v + 3] = q.w;
        }
        store_unit(c, e, f);
      }
      fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor-core (async) proxy
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(set_full(set));
        mbar_arrive(halo_empty(buf));
      }
      if (++buf == nb) { buf = 0; halo_phase ^= 1u; }
      if (++set == kPlSets) { set = 0; set_phase ^= 1u; }
    }
  } else if (warp == kPlLoaderWarp) {
    // ---- loader: lane 0 keeps the halo buffers full, lane 1 brings each pass's weight block -----------
    // Both run ahead of the producers by themselves: the 4-D copy of a halo tile and the wait for a
    // free buffer used to sit in the producers' path between two handshakes.
    if (lane == 0) {
      PlWalk a;
      a.start(my_tiles, apr, g.n_cb);
      const int nb = g.n_halo;
      int buf = 0;
      uint32_t phase = 0;
      for (; !a.done(); a.next()) {
        // the n-th use of a buffer waits for its use n - 1 to be released by every producer warp
        if (a.idx >= nb && !mbar_wait(halo_empty(buf), phase ^ 1u, status, kFaultPlReuse)) break;
        int img, oy0;
        tile_of(a.ti(), &img, &oy0);
        mbar_arrive_expect_tx(halo_full(buf), static_cast<uint32_t>(g.cb * g.ih_t * g.iwp * 4));
        tma_load_4d(base + halo_off + static_cast<uint32_t>(buf * g.halo_bytes), &tmap_x, halo_full(buf),
                    g.x0a, oy0 - g.ph, a.cb * g.cb, img);
        if (++buf == nb) { buf = 0; phase ^= 1u; }
      }
    } else if (lane == 1) {
      PlWalk b;
      b.start(my_tiles, apr, g.n_cb);
      int passes = 0;
      for (; !b.done(); b.next()) {
        if (!(b.first_of_pass() && (g.n_cb > 1 || b.idx == 0))) continue;
        // one bulk copy of the block's packed image, as soon as the MMAs of the previous pass have
        // finished reading the block it replaces
        if (passes >= 1 && !mbar_wait(w_free, static_cast<uint32_t>(passes - 1) & 1u, status, kFaultPlWeights)) break;
        mbar_arrive_expect_tx(w_full, static_cast<uint32_t>(g.w_bytes));
        bulk_load_1d(base + w_off, w_packed + static_cast<size_t>(b.cb) * (g.w_bytes / 4), static_cast<uint32_t>(g.w_bytes), w_full);
        ++passes;
      }
    }
  } else if (warp == kPlMmaWarp) {
    // The whole warp runs this loop and one elected lane issues (warp-uniform code keeps the
    // descriptors in uniform registers).
    bool ok = true;
    // A: MN-major, 32-pixel spans `lbo` bytes apart, 4-channel groups 512 bytes apart; one MMA
    // (K = 8 channels) covers two groups = 1024 bytes.  B: K-major, 8-row groups 1024 bytes apart;
    // a K step of 8 is 32 bytes inside the swizzled row.
    const uint64_t a_desc0 = make_smem_desc(base, static_cast<uint32_t>(g.lbo), 512, kLayoutSw128Base32);
    const uint64_t b_desc0 = make_smem_desc(base + w_off, 16, 1024, kLayoutSw128);
    const uint64_t plane_units = static_cast<uint64_t>(static_cast<uint32_t>(g.plane_bytes) >> 4);
    const uint64_t row_units = static_cast<uint64_t>(static_cast<uint32_t>(g.spr * g.lbo) >> 4);
    const uint64_t b_block_units = static_cast<uint64_t>(static_cast<uint32_t>(g.npad * 128) >> 4);
    int w_passes = 0;
    PlWalk it;
    it.start(my_tiles, apr, g.n_cb);
    int set = 0;
    uint32_t set_phase = 0;
    for (; !it.done() && ok; it.next()) {
      const int idx = it.idx;
      if (it.cb == 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(tmem_empty(it.acc), (static_cast<uint32_t>(it.round) & 1u) ^ 1u, status, kFaultPlMmaTmem));
        if (!ok) break;
      }
      ok = __all_sync(0xffffffffu, mbar_wait(set_full(set), set_phase, status, kFaultPlMmaSet));
      if (!ok) break;
      tcgen05_fence_after_sync();
      if (it.first_of_pass() && (g.n_cb > 1 || idx == 0)) {
        ok = __all_sync(0xffffffffu, mbar_wait(w_full, static_cast<uint32_t>(w_passes) & 1u, status, kFaultPlWeights));
        if (!ok) break;
        ++w_passes;
      }
      const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(it.acc * g.npad);
      // k = tap * cb + 8 j runs through 0, 8, 16, ...: the B operand moves 32 bytes per step inside a
      // 32-wide k-block and jumps to the next block every fourth step; A moves one plane per kx, `spr`
      // spans per ky and 1024 bytes per eight channels.  Every offset below is a compile-time
      // multiple of three per-kernel constants.
      const uint64_t a_item = a_desc0 + static_cast<uint64_t>(static_cast<uint32_t>(set * g.set_bytes) >> 4);
#pragma unroll
      for (int ky = 0; ky < KH; ++ky) {
#pragma unroll
        for (int kx = 0; kx < KW; ++kx) {
#pragma unroll
          for (int j = 0; j < GROUPS; ++j) {
            const int step = (ky * KW + kx) * GROUPS + j;
            const uint64_t a_desc = a_item + static_cast<uint64_t>(ky) * row_units + static_cast<uint64_t>(kx) * plane_units +
                                    static_cast<uint64_t>(j * 64);
            const uint64_t b_desc = b_desc0 + static_cast<uint64_t>(step >> 2) * b_block_units + static_cast<uint64_t>((step & 3) * 2);
            mma_tf32_elect(d_tmem, a_desc, b_desc, idesc, (it.cb > 0 || step > 0) ? 1u : 0u);
          }
        }
      }
      mma_commit_elect(set_empty(set));
      if (it.last_of_pass()) mma_commit_elect(w_free);
      if (it.cb == g.n_cb - 1) mma_commit_elect(tmem_full(it.acc));
      if (++set == kPlSets) { set = 0; set_phase ^= 1u; }
    }
  } else {
    // ---- epilogue warps 9..12 and 14..17: TMEM lane = pixel slot of the tile (row = lane / OWP); the two
    // warps of a lane quarter split the 32-channel chunks -----------------------------------------------
    const int quarter = warp & 3;
    const int ehalf = warp > kPlLoaderWarp ? 1 : 0;   // warps 9-12: first half of the 32-channel chunks; 14-17: second
    const int m = quarter * 32 + lane;
    const int pr = m / g.owp;
    const int px = m - pr * g.owp;
    const bool pix_ok = px < g.ow && pr < g.rows;
    const int64_t ohow = static_cast<int64_t>(g.oh) * g.ow;
    const bool use_tma_store = g.out_stage_bytes > 0;
    const int tile_px = g.rows * g.ow;
    const int e_chunks = g.npad / 32;
    const int ec_begin = ehalf * ((e_chunks + 1) / 2) * 32;
    const int ec_end = ehalf == 0 ? ((e_chunks + 1) / 2) * 32 : g.npad;
    bool ok = true;
    for (int ti = 0; ti < my_tiles && ok; ++ti) {
      const int acc = ti % apr, round = ti / apr;
      if (!mbar_wait(tmem_full(acc), static_cast<uint32_t>(round) & 1u, status, kFaultPlEpilogue)) { ok = false; break; }
      tcgen05_fence_after_sync();
      int img, oy0;
      tile_of(ti, &img, &oy0);
      const int oy = oy0 + pr;
      const bool valid = pix_ok && oy < g.oh;
      const int64_t pix = static_cast<int64_t>(oy) * g.ow + px;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(acc * g.npad);
#pragma unroll 1
      for (int c0 = ec_begin; c0 < ec_end; c0 += 32) {
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
            float* dst = ostage + static_cast<size_t>(c0) * tile_px + pr * g.ow + px;
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
        asm volatile("bar.sync 2, 256;" ::: "memory");   // the eight epilogue warps
        if (warp == kPlMmaWarp + 1 && lane == 0) {
          tma_store_4d(&tmap_out, base + ostage_off, 0, oy0, 0, img);
          tma_store_commit();
          tma_store_wait_read<0>();   // the staging tile may be overwritten by the next tile
        }
        asm volatile("bar.sync 2, 256;" ::: "memory");
      }
    }
    if (use_tma_store && warp == kPlMmaWarp + 1 && lane == 0) tma_store_wait_all();
  }

  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == kPlMmaWarp) {
    __syncwarp();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(g.tmem_cols));
  }
}

template <int KH, int KW, int XOFF, int GROUPS>
static int launch_planes(const CUtensorMap& tx, const CUtensorMap& tout, const float* w, const float* bias,
                         float* out, const PlanesGeom& g, uint32_t idesc, const EpilogueDev& epi, int* status,
                         size_t smem, int grid, cudaStream_t s) {
  auto kernel = conv2d_planes_tcgen05_kernel<KH, KW, XOFF, GROUPS>;
  FB200_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  kernel<<<grid, kPlThreads, smem, s>>>(tx, tout, w, bias, out, g, idesc, epi, status);
  return after_launch("conv2d_planes_tcgen05_kernel");
}

}  // namespace fb200

using namespace fb200;

// Returns FB200_UNIMPLEMENTED for shapes outside this kernel's reach (stride other than 1, input
// channels not a multiple of 8, filters other than square 1/3/5/7 with "same" padding or 3x3 without,
// rows longer than 128 pixels, ...): the caller then tries the halo kernel, the gather kernel and
// the direct kernel.
extern "C" int fb200_conv2d_planes_tcgen05(const void* x, const void* w, const void* bias, void* out,
                                           const fb200_conv2d_params* p, int dtype,
                                           const fb200_epilogue* epilogue, fb200_stream stream) {
  if (dtype != FB200_F32 || p->groups != 1 || p->cout > 256 || p->cout < 1) return FB200_UNIMPLEMENTED;
  if (p->stride_h != 1 || p->stride_w != 1 || p->cin % 8 != 0) return FB200_UNIMPLEMENTED;
  PlanesGeom g{};
  g.n = static_cast<int>(p->n); g.cin = static_cast<int>(p->cin); g.h = static_cast<int>(p->h);
  g.w = static_cast<int>(p->w); g.cout = static_cast<int>(p->cout); g.kh = static_cast<int>(p->kh);
  g.kw = static_cast<int>(p->kw); g.ph = static_cast<int>(p->pad_h); g.pw = static_cast<int>(p->pad_w);
  if (p->n * p->cin * p->h * p->w >= (int64_t(1) << 31) || p->n > 65535 * 64) return FB200_UNIMPLEMENTED;
  if (g.kh > 7 || g.pw > 3) return FB200_UNIMPLEMENTED;
  g.oh = g.h + 2 * g.ph - g.kh + 1;
  g.ow = g.w + 2 * g.pw - g.kw + 1;
  if (g.oh < 1 || g.ow < 4 || g.ow > kPlTileM || g.ow % 4 != 0 || g.w % 4 != 0 || !aligned16(x)) return FB200_UNIMPLEMENTED;
  g.owp = g.ow <= 32 ? 32 : (g.ow <= 64 ? 64 : 128);
  g.spr = g.owp / 32;
  g.rows = kPlTileM / g.owp;
  if (g.rows > g.oh) g.rows = g.oh;
  g.tiles_per_img = (g.oh + g.rows - 1) / g.rows;
  g.n_tiles = static_cast<int64_t>(g.n) * g.tiles_per_img;
  if (g.n_tiles <= 0) return FB200_UNIMPLEMENTED;
  // the halo tile always has the rows of a full tile (kPlTileM / owp output rows), so that every
  // descriptor stays inside a plane
  const int full_rows = kPlTileM / g.owp;
  g.ih_t = full_rows + g.kh - 1;
  g.x0a = -((g.pw + 3) / 4) * 4;
  const int xoff = -g.pw - g.x0a;
  g.iwp = (g.ow - 1 + g.kw + xoff + 3) / 4 * 4;
  if (g.iwp > 256 || g.ih_t > 256) return FB200_UNIMPLEMENTED;
  g.npad = (g.cout + 31) / 32 * 32;
  g.acc_per_round = 512 / g.npad < kPlMaxAcc ? 512 / g.npad : kPlMaxAcc;
  g.tmem_cols = 32;
  while (g.tmem_cols < g.acc_per_round * g.npad) g.tmem_cols *= 2;
  EpilogueDev epi{};
  if (int rc = make_epilogue(epilogue, &epi, "conv2d")) return rc;
  // channel block: the largest of 32, 16, 8 that divides Cin and fits, together with two plane sets,
  // at least two halo buffers and (when possible) the output staging tile
  const int64_t limit = 227 * 1024;
  const int64_t misc = 1024 /*align*/ + 512 /*barriers*/ + 1024 /*bias*/ + 256 +
                       static_cast<int64_t>(g.ih_t) * (g.ow / 4) * 8 /*pair table*/;
  int64_t stage_need = (static_cast<int64_t>(g.cout) * g.rows * g.ow * 4 + 127) / 128 * 128 + 128;
  if (!(g.ow % 4 == 0 && aligned16(out))) stage_need = 0;
  bool fits = false;
  for (int cb : {32, 16, 8}) {
    if (g.cin % cb != 0) continue;
    g.cb = cb;
    g.n_cb = g.cin / cb;
    g.kcb = cb * g.kh * g.kw;
    g.kblocks = (g.kcb + 31) / 32;
    g.w_bytes = g.kblocks * g.npad * 128;
    g.lbo = cb * 128;
    g.plane_bytes = g.ih_t * g.spr * g.lbo;
    g.set_bytes = (g.kw * g.plane_bytes + 1023) / 1024 * 1024;
    g.halo_bytes = (cb * g.ih_t * g.iwp * 4 + 64 + 1023) / 1024 * 1024;
    const int64_t fixed = misc + g.w_bytes + static_cast<int64_t>(kPlSets) * g.set_bytes;
    const int64_t room = limit - fixed;
    if (room < 2 * static_cast<int64_t>(g.halo_bytes)) continue;
    g.out_stage_bytes = 0;
    int64_t room_left = room;
    if (stage_need > 0 && room - stage_need >= 2 * static_cast<int64_t>(g.halo_bytes)) {
      g.out_stage_bytes = static_cast<int>(stage_need);
      room_left = room - stage_need;
    }
    g.n_halo = static_cast<int>(room_left / g.halo_bytes);
    if (g.n_halo > kPlMaxBufs) g.n_halo = kPlMaxBufs;
    fits = true;
    break;
  }
  if (!fits) return FB200_UNIMPLEMENTED;
  CUtensorMap tx;
  if (int rc = make_tmap_nchw_f32(&tx, x, g.n, g.cin, g.h, g.w, g.cb, g.ih_t, g.iwp)) return rc;
  CUtensorMap tout = tx;   // placeholder when the direct-store epilogue is used
  if (g.out_stage_bytes > 0) {
    if (int rc = make_tmap_nchw_f32(&tout, out, g.n, g.cout, g.oh, g.ow, g.cout, g.rows, g.ow)) return rc;
  }
  int* status = nullptr;
  if (int rc = device_status_word(&status)) return rc;
  const size_t smem = static_cast<size_t>(misc) + g.w_bytes + static_cast<size_t>(kPlSets) * g.set_bytes +
                      static_cast<size_t>(g.n_halo) * g.halo_bytes + static_cast<size_t>(g.out_stage_bytes);
  const uint32_t idesc = make_instr_desc(kFmtTF32, /*a MN-major*/ 1, /*b MN-major*/ 0, kPlTileM,
                                         static_cast<uint32_t>(g.npad));
  const int grid = static_cast<int>(g.n_tiles < kNumSMs ? g.n_tiles : kNumSMs);
  if (g.kh != g.kw) return FB200_UNIMPLEMENTED;
  const bool known = (g.kw == 3 && (xoff == 3 || xoff == 0)) || (g.kw == 1 && xoff == 0) || (g.kw == 5 && xoff == 2) ||
                     (g.kw == 7 && xoff == 1);
  if (!known) return FB200_UNIMPLEMENTED;
  const float* bp = static_cast<const float*>(bias);
  float* op = static_cast<float*>(out);
  cudaStream_t s = as_stream(stream);
  // the filter packed into the shared-memory image of each channel block (stream-ordered scratch)
  float* packed = nullptr;
  const size_t packed_floats = static_cast<size_t>(g.n_cb) * (g.w_bytes / 4);
  FB200_CUDA_OK(scratch_alloc_async(reinterpret_cast<void**>(&packed), packed_floats * sizeof(float), s));
  conv_pack_weights_kernel<<<grid_for(static_cast<int64_t>(packed_floats), 256, 4), 256, 0, s>>>(
      static_cast<const float*>(w), packed, g.cin, g.cout, g.kh * g.kw, g.cb, g.n_cb, g.kblocks, g.npad);
  int rc = after_launch("conv_pack_weights_kernel");
  const int groups = g.cb / 8;
#define FB200_PLANES_CASE(KV, XO)                                                                              \
  if (rc == FB200_OK && g.kw == KV && xoff == XO) {                                                             \
    if (groups == 4) rc = launch_planes<KV, KV, XO, 4>(tx, tout, packed, bp, op, g, idesc, epi, status, smem, grid, s);      \
    else if (groups == 2) rc = launch_planes<KV, KV, XO, 2>(tx, tout, packed, bp, op, g, idesc, epi, status, smem, grid, s); \
    else rc = launch_planes<KV, KV, XO, 1>(tx, tout, packed, bp, op, g, idesc, epi, status, smem, grid, s);                  \
  }
  FB200_PLANES_CASE(3, 3)   // 3x3, padding 1
  FB200_PLANES_CASE(1, 0)   // 1x1
  FB200_PLANES_CASE(3, 0)   // 3x3, no padding
  FB200_PLANES_CASE(5, 2)   // 5x5, padding 2
  FB200_PLANES_CASE(7, 1)   // 7x7, padding 3
#undef FB200_PLANES_CASE
  cudaFreeAsync(packed, s);
  return rc;
}
