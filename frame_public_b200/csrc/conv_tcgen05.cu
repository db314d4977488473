// conv2d as an implicit GEMM on the tensor cores (fp32 tensors, TF32 math, fp32 accumulation).
//
// Semantics: src/backends/cpu/kernels/conv.cpp:225-257 (NCHW cross-correlation, zero padding,
// bias per output channel added last); used when CompileOptions::allow_tf32 permits reduced
// precision (include/frame/hal/backend.h:51-63), groups == 1 and Cout <= 256.  Replaces
// cudnnConvolutionForward + cudnnAddTensor of src/backends/cuda/kernels/conv.cpp:385-520 and the
// separate activation / residual launches that followed it.
//
// GEMM view: D[pixel, co] = sum_k A[pixel, k] * W[co, k], k = (ci, kh, kw), pixel = (n, oh, ow).
//   * M = 128 pixels per tile.  Pixels of one image row are contiguous in NCHW, so the im2col
//     operand A is "MN-major"; the TMEM accumulator then has one pixel per lane and the epilogue
//     writes out[n, co, pixel] with 32 consecutive pixels per warp store: coalesced NCHW output
//     with no transpose anywhere.
//   * N = Cout (padded to 16), K-major operand straight from w[co][ci,kh,kw].
//   * A cannot be fetched by TMA: the +-1 pixel shifts of a 3x3 window start at addresses that are
//     not multiples of 16 bytes.  Four producer warps gather it with coalesced 4-byte loads (one
//     pixel per thread, zero for padding) and store it in the 128-byte-swizzled (32-byte units)
//     layout tcgen05 requires for 32-bit MN-major operands; the weights go the same way into the
//     K-major 128-byte-swizzled layout.  fence.proxy.async + mbarrier hand a stage to the MMA warp.
//   * warp 4 allocates TMEM (two accumulators) and issues 4 tcgen05.mma kind::tf32 (K = 8) per
//     32-wide k-block; warps 5-8 run the epilogue (bias, ReLU / residual chain, coalesced stores)
//     of tile i while tile i+1 accumulates.
// Every wait is bounded; a wait that gives up records a status code and the CTA exits cleanly.
// Bound: tensor pipe / LSU of the gather.  FLOPs per launch = 2 * N*OH*OW * Cout * Cin*KH*KW.
#include "common.cuh"
#include "epilogue.cuh"
#include "sm100_ptx.cuh"

namespace fb200 {

int device_status_word(int** dev_ptr);  // gemm_tcgen05.cu

using namespace sm100;

constexpr int kConvTileM = 128;
constexpr int kConvBlockK = 32;
constexpr int kConvProducers = 256;
constexpr int kConvThreads = 416;  // 8 producer warps, 1 MMA warp, 4 epilogue warps
constexpr int kConvMmaWarp = 8;
constexpr int kConvMaxK = 4608;    // rows of the k -> (offset, ky, kx) table kept in shared memory
constexpr int kConvAStage = kConvTileM * 128;  // 16 KiB: 4 chunks of 32 pixels x 32 k-rows x 128 B

enum ConvFault : int {
  kFaultConvProducerEmpty = 201,
  kFaultConvMmaFull = 202,
  kFaultConvMmaTmemEmpty = 203,
  kFaultConvEpilogueFull = 204,
};

struct ConvGeom {
  int64_t n, cin, h, w, cout, kh, kw, sh, sw, ph, pw, oh, ow;
  int64_t K;          // cin*kh*kw
  int64_t total_pix;  // n*oh*ow
  int npad;           // cout rounded up to 16
  int tmem_cols;      // power of two >= 2*npad
  int stages;         // depth of the shared-memory ring
};

__global__ void __launch_bounds__(kConvThreads, 1)
conv2d_tcgen05_kernel(const float* __restrict__ x, const float* __restrict__ w,
                      const float* __restrict__ bias, float* __restrict__ out, ConvGeom g,
                      uint32_t idesc, EpilogueDev epi, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw_addr);
  const int b_stage_bytes = g.npad * 128;
  const int stage_bytes = kConvAStage + b_stage_bytes;
  const uint32_t bars = base + g.stages * stage_bytes;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (g.stages + s); };
  auto tmem_full_bar = [&](int a) { return bars + 8u * (2 * g.stages + a); };
  auto tmem_empty_bar = [&](int a) { return bars + 8u * (2 * g.stages + 2 + a); };
  const uint32_t tmem_slot = bars + 8u * (2 * g.stages + 4);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(
      base_ptr + g.stages * stage_bytes + 8 * (2 * g.stages + 4));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t n_tiles = (g.total_pix + kConvTileM - 1) / kConvTileM;
  const int64_t k_blocks = (g.K + kConvBlockK - 1) / kConvBlockK;
  const int64_t ohow = g.oh * g.ow;

  if (threadIdx.x == 0) {
    for (int s = 0; s < g.stages; ++s) {
      mbar_init(full_bar(s), kConvProducers / 32);   // one arrival per producer warp
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), 4);
    }
    mbar_fence_init();
  }
  // k -> {offset of (ci, ky, kx) inside one image, ky | kx << 16}; rows past K are marked so that
  // the bounds test fails and the tap reads as zero.
  int2* ktab = reinterpret_cast<int2*>(base_ptr + g.stages * stage_bytes + 256);
  {
    const int64_t khkw0 = g.kh * g.kw;
    for (int64_t k = threadIdx.x; k < k_blocks * kConvBlockK; k += kConvThreads) {
      int2 e;
      if (k < g.K) {
        const int64_t ci = k / khkw0;
        const int64_t rem = k - ci * khkw0;
        const int64_t ky = rem / g.kw;
        const int64_t kx = rem - ky * g.kw;
        e.x = static_cast<int>((ci * g.h + ky) * g.w + kx);
        e.y = static_cast<int>(ky | (kx << 16));
      } else {
        e.x = 0;
        e.y = 0x4000;  // ky far outside any image
      }
      ktab[k] = e;
    }
  }
  if (warp == kConvMmaWarp) {
    __syncwarp();
    tmem_alloc(tmem_slot, static_cast<uint32_t>(g.tmem_cols));
    tmem_relinquish();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp < kConvMmaWarp) {
    // ---- producers: 256 threads = 128 pixels x 2 halves of the 32 k-rows of a block -------------
    const int tid = threadIdx.x;        // 0..255
    const int ptid = tid & 127;         // pixel inside the tile
    const int khalf = tid >> 7;         // which 16 k-rows of the block
    const uint32_t a_thread_off = static_cast<uint32_t>((ptid >> 5) * (kConvBlockK * 128) + (ptid & 7) * 4);
    const uint32_t a_unit = static_cast<uint32_t>((ptid & 31) >> 3);  // 32-byte unit inside the row
    const int H = static_cast<int>(g.h), W = static_cast<int>(g.w);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int64_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
      const int64_t p = tile * kConvTileM + ptid;
      const bool valid = p < g.total_pix;
      const int64_t img = valid ? p / ohow : 0;
      const int pix = static_cast<int>(valid ? p - img * ohow : 0);
      const int oy = pix / static_cast<int>(g.ow);
      const int ox = pix - oy * static_cast<int>(g.ow);
      const int ih0 = valid ? oy * static_cast<int>(g.sh) - static_cast<int>(g.ph) : -0x8000;
      const int iw0 = ox * static_cast<int>(g.sw) - static_cast<int>(g.pw);
      const float* xpix = x + img * g.cin * g.h * g.w + static_cast<int64_t>(ih0) * W + iw0;
      for (int64_t kb = 0; kb < k_blocks; ++kb) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, status, kFaultConvProducerEmpty)) { ok = false; break; }
        const uint32_t a_stage = base + stage * stage_bytes;
        const uint32_t b_stage = a_stage + kConvAStage;
        const int64_t k0 = kb * kConvBlockK;
        const int2* tab = ktab + k0 + khalf * 16;
        float v[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          const int2 e = tab[u];
          const int ky = e.y & 0xFFFF, kx = e.y >> 16;
          const bool inb = static_cast<unsigned>(ih0 + ky) < static_cast<unsigned>(H) &&
                           static_cast<unsigned>(iw0 + kx) < static_cast<unsigned>(W);
          v[u] = inb ? __ldg(xpix + e.x) : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          const uint32_t kk = static_cast<uint32_t>(khalf * 16 + u);
          const uint32_t addr = a_stage + a_thread_off + kk * 128u + ((a_unit ^ (kk & 3u)) << 5);
          asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v[u]) : "memory");
        }
        // B: npad rows x 32 k, K-major, 16-byte swizzle units over 8 rows
        for (int idx = tid; idx < g.npad * kConvBlockK; idx += kConvProducers) {
          const int co = idx >> 5;
          const uint32_t kk = static_cast<uint32_t>(idx & 31);
          const int64_t k = k0 + kk;
          const float wv = (co < g.cout && k < g.K) ? __ldg(w + co * g.K + k) : 0.0f;
          const uint32_t addr = b_stage + static_cast<uint32_t>((co >> 3) * 1024 + (co & 7) * 128) +
                                (((kk >> 2) ^ static_cast<uint32_t>(co & 7)) << 4) + (kk & 3u) * 4u;
          asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(wv) : "memory");
        }
        fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor-core (async) proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(full_bar(stage));   // 256 separate arrivals would serialise
        if (++stage == g.stages) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == kConvMmaWarp) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int64_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1u, status, kFaultConvMmaTmemEmpty)) { ok = false; break; }
        tcgen05_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * g.npad);
        for (int64_t kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, status, kFaultConvMmaFull)) { ok = false; break; }
          tcgen05_fence_after_sync();
          const uint32_t a_addr = base + stage * stage_bytes;
          const uint32_t b_addr = a_addr + kConvAStage;
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            // A: MN-major, 32-pixel spans kConvBlockK*128 bytes apart (LBO), 4-row k groups 512
            // bytes apart (SBO); one MMA (K = 8) covers two groups = 1024 bytes.
            const uint64_t a_desc = make_smem_desc(a_addr + ks * 1024, kConvBlockK * 128, 512, kLayoutSw128Base32);
            // B: K-major, 8-row groups 1024 bytes apart; a K step is 32 bytes inside the row.
            const uint64_t b_desc = make_smem_desc(b_addr + ks * 32, 16, 1024, kLayoutSw128);
            mma_tf32(d_tmem, a_desc, b_desc, idesc, (kb > 0 || ks > 0) ? 1u : 0u);
          }
          mma_commit(empty_bar(stage));
          if (++stage == g.stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        mma_commit(tmem_full_bar(acc));
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ---- epilogue warps 9..12: TMEM lane = pixel ------------------------------------------------------
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int64_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
      if (!mbar_wait(tmem_full_bar(acc), acc_phase, status, kFaultConvEpilogueFull)) { ok = false; break; }
      tcgen05_fence_after_sync();
      const int64_t p = tile * kConvTileM + quarter * 32 + lane;
      const bool valid = p < g.total_pix;
      const int64_t img = valid ? p / ohow : 0;
      const int64_t pix = valid ? p - img * ohow : 0;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(acc * g.npad);
#pragma unroll 1
      for (int c0 = 0; c0 < g.npad; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + static_cast<uint32_t>(c0), r);
        tmem_ld_wait();
        if (valid) {
          float v[32];
          const int64_t obase = (img * g.cout + c0) * ohow + pix;   // + j*ohow per channel
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            v[j] = __uint_as_float(r[j]);
            if (bias != nullptr && c0 + j < g.cout) v[j] += __ldg(bias + c0 + j);
          }
#pragma unroll 1
          for (int s = 0; s < epi.n_ops; ++s) {
            const int op = epi.ops[s];
            const float* opnd = static_cast<const float*>(epi.operands[s]);
            if (opnd != nullptr) {
              const int mode = epi.modes[s];
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (c0 + j < g.cout) {
                  const float rhs = mode == FB200_OPERAND_FULL ? __ldg(opnd + obase + j * ohow)
                                    : mode == FB200_OPERAND_ROW ? __ldg(opnd + c0 + j)
                                                                : __ldg(opnd + pix % g.ow);
                  v[j] = ew_binary(op, v[j], rhs);
                }
              }
            } else {
              ew_unary_vec<float, 32>(op, v);
            }
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (c0 + j < g.cout) out[obase + j * ohow] = v[j];
          }
        }
      }
      tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty_bar(acc));
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }

  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == kConvMmaWarp) {
    __syncwarp();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(g.tmem_cols));
  }
}

}  // namespace fb200

using namespace fb200;

extern "C" int fb200_conv2d_tcgen05(const void* x, const void* w, const void* bias, void* out,
                                    const fb200_conv2d_params* p, int dtype,
                                    const fb200_epilogue* epilogue, fb200_stream stream) {
  if (dtype != FB200_F32 || p->groups != 1 || p->cout > 256 || p->cout < 1) return FB200_UNIMPLEMENTED;
  ConvGeom g{};
  g.n = p->n; g.cin = p->cin; g.h = p->h; g.w = p->w; g.cout = p->cout; g.kh = p->kh; g.kw = p->kw;
  g.sh = p->stride_h; g.sw = p->stride_w; g.ph = p->pad_h; g.pw = p->pad_w;
  g.oh = (p->h + 2 * p->pad_h - p->kh) / p->stride_h + 1;
  g.ow = (p->w + 2 * p->pad_w - p->kw) / p->stride_w + 1;
  g.K = g.cin * g.kh * g.kw;
  g.total_pix = g.n * g.oh * g.ow;
  g.npad = static_cast<int>((g.cout + 15) / 16 * 16);
  if (g.npad > 32 && g.npad % 32 != 0) g.npad = (g.npad + 31) / 32 * 32;  // whole 32-column TMEM reads
  if (g.npad < 32) g.npad = 32;
  g.tmem_cols = 32;
  while (g.tmem_cols < 2 * g.npad) g.tmem_cols *= 2;
  const int64_t k_pad = (g.K + kConvBlockK - 1) / kConvBlockK * kConvBlockK;
  if (g.total_pix <= 0 || g.npad > 256 || k_pad > kConvMaxK) return FB200_UNIMPLEMENTED;
  if (g.n * g.cin * g.h * g.w >= (int64_t(1) << 31) || g.cin * g.h * g.w >= (int64_t(1) << 30)) {
    return FB200_UNIMPLEMENTED;  // 32-bit offsets inside one image
  }
  const int stage_bytes = kConvAStage + g.npad * 128;
  const int64_t table_bytes = k_pad * 8;
  g.stages = static_cast<int>((220 * 1024 - 1024 - 256 - table_bytes) / stage_bytes);
  if (g.stages > 4) g.stages = 4;
  if (g.stages < 2) return FB200_UNIMPLEMENTED;
  EpilogueDev epi{};
  if (int rc = make_epilogue(epilogue, &epi, "conv2d")) return rc;
  int* status = nullptr;
  if (int rc = device_status_word(&status)) return rc;
  const size_t smem = static_cast<size_t>(g.stages) * stage_bytes + 1024 + 256 + table_bytes;
  FB200_CUDA_OK(cudaFuncSetAttribute(conv2d_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(smem)));
  const uint32_t idesc = make_instr_desc(kFmtTF32, /*a MN-major*/ 1, /*b MN-major*/ 0, kConvTileM,
                                         static_cast<uint32_t>(g.npad));
  const int64_t tiles = (g.total_pix + kConvTileM - 1) / kConvTileM;
  const int grid = static_cast<int>(tiles < kNumSMs ? tiles : kNumSMs);
  conv2d_tcgen05_kernel<<<grid, kConvThreads, smem, as_stream(stream)>>>(
      static_cast<const float*>(x), static_cast<const float*>(w), static_cast<const float*>(bias),
      static_cast<float*>(out), g, idesc, epi, status);
  return after_launch("conv2d_tcgen05_kernel");
}
