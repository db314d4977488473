// matmul on the 5th-generation tensor cores: C[M,N] = A[M,K] * B[K,N] (+ fused epilogue), all
// row-major, bf16/f16 operands through tcgen05.mma kind::f16 and fp32 operands through
// kind::tf32, fp32 accumulation in TMEM, one rounding at the store.
//
// Semantics: src/backends/cpu/kernels/matmul.cpp:92-131 (fp32 accumulate, single rounding).
// Replaces the cublasLtMatmul call of src/backends/cuda/kernels/matmul.cpp:90-276, which also
// ran bias and activation as separate launches; here they are the epilogue of the same kernel.
//
// Design (one persistent CTA per SM, 352 threads, warp-specialised):
//   warps 0, 10  TMA producers: warp 0 loads the A tile [128*MH x BLOCK_K] (K-contiguous, "K-major"
//            operand), warp 10 the B tile [BLOCK_K x BLOCK_N] (N-contiguous, "MN-major" operand)
//            with one copy through a 3-D view [N/span][K][span] of the row-major matrix (or one copy
//            per 128-byte span when N is not a whole number of spans).  Both land in
//            128-byte-swizzled shared memory; a ring of STAGES slots is handed over with full/empty
//            mbarriers.  No host-side transposes: the row-major B is consumed as it lies in HBM.
//   warp 1   allocates TMEM (2 accumulators of BLOCK_N fp32 columns) and issues 4*MH tcgen05.mma
//            (M=128, N=BLOCK_N, K=32 bytes) per stage; tcgen05.commit releases the stage and, after
//            the last k-block, publishes the accumulator.
//   warps 2-9 epilogue: tcgen05.ld 32 lanes x 32 columns, the epilogue chain in fp32 registers
//            (operands fetched with 128-bit loads), 128-bit stores; two warps per TMEM lane
//            quarter, each on half of the tile's columns (with four warps a transcendental
//            epilogue behind a short K was bound by those 128 threads).  The second accumulator
//            lets the epilogue of tile i overlap the MMAs of tile i+1 (MH = 1; with MH = 2 the
//            256 x 256 tile takes both accumulators and each warp group drains one of them).
// Producer and MMA loops are run by the whole warp, one elected lane issuing each instruction
// (elect.sync + predicate): inside an `if (lane == 0)` branch the same loops fed the tensor pipe a
// quarter slower (166 instead of 128 cycles per M128 x N256 x K16 instruction with resident
// operands), because descriptors and coordinates then live in per-thread instead of uniform
// registers.
// Tiles are walked in groups of 16 M-blocks so that concurrently resident CTAs share A and B
// panels in the 126 MB L2 (B is then streamed from HBM tiles_m/16 times: 1.0 GB of DRAM reads per
// 8192^3 launch with groups of 8 measured by ncu, against 384 MB of distinct operands).  Edge tiles rely on TMA zero fill for loads and masked stores.
// Bound: tensor pipe.  FLOPs per launch = 2*M*N*K.
#include <cuda.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "epilogue.cuh"
#include "sm100_ptx.cuh"

namespace fb200 {

int gemm_simt(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k, int dtype,
              const EpilogueDev& epi, cudaStream_t s);

using namespace sm100;

constexpr int kBlockM = 128;
constexpr int kGemmThreads = 352;   // A-producer warp, MMA warp, eight epilogue warps, B-producer warp
constexpr int kGemmBProducerWarp = 10;
// M-blocks per group of the tile walk (8192^3 bf16: groups of 8 gave 1345, 16: 1362, 32: 1335,
// 64: 1278 TFLOP/s).
constexpr int kGemmGroupM = 16;

// An epilogue of binary ops, ReLU, square and the step function: a few instructions per element.
static bool light_epilogue(const EpilogueDev& epi) {
  for (int i = 0; i < epi.n_ops; ++i) {
    const int op = epi.ops[i];
    if (op != FB200_EW_ADD && op != FB200_EW_MUL && op != FB200_EW_RELU && op != FB200_EW_SQUARE &&
        op != FB200_EW_HEAVISIDE) {
      return false;
    }
  }
  return true;
}

// Where a tile of the result goes: one or several destination matrices of row pitch `ld`, at
// column offset `col0`.  One destination with ld == N, col0 == 0 is the ordinary matmul; several
// destinations are this GPU's and its peers' copies of a column-split result (the all-gather is
// fused into the epilogue as plain peer stores over NVLink).
constexpr int kMaxDest = 8;
struct GemmDest {
  void* ptr[kMaxDest];
  int n;
  int group_m;   // M-blocks per group of the tile walk
  int64_t ld;
  int64_t col0;
  // columns [tail_col, N) of the result go to a dense matrix of their own (row pitch tail_ld)
  // instead of `ptr`: a graph that only ever reads that column block as a `slice` gets it where the
  // slice would have copied it.  tail_ptr == nullptr: no split.  tail_col is a multiple of 32.
  void* tail_ptr;
  int64_t tail_col;
  int64_t tail_ld;
  // error-compensated fp32: the low parts x - trunc_tf32(x) of A and B (same shapes), or nullptr
  const void* a_lo;
  const void* b_lo;
};

enum GemmFault : int {
  kFaultProducerEmpty = 101,
  kFaultMmaFull = 102,
  kFaultMmaTmemEmpty = 103,
  kFaultEpilogueTmemFull = 104,
  kFaultSplitPartial = 105,
};

// Work of one launch.  The first `dp_tiles` tiles of the tile order are walked whole (tile = CTA,
// CTA + grid, ...).  The k-blocks of the remaining tiles, `sk_units` in all, are dealt out to the
// first `sk_ctas` CTAs in contiguous ranges of equal length, so that a last wave which would occupy a
// fraction of the SMs for a whole tile's time is spread over all of them ("stream-K").  A range cuts
// tiles into segments [kb0, kb1).  The CTA that holds a tile's FIRST k-blocks owns it: it keeps its
// segment in TMEM, adds the partial accumulators of the CTAs that follow (each CTA writes at most one:
// only its first segment can start inside a tile) and runs the epilogue.  A partial tile is the raw
// fp32 accumulator in `ws`, in the order the TMEM loads hand it out; flags[cta * 8 + epilogue warp]
// says that the warp's share is written.  Ranges are handed out against the order in which the CTAs
// START (a ticket taken at entry): an owner only ever waits for CTAs that started before it, each
// working on its FIRST segment, which never waits itself.  So a waiting CTA never depends on one
// that is not yet resident, whatever else shares the GPU, and the waits cannot form a cycle; every
// wait is bounded all the same.  sk_units == 0: no split.
struct GemmSplit {
  int64_t dp_tiles;
  int64_t sk_units;
  int sk_ctas;
  float* ws;     // [sk_ctas][BLOCK_N / 32][8][128] float4
  int* flags;    // [range][8], zero before the launch; every owner clears what it has consumed
  int* tickets;  // {CTAs started, CTAs finished}: zero before the launch, reset by the last CTA
};

struct GemmSegment {
  int64_t tile, kb0, kb1;
};

__device__ __forceinline__ int64_t split_range_begin(const GemmSplit& sp, int cta) {
  return sp.sk_units * cta / sp.sk_ctas;
}

// The segments of this CTA, in order; every role of the CTA walks the same list.  `rank` is the
// CTA's place in the order in which the grid's CTAs started (blockIdx.x when nothing is split):
// whole tiles go by rank, and rank r takes range sk_ctas - 1 - r, so that the ranges AFTER a CTA's
// own, the ones its epilogue may wait for, belong to CTAs that started before it.
template <bool SPLIT>
struct SegmentWalk {
  int64_t dp_next, dp_tiles, k_blocks, u, u1;
  __device__ SegmentWalk(const GemmSplit& sp, int64_t k_blocks_, int rank) {
    dp_next = rank;
    dp_tiles = sp.dp_tiles;
    k_blocks = k_blocks_;
    u = u1 = 0;
    if (SPLIT && sp.sk_units > 0 && rank < sp.sk_ctas) {
      const int range = sp.sk_ctas - 1 - rank;
      u = split_range_begin(sp, range);
      u1 = split_range_begin(sp, range + 1);
    }
  }
  __device__ __forceinline__ bool next(GemmSegment* sg) {
    if (dp_next < dp_tiles) {
      sg->tile = dp_next;
      sg->kb0 = 0;
      sg->kb1 = k_blocks;
      dp_next += gridDim.x;
      return true;
    }
    if (SPLIT && u < u1) {
      const int64_t t = u / k_blocks;
      sg->tile = dp_tiles + t;
      sg->kb0 = u - t * k_blocks;
      const int64_t left = u1 - u, room = k_blocks - sg->kb0;
      const int64_t len = left < room ? left : room;
      sg->kb1 = sg->kb0 + len;
      u += len;
      return true;
    }
    return false;
  }
};

// Bounded wait for a flag another CTA of this launch sets (lane 0 polls, the warp gets the result).
__device__ __forceinline__ bool split_flag_wait(const int* flag, int* status) {
  int ok = 1;
  if ((threadIdx.x & 31u) == 0u) {
    const unsigned long long t0 = globaltimer_ns();
    for (uint32_t i = 1;; ++i) {
      int v;
      asm volatile("ld.acquire.gpu.global.b32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
      if (v != 0) break;
      if ((i & 255u) == 0u) {
        if (*reinterpret_cast<volatile int*>(status) != 0) { ok = 0; break; }
        if (globaltimer_ns() - t0 > kWaitBudgetNs) {
          *reinterpret_cast<volatile int*>(status) = kFaultSplitPartial;
          ok = 0;
          break;
        }
      }
    }
  }
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// EG: epilogue groups.  1: eight epilogue warps drain every tile.  2: a second group of eight warps
// (warps 11-18), each group draining the tiles of ONE of the two TMEM accumulators, so that the
// epilogue of tile i runs beside that of tile i + 1: for products whose K is so short that the
// launch IS its epilogue (one 32-column chunk in flight per warp is latency-bound).  The second
// group's transposition buffers cost a ring stage.
template <int ELT, int BLOCK_N, int MH = 1, int KB = 128, int EG = 1>
struct GemmCfg {
  // KB: bytes of K per A row in a ring stage (128, or 64 with the 64-byte swizzle).  What bounds the
  // mainloop is the ring's turnaround (per-role cycle counters, 8192^3 bf16: about 2400 cycles from
  // the first MMA of a slot to its refill having landed: 512 of MMAs, 450 until the producer sees the
  // commit, the copy's issue, 1300 of L2 latency and transfer; four 48 KiB slots give one k-block
  // per 600 cycles against 512 of tensor work).  Half-size slots (KB = 64, twice as many) would turn
  // around faster, but the producers then cannot issue fast enough: measured 0.955 ms against
  // 0.764 ms for 8192^3 on 128 x 256 tiles, 0.728 against 0.711 on 256 x 256.  Only KB = 128 is
  // instantiated.
  static constexpr int kTileM = kBlockM * MH;          // MH = 2: two M = 128 instructions share each B stage
  static constexpr int kBlockK = KB / ELT;           // K elements per stage: one swizzle span of the A rows
  static constexpr int kUmmaKBytes = 32;              // K extent of one tcgen05.mma
  static constexpr int kStepsPerBlock = KB / 32;
  static constexpr int kAStageBytes = kTileM * KB;    // 16 KiB per 128 rows of 128 bytes
  static constexpr int kBChunkCols = 128 / ELT;       // N columns per 128-byte span
  static constexpr int kBChunks = BLOCK_N / kBChunkCols;
  static constexpr int kBChunkBytes = kBlockK * 128;
  static constexpr int kBStageBytes = kBChunks * kBChunkBytes;
  static constexpr int kStageBytes = kAStageBytes + kBStageBytes;
  static constexpr int kRingBytes = (192 - 32 * (EG - 1)) * 1024;
  static constexpr int kStages = kRingBytes / kStageBytes > 12 ? 12 : kRingBytes / kStageBytes;
  static constexpr int kThreads = kGemmThreads + (EG - 1) * 256;
  static constexpr int kTmemCols = 2 * BLOCK_N;
  // B operand, MN-major, 128-byte swizzle: 8-row K groups are 1024 bytes apart (SBO); the next
  // 128-byte span along N is one chunk further (LBO).  One MMA covers 32 bytes of K:
  // 16 rows (two groups) for 2-byte elements, 8 rows (one group) for 4-byte elements.
  static constexpr int kBKStepBytes = (kUmmaKBytes / ELT / 8) * 1024;
  // after the ring: 512 bytes of barriers, then one 4 KiB transpose buffer per epilogue warp
  static constexpr int kEpiStageBytes = 32 * 128;
  static constexpr size_t kSmemBytes = size_t(kStages) * kStageBytes + 1024 /*align*/ + 512 /*barriers*/ +
                                       8 * EG * kEpiStageBytes;
};

__device__ __forceinline__ void tile_coords(int64_t tile, int64_t tiles_m, int64_t tiles_n, int kGroupM,
                                            int64_t* tm, int64_t* tn) {
  const int64_t per_group = kGroupM * tiles_n;
  const int64_t group = tile / per_group;
  const int64_t first_m = group * kGroupM;
  const int64_t group_rows = tiles_m - first_m < kGroupM ? tiles_m - first_m : kGroupM;
  const int64_t in_group = tile - group * per_group;
  *tm = first_m + in_group % group_rows;
  *tn = in_group / group_rows;
}


// ---- epilogue ------------------------------------------------------------------------------------
// tcgen05.ld hands lane r of a warp the 32 columns of ROW r: stores straight from that layout are
// 32 separate 16-byte pieces per instruction, one per row.  The chunk is therefore turned through a
// 4 KiB shared-memory buffer (16-byte pieces XOR-swizzled by the row, conflict-free both ways) into
// a layout in which the lanes of a warp cover whole rows: 32 / W lanes per row, W = 16 / sizeof(T)
// output elements per lane and pass.  Operand loads (a full-shape bias or residual) and the result
// stores are then 16 bytes per lane over contiguous row segments: whole 128-byte lines for fp32,
// 64-byte half lines for 16-bit results.
//
// Chains the kernel is instantiated for with the step codes as compile-time constants (the
// per-fused-group specialisation of the GEMM epilogue); every other chain runs the same code with
// the step list read at run time.
enum EpiKind : int {
  kEpiGeneric = 0,       // interpreter over epi.ops
  kEpiNone = 1,          // plain store
  kEpiAddFullGelu = 2,   // + full-shape bias, GELU         (Linear + GELU)
  kEpiAddColSoftplus = 3,// + row-broadcast bias, softplus  (Mamba dt_proj)
  kEpiGelu = 4,          // GELU                            (bias-free FFN)
  kEpiAddFull = 5,       // + full-shape tensor             (Linear bias or residual)
};

static int classify_epilogue(const EpilogueDev& e) {
  if (e.n_ops == 0) return kEpiNone;
  if (e.n_ops == 1 && e.ops[0] == FB200_EW_GELU) return kEpiGelu;
  if (e.n_ops == 1 && e.ops[0] == FB200_EW_ADD && e.modes[0] == FB200_OPERAND_FULL) return kEpiAddFull;
  if (e.n_ops == 2 && e.ops[0] == FB200_EW_ADD && e.modes[0] == FB200_OPERAND_FULL && e.ops[1] == FB200_EW_GELU) return kEpiAddFullGelu;
  if (e.n_ops == 2 && e.ops[0] == FB200_EW_ADD && e.modes[0] == FB200_OPERAND_COL && e.ops[1] == FB200_EW_SOFTPLUS) return kEpiAddColSoftplus;
  return kEpiGeneric;
}

// Geometry of one 32 x 32 chunk in the row-covering layout.
template <typename T>
struct ChunkView {
  static constexpr int W = 16 / sizeof(T);   // elements per lane and pass
  static constexpr int LPR = 32 / W;         // lanes per row
  static constexpr int RPP = W;              // rows per pass
  static constexpr int P = 32 / W;           // passes
  int64_t row0;      // first row of the warp's 32 rows
  int64_t col;       // this lane's first column
  int sub_row;       // lane / LPR
  int64_t M, N;
  bool vec;          // 16-byte accesses are legal for this chunk
  __device__ __forceinline__ int64_t row(int j) const { return row0 + j * RPP + sub_row; }
};

// One step of the chain over the lane's 32 values.  `op` and `mode` are compile-time constants in the
// specialised kernels (the switch folds away) and run-time values in the interpreter.
// `pre` holds the lane's pieces of a FULL operand fetched ahead of the accumulator (use_pre).
template <typename T>
__device__ __forceinline__ void chain_step(int op, int mode, const void* operand, float (&v)[32],
                                           const ChunkView<T>& g, const Vec16<T> (&pre)[32 / ChunkView<T>::W],
                                           bool use_pre) {
  constexpr int W = ChunkView<T>::W, P = ChunkView<T>::P;
  const T* opnd = static_cast<const T*>(operand);
  if (opnd == nullptr) {
    ew_unary_vec<T, 32>(op, v);
    return;
  }
  if (mode == FB200_OPERAND_ROW) {
#pragma unroll
    for (int j = 0; j < P; ++j) {
      const int64_t r = g.row(j);
      const float rhs = r < g.M ? to_f32(opnd[r]) : 0.0f;
#pragma unroll
      for (int e = 0; e < W; ++e) v[j * W + e] = round_through<T>(ew_binary(op, v[j * W + e], rhs));
    }
    return;
  }
  if (mode == FB200_OPERAND_COL) {
    float rhs[W];
    if (g.vec && (reinterpret_cast<uintptr_t>(opnd) & 15u) == 0) {
      load_vec<T>(opnd + g.col, rhs);
    } else {
#pragma unroll
      for (int e = 0; e < W; ++e) rhs[e] = g.col + e < g.N ? to_f32(opnd[g.col + e]) : 0.0f;
    }
#pragma unroll
    for (int j = 0; j < P; ++j) ew_binary_round_vec<T, W>(op, &v[j * W], rhs);
    return;
  }
  const bool vec = g.vec && (reinterpret_cast<uintptr_t>(opnd) & 15u) == 0;
#pragma unroll
  for (int j = 0; j < P; ++j) {
    const int64_t r = g.row(j);
    if (r >= g.M) continue;
    const T* src = opnd + r * g.N + g.col;
    float rhs[W];
    if (use_pre) {
#pragma unroll
      for (int e = 0; e < W; ++e) rhs[e] = to_f32(pre[j].v[e]);
    } else if (vec) {
      load_vec<T>(src, rhs);
    } else {
#pragma unroll
      for (int e = 0; e < W; ++e) rhs[e] = g.col + e < g.N ? to_f32(src[e]) : 0.0f;
    }
    ew_binary_round_vec<T, W>(op, &v[j * W], rhs);
  }
}

// Step of the chain whose FULL operand is fetched ahead of the accumulator: the first such step.
template <int EPI>
__device__ __forceinline__ int prefetch_step(const EpilogueDev& epi) {
  if constexpr (EPI == kEpiAddFull || EPI == kEpiAddFullGelu) {
    return 0;
  } else if constexpr (EPI != kEpiGeneric) {
    return -1;
  } else {
    for (int s = 0; s < epi.n_ops; ++s) {
      if (epi.operands[s] != nullptr && epi.modes[s] == FB200_OPERAND_FULL) return s;
    }
    return -1;
  }
}

template <typename T, int EPI>
__device__ __forceinline__ void apply_chain(const EpilogueDev& epi, float (&v)[32], const ChunkView<T>& g,
                                            const Vec16<T> (&pre)[32 / ChunkView<T>::W], int pre_step) {
  if constexpr (EPI == kEpiNone) {
    return;
  } else if constexpr (EPI == kEpiGelu) {
    chain_step<T>(FB200_EW_GELU, 0, nullptr, v, g, pre, false);
  } else if constexpr (EPI == kEpiAddFull) {
    chain_step<T>(FB200_EW_ADD, FB200_OPERAND_FULL, epi.operands[0], v, g, pre, pre_step == 0);
  } else if constexpr (EPI == kEpiAddFullGelu) {
    chain_step<T>(FB200_EW_ADD, FB200_OPERAND_FULL, epi.operands[0], v, g, pre, pre_step == 0);
    chain_step<T>(FB200_EW_GELU, 0, nullptr, v, g, pre, false);
  } else if constexpr (EPI == kEpiAddColSoftplus) {
    chain_step<T>(FB200_EW_ADD, FB200_OPERAND_COL, epi.operands[0], v, g, pre, false);
    chain_step<T>(FB200_EW_SOFTPLUS, 0, nullptr, v, g, pre, false);
  } else {
#pragma unroll 1
    for (int s = 0; s < epi.n_ops; ++s) chain_step<T>(epi.ops[s], epi.modes[s], epi.operands[s], v, g, pre, s == pre_step);
  }
}

// Row r's 32 accumulator columns (held by lane r) -> the row-covering layout, through `stage`.
template <typename T>
__device__ __forceinline__ void transpose_chunk(const uint32_t (&r)[32], float (&v)[32], uint32_t stage, int lane) {
  constexpr int W = ChunkView<T>::W, LPR = ChunkView<T>::LPR, P = ChunkView<T>::P;
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const uint32_t addr = stage + static_cast<uint32_t>(lane * 128 + ((q ^ (lane & 7)) << 4));
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(r[4 * q]), "r"(r[4 * q + 1]),
                 "r"(r[4 * q + 2]), "r"(r[4 * q + 3]) : "memory");
  }
  __syncwarp();
  const int sub_row = lane / LPR, piece0 = (lane % LPR) * (W / 4);
#pragma unroll
  for (int j = 0; j < P; ++j) {
    const int row = j * W + sub_row;
#pragma unroll
    for (int h = 0; h < W / 4; ++h) {
      const uint32_t addr = stage + static_cast<uint32_t>(row * 128 + (((piece0 + h) ^ (row & 7)) << 4));
      uint32_t a, b, c, d;
      asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr) : "memory");
      const float2 lo = round_pair_through<T>(make_float2(__uint_as_float(a), __uint_as_float(b)));
      const float2 hi = round_pair_through<T>(make_float2(__uint_as_float(c), __uint_as_float(d)));
      v[j * W + 4 * h + 0] = lo.x;
      v[j * W + 4 * h + 1] = lo.y;
      v[j * W + 4 * h + 2] = hi.x;
      v[j * W + 4 * h + 3] = hi.y;
    }
  }
  __syncwarp();   // every lane has read its pieces before the next chunk overwrites the buffer
}

template <typename T, int ELT, int BLOCK_N, int MH, int KB, int EPI, bool SPLIT, int EG = 1>
__global__ void __launch_bounds__(kGemmThreads + (EG - 1) * 256, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                    const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_a_lo,
                    const __grid_constant__ CUtensorMap tmap_b_lo, int parts, int b_spans_map, GemmDest dest, int64_t M,
                    int64_t N, int64_t K, uint32_t idesc, EpilogueDev epi, GemmSplit split, int* status) {
  using Cfg = GemmCfg<ELT, BLOCK_N, MH, KB, EG>;
  static_assert(MH == 1 || (MH == 2 && BLOCK_N == 256), "two M halves fill TMEM with one 256 x 256 tile");
  static_assert(EG == 1 || (MH == 1 && !SPLIT), "a second epilogue group drains the second accumulator");
  static_assert(!SPLIT || MH == 1, "split ranges keep one accumulator per segment");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;  // swizzle atoms need 1024-byte alignment
  uint8_t* base_ptr = smem_raw + (base - raw_addr);
  const uint32_t bars = base + Cfg::kStages * Cfg::kStageBytes;
  // barrier layout (8 bytes each): full[S], empty[S], tmem_full[2], tmem_empty[2], then tmem ptr
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (Cfg::kStages + s); };
  auto tmem_full_bar = [&](int a) { return bars + 8u * (2 * Cfg::kStages + a); };
  auto tmem_empty_bar = [&](int a) { return bars + 8u * (2 * Cfg::kStages + 2 + a); };
  const uint32_t tmem_slot = bars + 8u * (2 * Cfg::kStages + 4);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(
      base_ptr + Cfg::kStages * Cfg::kStageBytes + 8 * (2 * Cfg::kStages + 4));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t tiles_m = (M + Cfg::kTileM - 1) / Cfg::kTileM;
  const int64_t tiles_n = (N + BLOCK_N - 1) / BLOCK_N;
  const int group_m = dest.group_m / MH > 0 ? dest.group_m / MH : 1;
  // parts == 3: the contraction runs three times over K into the same accumulator, with the operand
  // pairs (A_lo, B), (A, B_lo), (A, B): fp32 operands split as x = trunc_tf32(x) + x_lo, the tensor
  // core truncating every operand it reads to TF32 itself (error-compensated "3xTF32": all product
  // terms but lo x lo, small terms first).
  const int64_t k_blocks_part = (K + Cfg::kBlockK - 1) / Cfg::kBlockK;
  const int64_t k_blocks = k_blocks_part * parts;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(full_bar(s), 2);   // the A producer's and the B producer's expect_tx arrivals
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), 8 / MH);  // one arrival per epilogue warp that drains it
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (parts > 1) {
      tma_prefetch_desc(&tmap_a_lo);
      tma_prefetch_desc(&tmap_b_lo);
    }
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  volatile int* rank_slot_ptr = reinterpret_cast<volatile int*>(
      base_ptr + Cfg::kStages * Cfg::kStageBytes + 8 * (2 * Cfg::kStages + 5));
  if (threadIdx.x == 32 * 2) {
    *rank_slot_ptr = SPLIT ? atomicAdd(split.tickets, 1) : static_cast<int>(blockIdx.x);
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;
  const int rank = SPLIT ? *rank_slot_ptr : static_cast<int>(blockIdx.x);
  const int my_range = split.sk_ctas - 1 - rank;   // meaningful when rank < sk_ctas

  if (warp == 0 || warp == kGemmBProducerWarp) {
    // Producers: warp 0 loads the A tiles, warp 10 the B tiles, each with its own expect_tx arrival
    // on the stage's full barrier (two short issue paths instead of one long one: the reaction to
    // a freed slot is part of the ring's turnaround).  The whole warp runs the loop, one elected
    // lane issues the copies (warp-uniform code keeps the tensor-map address, the coordinates and
    // the barrier address in uniform registers).
    const bool loads_b = warp != 0;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    SegmentWalk<SPLIT> walk(split, k_blocks, rank);
    GemmSegment sg;
    while (ok && walk.next(&sg)) {
      int64_t tm, tn;
      tile_coords(sg.tile, tiles_m, tiles_n, group_m, &tm, &tn);
      const int32_t a_row = static_cast<int32_t>(tm * Cfg::kTileM);
      const int32_t b_col = static_cast<int32_t>(tn * BLOCK_N);
      for (int64_t kb = SPLIT ? sg.kb0 : 0; kb < (SPLIT ? sg.kb1 : k_blocks); ++kb) {
        ok = __all_sync(0xffffffffu, mbar_wait(empty_bar(stage), phase ^ 1u, status, kFaultProducerEmpty));
        if (!ok) break;
        const uint32_t a_dst = base + stage * Cfg::kStageBytes;
        const uint32_t b_dst = a_dst + Cfg::kAStageBytes;
        const int64_t part = kb / k_blocks_part;                 // warp-uniform
        const int32_t k0 = static_cast<int32_t>((kb - part * k_blocks_part) * Cfg::kBlockK);
        if (!loads_b) {
          const CUtensorMap* ma = (parts > 1 && part == 0) ? &tmap_a_lo : &tmap_a;
          mbar_arrive_expect_tx_elect(full_bar(stage), Cfg::kAStageBytes);
          tma_load_2d_elect(a_dst, ma, full_bar(stage), k0, a_row);
        } else {
          const CUtensorMap* mb = (parts > 1 && part == 1) ? &tmap_b_lo : &tmap_b;
          mbar_arrive_expect_tx_elect(full_bar(stage), Cfg::kBStageBytes);
          if (b_spans_map) {
            // B seen as [N / span][K][span columns]: the whole B stage is one copy
            tma_load_3d_elect(b_dst, mb, full_bar(stage), 0, k0, b_col / Cfg::kBChunkCols);
          } else {
#pragma unroll
            for (int c = 0; c < Cfg::kBChunks; ++c) {
              tma_load_2d_elect(b_dst + c * Cfg::kBChunkBytes, mb, full_bar(stage), b_col + c * Cfg::kBChunkCols, k0);
            }
          }
        }
        if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // The whole warp runs the loop and one elected lane issues: in warp-uniform code the
    // descriptors live in uniform registers, and the tensor pipe gets an instruction every 128
    // cycles (M128 x N256 x K16) instead of every 166 from a single-lane branch.
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    // A rows are KB bytes long: 128-byte swizzle with 8-row groups 1024 bytes apart, or 64-byte
    // swizzle with 8-row groups 512 bytes apart.
    const uint64_t a_desc0 = make_smem_desc(base, 16, 8 * KB, KB == 64 ? kLayoutSw64 : kLayoutSw128);
    const uint64_t b_desc0 = ELT == 2 ? make_smem_desc(base + Cfg::kAStageBytes, Cfg::kBChunkBytes, 1024, kLayoutSw128)
                                      : make_smem_desc(base + Cfg::kAStageBytes, Cfg::kBChunkBytes, 512, kLayoutSw128Base32);
    SegmentWalk<SPLIT> walk(split, k_blocks, rank);
    GemmSegment sg;
    while (ok && walk.next(&sg)) {
      // MH = 1: the tile's accumulator alternates between the two TMEM halves; MH = 2: the tile
      // uses both (rows 0-127 and 128-255), so nothing of the next tile overlaps this epilogue.
      ok = __all_sync(0xffffffffu, mbar_wait(tmem_empty_bar(MH == 2 ? 0 : acc), acc_phase ^ 1u, status, kFaultMmaTmemEmpty));
      if (MH == 2 && ok) ok = __all_sync(0xffffffffu, mbar_wait(tmem_empty_bar(1), acc_phase ^ 1u, status, kFaultMmaTmemEmpty));
      if (!ok) break;
      tcgen05_fence_after_sync();
      const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(MH == 2 ? 0 : acc * BLOCK_N);
      for (int64_t kb = SPLIT ? sg.kb0 : 0; kb < (SPLIT ? sg.kb1 : k_blocks); ++kb) {
        ok = __all_sync(0xffffffffu, mbar_wait(full_bar(stage), phase, status, kFaultMmaFull));
        if (!ok) break;
        tcgen05_fence_after_sync();
        // A: K-major, rows of 128 bytes, 8-row groups 1024 bytes apart; a K step is 32 bytes
        // further inside the swizzled row.  B: MN-major; 2-byte elements: 16-byte swizzle units,
        // 8-row K groups 1024 bytes apart; 4-byte elements: 32-byte swizzle units, 4-row K groups
        // 512 bytes apart.  Only the address field (bytes >> 4) changes between instructions, so
        // the descriptors are built once per kernel and advanced by additions.
        const uint32_t stage_units = static_cast<uint32_t>(stage * Cfg::kStageBytes) >> 4;
#pragma unroll
        for (int ks = 0; ks < Cfg::kStepsPerBlock; ++ks) {
          const uint64_t b_desc = b_desc0 + (stage_units + static_cast<uint32_t>(ks * Cfg::kBKStepBytes) / 16u);
          const uint32_t accumulate = (kb > (SPLIT ? sg.kb0 : 0) || ks > 0) ? 1u : 0u;
#pragma unroll
          for (int h = 0; h < MH; ++h) {
            const uint64_t a_desc = a_desc0 + (stage_units + static_cast<uint32_t>(h * kBlockM * KB + ks * Cfg::kUmmaKBytes) / 16u);
            const uint32_t d = d_tmem + static_cast<uint32_t>(h * BLOCK_N);
            if (ELT == 2) mma_f16_elect(d, a_desc, b_desc, idesc, accumulate);
            else mma_tf32_elect(d, a_desc, b_desc, idesc, accumulate);
          }
        }
        mma_commit_elect(empty_bar(stage));  // the slot is free once these MMAs have read it
        if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
      }
      if (!ok) break;
      if (MH == 2) {
        mma_commit_elect(tmem_full_bar(0));
        mma_commit_elect(tmem_full_bar(1));
        acc_phase ^= 1u;
      } else {
        mma_commit_elect(tmem_full_bar(acc));
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // Epilogue warps 2..9 (and 11..18 with a second group); a warp may only touch TMEM lanes
    // 32*(warp%4) .. +31, so two warps of a group share each lane quarter and split the tile's columns
    // between them.
    const int egroup = warp > kGemmBProducerWarp ? 1 : 0;
    const int ewarp = egroup == 0 ? warp - 2 : warp - (kGemmBProducerWarp + 1);
    const int quarter = warp & 3;
    const int half = ewarp >> 2;
    // MH = 1: the two warps of a lane quarter split the tile's columns; MH = 2: each drains one of
    // the two accumulators (rows 0-127 / 128-255 of the tile) over all its columns.
    constexpr int kChunksPerWarp = MH == 2 ? BLOCK_N / 32 : BLOCK_N / 64;
    int acc = MH == 2 ? half : (EG == 2 ? egroup : 0);
    uint32_t acc_phase = 0;
    int seg_index = 0;
    using View = ChunkView<T>;
    constexpr int W = View::W;
    bool vec_n = (N % W == 0) && (dest.ld % W == 0) && (dest.col0 % W == 0);
    for (int d = 0; d < dest.n; ++d) vec_n = vec_n && ((reinterpret_cast<uintptr_t>(dest.ptr[d]) & 15u) == 0);
    if (dest.tail_ptr != nullptr) {
      vec_n = vec_n && (dest.tail_ld % W == 0) && ((reinterpret_cast<uintptr_t>(dest.tail_ptr) & 15u) == 0);
    }
    const uint32_t stage_buf = bars + 512u + static_cast<uint32_t>((egroup * 8 + ewarp) * Cfg::kEpiStageBytes);
    const int pf_step = prefetch_step<EPI>(epi);
    bool ok = true;
    SegmentWalk<SPLIT> walk(split, k_blocks, rank);
    GemmSegment sg;
    while (ok && walk.next(&sg)) {
      if (EG == 2 && ((seg_index++ & 1) != egroup)) continue;   // the other group's accumulator
      int64_t tm, tn;
      tile_coords(sg.tile, tiles_m, tiles_n, group_m, &tm, &tn);
      // A segment that starts inside a tile leaves as a partial accumulator; the segment with the
      // tile's first k-blocks collects the partials of the CTAs after this one (MH = 1 only).
      const bool partial_out = SPLIT && sg.kb0 > 0;
      int n_peers = 0;
      if (SPLIT && sg.kb0 == 0 && sg.kb1 < k_blocks) {
        int64_t missing = k_blocks - sg.kb1;
        for (int peer = my_range + 1; missing > 0 && peer < split.sk_ctas; ++peer) {
          const int64_t len = split_range_begin(split, peer + 1) - split_range_begin(split, peer);
          missing -= len < missing ? len : missing;
          ++n_peers;
        }
      }
      if (!mbar_wait(tmem_full_bar(acc), acc_phase, status, kFaultEpilogueTmemFull)) { ok = false; break; }
      tcgen05_fence_after_sync();
      for (int p = 1; p <= n_peers && ok; ++p) {
        ok = split_flag_wait(split.flags + (my_range + p) * 8 + (warp - 2), status);
      }
      if (!ok) break;
      // partial tiles: float4 index ((chunk * 8 + q) * 128 + row of the tile), q = 4 columns
      float4* const my_partial = reinterpret_cast<float4*>(split.ws) +
                                 static_cast<int64_t>(my_range > 0 ? my_range : 0) * (BLOCK_N * 32) + quarter * 32 + lane;
      View g;
      g.row0 = tm * Cfg::kTileM + (MH == 2 ? half * kBlockM : 0) + quarter * 32;
      g.sub_row = lane / View::LPR;
      g.M = M;
      g.N = N;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(acc * BLOCK_N);
#pragma unroll 1
      for (int c = (MH == 2 ? 0 : half * kChunksPerWarp); c < (MH == 2 ? kChunksPerWarp : (half + 1) * kChunksPerWarp); ++c) {
        const int64_t col0 = tn * BLOCK_N + c * 32;
        if (col0 >= N) break;  // warp-uniform
        g.col = col0 + (lane % View::LPR) * W;
        g.vec = vec_n && col0 + 32 <= N;
        // The chain's full-shape operand (a Linear bias, a residual) does not depend on the
        // accumulator: its loads go out first and are in flight during the TMEM read and the
        // transposition; the next chunk's lines are pulled into L2 meanwhile.
        Vec16<T> pre[View::P];
        int pre_step = -1;
        if (!partial_out && pf_step >= 0 && g.vec && g.row0 < M && (reinterpret_cast<uintptr_t>(epi.operands[pf_step]) & 15u) == 0) {
          pre_step = pf_step;
          const T* opnd = static_cast<const T*>(epi.operands[pf_step]);
#pragma unroll
          for (int j = 0; j < View::P; ++j) {
            const int64_t row = g.row(j) < M ? g.row(j) : M - 1;
            const T* src = opnd + row * N + g.col;
            pre[j] = *reinterpret_cast<const Vec16<T>*>(src);
            if (col0 + 64 <= N) asm volatile("prefetch.global.L2 [%0];" ::"l"(src + 32));
          }
        }
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + static_cast<uint32_t>(c * 32), r);
        tmem_ld_wait();
        if (g.row0 >= M) continue;  // warp-uniform: the whole 32-row band lies below the matrix
        if constexpr (SPLIT) {
          if (partial_out) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              __stcg(my_partial + (c * 8 + q) * 128,
                     make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                 __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3])));
            }
            continue;
          }
          for (int p = 1; p <= n_peers; ++p) {   // fixed order: the result does not depend on timing
            const float4* src = my_partial + static_cast<int64_t>(p) * (BLOCK_N * 32) + c * 8 * 128;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const float4 t = __ldcg(src + q * 128);
              r[4 * q] = __float_as_uint(__uint_as_float(r[4 * q]) + t.x);
              r[4 * q + 1] = __float_as_uint(__uint_as_float(r[4 * q + 1]) + t.y);
              r[4 * q + 2] = __float_as_uint(__uint_as_float(r[4 * q + 2]) + t.z);
              r[4 * q + 3] = __float_as_uint(__uint_as_float(r[4 * q + 3]) + t.w);
            }
          }
        }
        float v[32];
        transpose_chunk<T>(r, v, stage_buf, lane);
        apply_chain<T, EPI>(epi, v, g, pre, pre_step);
        const bool tail = dest.tail_ptr != nullptr && col0 >= dest.tail_col;   // warp-uniform
        const int64_t dst_ld = tail ? dest.tail_ld : dest.ld;
        for (int d = 0; d < dest.n; ++d) {
          T* base_dst = tail ? static_cast<T*>(dest.tail_ptr) + (g.col - dest.tail_col)
                             : static_cast<T*>(dest.ptr[d]) + dest.col0 + g.col;
#pragma unroll
          for (int j = 0; j < View::P; ++j) {
            const int64_t row = g.row(j);
            if (row >= M) continue;
            T* dst = base_dst + row * dst_ld;
            if (g.vec) {
              float o[W];
#pragma unroll
              for (int e = 0; e < W; ++e) o[e] = v[j * W + e];
              store_vec<T>(dst, o);
            } else {
#pragma unroll
              for (int e = 0; e < W; ++e) {
                if (g.col + e < N) dst[e] = from_f32<T>(v[j * W + e]);
              }
            }
          }
        }
      }
      if (SPLIT && n_peers > 0 && lane == 0) {
        // consumed: the flags are zero again when the launch ends
        for (int p = 1; p <= n_peers; ++p) split.flags[(my_range + p) * 8 + (warp - 2)] = 0;
      }
      if (SPLIT && partial_out) {
        __threadfence();   // every lane's share of the partial tile is visible before the flag
        __syncwarp();
        if (lane == 0) {
          int* flag = split.flags + my_range * 8 + (warp - 2);
          asm volatile("st.release.gpu.global.b32 [%0], %1;" ::"l"(flag), "r"(1) : "memory");
        }
      }
      tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty_bar(acc));
      if (MH == 2 || EG == 2) {
        acc_phase ^= 1u;
      } else if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
  }

  // Common exit: every role arrives here, on success or after a bounded wait gave up.
  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  if (SPLIT && threadIdx.x == 0) {
    // the last CTA to leave puts the tickets back to zero for the next launch on this stream
    if (atomicAdd(split.tickets + 1, 1) == static_cast<int>(gridDim.x) - 1) {
      split.tickets[0] = 0;
      split.tickets[1] = 0;
    }
  }
}

// ---- host side ----------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    (void)cudaGetLastError();
  });
  return fn;
}

// 2-D row-major tensor [rows, cols] of `elt`-byte elements; box = 128 bytes x box_rows,
// 128-byte swizzle (16-byte units, or 32-byte units for an MN-major 32-bit operand), zero fill
// outside the tensor.
int make_tmap_2d(CUtensorMap* map, const void* ptr, int dtype, int64_t rows, int64_t cols,
                 int box_rows, bool swizzle_32b_units) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return set_error(FB200_DEVICE_ERROR, "cuTensorMapEncodeTiled is not available");
  const int elt = itemsize_of(dtype);
  CUtensorMapDataType dt = dtype == FB200_F32    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                           : dtype == FB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  cuuint64_t gdim[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t gstride[1] = {static_cast<cuuint64_t>(cols) * elt};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / elt), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle_32b_units ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    return set_error(FB200_INTERNAL, "cuTensorMapEncodeTiled failed with code %d (rows %lld cols %lld)",
                     static_cast<int>(r), (long long)rows, (long long)cols);
  }
  return FB200_OK;
}

// 2-D row-major tensor [rows, cols]; box = row_bytes (128 or 64) x box_rows with the swizzle of that
// width (16-byte units): the K-major A operand.
int make_tmap_rows(CUtensorMap* map, const void* ptr, int dtype, int64_t rows, int64_t cols, int box_rows,
                   int row_bytes) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return set_error(FB200_DEVICE_ERROR, "cuTensorMapEncodeTiled is not available");
  const int elt = itemsize_of(dtype);
  CUtensorMapDataType dt = dtype == FB200_F32    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                           : dtype == FB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  cuuint64_t gdim[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t gstride[1] = {static_cast<cuuint64_t>(cols) * elt};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(row_bytes / elt), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt, 2, const_cast<void*>(ptr), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    return set_error(FB200_INTERNAL, "cuTensorMapEncodeTiled failed with code %d (rows %lld cols %lld)",
                     static_cast<int>(r), (long long)rows, (long long)cols);
  }
  return FB200_OK;
}

// The B operand [k, n] (row-major, n a multiple of the 128-byte span) seen as
// [n / span][k][span columns]: one box of `spans` x box_k x span elements is a whole B stage, written
// to shared memory span after span, i.e. what `spans` 2-D copies of 128-byte-wide boxes would write.
int make_tmap_b_spans(CUtensorMap* map, const void* ptr, int dtype, int64_t k, int64_t n, int box_k,
                      int spans, bool swizzle_32b_units) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return set_error(FB200_DEVICE_ERROR, "cuTensorMapEncodeTiled is not available");
  const int elt = itemsize_of(dtype);
  const int span = 128 / elt;
  CUtensorMapDataType dt = dtype == FB200_F32    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                           : dtype == FB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  cuuint64_t gdim[3] = {static_cast<cuuint64_t>(span), static_cast<cuuint64_t>(k),
                        static_cast<cuuint64_t>(n / span)};
  cuuint64_t gstride[2] = {static_cast<cuuint64_t>(n) * elt, static_cast<cuuint64_t>(span) * elt};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(span), static_cast<cuuint32_t>(box_k), static_cast<cuuint32_t>(spans)};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, dt, 3, const_cast<void*>(ptr), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle_32b_units ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    return set_error(FB200_INTERNAL, "cuTensorMapEncodeTiled (B spans) failed with code %d (k %lld n %lld)",
                     static_cast<int>(r), (long long)k, (long long)n);
  }
  return FB200_OK;
}

// Row-major fp32 tensor [n, c, h, w] with a box of [1, box_c, box_h, box_w] elements, no swizzle: the
// halo tile of a convolution lands in shared memory as plain [box_c][box_h][box_w].  w must be a
// multiple of 4 elements (strides are multiples of 16 bytes) and box_w too.
int make_tmap_nchw_f32(CUtensorMap* map, const void* ptr, int64_t n, int64_t c, int64_t h, int64_t w,
                       int box_c, int box_h, int box_w) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return set_error(FB200_DEVICE_ERROR, "cuTensorMapEncodeTiled is not available");
  cuuint64_t gdim[4] = {static_cast<cuuint64_t>(w), static_cast<cuuint64_t>(h), static_cast<cuuint64_t>(c),
                        static_cast<cuuint64_t>(n)};
  cuuint64_t gstride[3] = {static_cast<cuuint64_t>(w) * 4, static_cast<cuuint64_t>(w * h) * 4,
                           static_cast<cuuint64_t>(w * h * c) * 4};
  cuuint32_t box[4] = {static_cast<cuuint32_t>(box_w), static_cast<cuuint32_t>(box_h),
                       static_cast<cuuint32_t>(box_c), 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(ptr), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    return set_error(FB200_INTERNAL, "cuTensorMapEncodeTiled (nchw) failed with code %d", static_cast<int>(r));
  }
  return FB200_OK;
}

// Per-device status word the kernels write when a bounded wait gives up (host-mapped, so the
// host can read it after a stream synchronise without a copy).
struct StatusWord { int* host = nullptr; int* dev = nullptr; };
static StatusWord g_status[16];
static std::mutex g_status_mu;

int device_status_word(int** dev_ptr) {
  int device = 0;
  FB200_CUDA_OK(cudaGetDevice(&device));
  if (device < 0 || device >= 16) return set_error(FB200_INVALID_ARGUMENT, "device index %d", device);
  std::lock_guard<std::mutex> lock(g_status_mu);
  if (g_status[device].host == nullptr) {
    int* h = nullptr;
    FB200_CUDA_OK(cudaHostAlloc(&h, sizeof(int), cudaHostAllocMapped));
    *h = 0;
    int* d = nullptr;
    FB200_CUDA_OK(cudaHostGetDevicePointer(&d, h, 0));
    g_status[device].host = h;
    g_status[device].dev = d;
  }
  *dev_ptr = g_status[device].dev;
  return FB200_OK;
}

// Scratch of a split launch: 8 flags per CTA, then one fp32 partial tile of 128 x 256 per CTA.  Kept
// per (device, stream): launches on one stream run one after the other, so they can share it, and
// the owners clear every flag they have consumed, so it is all zeros between launches (after a
// launch that gave up, the status word is set and the flags are cleared here).  More than eight
// streams at a time: stream-ordered scratch, cleared per launch.
constexpr size_t kSplitFlagBytes = 8192;   // 148 * 8 flags, then (at kSplitTicketOffset) two tickets
constexpr size_t kSplitTicketOffset = 6144;
constexpr size_t kSplitBytes = kSplitFlagBytes + size_t(kNumSMs) * 256 * kBlockM * sizeof(float);
struct SplitWorkspace { int device = -1; cudaStream_t stream = nullptr; uint8_t* ptr = nullptr; uint64_t clean_at = 0; };
static SplitWorkspace g_split_ws[8];
static std::mutex g_split_mu;
static uint64_t g_fault_epoch = 0;   // counts the times a kernel was seen to have given up (under g_split_mu)

static int split_workspace(cudaStream_t s, uint8_t** out, bool* pooled) {
  int device = 0;
  FB200_CUDA_OK(cudaGetDevice(&device));
  *pooled = false;
  {
    std::lock_guard<std::mutex> lock(g_split_mu);
    SplitWorkspace* slot = nullptr;
    for (auto& w : g_split_ws) {
      if (w.ptr != nullptr && w.device == device && w.stream == s) { slot = &w; break; }
    }
    if (slot == nullptr) {
      for (auto& w : g_split_ws) if (w.ptr == nullptr) { slot = &w; break; }
      if (slot != nullptr) {
        uint8_t* p = nullptr;
        FB200_CUDA_OK(cudaMalloc(reinterpret_cast<void**>(&p), kSplitBytes));
        FB200_CUDA_OK(cudaMemset(p, 0, kSplitFlagBytes));
        slot->device = device;
        slot->stream = s;
        slot->ptr = p;
        slot->clean_at = g_fault_epoch;
      }
    }
    if (slot != nullptr) {
      const StatusWord& sw = g_status[device < 16 ? device : 0];
      if (sw.host != nullptr && *reinterpret_cast<volatile int*>(sw.host) != 0) ++g_fault_epoch;
      if (slot->clean_at != g_fault_epoch) {
        // a kernel gave up since this workspace was last known clean: flags or tickets may be left set
        FB200_CUDA_OK(cudaMemsetAsync(slot->ptr, 0, kSplitFlagBytes, s));
        slot->clean_at = g_fault_epoch;
      }
      *out = slot->ptr;
      return FB200_OK;
    }
  }
  uint8_t* p = nullptr;
  FB200_CUDA_OK(scratch_alloc_async(reinterpret_cast<void**>(&p), kSplitBytes, s));
  FB200_CUDA_OK(cudaMemsetAsync(p, 0, kSplitFlagBytes, s));
  *pooled = true;
  *out = p;
  return FB200_OK;
}

// Decides whether the tiles' k-blocks are split over more CTAs than there are tiles.  Measured on
// B200 (back-to-back launches, CUDA events): with more than about a quarter of the SMs busy the
// mainloop is bound by what the L2 can deliver to all SMs together, not by any one SM, so spreading a
// partial last wave over the idle SMs moves the same bytes in the same time and only adds the
// partial tiles' round trip (4096 x 1024 x 4096 bf16: 39.6 us as 128 whole tiles on 128 SMs, 47.7 us
// split over 148; 2048 x 8192 x 8192: 212 -> 196 us, but 185 us on 256 x 256 tiles).  It pays when a
// few tiles carry a long K (a quarter of the SMs or fewer, 128 k-blocks or more): the weight-gradient
// shape, out[in, out] summed over all tokens (768 x 1024 x 32768 TF32: 370 -> 165 us; 128 x 256 x
// 65536 bf16: 365 -> 70 us; 256 x 512 x 8192: 52 -> 32 us; at 64 k-blocks it saved nothing).  Ranges
// are at least an eighth of a tile's k-blocks, so an owner adds at most eight partial tiles.
constexpr int64_t kSplitMaxTiles = kNumSMs / 4;
constexpr int64_t kSplitMinKBlocks = 128;
static GemmSplit plan_split(int64_t tiles, int64_t k_blocks, int mh) {
  GemmSplit sp{};
  sp.dp_tiles = tiles;
  if (mh != 1 || k_blocks < kSplitMinKBlocks) return sp;
  if (tiles <= kSplitMaxTiles) {
    const int64_t units = tiles * k_blocks;
    const int64_t min_range = k_blocks / 8 > 8 ? k_blocks / 8 : 8;
    const int64_t ctas = units / min_range < kNumSMs ? units / min_range : kNumSMs;
    if (ctas < 2 * tiles) return sp;
    sp.dp_tiles = 0;
    sp.sk_units = units;
    sp.sk_ctas = static_cast<int>(ctas);
    return sp;
  }
  // Whole waves followed by a light last wave (the 2048-row shard of an 8192^3 product: 3.46 waves of
  // 148 tiles) are NOT split: dealing the last wave's k-blocks out to all SMs measured 212 -> 196 us
  // for the plain product, which 256 x 256 tiles beat anyway (185 us), and nothing with a bias + GELU
  // epilogue (0.2418 against 0.2403 ms per shard).
  return sp;
}

// Two epilogue groups pay when the mainloop of a tile is shorter than its epilogue and every SM has
// several tiles to alternate between.
// (Measured: dt_proj + bias + softplus, K = 48, 0.101 -> 0.084 ms; at 16 k-blocks, the K = 1024 GEMMs
// of the transformer block, the lost ring stage costs more than the second group gains: 0.050 ->
// 0.054 ms.)
static bool two_epilogue_groups(int64_t tiles, int64_t k_blocks) {
  return k_blocks <= 4 && tiles >= 2 * kNumSMs;
}

template <typename T, int ELT, int BLOCK_N, int MH, int KB, int EPI>
static int launch_tc_epi(const void* a, const void* b, const GemmDest& c, int64_t m, int64_t n, int64_t k,
                         int dtype, const EpilogueDev& epi, cudaStream_t s) {
  using Cfg = GemmCfg<ELT, BLOCK_N, MH, KB>;
  CUtensorMap ta, tb;
  if (int rc = make_tmap_rows(&ta, a, dtype, m, k, Cfg::kTileM, KB)) return rc;
  // one copy per B stage when n is a whole number of 128-byte spans (else the last span would run
  // into the next row), `kBChunks` copies of one span otherwise
  const int b_spans_map = (n % Cfg::kBChunkCols == 0 && Cfg::kBChunks > 1) ? 1 : 0;
  if (b_spans_map) {
    if (int rc = make_tmap_b_spans(&tb, b, dtype, k, n, Cfg::kBlockK, Cfg::kBChunks, ELT == 4)) return rc;
  } else {
    if (int rc = make_tmap_2d(&tb, b, dtype, k, n, Cfg::kBlockK, ELT == 4)) return rc;
  }
  CUtensorMap ta_lo = ta, tb_lo = tb;
  const int parts = (c.a_lo != nullptr && c.b_lo != nullptr) ? 3 : 1;
  if (parts == 3) {
    if (int rc = make_tmap_rows(&ta_lo, c.a_lo, dtype, m, k, Cfg::kTileM, KB)) return rc;
    if (b_spans_map) {
      if (int rc = make_tmap_b_spans(&tb_lo, c.b_lo, dtype, k, n, Cfg::kBlockK, Cfg::kBChunks, ELT == 4)) return rc;
    } else {
      if (int rc = make_tmap_2d(&tb_lo, c.b_lo, dtype, k, n, Cfg::kBlockK, ELT == 4)) return rc;
    }
  }
  int* status = nullptr;
  if (int rc = device_status_word(&status)) return rc;
  const uint32_t fmt = dtype == FB200_F32 ? kFmtTF32 : (dtype == FB200_BF16 ? kFmtBF16 : kFmtF16);
  const uint32_t idesc = make_instr_desc(fmt, /*a MN-major*/ 0, /*b MN-major*/ 1, kBlockM, BLOCK_N);
  const int64_t tiles = ((m + Cfg::kTileM - 1) / Cfg::kTileM) * ((n + BLOCK_N - 1) / BLOCK_N);
  const int64_t k_blocks = ((k + Cfg::kBlockK - 1) / Cfg::kBlockK) * parts;
  GemmSplit split{};
  split.dp_tiles = tiles;
  // The split form exists for 128 x 256 tiles with a plain store or the interpreted chain.
  constexpr bool kCanSplit = MH == 1 && BLOCK_N == 256 && (EPI == kEpiNone || EPI == kEpiGeneric);
  if constexpr (kCanSplit) {
    const GemmSplit planned = plan_split(tiles, k_blocks, MH);
    if (planned.sk_units > 0) {
      // One partial-tile slot and eight flags per range, from this stream's persistent workspace (or
      // stream-ordered scratch when the table is full); one CTA per SM.
      split = planned;
      auto kernel = gemm_tcgen05_kernel<T, ELT, BLOCK_N, MH, KB, EPI, true>;
      FB200_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(Cfg::kSmemBytes)));
      uint8_t* scratch = nullptr;
      bool pooled = false;
      if (int rc = split_workspace(s, &scratch, &pooled)) return rc;
      split.flags = reinterpret_cast<int*>(scratch);
      split.ws = reinterpret_cast<float*>(scratch + kSplitFlagBytes);
      split.tickets = reinterpret_cast<int*>(scratch + kSplitTicketOffset);
      kernel<<<kNumSMs, kGemmThreads, Cfg::kSmemBytes, s>>>(ta, tb, ta_lo, tb_lo, parts, b_spans_map, c, m, n, k,
                                                             idesc, epi, split, status);
      const int rc = after_launch("gemm_tcgen05_kernel");
      if (pooled) cudaFreeAsync(scratch, s);
      return rc;
    }
  }
  const int grid = static_cast<int>(tiles < kNumSMs ? tiles : kNumSMs);
  // Products that are all epilogue (a K of a few k-blocks under a wide result: Mamba's dt_proj, K = 48)
  // take the form with two epilogue groups.
  if constexpr (MH == 1 && BLOCK_N == 256 && KB == 128 && !std::is_same<T, __half>::value) {
    if (two_epilogue_groups(tiles, k_blocks)) {
      using Cfg2 = GemmCfg<ELT, BLOCK_N, MH, KB, 2>;
      auto kernel2 = gemm_tcgen05_kernel<T, ELT, BLOCK_N, MH, KB, EPI, false, 2>;
      FB200_CUDA_OK(cudaFuncSetAttribute(kernel2, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(Cfg2::kSmemBytes)));
      kernel2<<<grid, Cfg2::kThreads, Cfg2::kSmemBytes, s>>>(ta, tb, ta_lo, tb_lo, parts, b_spans_map, c, m, n, k, idesc,
                                                              epi, split, status);
      return after_launch("gemm_tcgen05_kernel");
    }
  }
  auto kernel = gemm_tcgen05_kernel<T, ELT, BLOCK_N, MH, KB, EPI, false>;
  FB200_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(Cfg::kSmemBytes)));
  kernel<<<grid, kGemmThreads, Cfg::kSmemBytes, s>>>(ta, tb, ta_lo, tb_lo, parts, b_spans_map, c, m, n, k, idesc,
                                                      epi, split, status);
  return after_launch("gemm_tcgen05_kernel");
}

// Picks the kernel instantiated for this epilogue chain; 16-bit float (f16) tensors and 256 x 256
// tiles (light epilogues only) keep to the plain store and the interpreter.
template <typename T, int ELT, int BLOCK_N, int MH = 1, int KB = 128>
static int launch_tc(const void* a, const void* b, const GemmDest& c, int64_t m, int64_t n, int64_t k,
                     int dtype, const EpilogueDev& epi, cudaStream_t s) {
  const int kind = classify_epilogue(epi);
  if (kind == kEpiNone) return launch_tc_epi<T, ELT, BLOCK_N, MH, KB, kEpiNone>(a, b, c, m, n, k, dtype, epi, s);
  bool split_planned = false;   // split products take the interpreted chain
  if constexpr (MH == 1 && BLOCK_N == 256) {
    const int parts = (c.a_lo != nullptr && c.b_lo != nullptr) ? 3 : 1;
    const int64_t tiles = ((m + kBlockM - 1) / kBlockM) * ((n + BLOCK_N - 1) / BLOCK_N);
    split_planned = plan_split(tiles, ((k * ELT + KB - 1) / KB) * parts, MH).sk_units > 0;
  }
  if constexpr (MH == 1 && !std::is_same<T, __half>::value) {
    if (!split_planned) switch (kind) {
      case kEpiAddFullGelu: return launch_tc_epi<T, ELT, BLOCK_N, MH, KB, kEpiAddFullGelu>(a, b, c, m, n, k, dtype, epi, s);
      case kEpiAddColSoftplus: return launch_tc_epi<T, ELT, BLOCK_N, MH, KB, kEpiAddColSoftplus>(a, b, c, m, n, k, dtype, epi, s);
      case kEpiGelu: return launch_tc_epi<T, ELT, BLOCK_N, MH, KB, kEpiGelu>(a, b, c, m, n, k, dtype, epi, s);
      case kEpiAddFull: return launch_tc_epi<T, ELT, BLOCK_N, MH, KB, kEpiAddFull>(a, b, c, m, n, k, dtype, epi, s);
      default: break;
    }
  }
  return launch_tc_epi<T, ELT, BLOCK_N, MH, KB, kEpiGeneric>(a, b, c, m, n, k, dtype, epi, s);
}

// Tile shape for a product: BLOCK_N in {64, 128, 256} and MH (1: 128-row tiles, 2: 256 x 256).
struct TileChoice { int block_n, mh; };
static TileChoice choose_tile(int64_t m, int64_t n, int64_t k, int elt, int parts, bool light) {
  const int64_t tiles_m = (m + kBlockM - 1) / kBlockM;
  auto tiles = [&](int bn) { return tiles_m * ((n + bn - 1) / bn); };
  if (n > 128 && tiles(256) >= kNumSMs) {
    // 256 x 256 tiles (two M halves per B stage) need a third less operand traffic from L2 per FLOP
    // (8192^3 bf16: 1418 -> 1509 TFLOP/s, TF32 4096^3: 622 -> 690), but the tile fills TMEM, so its
    // epilogue no longer overlaps the next mainloop: a transcendental epilogue (GELU over 64 Ki
    // elements is about 18 K issue cycles per tile) costs more than the traffic saves.  They are
    // taken for chains of adds, multiplies and ReLU over a long K, when the waves of tiles do not get
    // longer by more than an eighth.
    const int64_t t2 = ((m + 255) / 256) * ((n + 255) / 256);
    const int64_t waves1 = (tiles(256) + kNumSMs - 1) / kNumSMs, waves2 = (t2 + kNumSMs - 1) / kNumSMs;
    // The exposed epilogue costs about 8-10 K cycles per tile against a gain of 6-11 % of the mainloop:
    // for 16-bit operands only worth it from 128 k-blocks per tile on (39-68 us against 35-46 us at
    // K = 1024 bf16); fp32 k-blocks take twice as long per byte of K, and there it pays from K = 768
    // (32768 x 768 x 1536 TF32: 139 -> 131 us, 32768 x 3072 x 768: 269 -> 259 us).
    const int64_t min_k_bytes = elt == 4 ? 3072 : 128 * 128;
    if (light && m > 128 && k * elt >= min_k_bytes && t2 >= kNumSMs && 16 * waves2 <= 9 * waves1) return {256, 2};
    return {256, 1};
  }
  // One wave of 128 x 256 tiles beats two waves of 128 x 128 (4096 x 1024 x 4096 bf16: 39.6 against
  // 58.0 us; 4096 x 1024 x 1024: 16.9 against 21.0 us): wide tiles move a third less operand data per
  // FLOP through the L2.  A few tiles with a long K are split over the SMs (plan_split).
  const int64_t k_blocks = ((k * elt + 127) / 128) * parts;
  if (n > 128 && (tiles(128) > kNumSMs || plan_split(tiles(256), k_blocks, 1).sk_units > 0)) return {256, 1};
  if (n > 64 && tiles(128) >= kNumSMs) return {128, 1};
  if (n > 128 && tiles(64) < kNumSMs / 2) return {128, 1};
  return {64, 1};
}

template <typename T, int ELT>
static int launch_tc_n(const void* a, const void* b, const GemmDest& c, int64_t m, int64_t n, int64_t k,
                       int dtype, const EpilogueDev& epi, cudaStream_t s) {
  const int parts = (c.a_lo != nullptr && c.b_lo != nullptr) ? 3 : 1;
  const TileChoice t = choose_tile(m, n, k, ELT, parts, light_epilogue(epi));
  if (t.mh == 2) return launch_tc<T, ELT, 256, 2>(a, b, c, m, n, k, dtype, epi, s);
  if (t.block_n == 256) return launch_tc<T, ELT, 256>(a, b, c, m, n, k, dtype, epi, s);
  if (t.block_n == 128) return launch_tc<T, ELT, 128>(a, b, c, m, n, k, dtype, epi, s);
  return launch_tc<T, ELT, 64>(a, b, c, m, n, k, dtype, epi, s);
}

// x_lo = x - trunc_tf32(x): what the tensor core drops when it reads an fp32 operand as TF32 (it
// truncates: the low 13 mantissa bits are ignored).  Exact in fp32.
__global__ void __launch_bounds__(256)
tf32_low_part_kernel(const float4* __restrict__ x, float4* __restrict__ lo, int64_t n_vec) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
    const float4 v = x[i];
    float4 r;
    r.x = v.x - __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u);
    r.y = v.y - __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u);
    r.z = v.z - __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u);
    r.w = v.w - __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u);
    lo[i] = r;
  }
}

// Strict fp32 products from this many multiply-adds on run on the tensor cores with error
// compensation instead of on the CUDA cores (about 0.1 ms of the SIMT kernel).
constexpr int64_t kCompensatedMinMacs = int64_t(1) << 30;

static bool tensor_core_eligible(const void* a, const void* b, const void* c, int64_t m, int64_t n,
                                 int64_t k, int dtype, int allow_tf32) {
  (void)m;
  const int elt = itemsize_of(dtype);
  if (dtype == FB200_F32 && !allow_tf32) return false;
  if (dtype != FB200_F32 && dtype != FB200_BF16 && dtype != FB200_F16) return false;
  // TMA: 16-byte aligned base and row pitch; coordinates must fit int32.
  if ((k * elt) % 16 != 0 || (n * elt) % 16 != 0) return false;
  if (a != nullptr && !aligned16(a)) return false;
  if (b != nullptr && !aligned16(b)) return false;
  (void)c;
  if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX) return false;
  return true;
}

}  // namespace fb200

using namespace fb200;

extern "C" int fb200_matmul_uses_tensor_cores(int64_t m, int64_t n, int64_t k, int dtype,
                                              int allow_tf32) {
  return tensor_core_eligible(nullptr, nullptr, nullptr, m, n, k, dtype, allow_tf32) ? 1 : 0;
}

// How fb200_matmul would run a tensor-core product: out = {BLOCK_N, tile rows, tiles walked whole,
// k-blocks dealt out in ranges, CTAs that take a range, k-blocks per tile}.  `light_epilogue`: the
// chain is adds, multiplies and ReLU only.  `compensated`: the three-pass strict fp32 form.
extern "C" int fb200_matmul_schedule(int64_t m, int64_t n, int64_t k, int dtype, int light_epilogue_chain,
                                     int compensated, int64_t* out6) {
  if (out6 == nullptr || m < 1 || n < 1 || k < 1) return set_error(FB200_INVALID_ARGUMENT, "matmul_schedule: invalid argument");
  if (!tensor_core_eligible(nullptr, nullptr, nullptr, m, n, k, dtype, 1)) {
    return set_error(FB200_UNIMPLEMENTED, "matmul_schedule: not a tensor-core shape");
  }
  const int elt = itemsize_of(dtype), parts = compensated ? 3 : 1;
  const TileChoice t = choose_tile(m, n, k, elt, parts, light_epilogue_chain != 0);
  const int64_t tile_m = kBlockM * t.mh;
  const int64_t tiles = ((m + tile_m - 1) / tile_m) * ((n + t.block_n - 1) / t.block_n);
  const int64_t k_blocks = ((k * elt + 127) / 128) * parts;
  const GemmSplit sp = plan_split(tiles, k_blocks, t.mh);
  out6[0] = t.block_n;
  out6[1] = tile_m;
  out6[2] = sp.dp_tiles;
  out6[3] = sp.sk_units;
  out6[4] = sp.sk_ctas;
  out6[5] = k_blocks;
  return FB200_OK;
}

static int matmul_impl(const void* a, const void* b, void* c, void* c_tail, int64_t tail_col, int64_t m,
                       int64_t n, int64_t k, int dtype, int allow_tf32, const fb200_epilogue* epilogue,
                       fb200_stream stream, const char* who) {
  if (m < 0 || n < 0 || k < 0) return set_error(FB200_INVALID_ARGUMENT, "%s: negative dimension", who);
  if (!is_float_dtype(dtype)) {
    return set_error(FB200_INVALID_ARGUMENT,
                     "%s: dtype code %d is not float32/float16/bfloat16", who, dtype);
  }
  if (m == 0 || n == 0) return FB200_OK;
  if (c == nullptr || (k > 0 && (a == nullptr || b == nullptr))) {
    return set_error(FB200_INVALID_ARGUMENT, "%s: null argument", who);
  }
  EpilogueDev epi{};
  if (int rc = make_epilogue(epilogue, &epi, who)) return rc;
  cudaStream_t s = as_stream(stream);
  const bool exact_order = allow_tf32 < 0;   // the CPU reference's order of additions, whatever the size
  if (exact_order) allow_tf32 = 0;
  // Strict fp32 (allow_tf32 == 0) of a size worth it: three TF32 products with the operands' low
  // parts ("3xTF32") at about a third of the TF32 rate.  Operand rounding is gone; the error left is
  // the tensor core's truncating fp32 accumulation (about 2^-23 * K/8 of the result's scale).
  const bool compensated = dtype == FB200_F32 && allow_tf32 == 0 && !exact_order && k > 0 && m * n >= 128 * 128 &&
                           m * n * k >= kCompensatedMinMacs && (m * k) % 4 == 0 && (k * n) % 4 == 0 &&
                           tensor_core_eligible(a, b, c, m, n, k, dtype, 1);
  if (k > 0 && (compensated || tensor_core_eligible(a, b, c, m, n, k, dtype, allow_tf32))) {
    GemmDest dest{};
    dest.group_m = kGemmGroupM;
    dest.ptr[0] = c;
    dest.n = 1;
    dest.ld = n;
    dest.col0 = 0;
    dest.tail_ptr = c_tail;
    dest.tail_col = tail_col;
    dest.tail_ld = n - tail_col;
    if (compensated) {
      float* lo = nullptr;
      const size_t na = static_cast<size_t>(m) * k, nb = static_cast<size_t>(k) * n;
      FB200_CUDA_OK(scratch_alloc_async(reinterpret_cast<void**>(&lo), (na + nb) * sizeof(float), s));
      tf32_low_part_kernel<<<grid_for(na / 4, 256, 8), 256, 0, s>>>(static_cast<const float4*>(a), reinterpret_cast<float4*>(lo), na / 4);
      int rc = after_launch("tf32_low_part_kernel");
      if (rc == FB200_OK) {
        tf32_low_part_kernel<<<grid_for(nb / 4, 256, 8), 256, 0, s>>>(static_cast<const float4*>(b), reinterpret_cast<float4*>(lo + na), nb / 4);
        rc = after_launch("tf32_low_part_kernel");
      }
      if (rc == FB200_OK) {
        dest.a_lo = lo;
        dest.b_lo = lo + na;
        rc = launch_tc_n<float, 4>(a, b, dest, m, n, k, dtype, epi, s);
      }
      cudaFreeAsync(lo, s);
      return rc;
    }
    switch (dtype) {
      case FB200_F32: return launch_tc_n<float, 4>(a, b, dest, m, n, k, dtype, epi, s);
      case FB200_BF16: return launch_tc_n<__nv_bfloat16, 2>(a, b, dest, m, n, k, dtype, epi, s);
      default: return launch_tc_n<__half, 2>(a, b, dest, m, n, k, dtype, epi, s);
    }
  }
  if (c_tail != nullptr) {
    return set_error(FB200_UNIMPLEMENTED, "%s: the split result needs a tensor-core shape "
                     "(fb200_matmul_uses_tensor_cores)", who);
  }
  return gemm_simt(a, b, c, m, n, k, dtype, epi, s);
}

extern "C" int fb200_matmul(const void* a, const void* b, void* c, int64_t m, int64_t n,
                            int64_t k, int dtype, int allow_tf32, const fb200_epilogue* epilogue,
                            fb200_stream stream) {
  return matmul_impl(a, b, c, nullptr, 0, m, n, k, dtype, allow_tf32, epilogue, stream, "matmul");
}

// matmul whose result leaves in two pieces: columns [0, tail_col) into `c` (row pitch n, as
// fb200_matmul writes them; the columns from tail_col on are left untouched there) and columns
// [tail_col, n) into the dense matrix `c_tail` [m, n - tail_col].  For graphs that read a column
// block of a projection only through a `slice` (the gate half of Mamba's in_proj): the block lands
// where the slice would have copied it and the copy disappears.  tail_col must be a multiple of 32
// and the shape a tensor-core one.
extern "C" int fb200_matmul_split(const void* a, const void* b, void* c, void* c_tail, int64_t tail_col,
                                  int64_t m, int64_t n, int64_t k, int dtype, int allow_tf32,
                                  const fb200_epilogue* epilogue, fb200_stream stream) {
  if (c_tail == nullptr || tail_col <= 0 || tail_col >= n || tail_col % 32 != 0) {
    return set_error(FB200_INVALID_ARGUMENT,
                     "matmul_split: tail_col %lld must be a multiple of 32 inside (0, n) and c_tail non-null",
                     static_cast<long long>(tail_col));
  }
  return matmul_impl(a, b, c, c_tail, tail_col, m, n, k, dtype, allow_tf32, epilogue, stream, "matmul_split");
}

// Reads and clears the per-device kernel status word: 0 = no bounded wait has given up.
extern "C" int fb200_kernel_status(int device, int* code) {
  if (code == nullptr) return set_error(FB200_INVALID_ARGUMENT, "fb200_kernel_status: null out");
  *code = 0;
  if (device < 0 || device >= 16) return set_error(FB200_INVALID_ARGUMENT, "device index %d", device);
  std::lock_guard<std::mutex> lock(g_status_mu);
  if (g_status[device].host != nullptr) {
    *code = *reinterpret_cast<volatile int*>(g_status[device].host);
    if (*code != 0) {
      std::lock_guard<std::mutex> lock(g_split_mu);
      ++g_fault_epoch;   // split workspaces clear their flags before their next launch
    }
    *g_status[device].host = 0;
  }
  return FB200_OK;
}

// Column-split matmul with the all-gather of C fused into the epilogue.  This rank multiplies A
// [m,k] by its own column block of B (`b_local`, [k, n_local], contiguous) and stores
// epilogue(A.B_local) into columns [col0, col0+n_local) of every destination matrix in `c_dest`
// (row pitch n_total): its own copy of C and its peers' copies, mapped into this process with
// fb200_ipc_import.  Peer stores are ordinary global stores that travel over NVLink; when every
// rank has finished (stream synchronise + a host-side barrier) each GPU holds the whole C.
// Epilogue operands are indexed in the local [m, n_local] layout.  Tensor-core shapes only.
extern "C" int fb200_matmul_colsplit(const void* a, const void* b_local, void* const* c_dest,
                                     int n_dest, int64_t m, int64_t n_local, int64_t n_total,
                                     int64_t col0, int64_t k, int dtype, int allow_tf32,
                                     const fb200_epilogue* epilogue, fb200_stream stream) {
  if (c_dest == nullptr || n_dest < 1 || n_dest > kMaxDest) {
    return set_error(FB200_INVALID_ARGUMENT, "matmul_colsplit: between 1 and %d destinations", kMaxDest);
  }
  if (m < 1 || n_local < 1 || k < 1 || col0 < 0 || col0 + n_local > n_total) {
    return set_error(FB200_INVALID_ARGUMENT, "matmul_colsplit: invalid geometry");
  }
  if (!tensor_core_eligible(a, b_local, nullptr, m, n_local, k, dtype, allow_tf32)) {
    return set_error(FB200_UNIMPLEMENTED,
                     "matmul_colsplit: shape/dtype outside the tensor-core kernel (16-byte row pitches, "
                     "bf16/f16, or fp32 with allow_tf32)");
  }
  EpilogueDev epi{};
  if (int rc = make_epilogue(epilogue, &epi, "matmul_colsplit")) return rc;
  GemmDest dest{};
  dest.group_m = kGemmGroupM;
  for (int d = 0; d < n_dest; ++d) {
    if (c_dest[d] == nullptr) return set_error(FB200_INVALID_ARGUMENT, "matmul_colsplit: destination %d is null", d);
    dest.ptr[d] = c_dest[d];
  }
  dest.n = n_dest;
  dest.ld = n_total;
  dest.col0 = col0;
  cudaStream_t s = as_stream(stream);
  switch (dtype) {
    case FB200_F32: return launch_tc_n<float, 4>(a, b_local, dest, m, n_local, k, dtype, epi, s);
    case FB200_BF16: return launch_tc_n<__nv_bfloat16, 2>(a, b_local, dest, m, n_local, k, dtype, epi, s);
    default: return launch_tc_n<__half, 2>(a, b_local, dest, m, n_local, k, dtype, epi, s);
  }
}

// ---- peer memory plumbing for the column-split variant ------------------------------------------------
extern "C" int fb200_ipc_export(int device, void* ptr, void* handle64) {
  if (ptr == nullptr || handle64 == nullptr) return set_error(FB200_INVALID_ARGUMENT, "fb200_ipc_export: null argument");
  FB200_CUDA_OK(cudaSetDevice(device));
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  FB200_CUDA_OK(cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle64), ptr));
  return FB200_OK;
}

extern "C" int fb200_ipc_import(int device, const void* handle64, void** ptr) {
  if (ptr == nullptr || handle64 == nullptr) return set_error(FB200_INVALID_ARGUMENT, "fb200_ipc_import: null argument");
  FB200_CUDA_OK(cudaSetDevice(device));
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  FB200_CUDA_OK(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return FB200_OK;
}

extern "C" int fb200_ipc_close(int device, void* ptr) {
  if (ptr == nullptr) return FB200_OK;
  FB200_CUDA_OK(cudaSetDevice(device));
  FB200_CUDA_OK(cudaIpcCloseMemHandle(ptr));
  return FB200_OK;
}

// ---- gradients of matmul ------------------------------------------------------------------------
// matmul_grad_lhs_internal: ga[m, k] = gy[m, n] * b[k, n]^T; matmul_grad_rhs_internal:
// gb[k, n] = a[m, k]^T * gy[m, n] (src/backends/cpu/kernels/matmul.cpp:187-232, :289-330: fp32
// accumulation over the contracted index in increasing order, one rounding).  Strict fp32 and
// shapes TMA cannot address run the SIMT kernel with the transposed operand read in place, in the
// CPU's order (bit-identical).  Where reduced-precision tensor-core math is allowed (bf16 / f16,
// fp32 with allow_tf32) the transposed operand is materialised once in a stream-ordered scratch by
// the tiled transpose kernel (an HBM-bound pass, small beside the product) and the product runs on
// the tcgen05 GEMM above.
namespace fb200 {
int gemm_simt_strided(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k,
                      int64_t a_row, int64_t a_k, int64_t b_k, int64_t b_col, int dtype,
                      const EpilogueDev& epi, cudaStream_t s);
}

static int matmul_grad_check(const char* op, const void* x, const void* y, const void* out, int64_t m,
                             int64_t n, int64_t k, int dtype, int64_t out_elems, int64_t contracted) {
  if (m < 0 || n < 0 || k < 0) return set_error(FB200_INVALID_ARGUMENT, "%s: negative dimension", op);
  if (!is_float_dtype(dtype)) {
    return set_error(FB200_INVALID_ARGUMENT, "%s: dtype code %d is not float32/float16/bfloat16", op, dtype);
  }
  if (out_elems > 0 && (out == nullptr || (contracted > 0 && (x == nullptr || y == nullptr)))) {
    return set_error(FB200_INVALID_ARGUMENT, "%s: null argument", op);
  }
  return FB200_OK;
}

extern "C" int fb200_matmul_grad_lhs(const void* gy, const void* b, void* ga, int64_t m, int64_t n,
                                     int64_t k, int dtype, int allow_tf32, fb200_stream stream) {
  if (int rc = matmul_grad_check("matmul_grad_lhs_internal", gy, b, ga, m, n, k, dtype, m * k, n)) return rc;
  if (m == 0 || k == 0) return FB200_OK;
  cudaStream_t s = as_stream(stream);
  EpilogueDev epi{};
  // as a plain product: [m, n] x [n, k]
  if (n > 0 && m * k >= 128 * 128 && tensor_core_eligible(gy, b, ga, m, k, n, dtype, allow_tf32) &&
      (k * itemsize_of(dtype)) % 16 == 0) {
    void* bt = nullptr;
    FB200_CUDA_OK(scratch_alloc_async(&bt, static_cast<size_t>(n) * k * itemsize_of(dtype), s));
    const int64_t dims[2] = {k, n}, perm[2] = {1, 0};
    int rc = fb200_transpose(b, bt, 2, dims, perm, itemsize_of(dtype), stream);
    if (rc == FB200_OK) rc = fb200_matmul(gy, bt, ga, m, k, n, dtype, allow_tf32, nullptr, stream);
    cudaFreeAsync(bt, s);
    return rc;
  }
  // ga[i, p] = sum_j gy[i*n + j] * b[p*n + j]
  return gemm_simt_strided(gy, b, ga, m, k, n, n, 1, 1, n, dtype, epi, s);
}

extern "C" int fb200_matmul_grad_rhs(const void* a, const void* gy, void* gb, int64_t m, int64_t n,
                                     int64_t k, int dtype, int allow_tf32, fb200_stream stream) {
  if (int rc = matmul_grad_check("matmul_grad_rhs_internal", a, gy, gb, m, n, k, dtype, k * n, m)) return rc;
  if (k == 0 || n == 0) return FB200_OK;
  cudaStream_t s = as_stream(stream);
  EpilogueDev epi{};
  // as a plain product: [k, m] x [m, n]
  if (m > 0 && k * n >= 128 * 128 && tensor_core_eligible(a, gy, gb, k, n, m, dtype, allow_tf32) &&
      (k * itemsize_of(dtype)) % 16 == 0) {
    void* at = nullptr;
    FB200_CUDA_OK(scratch_alloc_async(&at, static_cast<size_t>(m) * k * itemsize_of(dtype), s));
    const int64_t dims[2] = {m, k}, perm[2] = {1, 0};
    int rc = fb200_transpose(a, at, 2, dims, perm, itemsize_of(dtype), stream);
    if (rc == FB200_OK) rc = fb200_matmul(at, gy, gb, k, n, m, dtype, allow_tf32, nullptr, stream);
    cudaFreeAsync(at, s);
    return rc;
  }
  // gb[p, j] = sum_i a[i*k + p] * gy[i*n + j]
  return gemm_simt_strided(a, gy, gb, k, n, m, 1, k, n, 1, dtype, epi, s);
}
