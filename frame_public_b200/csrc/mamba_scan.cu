// mamba_scan — a NEW op with no counterpart in the reference: the Mamba SSM recurrence with
// delta, A, B, C, D un-materialised (the reference's selective_scan needs five materialised
// [B, D, N, L] operands: 19 GB per run at the Mamba config instead of 0.8 GB) and the d_state-wide
// state held in registers.  fp32.
//     h[n] = exp(delta*A[d,n]) * h[n] + (delta*B[n]) * u
//     y    = sum_n C[n]*h[n] + D[d]*u ;   y *= silu(z) when a gate is given
// u / delta / z / y are time-major [batch, len, dm] (the layout the surrounding GEMMs produce);
// A is [dm, nstate]; B, C are [batch, len, nstate]; D is [dm].
//
// Mapping: LANES lanes share one (batch, channel), each holding NS/LANES states.  The recurrence is
// bound by instruction issue and by the exp2 unit, not by HBM (0.8 GB per run at the Mamba
// configuration), so what matters is instructions per channel-step: the per-lane overhead (loads of
// u and delta, addressing, the cross-lane sum, the finishing of y) is paid LANES times, the state
// arithmetic once.  Two lanes of eight states keep enough threads for one wave on 148 SMs and
// cost a third of the instructions of four lanes of four.
// Four time steps are processed per iteration: u, delta and z of the NEXT four steps are in flight
// (two register sets) while the current four are computed; B and C rows, shared by all channels
// of a batch and therefore L1/L2 hits, are fetched with 128-bit loads at the start of the
// iteration.  The partial sums are combined with log2(LANES) shuffles per step, after which every
// lane holds all four sums and lane s finishes (D skip, gate, store) the steps j with j % LANES == s.
// exp(delta*A) is evaluated as ex2.approx(delta * (A*log2 e)): 2 ulp, and the recurrence contracts,
// so the error does not grow.  Algorithmic bytes = (4*B*L*D + 2*B*L*N) * 4.
#include <cstdlib>

#include "common.cuh"

namespace fb200 {

constexpr int kMambaThreads = 128;
// The pipelined kernel's warps never talk to each other, so a CTA is ONE warp: 1536 CTAs of the
// benchmark shape spread over 148 SMs as 10 or 11 each (four-warp CTAs: 2 or 3 each, i.e. a sixth of
// the SMs' time idle at the end).
constexpr int kPipeThreads = 32;
constexpr int kMambaSteps = 4;  // time steps per iteration

__device__ __forceinline__ float mamba_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int NS, int LANES>
__global__ void __launch_bounds__(kMambaThreads)
mamba_scan_kernel(const float* __restrict__ u, const float* __restrict__ delta,
                  const float* __restrict__ A, const float* __restrict__ B,
                  const float* __restrict__ C, const float* __restrict__ D,
                  const float* __restrict__ z, float* __restrict__ y, int64_t len, int64_t dm) {
  constexpr int PER = NS / LANES;  // states per lane
  constexpr int U = kMambaSteps;
  constexpr int FIN = U / LANES;   // steps each lane finishes per iteration
  constexpr int kChannelsPerCta = kMambaThreads / LANES;
  static_assert(PER % 4 == 0 && U % LANES == 0, "states per lane must fill 128-bit loads");
  const int64_t bidx = blockIdx.y;
  const int sg = threadIdx.x % LANES;
  const int64_t ch_raw = static_cast<int64_t>(blockIdx.x) * kChannelsPerCta + threadIdx.x / LANES;
  const bool live = ch_raw < dm;
  const int64_t ch = live ? ch_raw : dm - 1;  // dead lanes shadow a valid channel and never store
  float h[PER], Ar[PER];
#pragma unroll
  for (int n = 0; n < PER; ++n) {
    h[n] = 0.0f;
    Ar[n] = A[ch * NS + sg * PER + n] * 1.4426950408889634f;
  }
  const float Dd = D[ch];
  const float* up = u + bidx * len * dm + ch;
  const float* dp = delta + bidx * len * dm + ch;
  const float* zp = z != nullptr ? z + bidx * len * dm + ch : nullptr;
  float* yp = y + bidx * len * dm + ch;
  const float4* Bp = reinterpret_cast<const float4*>(B + bidx * len * NS + sg * PER);
  const float4* Cp = reinterpret_cast<const float4*>(C + bidx * len * NS + sg * PER);
  struct Ahead {
    float uu[U], dd[U], zz[FIN];
  };
  auto load = [&](int64_t t0, Ahead& a) {
#pragma unroll
    for (int j = 0; j < U; ++j) {
      const int64_t t = t0 + j < len ? t0 + j : len - 1;
      a.uu[j] = __ldg(up + t * dm);
      a.dd[j] = __ldg(dp + t * dm);
    }
#pragma unroll
    for (int f = 0; f < FIN; ++f) {   // gate operands of the steps this lane finishes
      const int64_t tm = t0 + f * LANES + sg;
      const int64_t t = tm < len ? tm : len - 1;
      a.zz[f] = zp != nullptr ? __ldg(zp + t * dm) : 0.0f;
    }
  };
  auto compute = [&](int64_t t0, const Ahead& a) {
    float4 bb[U][PER / 4], cc[U][PER / 4];
#pragma unroll
    for (int j = 0; j < U; ++j) {
      const int64_t t = t0 + j < len ? t0 + j : len - 1;
#pragma unroll
      for (int q = 0; q < PER / 4; ++q) {
        bb[j][q] = __ldg(Bp + t * (NS / 4) + q);
        cc[j][q] = __ldg(Cp + t * (NS / 4) + q);
      }
    }
    float acc[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
      const float du = a.dd[j] * a.uu[j];
      float s = 0.0f;
#pragma unroll
      for (int q = 0; q < PER / 4; ++q) {
        const float bq[4] = {bb[j][q].x, bb[j][q].y, bb[j][q].z, bb[j][q].w};
        const float cq[4] = {cc[j][q].x, cc[j][q].y, cc[j][q].z, cc[j][q].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int n = q * 4 + e;
          h[n] = mamba_ex2(a.dd[j] * Ar[n]) * h[n] + du * bq[e];
          s = s + cq[e] * h[n];
        }
      }
      acc[j] = s;
    }
#pragma unroll
    for (int j = 0; j < U; ++j) {
#pragma unroll
      for (int o = 1; o < LANES; o <<= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
    }
#pragma unroll
    for (int f = 0; f < FIN; ++f) {
      float mine = acc[f * LANES], umine = a.uu[f * LANES];
#pragma unroll
      for (int l = 1; l < LANES; ++l) {
        if (sg == l) { mine = acc[f * LANES + l]; umine = a.uu[f * LANES + l]; }
      }
      const int64_t t = t0 + f * LANES + sg;
      if (live && t < len) {
        float out = mine + Dd * umine;
        if (zp != nullptr) out = out * (a.zz[f] * ew_sigmoid(a.zz[f]));
        yp[t * dm] = out;
      }
    }
  };
  Ahead a0, a1;
  load(0, a0);
  for (int64_t t0 = 0; t0 < len; t0 += 2 * U) {
    load(t0 + U, a1);
    compute(t0, a0);
    load(t0 + 2 * U, a0);
    if (t0 + U < len) compute(t0 + U, a1);   // uniform across the CTA
  }
}

// ---- the same recurrence behind a per-warp cp.async pipeline ---------------------------------------
// The direct kernel above has every thread wait for its own global loads once per iteration: with
// 2048 sequential steps per thread that latency, not throughput, set the run time.  Here each warp
// streams its operands (u, delta, z for its 32/LANES channels, the B and C rows) for kPipeTile time
// steps per stage into shared memory with 16-byte cp.async copies, kPipeStages - 1 stages ahead,
// and computes from shared memory; warps are independent (no CTA-wide barrier).  Needs
// dm % (32/LANES) == 0 and 16-byte aligned operands; other shapes take the direct kernel.
constexpr int kPipeTile = 8;
constexpr int kPipeStages = 4;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int NS, int LANES>
__host__ __device__ constexpr int mamba_pipe_stage_floats() { return 3 * kPipeTile * (32 / LANES) + 2 * kPipeTile * NS; }

// Which part of the time axis a launch covers.
//   kScanWhole    the whole sequence from h = 0, results written: one pass, used when batch x
//                 channels alone fill the machine.
//   kScanSummary  chunk `blockIdx.z` of the sequence from h = 0, nothing written but the chunk's end
//                 state S[n] and the sum of its deltas (the chunk's decay is exp(A[n] * sum delta),
//                 one exponential per state instead of a product over the chunk).
//   kScanApply    chunk `blockIdx.z` from the state the earlier chunks leave behind
//                 (h = P_c' * h + S_c' over c' < chunk), results written.
// Summary + apply evaluate every exponential twice, but give `chunks` times the threads: with a few
// samples per GPU (a batch sharded over 8 GPUs leaves 2) the single pass has 2 warps per SM and
// runs at the latency of 2048 dependent steps.
enum MambaScanMode : int { kScanWhole = 0, kScanSummary = 1, kScanApply = 2 };

struct MambaChunks {
  int64_t chunks;      // time chunks (1 for kScanWhole)
  int64_t chunk_len;   // steps per chunk, a multiple of kPipeTile
  float* state;        // [batch][chunks][dm][NS]  end state of each chunk started from zero
  float* dsum;         // [batch][chunks][dm]      sum of delta over each chunk
};

__device__ __forceinline__ float2 f2(float a, float b) { return make_float2(a, b); }

// Arithmetic on pairs of states goes through the packed fp32 instructions of sm_100
// (fma.rn.f32x2 / mul.rn.f32x2): half the issue slots per state update; the exponentials stay
// one ex2.approx each.
template <int NS, int LANES, int MODE>
__global__ void __launch_bounds__(kPipeThreads)
mamba_scan_pipe_kernel(const float* __restrict__ u, const float* __restrict__ delta,
                       const float* __restrict__ A, const float* __restrict__ B,
                       const float* __restrict__ C, const float* __restrict__ D,
                       const float* __restrict__ z, float* __restrict__ y, int64_t len, int64_t dm,
                       MambaChunks ck) {
  constexpr int PER = NS / LANES;            // states per lane
  constexpr int PAIRS = PER / 2;
  constexpr int CW = 32 / LANES;             // channels per warp
  constexpr int TT = kPipeTile, ST = kPipeStages, U = kMambaSteps;
  constexpr int FIN = TT / LANES;            // steps of a tile each lane finishes
  constexpr int kStageFloats = mamba_pipe_stage_floats<NS, LANES>();
  static_assert(PER % 4 == 0 && TT % LANES == 0 && TT % U == 0 && CW % 4 == 0, "tile geometry");
  extern __shared__ float4 mamba_smem4[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* ws = reinterpret_cast<float*>(mamba_smem4) + warp * ST * kStageFloats;
  const int64_t ch0 = (static_cast<int64_t>(blockIdx.x) * (kPipeThreads / 32) + warp) * CW;
  if (ch0 >= dm) return;                     // whole warp; warps never wait on each other
  const int64_t bidx = blockIdx.y;
  const int64_t chunk = MODE == kScanWhole ? 0 : blockIdx.z;
  if (MODE == kScanSummary && chunk + 1 >= ck.chunks) return;   // nobody needs the last chunk's end state
  const int64_t t_begin = chunk * ck.chunk_len;
  const int64_t t_end = (MODE == kScanWhole || t_begin + ck.chunk_len > len) ? len : t_begin + ck.chunk_len;
  const int sg = lane % LANES, c = lane / LANES;
  const int64_t ch = ch0 + c;
  float2 h[PAIRS], Ar[PAIRS];
#pragma unroll
  for (int p = 0; p < PAIRS; ++p) {
    h[p] = f2(0.0f, 0.0f);
    Ar[p] = f2(A[ch * NS + sg * PER + 2 * p] * 1.4426950408889634f, A[ch * NS + sg * PER + 2 * p + 1] * 1.4426950408889634f);
  }
  if (MODE == kScanApply) {
    // the state the chunks before this one leave behind
    for (int64_t cp = 0; cp < chunk; ++cp) {
      const float ds = ck.dsum[(bidx * ck.chunks + cp) * dm + ch];
      const float* sp = ck.state + ((bidx * ck.chunks + cp) * dm + ch) * NS + sg * PER;
#pragma unroll
      for (int p = 0; p < PAIRS; ++p) {
        const float2 x = __fmul2_rn(f2(ds, ds), Ar[p]);
        h[p] = __ffma2_rn(f2(mamba_ex2(x.x), mamba_ex2(x.y)), h[p], f2(sp[2 * p], sp[2 * p + 1]));
      }
    }
  }
  const float Dd = D[ch];
  const float* ub = u + bidx * len * dm + ch0;
  const float* db = delta + bidx * len * dm + ch0;
  const float* zb = (z != nullptr && MODE != kScanSummary) ? z + bidx * len * dm + ch0 : nullptr;
  const float* Bb = B + bidx * len * NS;
  const float* Cb = C + bidx * len * NS;
  float* yp = y + bidx * len * dm + ch;
  const int64_t n_tiles = (t_end - t_begin + TT - 1) / TT;
  // stage layout (floats): u[TT][CW] | delta[TT][CW] | z[TT][CW] | B[TT][NS] | C[TT][NS]
  auto issue = [&](int64_t tile) {
    if (tile < n_tiles) {
      float* st = ws + (tile % ST) * kStageFloats;
      const int64_t t0 = t_begin + tile * TT;
      constexpr int kChunksX = TT * CW / 4, kChunksS = TT * NS / 4;
      for (int i = lane; i < kChunksX; i += 32) {
        const int r = i / (CW / 4), q = i % (CW / 4);
        const int64_t t = t0 + r < len ? t0 + r : len - 1;
        cp_async16(st + r * CW + q * 4, ub + t * dm + q * 4);
        cp_async16(st + TT * CW + r * CW + q * 4, db + t * dm + q * 4);
        if (zb != nullptr) cp_async16(st + 2 * TT * CW + r * CW + q * 4, zb + t * dm + q * 4);
      }
      for (int i = lane; i < kChunksS; i += 32) {
        const int r = i / (NS / 4), q = i % (NS / 4);
        const int64_t t = t0 + r < len ? t0 + r : len - 1;
        cp_async16(st + 3 * TT * CW + r * NS + q * 4, Bb + t * NS + q * 4);
        if (MODE != kScanSummary) cp_async16(st + 3 * TT * CW + TT * NS + r * NS + q * 4, Cb + t * NS + q * 4);
      }
    }
    cp_async_commit();   // an empty group keeps the group count uniform
  };
  float dsum = 0.0f;
  for (int s = 0; s < ST - 1; ++s) issue(s);
  for (int64_t tile = 0; tile < n_tiles; ++tile) {
    issue(tile + ST - 1);
    cp_async_wait<ST - 1>();
    __syncwarp();
    const float* st = ws + (tile % ST) * kStageFloats;
    const float* su = st;
    const float* sd = st + TT * CW;
    const float* sz = st + 2 * TT * CW;
    const float* sB = st + 3 * TT * CW + sg * PER;
    const float* sC = sB + TT * NS;
    float acc[TT], uu[TT];
#pragma unroll
    for (int g = 0; g < TT / U; ++g) {
      // everything that does not depend on the state first: U x PER exponentials and input terms
      float2 dA[U][PAIRS], dBx[U][PAIRS];
#pragma unroll
      for (int j = 0; j < U; ++j) {
        const int r = g * U + j;
        const float dd = sd[r * CW + c];
        uu[r] = su[r * CW + c];
        if (MODE == kScanSummary) dsum += dd;
        const float du = dd * uu[r];
#pragma unroll
        for (int q = 0; q < PER / 4; ++q) {
          const float4 b4 = *reinterpret_cast<const float4*>(sB + r * NS + q * 4);
          const float2 x0 = __fmul2_rn(f2(dd, dd), Ar[2 * q]), x1 = __fmul2_rn(f2(dd, dd), Ar[2 * q + 1]);
          dA[j][2 * q] = f2(mamba_ex2(x0.x), mamba_ex2(x0.y));
          dA[j][2 * q + 1] = f2(mamba_ex2(x1.x), mamba_ex2(x1.y));
          dBx[j][2 * q] = __fmul2_rn(f2(du, du), f2(b4.x, b4.y));
          dBx[j][2 * q + 1] = __fmul2_rn(f2(du, du), f2(b4.z, b4.w));
        }
      }
      // the recurrence itself: PAIRS independent packed FMAs per step
#pragma unroll
      for (int j = 0; j < U; ++j) {
        const int r = g * U + j;
        float2 sum = f2(0.0f, 0.0f);
#pragma unroll
        for (int q = 0; q < PER / 4; ++q) {
          h[2 * q] = __ffma2_rn(dA[j][2 * q], h[2 * q], dBx[j][2 * q]);
          h[2 * q + 1] = __ffma2_rn(dA[j][2 * q + 1], h[2 * q + 1], dBx[j][2 * q + 1]);
          if (MODE != kScanSummary) {
            const float4 c4 = *reinterpret_cast<const float4*>(sC + r * NS + q * 4);
            sum = __ffma2_rn(f2(c4.x, c4.y), h[2 * q], sum);
            sum = __ffma2_rn(f2(c4.z, c4.w), h[2 * q + 1], sum);
          }
        }
        acc[r] = sum.x + sum.y;
      }
    }
    if (MODE != kScanSummary) {
      // the tile's TT sums across the lanes of a channel, then each lane finishes TT / LANES steps
#pragma unroll
      for (int r = 0; r < TT; ++r) {
#pragma unroll
        for (int o = 1; o < LANES; o <<= 1) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], o);
      }
#pragma unroll
      for (int f = 0; f < FIN; ++f) {
        float mine = acc[f * LANES], umine = uu[f * LANES];
#pragma unroll
        for (int l = 1; l < LANES; ++l) {
          if (sg == l) { mine = acc[f * LANES + l]; umine = uu[f * LANES + l]; }
        }
        const int r = f * LANES + sg;
        const int64_t t = t_begin + tile * TT + r;
        if (t < t_end) {
          float out = mine + Dd * umine;
          if (zb != nullptr) {
            const float zz = sz[r * CW + c];
            out = out * (zz * ew_sigmoid(zz));
          }
          yp[t * dm] = out;
        }
      }
    }
    __syncwarp();   // every lane is done with this stage before the next issue overwrites it
  }
  if (MODE == kScanSummary) {
    float* sp = ck.state + ((bidx * ck.chunks + chunk) * dm + ch) * NS + sg * PER;
#pragma unroll
    for (int p = 0; p < PAIRS; ++p) { sp[2 * p] = h[p].x; sp[2 * p + 1] = h[p].y; }
    if (sg == 0) ck.dsum[(bidx * ck.chunks + chunk) * dm + ch] = dsum;
  }
}

// Lanes per channel for a state size: two lanes with nstate / 2 states each from 8 states on.
static int mamba_lanes(int64_t nstate) { return nstate >= 8 ? 2 : 1; }

}  // namespace fb200

using namespace fb200;

extern "C" int fb200_mamba_scan(const void* u, const void* delta, const void* A, const void* B,
                                const void* C, const void* D, const void* z, void* y,
                                int64_t batch, int64_t len, int64_t dm, int64_t nstate,
                                fb200_stream stream) {
  if (batch < 0 || len < 0 || dm < 0) return set_error(FB200_INVALID_ARGUMENT, "mamba_scan: negative shape");
  if (nstate != 16 && nstate != 8 && nstate != 4) {
    return set_error(FB200_UNIMPLEMENTED, "mamba_scan: nstate must be 4, 8 or 16, got %lld",
                     static_cast<long long>(nstate));
  }
  if (batch == 0 || len == 0 || dm == 0) return FB200_OK;
  if (!u || !delta || !A || !B || !C || !D || !y) {
    return set_error(FB200_INVALID_ARGUMENT, "mamba_scan: null argument");
  }
  if (batch > 65535) return set_error(FB200_INVALID_ARGUMENT, "mamba_scan: batch > 65535");
  cudaStream_t s = as_stream(stream);
  const float* up = static_cast<const float*>(u);
  const float* dp = static_cast<const float*>(delta);
  const float* Ap = static_cast<const float*>(A);
  const float* Bp = static_cast<const float*>(B);
  const float* Cp = static_cast<const float*>(C);
  const float* Dp = static_cast<const float*>(D);
  const float* zp = static_cast<const float*>(z);
  float* yp = static_cast<float*>(y);
  if (!aligned16(B) || !aligned16(C)) return set_error(FB200_INVALID_ARGUMENT, "mamba_scan: B and C must be 16-byte aligned");
  int lanes = mamba_lanes(nstate);
  // 16 states: four lanes per channel (four states each) repeat the per-channel work twice as often
  // (b16: 0.395 against 0.364 ms) but double the warps; taken when that alone fills the GPU and saves
  // the second pass of the time chunks (b8: 0.227 against 0.279 ms).
  if (nstate == 16 && dm % 8 == 0) {
    const int64_t warps2 = batch * (dm / 16), warps4 = batch * (dm / 8);
    if (warps2 < int64_t(kNumSMs) * 8 && warps4 >= int64_t(kNumSMs) * 8) lanes = 4;
  }
  const int per_cta = kMambaThreads / lanes;
  dim3 grid(static_cast<unsigned>((dm + per_cta - 1) / per_cta), static_cast<unsigned>(batch));
  const int cw = 32 / lanes;
  const bool piped = dm % cw == 0 && dm % 4 == 0 && aligned16(u) && aligned16(delta) &&
                     (z == nullptr || aligned16(z));
  if (piped) grid.x = static_cast<unsigned>((dm / cw + kPipeThreads / 32 - 1) / (kPipeThreads / 32));
  // Time chunks: one pass when batch x channels give every SM at least 8 warps; otherwise enough
  // chunks for about 16 warps per SM, each at least 64 steps long (a multiple of the pipeline tile).
  MambaChunks ck{1, len, nullptr, nullptr};
  if (piped) {
    const int64_t warps = batch * (dm / cw);
    if (warps < int64_t(kNumSMs) * 8) {
      int64_t chunks = (int64_t(kNumSMs) * 16 + warps - 1) / warps;
      if (chunks > len / 64) chunks = len / 64;
      if (chunks > 65535) chunks = 65535;
      if (chunks >= 2) {
        int64_t cl = (len + chunks - 1) / chunks;
        cl = (cl + kPipeTile - 1) / kPipeTile * kPipeTile;
        ck.chunks = (len + cl - 1) / cl;
        ck.chunk_len = cl;
      }
    }
  }
  float* scratch = nullptr;
  if (ck.chunks > 1) {
    const size_t n_state = static_cast<size_t>(batch) * ck.chunks * dm * nstate;
    const size_t n_dsum = static_cast<size_t>(batch) * ck.chunks * dm;
    FB200_CUDA_OK(scratch_alloc_async(reinterpret_cast<void**>(&scratch), (n_state + n_dsum) * sizeof(float), s));
    ck.state = scratch;
    ck.dsum = scratch + n_state;
  }
  int rc = FB200_OK;
#define FB200_MAMBA_PIPE(NS, LN, MODE, GRID)                                                         \
  do {                                                                                               \
    const size_t smem = size_t(kPipeThreads / 32) * kPipeStages * mamba_pipe_stage_floats<NS, LN>() * 4; \
    auto kernel = mamba_scan_pipe_kernel<NS, LN, MODE>;                                              \
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,        \
                                         static_cast<int>(smem));                                    \
    if (e != cudaSuccess) { rc = cuda_error(e, "cudaFuncSetAttribute(mamba_scan)"); break; }         \
    kernel<<<GRID, kPipeThreads, smem, s>>>(up, dp, Ap, Bp, Cp, Dp, zp, yp, len, dm, ck);            \
    rc = after_launch("mamba_scan_pipe_kernel");                                                     \
  } while (0)
#define FB200_MAMBA_LAUNCH(NS, LN)                                                                   \
  do {                                                                                               \
    if (piped && ck.chunks > 1) {                                                                    \
      dim3 g3(grid.x, grid.y, static_cast<unsigned>(ck.chunks));                                     \
      FB200_MAMBA_PIPE(NS, LN, kScanSummary, g3);                                                    \
      if (rc == FB200_OK) FB200_MAMBA_PIPE(NS, LN, kScanApply, g3);                                  \
    } else if (piped) {                                                                              \
      FB200_MAMBA_PIPE(NS, LN, kScanWhole, grid);                                                    \
    } else {                                                                                         \
      mamba_scan_kernel<NS, LN><<<grid, kMambaThreads, 0, s>>>(up, dp, Ap, Bp, Cp, Dp, zp, yp, len, dm); \
      rc = after_launch("mamba_scan_kernel");                                                        \
    }                                                                                                \
  } while (0)
  if (nstate == 16 && lanes == 4) {
    FB200_MAMBA_LAUNCH(16, 4);
  } else if (nstate == 16) {
    FB200_MAMBA_LAUNCH(16, 2);
  } else if (nstate == 8) {
    FB200_MAMBA_LAUNCH(8, 2);
  } else {
    FB200_MAMBA_LAUNCH(4, 1);
  }
#undef FB200_MAMBA_LAUNCH
#undef FB200_MAMBA_PIPE
  if (scratch != nullptr) cudaFreeAsync(scratch, s);
  return rc;
}
