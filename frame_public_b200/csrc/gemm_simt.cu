// matmul, strict-fp32 form: C[m,n] = sum_p A[m,p]*B[p,n] with an fp32 accumulator that visits
// p in increasing order, one rounding at the store — src/backends/cpu/kernels/matmul.cpp:92-131.
//
// This is the kernel fb200_matmul uses when reduced-precision math is not allowed for fp32
// (CompileOptions::allow_tf32 == false, include/frame/hal/backend.h:51-63) and for shapes whose
// row pitch is not a multiple of 16 bytes (TMA cannot address them).  Each thread owns a
// register micro-tile and accumulates every output over p = 0..K-1 in order; compiled with
// -fmad=false the multiply and the add round separately exactly as the CPU reference (built
// with -ffp-contract=off) does, so fp32 and bf16 results are BIT-IDENTICAL to the CPU backend.
// The tensor-core path lives in gemm_tcgen05.cu.
#include "common.cuh"
#include "epilogue.cuh"

namespace fb200 {

// Element strides of the two operands: A[i, p] = A[i*a_row + p*a_k], B[p, j] = B[p*b_k + j*b_col].
// The plain product has (K, 1, N, 1); the gradient forms read one operand transposed in place
// (src/backends/cpu/kernels/matmul.cpp:187-232, :289-330) with the same p-increasing accumulation.
struct GemmStrides { int64_t a_row, a_k, b_k, b_col; };

template <typename T, int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_simt_kernel(const T* __restrict__ A, const T* __restrict__ B, T* __restrict__ C, int64_t M,
                 int64_t N, int64_t K, GemmStrides st, EpilogueDev epi) {
  constexpr int THREADS = (BM / TM) * (BN / TN);
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN);
  const int ty = tid / (BN / TN);
  const int64_t tiles_n = (N + BN - 1) / BN;
  const int64_t tiles_m = (M + BM - 1) / BM;
  for (int64_t tile = blockIdx.x; tile < tiles_m * tiles_n; tile += gridDim.x) {
    const int64_t m0 = (tile / tiles_n) * BM;
    const int64_t n0 = (tile % tiles_n) * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;
    // The next k-block is fetched into registers while the current one is multiplied out of shared
    // memory: with a handful of CTAs (a [64, 256] x [256, 10] product is two tiles) every global
    // round trip would otherwise be exposed once per k-block.
    constexpr int A_PER = (BM * BK + THREADS - 1) / THREADS;
    constexpr int B_PER = (BK * BN + THREADS - 1) / THREADS;
    float a_reg[A_PER], b_reg[B_PER];
    auto fetch = [&](int64_t k0) {
#pragma unroll
      for (int q = 0; q < A_PER; ++q) {
        const int e = tid + q * THREADS;
        const int r = e / BK, kk = e % BK;
        const int64_t gm = m0 + r, gk = k0 + kk;
        a_reg[q] = (e < BM * BK && gm < M && gk < K) ? to_f32(A[gm * st.a_row + gk * st.a_k]) : 0.0f;
      }
#pragma unroll
      for (int q = 0; q < B_PER; ++q) {
        const int e = tid + q * THREADS;
        const int kk = e / BN, c = e % BN;
        const int64_t gk = k0 + kk, gn = n0 + c;
        b_reg[q] = (e < BK * BN && gk < K && gn < N) ? to_f32(B[gk * st.b_k + gn * st.b_col]) : 0.0f;
      }
    };
    fetch(0);
    for (int64_t k0 = 0; k0 < K; k0 += BK) {
      // A tile: BM rows x BK, stored k-major in shared memory; B tile: BK x BN.
#pragma unroll
      for (int q = 0; q < A_PER; ++q) {
        const int e = tid + q * THREADS;
        if (e < BM * BK) As[e % BK][e / BK] = a_reg[q];
      }
#pragma unroll
      for (int q = 0; q < B_PER; ++q) {
        const int e = tid + q * THREADS;
        if (e < BK * BN) Bs[e / BN][e % BN] = b_reg[q];
      }
      __syncthreads();
      if (k0 + BK < K) fetch(k0 + BK);
      const int klen = static_cast<int>(K - k0 < BK ? K - k0 : BK);
      for (int kk = 0; kk < klen; ++kk) {
        float a[TM], b[TN];
#pragma unroll
        for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
        for (int j = 0; j < TN; ++j) b[j] = Bs[kk][tx * TN + j];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
          for (int j = 0; j < TN; ++j) acc[i][j] += a[i] * b[j];
      }
      __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
      const int64_t gm = m0 + ty * TM + i;
      if (gm >= M) continue;
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        const int64_t gn = n0 + tx * TN + j;
        if (gn >= N) continue;
        const int64_t idx = gm * N + gn;
        C[idx] = from_f32<T>(apply_epilogue<T>(epi, acc[i][j], idx, gn, gm));
      }
    }
  }
}

template <typename T>
static int launch_simt(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k,
                       const GemmStrides& st, const EpilogueDev& epi, cudaStream_t s) {
  const T* ap = static_cast<const T*>(a);
  const T* bp = static_cast<const T*>(b);
  T* cp = static_cast<T*>(c);
  const int64_t big_tiles = ((m + 127) / 128) * ((n + 127) / 128);
  if (big_tiles >= kNumSMs) {
    const int grid = static_cast<int>(big_tiles < int64_t(kNumSMs) * 4 ? big_tiles : int64_t(kNumSMs) * 4);
    gemm_simt_kernel<T, 128, 128, 16, 8, 8><<<grid, 256, 0, s>>>(ap, bp, cp, m, n, k, st, epi);
  } else if (((m + 31) / 32) * ((n + 63) / 64) < 16) {
    // a handful of outputs (the [64, 10] head of an MLP): one output per thread, 16 x 16 tiles, so
    // that more than one or two SMs take part
    const int64_t tiles = ((m + 15) / 16) * ((n + 15) / 16);
    const int grid = static_cast<int>(tiles < int64_t(kNumSMs) * 8 ? tiles : int64_t(kNumSMs) * 8);
    gemm_simt_kernel<T, 16, 16, 64, 1, 1><<<grid, 256, 0, s>>>(ap, bp, cp, m, n, k, st, epi);
  } else {
    const int64_t tiles = ((m + 31) / 32) * ((n + 63) / 64);
    const int grid = static_cast<int>(tiles < int64_t(kNumSMs) * 8 ? tiles : int64_t(kNumSMs) * 8);
    gemm_simt_kernel<T, 32, 64, 32, 2, 4><<<grid, 256, 0, s>>>(ap, bp, cp, m, n, k, st, epi);
  }
  return after_launch("gemm_simt_kernel");
}

// C[m, n] = sum_p A[i, p] * B[p, j] with explicit operand strides (see GemmStrides).
int gemm_simt_strided(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k,
                      int64_t a_row, int64_t a_k, int64_t b_k, int64_t b_col, int dtype,
                      const EpilogueDev& epi, cudaStream_t s) {
  const GemmStrides st{a_row, a_k, b_k, b_col};
  switch (dtype) {
    case FB200_F32: return launch_simt<float>(a, b, c, m, n, k, st, epi, s);
    case FB200_BF16: return launch_simt<__nv_bfloat16>(a, b, c, m, n, k, st, epi, s);
    case FB200_F16: return launch_simt<__half>(a, b, c, m, n, k, st, epi, s);
    default:
      return set_error(FB200_INVALID_ARGUMENT,
                       "matmul: dtype code %d is not float32/float16/bfloat16", dtype);
  }
}

int gemm_simt(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k, int dtype,
              const EpilogueDev& epi, cudaStream_t s) {
  return gemm_simt_strided(a, b, c, m, n, k, k, 1, n, 1, dtype, epi, s);
}

}  // namespace fb200
