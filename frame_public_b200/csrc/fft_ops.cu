// rfft / irfft along the last axis (fp32 only, like the reference).
//
// Semantics: src/ops/schemas/fft.cpp:8-9 — rfft(x[..., n]) -> out[..., k, 2] with k = n/2 + 1,
// interleaved (re, im), forward sign exp(-2*pi*i*j*k/n), no scaling; irfft(z[..., k, 2]; n) ->
// out[..., n], the inverse of a Hermitian spectrum scaled by 1/n (the imaginary parts of the DC
// term and, for even n, of the Nyquist term do not enter).  They replace the cuFFT R2C / C2R plans
// of src/backends/cuda/kernels/fft.cpp; the CPU reference (src/backends/cpu/kernels/fft.cpp) calls
// pocketfft's r2c / c2r.
//
// These are direct transforms: one thread per output element sums its n (resp. k) terms in double
// precision, with the twiddle factor advanced by a complex multiplication per term and recomputed
// exactly (index reduced mod n, sincospi) every 32 terms, and rounds once to fp32.  The result is
// the correctly rounded transform up to double-precision error, i.e. closer to the exact DFT than
// an fp32 FFT; the cost is O(n^2) per row, meant for the short transforms of the reference's tests
// and examples (n up to a few thousand), not for long signals.
// Bound: fp64 pipe.  Work per launch: rows * k * n complex multiply-adds.
#include "common.cuh"

namespace fb200 {

constexpr int kTwiddleResync = 32;

// exp(-2*pi*i*m/n) for 0 <= m < n
__device__ __forceinline__ void twiddle(int64_t m, int64_t n, double* c, double* s) {
  double sn, cs;
  sincospi(2.0 * static_cast<double>(m) / static_cast<double>(n), &sn, &cs);
  *c = cs;
  *s = -sn;
}

__global__ void __launch_bounds__(128)
rfft_direct_kernel(const float* __restrict__ x, float* __restrict__ out, int64_t rows, int64_t n, int64_t k) {
  const int64_t total = rows * k;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t row = i / k;
    const int64_t f = i - row * k;
    const float* xr = x + row * n;
    double step_c, step_s;
    twiddle(f, n, &step_c, &step_s);
    double re = 0.0, im = 0.0;
    for (int64_t j0 = 0; j0 < n; j0 += kTwiddleResync) {
      double wc, ws;
      twiddle((j0 * f) % n, n, &wc, &ws);
      const int64_t j1 = j0 + kTwiddleResync < n ? j0 + kTwiddleResync : n;
      for (int64_t j = j0; j < j1; ++j) {
        const double v = static_cast<double>(xr[j]);
        re += v * wc;
        im += v * ws;
        const double nc = wc * step_c - ws * step_s;
        ws = wc * step_s + ws * step_c;
        wc = nc;
      }
    }
    out[2 * i] = static_cast<float>(re);
    out[2 * i + 1] = static_cast<float>(im);
  }
}

__global__ void __launch_bounds__(128)
irfft_direct_kernel(const float* __restrict__ z, float* __restrict__ out, int64_t rows, int64_t n, int64_t k) {
  const int64_t total = rows * n;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const bool even = (n % 2) == 0;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t row = i / n;
    const int64_t t = i - row * n;
    const float* zr = z + row * k * 2;
    double step_c, step_s;
    twiddle(t, n, &step_c, &step_s);   // exp(-2*pi*i*t/n); the inverse uses its conjugate
    double acc = static_cast<double>(zr[0]);
    const int64_t last = even ? k - 1 : k;   // exclusive end of the doubled terms
    for (int64_t f0 = 1; f0 < last; f0 += kTwiddleResync) {
      double wc, ws;
      twiddle((f0 * t) % n, n, &wc, &ws);
      const int64_t f1 = f0 + kTwiddleResync < last ? f0 + kTwiddleResync : last;
      for (int64_t f = f0; f < f1; ++f) {
        // Re(z_f * exp(+i*theta)) = re*cos(theta) - im*sin(theta) = re*wc + im*ws  (ws = -sin)
        acc += 2.0 * (static_cast<double>(zr[2 * f]) * wc + static_cast<double>(zr[2 * f + 1]) * ws);
        const double nc = wc * step_c - ws * step_s;
        ws = wc * step_s + ws * step_c;
        wc = nc;
      }
    }
    if (even) {
      // Nyquist term: exp(i*pi*t) = +-1, imaginary part ignored
      acc += (t % 2 == 0 ? 1.0 : -1.0) * static_cast<double>(zr[2 * (k - 1)]);
    }
    out[i] = static_cast<float>(acc / static_cast<double>(n));
  }
}

}  // namespace fb200

using namespace fb200;

extern "C" int fb200_rfft(const void* x, void* out, int64_t rows, int64_t n, int dtype, fb200_stream stream) {
  if (dtype != FB200_F32) return set_error(FB200_INVALID_ARGUMENT, "rfft: dtype code %d is not float32", dtype);
  if (rows < 0 || n < 2) return set_error(FB200_INVALID_ARGUMENT, "rfft: the last dimension must be >= 2, got n=%lld", (long long)n);
  if (rows == 0) return FB200_OK;
  if (x == nullptr || out == nullptr) return set_error(FB200_INVALID_ARGUMENT, "rfft: null argument");
  const int64_t k = n / 2 + 1;
  rfft_direct_kernel<<<grid_for(rows * k, 128, 1), 128, 0, as_stream(stream)>>>(
      static_cast<const float*>(x), static_cast<float*>(out), rows, n, k);
  return after_launch("rfft_direct_kernel");
}

extern "C" int fb200_irfft(const void* z, void* out, int64_t rows, int64_t n, int dtype, fb200_stream stream) {
  if (dtype != FB200_F32) return set_error(FB200_INVALID_ARGUMENT, "irfft: dtype code %d is not float32", dtype);
  if (rows < 0 || n < 2) return set_error(FB200_INVALID_ARGUMENT, "irfft: attribute n must be >= 2, got n=%lld", (long long)n);
  if (rows == 0) return FB200_OK;
  if (z == nullptr || out == nullptr) return set_error(FB200_INVALID_ARGUMENT, "irfft: null argument");
  const int64_t k = n / 2 + 1;
  irfft_direct_kernel<<<grid_for(rows * n, 128, 1), 128, 0, as_stream(stream)>>>(
      static_cast<const float*>(z), static_cast<float*>(out), rows, n, k);
  return after_launch("irfft_direct_kernel");
}
