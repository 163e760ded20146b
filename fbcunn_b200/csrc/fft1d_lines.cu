// Batched 1-D R2C / C2R transforms of 64, 128 and 256 points (the stand-alone 1-D entry points; a
// convolution never reaches this file).  Stands where fbfft1dHost dispatches the reference's 1-D
// kernels (src/fft/FBFFTHost.cpp:119-160); 256 is the largest size of the reference's 1-D test list
// (test/test_FFTModule.lua:170-260).
//
// Two real rows ride one complex line z = a + i b.  A line of N = R1 * R2 points is transformed by two
// register steps around one pass through shared memory (input index n = R2 n1 + n2, output index
// k = k1 + R1 k2): R2 threads each do an R1-point transform and a twiddle, then R1 threads each do an
// R2-point transform.  Afterwards the pair is untangled into the two half spectra (forward), or was
// tangled from them before (inverse).  Blocks are light (48 registers, 35 KB of shared memory: five
// per SM), which is what a transform with this little arithmetic per byte wants: 5.0 TB/s forward at
// 256 points.
#include "kernels.h"

namespace fbfft {

namespace {

constexpr int kThreads = 256;

template <int N>
struct Lines {
  static constexpr int R1 = N == 64 ? 8 : 16;          // points of the first register step
  static constexpr int R2 = N / R1;                    // ... of the second: 8, 8, 16
  static constexpr int LINES = kThreads / (R1 < R2 ? R1 : R2);  // complex lines per block: 32, 32, 16
  static constexpr int BINS = N / 2 + 1;
  static constexpr int PITCH_SPLIT = R1 * (R2 + 1) + 1;  // [line][k1 * (R2 + 1) + n2]
  static constexpr int PITCH_LINE = N + 1;               // [line][k]
  static constexpr int PITCH = PITCH_SPLIT > PITCH_LINE ? PITCH_SPLIT : PITCH_LINE;
  static_assert(N == 64 || N == 128 || N == 256, "sizes of this file");
};

// exp(-+ 2 pi i j / N)
template <int N, bool INV>
__device__ __forceinline__ float2 twiddle(int j) {
  float s, c;
  sincospif((float)j * (2.f / N), &s, &c);
  return make_float2(c, INV ? s : -s);
}

// The two register steps on the block's lines.  `z(line, n)` yields element n of a line; `out(line, k, v)`
// takes element k of its transform.  FROM_BUF: `z` reads the memory `buf`, so everybody fetches before
// anybody stores.  INTO_BUF: `out` writes the memory `buf`, so everybody finishes loading before
// anybody emits.  Every thread has exactly one first-step item and one or two second-step items.
template <int N, bool INV, bool FROM_BUF, bool INTO_BUF, class Fetch, class Emit>
__device__ __forceinline__ void transform_lines(float2* buf, Fetch z, Emit out) {
  using L = Lines<N>;
  constexpr int R1 = L::R1, R2 = L::R2;
  static_assert(L::LINES * R2 == kThreads, "one first-step item per thread");
  static_assert((L::LINES * R1) % kThreads == 0, "whole rounds of second-step items");
  constexpr int PER2 = L::LINES * R1 / kThreads;
  const int tid = threadIdx.x;
  {
    float2 v[R1];
    const int line = tid / R2, n2 = tid % R2;
#pragma unroll
    for (int n1 = 0; n1 < R1; ++n1) v[n1] = z(line, R2 * n1 + n2);
    if (FROM_BUF) __syncthreads();
    fft_inreg<R1, INV>(v);
    float2* dst = buf + line * L::PITCH_SPLIT + n2;
    dst[0] = v[0];
#pragma unroll
    for (int k1 = 1; k1 < R1; ++k1) dst[k1 * (R2 + 1)] = cmul(v[k1], twiddle<N, INV>(n2 * k1));
  }
  __syncthreads();
  float2 u[PER2][R2];
#pragma unroll
  for (int i = 0; i < PER2; ++i) {
    const int item = tid + i * kThreads;
    const float2* src = buf + (item / R1) * L::PITCH_SPLIT + (item % R1) * (R2 + 1);
#pragma unroll
    for (int n2 = 0; n2 < R2; ++n2) u[i][n2] = src[n2];
    fft_inreg<R2, INV>(u[i]);
  }
  if (INTO_BUF) __syncthreads();
#pragma unroll
  for (int i = 0; i < PER2; ++i) {
    const int item = tid + i * kThreads;
#pragma unroll
    for (int k2 = 0; k2 < R2; ++k2) out(item / R1, item % R1 + R1 * k2, u[i][k2]);
  }
}

// rows [0, rows) of n floats, each placed at `pad` of a zero line of N -> spectrum[row][0 .. N/2]
template <int N>
__global__ void __launch_bounds__(kThreads)
fft1d_forward_lines_kernel(const float* __restrict__ real, float2* __restrict__ spec, long long rows, int n, int pad) {
  using L = Lines<N>;
  __shared__ float2 buf[L::LINES * L::PITCH];  // the split buffer, then (same memory) the transformed lines
  const long long pair0 = (long long)blockIdx.x * L::LINES;
  float2* zbuf = buf;
  transform_lines<N, false, false, true>(
      buf,
      [&](int line, int x) {
        const long long ra = 2 * (pair0 + line);
        const bool vx = x >= pad && x < pad + n;
        const float* pa = real + ra * n - pad;
        return make_float2(ra < rows && vx ? pa[x] : 0.f, ra + 1 < rows && vx ? pa[n + x] : 0.f);
      },
      [&](int line, int k, float2 v) { zbuf[line * L::PITCH_LINE + k] = v; });
  __syncthreads();
  for (int item = threadIdx.x; item < L::LINES * L::BINS; item += kThreads) {
    const int l = item / L::BINS, k = item - l * L::BINS;
    const long long r0 = 2 * (pair0 + l);
    if (r0 >= rows) break;
    float2 a, b;
    untangle_pair(zbuf[l * L::PITCH_LINE + k], zbuf[l * L::PITCH_LINE + ((N - k) & (N - 1))], a, b);
    spec[r0 * L::BINS + k] = a;
    if (r0 + 1 < rows) spec[(r0 + 1) * L::BINS + k] = b;
  }
}

// spectrum[row][0 .. N/2] -> the un-normalised inverse, columns [offset, offset + n) of every row
template <int N>
__global__ void __launch_bounds__(kThreads)
fft1d_inverse_lines_kernel(const float2* __restrict__ spec, float* __restrict__ real, long long rows, int n, int offset) {
  using L = Lines<N>;
  __shared__ float2 buf[L::LINES * L::PITCH];  // first the tangled lines, then the split buffer
  const long long pair0 = (long long)blockIdx.x * L::LINES;
  for (int item = threadIdx.x; item < L::LINES * L::BINS; item += kThreads) {
    const int l = item / L::BINS, k = item - l * L::BINS;
    const long long r0 = 2 * (pair0 + l);
    const float2 zero = make_float2(0.f, 0.f);
    const float2 a = r0 < rows ? spec[r0 * L::BINS + k] : zero;
    const float2 b = r0 + 1 < rows ? spec[(r0 + 1) * L::BINS + k] : zero;
    buf[l * L::PITCH_LINE + k] = tangle_low(a, b);
    if (k > 0 && k < N / 2) buf[l * L::PITCH_LINE + N - k] = tangle_high(a, b);
  }
  __syncthreads();
  transform_lines<N, true, true, false>(
      buf, [&](int line, int k) { return buf[line * L::PITCH_LINE + k]; },
      [&](int line, int x, float2 v) {
        const long long ra = 2 * (pair0 + line);
        if (ra >= rows || x < offset || x >= offset + n) return;
        float* pa = real + ra * n - offset;
        pa[x] = v.x;
        if (ra + 1 < rows) pa[n + x] = v.y;
      });
}

template <int N>
cudaError_t launch_lines(bool inverse, const float* real_in, float* real_out, float2* spec, long long rows, int n,
                         int offset, cudaStream_t stream) {
  const long long pairs = (rows + 1) / 2;
  const long long blocks = (pairs + Lines<N>::LINES - 1) / Lines<N>::LINES;
  if (blocks > 0x7fffffff) return cudaErrorInvalidValue;
  if (inverse)
    fft1d_inverse_lines_kernel<N><<<(unsigned)blocks, kThreads, 0, stream>>>(spec, real_out, rows, n, offset);
  else
    fft1d_forward_lines_kernel<N><<<(unsigned)blocks, kThreads, 0, stream>>>(real_in, spec, rows, n, offset);
  count_launch();
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_fft1d_lines(bool inverse, const float* real_in, float* real_out, float2* spec, long long rows,
                               int n, int N, int offset, cudaStream_t stream) {
  if (rows <= 0 || n <= 0 || offset < 0 || n + offset > N) return cudaErrorInvalidValue;
  switch (N) {
    case 64: return launch_lines<64>(inverse, real_in, real_out, spec, rows, n, offset, stream);
    case 128: return launch_lines<128>(inverse, real_in, real_out, spec, rows, n, offset, stream);
    case 256: return launch_lines<256>(inverse, real_in, real_out, spec, rows, n, offset, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace fbfft
