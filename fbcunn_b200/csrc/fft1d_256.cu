// 256-point batched 1-D R2C / C2R transforms: the largest size of the reference's 1-D test list
// (test/test_FFTModule.lua:170-260; fbfft1dHost in src/fft/FBFFTHost.cpp:119-160 dispatches it to
// its own kernel).  Only the stand-alone 1-D entry points reach this file; a convolution never
// transforms more than 128 points.
//
// Two real rows ride one complex line z = a + i b.  A block of 256 threads owns 16 lines; 16 threads
// share a line and each does a 16-point transform in registers, twice (256 = 16 x 16: input index
// n = 16 n1 + n2, output index k = k1 + 16 k2), with the 256-point twiddle and a pass through shared
// memory in between.  Afterwards the pair is untangled into the two half spectra (forward), or was
// tangled from them before (inverse).
#include "kernels.h"

namespace fbfft {

namespace {

constexpr int kN = 256, kRadix = 16, kLines = 16, kBins = kN / 2 + 1;
constexpr int kPitchSplit = kRadix * (kRadix + 1) + 1;  // [line][k1 * 17 + n2]: conflict-free both ways
constexpr int kPitchLine = kN + 1;                      // [line][k]
static_assert(kLines * kRadix == 256, "one thread per (line, residue)");

// exp(-+ 2 pi i j / 256)
template <bool INV>
__device__ __forceinline__ float2 twiddle256(int j) {
  float s, c;
  sincospif((float)j * (1.f / 128.f), &s, &c);
  return make_float2(c, INV ? s : -s);
}

// The two 16-point steps on the complex line this thread group owns.  In: `z` yields element n of
// the line.  Out: element k1 + 16 k2 of the transform in u[k2], for this thread's k1 = lane16.
// FROM_SPLIT: `z` reads the memory `split` aliases, so everybody fetches before anybody stores.
template <bool INV, bool FROM_SPLIT, class Fetch>
__device__ __forceinline__ void transform256(float2* split, int line, int lane16, Fetch z, float2 (&u)[kRadix]) {
  float2 v[kRadix];
#pragma unroll
  for (int n1 = 0; n1 < kRadix; ++n1) v[n1] = z(kRadix * n1 + lane16);
  if (FROM_SPLIT) __syncthreads();
  fft_inreg<kRadix, INV>(v);
  float2* dst = split + line * kPitchSplit + lane16;
  dst[0] = v[0];
#pragma unroll
  for (int k1 = 1; k1 < kRadix; ++k1) dst[k1 * (kRadix + 1)] = cmul(v[k1], twiddle256<INV>(lane16 * k1));
  __syncthreads();
  const float2* src = split + line * kPitchSplit + lane16 * (kRadix + 1);
#pragma unroll
  for (int n2 = 0; n2 < kRadix; ++n2) u[n2] = src[n2];
  fft_inreg<kRadix, INV>(u);
}

// rows [0, rows) of n floats, each placed at `pad` of a zero line of 256 -> spectrum[row][0..128]
__global__ void __launch_bounds__(256)
fft1d_256_forward_kernel(const float* __restrict__ real, float2* __restrict__ spec, long long rows, int n, int pad) {
  __shared__ float2 buf[kLines * kPitchSplit];  // the split buffer, then (aliased) the 16 transformed lines
  static_assert(kLines * kPitchSplit >= kLines * kPitchLine, "the lines fit the split buffer");
  const int tid = threadIdx.x, line = tid / kRadix, lane16 = tid % kRadix;
  const long long pair0 = (long long)blockIdx.x * kLines;
  const long long ra = 2 * (pair0 + line), rb = ra + 1;
  const float* pa = real + ra * n - pad;
  const float* pb = real + rb * n - pad;
  const bool va = ra < rows, vb = rb < rows;
  float2 u[kRadix];
  transform256<false, false>(buf, line, lane16, [&](int x) {
    const bool vx = x >= pad && x < pad + n;
    return make_float2(va && vx ? pa[x] : 0.f, vb && vx ? pb[x] : 0.f);
  }, u);
  __syncthreads();  // everybody has read the split buffer
#pragma unroll
  for (int k2 = 0; k2 < kRadix; ++k2) buf[line * kPitchLine + lane16 + kRadix * k2] = u[k2];
  __syncthreads();
  for (int item = tid; item < kLines * kBins; item += 256) {
    const int l = item / kBins, k = item - l * kBins;
    const long long r0 = 2 * (pair0 + l);
    if (r0 >= rows) break;
    float2 a, b;
    untangle_pair(buf[l * kPitchLine + k], buf[l * kPitchLine + ((kN - k) & (kN - 1))], a, b);
    spec[r0 * kBins + k] = a;
    if (r0 + 1 < rows) spec[(r0 + 1) * kBins + k] = b;
  }
}

// spectrum[row][0..128] -> the un-normalised inverse, columns [offset, offset + n) of every row
__global__ void __launch_bounds__(256)
fft1d_256_inverse_kernel(const float2* __restrict__ spec, float* __restrict__ real, long long rows, int n, int offset) {
  __shared__ float2 split[kLines * kPitchSplit];  // first the 16 tangled lines, then the split buffer
  float2* lines = split;
  const int tid = threadIdx.x, line = tid / kRadix, lane16 = tid % kRadix;
  const long long pair0 = (long long)blockIdx.x * kLines;
  for (int item = tid; item < kLines * kBins; item += 256) {
    const int l = item / kBins, k = item - l * kBins;
    const long long r0 = 2 * (pair0 + l);
    const float2 zero = make_float2(0.f, 0.f);
    const float2 a = r0 < rows ? spec[r0 * kBins + k] : zero;
    const float2 b = r0 + 1 < rows ? spec[(r0 + 1) * kBins + k] : zero;
    lines[l * kPitchLine + k] = tangle_low(a, b);
    if (k > 0 && k < kN / 2) lines[l * kPitchLine + kN - k] = tangle_high(a, b);
  }
  __syncthreads();
  float2 u[kRadix];
  transform256<true, true>(split, line, lane16, [&](int k) { return lines[line * kPitchLine + k]; }, u);
  const long long ra = 2 * (pair0 + line), rb = ra + 1;
  if (ra >= rows) return;
  float* pa = real + ra * n - offset;
  float* pb = real + rb * n - offset;
#pragma unroll
  for (int k2 = 0; k2 < kRadix; ++k2) {
    const int x = lane16 + kRadix * k2;
    if (x < offset || x >= offset + n) continue;
    pa[x] = u[k2].x;
    if (rb < rows) pb[x] = u[k2].y;
  }
}

}  // namespace

cudaError_t launch_fft1d_256(bool inverse, const float* real_in, float* real_out, float2* spec, long long rows, int n,
                             int offset, cudaStream_t stream) {
  if (rows <= 0 || n <= 0 || offset < 0 || n + offset > kN) return cudaErrorInvalidValue;
  const long long pairs = (rows + 1) / 2;
  const long long blocks = (pairs + kLines - 1) / kLines;
  if (blocks > 0x7fffffff) return cudaErrorInvalidValue;
  if (inverse)
    fft1d_256_inverse_kernel<<<(unsigned)blocks, 256, 0, stream>>>(spec, real_out, rows, n, offset);
  else
    fft1d_256_forward_kernel<<<(unsigned)blocks, 256, 0, stream>>>(real_in, spec, rows, n, offset);
  count_launch();
  return cudaGetLastError();
}

}  // namespace fbfft
