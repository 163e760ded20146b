// Batched 2-D real<->complex FFT building blocks for power-of-two sizes 8..128.
//
// Everything here is written so that the same text compiles as CUDA device code
// and as plain host C++: the kernels are split into phases between barriers, each
// phase a function of the thread index, so a host harness can run a block by
// looping over thread indices phase by phase and check the index arithmetic
// without a GPU.
//
// Replaces the transform contract of the reference's fbfft entry points
// (src/fft/FBFFTHost.cpp:39-116, src/fft/FBFFTDevice.cu:15-48): a real h x w plane
// placed at (padU, padL) of a zero N x N square, forward sign exp(-2 pi i ..),
// Hermitian half kept, inverse un-normalised and cropped to the real tensor's
// extent.  The layout of the half spectrum is private to this library:
//
//     spectrum[bin][row][inner]   complex fp32,  bin = kx * N + ky,  kx in [0, N/2]
//
// i.e. bin-major with the plane index innermost, which is what the per-bin
// contraction reads (the reference needed a separate transpose for that,
// src/CuBLASWrapper.cpp:33-172).
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#include <cuda_runtime.h>
#define FBF_HD __host__ __device__ __forceinline__
#else
#include <cmath>
#define FBF_HD inline
struct float2 {
  float x, y;
};
static inline float2 make_float2(float x, float y) {
  float2 r;
  r.x = x;
  r.y = y;
  return r;
}
#endif

namespace fbfft {

// ---------------------------------------------------------------------------
// complex helpers and twiddles
// ---------------------------------------------------------------------------
FBF_HD float2 cadd(float2 a, float2 b) { return make_float2(a.x + b.x, a.y + b.y); }
FBF_HD float2 csub(float2 a, float2 b) { return make_float2(a.x - b.x, a.y - b.y); }
FBF_HD float2 cmul(float2 a, float2 b) {
  return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x);
}

// (cos, sin)(2 pi i / 128) as literals: with a compile-time index the switch folds
// into immediates.
FBF_HD float2 tw128_literal(int i) {
  switch (i & 127) {
#define FBF_TW(idx, c, s) \
  case idx:               \
    return make_float2(c, s);
#include "twiddle128.inc"
#undef FBF_TW
  }
  return make_float2(1.f, 0.f);
}

// Same table for indices only known at run time (uniform across a warp in the
// callers below, so the constant cache broadcasts it).
#if defined(__CUDACC__)
static __constant__ float2 c_tw128[128] = {
#define FBF_TW(idx, c, s) {c, s},
#include "twiddle128.inc"
#undef FBF_TW
};
#endif
static const float2 h_tw128[128] = {
#define FBF_TW(idx, c, s) {c, s},
#include "twiddle128.inc"
#undef FBF_TW
};

template <bool INV>
FBF_HD float2 tw128_runtime(int i) {
#if defined(__CUDA_ARCH__)
  float2 w = c_tw128[i & 127];
#else
  float2 w = h_tw128[i & 127];
#endif
  if (!INV) w.y = -w.y;
  return w;
}

// d * exp(-+ 2 pi i idx / 128), idx a compile-time constant after unrolling.
template <bool INV>
FBF_HD float2 mul_tw(float2 d, int idx) {
  if (idx == 0) return d;
  if (idx == 32) return INV ? make_float2(-d.y, d.x) : make_float2(d.y, -d.x);
  if (idx == 64) return make_float2(-d.x, -d.y);
  float2 w = tw128_literal(idx);
  const float s = INV ? w.y : -w.y;
  return make_float2(d.x * w.x - d.y * s, d.x * s + d.y * w.x);
}

template <int N>
struct Log2 {
  static constexpr int value = 1 + Log2<N / 2>::value;
};
template <>
struct Log2<1> {
  static constexpr int value = 0;
};

FBF_HD int bit_reverse(int k, int bits) {
  int r = 0;
#pragma unroll
  for (int i = 0; i < 7; ++i)
    if (i < bits) r |= ((k >> i) & 1) << (bits - 1 - i);
  return r;
}

// N-point complex FFT held entirely in one thread's registers (N <= 32), natural
// order in and out.  Decimation in frequency; the final bit reversal is a
// renaming once the loops are unrolled.
template <int N, bool INV>
FBF_HD void fft_inreg(float2 (&v)[N]) {
  constexpr int LG = Log2<N>::value;
#pragma unroll
  for (int s = 0; s < LG; ++s) {
    const int len = N >> s;
    const int half = len >> 1;
    const int tstep = 128 / len;
#pragma unroll
    for (int base = 0; base < N; base += len) {
#pragma unroll
      for (int j = 0; j < half; ++j) {
        const float2 a = v[base + j];
        const float2 b = v[base + j + half];
        v[base + j] = cadd(a, b);
        v[base + j + half] = mul_tw<INV>(csub(a, b), j * tstep);
      }
    }
  }
  float2 t[N];
#pragma unroll
  for (int k = 0; k < N; ++k) t[k] = v[k];
#pragma unroll
  for (int k = 0; k < N; ++k) v[k] = t[bit_reverse(k, LG)];
}

// Sizes above 32 are done by one thread in two steps through a private line of
// shared memory: N = N1 * N2, input index n = N2*n1 + n2, output index
// k = k1 + N1*k2.  After both steps slot N2*k1 + k2 holds frequency k1 + N1*k2.
template <int N>
struct Split {
  static constexpr int N1 = N, N2 = 1;
};
template <>
struct Split<64> {
  static constexpr int N1 = 8, N2 = 8;
};
template <>
struct Split<128> {
  static constexpr int N1 = 8, N2 = 16;
};

template <int N>
FBF_HD int slot_of_frequency(int k) {
  return Split<N>::N2 * (k % Split<N>::N1) + (k / Split<N>::N1);
}

// ld(n) returns input element n (already zero where pruned); st(slot, value).
template <int N, bool INV, class LoadFn, class StoreFn>
FBF_HD void fft_two_step_first(LoadFn ld, StoreFn st) {
  constexpr int N1 = Split<N>::N1, N2 = Split<N>::N2;
#pragma unroll 1
  for (int n2 = 0; n2 < N2; ++n2) {
    float2 v[N1];
#pragma unroll
    for (int n1 = 0; n1 < N1; ++n1) v[n1] = ld(N2 * n1 + n2);
    fft_inreg<N1, INV>(v);
#pragma unroll
    for (int k1 = 1; k1 < N1; ++k1) v[k1] = cmul(v[k1], tw128_runtime<INV>(n2 * k1 * (128 / N)));
#pragma unroll
    for (int k1 = 0; k1 < N1; ++k1) st(N2 * k1 + n2, v[k1]);
  }
}

// ld(slot); out(frequency, slot, value).
template <int N, bool INV, class LoadFn, class OutFn>
FBF_HD void fft_two_step_second(LoadFn ld, OutFn out) {
  constexpr int N1 = Split<N>::N1, N2 = Split<N>::N2;
#pragma unroll 1
  for (int k1 = 0; k1 < N1; ++k1) {
    float2 u[N2];
#pragma unroll
    for (int n2 = 0; n2 < N2; ++n2) u[n2] = ld(N2 * k1 + n2);
    fft_inreg<N2, INV>(u);
#pragma unroll
    for (int k2 = 0; k2 < N2; ++k2) out(k1 + N1 * k2, N2 * k1 + k2, u[k2]);
  }
}

// Two real rows a, b transformed as one complex line z = a + i b:
//   A[k] = (Z[k] + conj(Z[N-k])) / 2,   B[k] = (Z[k] - conj(Z[N-k])) / (2i).
FBF_HD void untangle_pair(float2 zk, float2 znk, float2& a, float2& b) {
  a = make_float2(0.5f * (zk.x + znk.x), 0.5f * (zk.y - znk.y));
  b = make_float2(0.5f * (zk.y + znk.y), -0.5f * (zk.x - znk.x));
}
// Inverse of the above for the two half spectra of real rows:
//   Z[k] = A[k] + i B[k]  (k <= N/2),   Z[N-k] = conj(A[k]) + i conj(B[k]).
FBF_HD float2 tangle_low(float2 a, float2 b) { return make_float2(a.x - b.y, a.y + b.x); }
FBF_HD float2 tangle_high(float2 a, float2 b) { return make_float2(a.x + b.y, b.x - a.y); }

// ---------------------------------------------------------------------------
// Geometry shared by host launch code, device code and the host harness
// ---------------------------------------------------------------------------
static inline int round_up(int v, int m) { return (v + m - 1) / m * m; }

// Smallest pitch >= n (in float2 units) such that groups of T consecutive planes
// of neighbouring lines fall on different banks.
static inline int plane_pitch(int n, int T) {
  if (T >= 16) return round_up(n, 16);
  int p = round_up(n, 16) + T;
  while (p - 16 >= n) p -= 16;
  return p;
}

struct FftGeom {
  int N, T;
  int he, we;      // extent of the non-zero region inside the N x N square (offset included)
  int hh;          // row pairs: rows (j, j + hh) share one complex line
  int pitch1;      // line pitch of the row-pass buffer  [x][line1], odd
  int pitch2;      // line pitch of the column buffers   [y][line2]
  int lines1;      // hh * T
  int lines2;      // (N/2 + 1) * T
  int rows1;       // rows of the row-pass buffer
  int threads;
  int off_a, off_b;  // byte offsets of the two shared-memory regions
  int smem_bytes;
};

static inline bool two_step(int N) { return N > 32; }

// Forward: region A = row-pass buffer, region B = column buffer ("mid").  For the
// single-step sizes both alias (a thread takes its whole line into registers
// before the barrier that precedes the first write of mid).
static inline FftGeom forward_geom(int N, int T, int h, int w, int pad_u, int pad_l) {
  FftGeom g;
  g.N = N;
  g.T = T;
  g.he = h + pad_u;
  g.we = w + pad_l;
  g.hh = (g.he + 1) / 2;
  g.lines1 = g.hh * T;
  g.lines2 = (N / 2 + 1) * T;
  g.pitch1 = g.lines1 | 1;
  g.pitch2 = plane_pitch(g.lines2, T);
  g.rows1 = two_step(N) ? N : g.we;
  const int bytes_a = g.rows1 * g.pitch1 * 8;
  const int bytes_b = (two_step(N) ? N : g.he) * g.pitch2 * 8;
  g.off_a = 0;
  if (two_step(N)) {
    g.off_b = round_up(bytes_a, 16);
    g.smem_bytes = g.off_b + bytes_b;
  } else {
    g.off_b = 0;
    g.smem_bytes = bytes_a > bytes_b ? bytes_a : bytes_b;
  }
  const int need = g.lines1 > g.lines2 ? g.lines1 : g.lines2;
  g.threads = round_up(need < 64 ? 64 : need, 32);
  if (g.threads > 512) g.threads = 512;
  return g;
}

// Inverse: he x we is the crop window (oh x ow); region A = column scratch
// (two-step only) and later the row-pass lines, region B = mid and later the
// staged real output.
static inline FftGeom inverse_geom(int N, int T, int oh, int ow) {
  FftGeom g;
  g.N = N;
  g.T = T;
  g.he = oh;
  g.we = ow;
  g.hh = (oh + 1) / 2;
  g.lines1 = g.hh * T;
  g.lines2 = (N / 2 + 1) * T;
  g.pitch1 = g.lines1 | 1;
  g.pitch2 = plane_pitch(g.lines2, T);
  g.rows1 = N;
  int bytes_a = 0;
  if (two_step(N)) {
    const int col = N * g.pitch2 * 8, row = N * g.pitch1 * 8;
    bytes_a = col > row ? col : row;
  }
  const int mid = oh * g.pitch2 * 8;
  const int stage = T * ((oh * ow) | 1) * 4;
  const int bytes_b = mid > stage ? mid : stage;
  g.off_a = 0;
  g.off_b = round_up(bytes_a, 16);
  g.smem_bytes = g.off_b + bytes_b;
  const int need = g.lines1 > g.lines2 ? g.lines1 : g.lines2;
  g.threads = round_up(need < 64 ? 64 : need, 32);
  if (g.threads > 512) g.threads = 512;
  return g;
}

// ---------------------------------------------------------------------------
// Kernel parameters
// ---------------------------------------------------------------------------
// A tile is T planes with consecutive `inner` index at one `row` of the spectrum.
// Real plane of (row, inner) starts at real + (row*real_row_stride +
// inner*real_inner_stride) * h * w  (strides counted in planes), so the same
// kernel writes the spectrum as [bin][d1][d2] or [bin][d2][d1].
struct FftParams {
  const float* real_in;   // forward input
  float* real_out;        // inverse output
  float2* spec;           // [bins][n_rows][kc]
  const float* bias;      // inverse only: added per inner index, may be null
  int h, w;               // extent of the real planes
  int off_y, off_x;       // forward: placement offset; inverse: crop origin
  int n_rows, n_inner;    // valid rows / planes along inner
  int kc;                 // padded inner extent of the spectrum (multiple of 4)
  long long real_row_stride, real_inner_stride;
  int accumulate;         // inverse only: real_out += result
};

// Registers a thread keeps across a barrier (single-step sizes only).
template <int N>
struct LineRegs {
  float2 v[N <= 32 ? N : 1];
};

// ===========================================================================
// Forward kernel phases.  Block (tile, row): planes inner0 .. inner0+T-1 of `row`.
// ===========================================================================
template <int N, int T>
struct Forward {
  static constexpr bool kTwoStep = (N > 32);

  // Phase 0: real planes -> row-pass buffer, rows (j, j+hh) packed as (re, im).
  static FBF_HD void load(const FftParams& p, const FftGeom& g, char* smem, int tid, int nthreads,
                          int row, int inner0) {
    float2* ra = reinterpret_cast<float2*>(smem + g.off_a);
    const int per_plane = g.hh * g.we;
    const int total = per_plane * T;
    for (int i = tid; i < total; i += nthreads) {
      const int t = i / per_plane;
      const int r = i - t * per_plane;
      const int j = r / g.we;
      const int xx = r - j * g.we;
      float a = 0.f, b = 0.f;
      const int inner = inner0 + t;
      if (inner < p.n_inner) {
        const float* plane =
            p.real_in + (row * p.real_row_stride + inner * p.real_inner_stride) * (long long)(p.h * p.w);
        const int x = xx - p.off_x;
        const int ya = j - p.off_y, yb = j + g.hh - p.off_y;
        if (x >= 0) {
          if (ya >= 0 && ya < p.h) a = plane[ya * p.w + x];
          if (yb >= 0 && yb < p.h) b = plane[yb * p.w + x];
        }
      }
      ra[xx * g.pitch1 + j * T + t] = make_float2(a, b);
    }
    if (kTwoStep) {  // columns the in-place transform reads beyond the data
      const int extra = (N - g.we) * g.lines1;
      for (int i = tid; i < extra; i += nthreads) {
        const int xx = g.we + i / g.lines1;
        ra[xx * g.pitch1 + (i % g.lines1)] = make_float2(0.f, 0.f);
      }
    }
  }

  // Phase 1a (single step): a line into registers.
  static FBF_HD void row_fetch(const FftGeom& g, const char* smem, int line, LineRegs<N>& regs) {
    if constexpr (!kTwoStep) {
      if (line >= g.lines1) return;
      const float2* ra = reinterpret_cast<const float2*>(smem + g.off_a);
#pragma unroll
      for (int xx = 0; xx < N; ++xx)
        regs.v[xx] = xx < g.we ? ra[xx * g.pitch1 + line] : make_float2(0.f, 0.f);
    }
  }

  // Phase 1b: transform along x, split the row pair, write mid[y][kx*T + t].
  static FBF_HD void row_pass(const FftGeom& g, char* smem, int line, LineRegs<N>& regs) {
    if (line >= g.lines1) return;
    float2* mid = reinterpret_cast<float2*>(smem + g.off_b);
    const int j = line / T, t = line - j * T;
    const bool has_b = (j + g.hh) < g.he;
    if constexpr (!kTwoStep) {
      fft_inreg<N, false>(regs.v);
#pragma unroll
      for (int k = 0; k <= N / 2; ++k) {
        float2 a, b;
        untangle_pair(regs.v[k], regs.v[(N - k) % N], a, b);
        mid[j * g.pitch2 + k * T + t] = a;
        if (has_b) mid[(j + g.hh) * g.pitch2 + k * T + t] = b;
      }
    } else {
      float2* ra = reinterpret_cast<float2*>(smem + g.off_a) + line;
      const int pitch = g.pitch1;
      fft_two_step_first<N, false>([&](int n) { return ra[n * pitch]; },
                                   [&](int slot, float2 v) { ra[slot * pitch] = v; });
      fft_two_step_second<N, false>([&](int slot) { return ra[slot * pitch]; },
                                    [&](int, int slot, float2 v) { ra[slot * pitch] = v; });
#pragma unroll 1
      for (int k = 0; k <= N / 2; ++k) {
        float2 a, b;
        untangle_pair(ra[slot_of_frequency<N>(k) * pitch],
                      ra[slot_of_frequency<N>((N - k) % N) * pitch], a, b);
        mid[j * g.pitch2 + k * T + t] = a;
        if (has_b) mid[(j + g.hh) * g.pitch2 + k * T + t] = b;
      }
    }
  }

  // Phase 2: transform along y for line2 = kx*T + t and write the spectrum.
  static FBF_HD void col_pass(const FftParams& p, const FftGeom& g, char* smem, int line, int row,
                              int inner0) {
    if (line >= g.lines2) return;
    float2* mid = reinterpret_cast<float2*>(smem + g.off_b) + line;
    const int kx = line / T, t = line - kx * T;
    const int inner = inner0 + t;
    if (inner >= p.kc) return;
    const long long bin_stride = (long long)p.n_rows * p.kc;
    float2* dst = p.spec + ((long long)kx * N) * bin_stride + (long long)row * p.kc + inner;
    const int pitch = g.pitch2;
    const int he = g.he;
    if constexpr (!kTwoStep) {
      float2 u[N];
#pragma unroll
      for (int y = 0; y < N; ++y) u[y] = y < he ? mid[y * pitch] : make_float2(0.f, 0.f);
      fft_inreg<N, false>(u);
#pragma unroll
      for (int ky = 0; ky < N; ++ky) dst[ky * bin_stride] = u[ky];
    } else {
      fft_two_step_first<N, false>(
          [&](int n) { return n < he ? mid[n * pitch] : make_float2(0.f, 0.f); },
          [&](int slot, float2 v) { mid[slot * pitch] = v; });
      fft_two_step_second<N, false>([&](int slot) { return mid[slot * pitch]; },
                                    [&](int ky, int, float2 v) { dst[ky * bin_stride] = v; });
    }
  }
};

// ===========================================================================
// Inverse kernel phases.
// ===========================================================================
template <int N, int T>
struct Inverse {
  static constexpr bool kTwoStep = (N > 32);

  // Phase 1: inverse transform along y of line2 = kx*T + t, keep the crop rows.
  static FBF_HD void col_pass(const FftParams& p, const FftGeom& g, char* smem, int line, int row,
                              int inner0) {
    if (line >= g.lines2) return;
    float2* mid = reinterpret_cast<float2*>(smem + g.off_b) + line;
    const int kx = line / T, t = line - kx * T;
    const int inner = inner0 + t;
    const bool live = inner < p.n_inner;
    const long long bin_stride = (long long)p.n_rows * p.kc;
    const float2* src = p.spec + ((long long)kx * N) * bin_stride + (long long)row * p.kc + inner;
    const int pitch = g.pitch2;
    const int y0 = p.off_y, y1 = p.off_y + g.he;
    if constexpr (!kTwoStep) {
      float2 u[N];
#pragma unroll
      for (int ky = 0; ky < N; ++ky) u[ky] = live ? src[ky * bin_stride] : make_float2(0.f, 0.f);
      fft_inreg<N, true>(u);
#pragma unroll
      for (int y = 0; y < N; ++y)
        if (y >= y0 && y < y1) mid[(y - y0) * pitch] = u[y];
    } else {
      float2* col = reinterpret_cast<float2*>(smem + g.off_a) + line;
      fft_two_step_first<N, true>(
          [&](int n) { return live ? src[n * bin_stride] : make_float2(0.f, 0.f); },
          [&](int slot, float2 v) { col[slot * pitch] = v; });
      fft_two_step_second<N, true>([&](int slot) { return col[slot * pitch]; },
                                   [&](int y, int, float2 v) {
                                     if (y >= y0 && y < y1) mid[(y - y0) * pitch] = v;
                                   });
    }
  }

  // Phase 2a: gather the two half spectra of rows (j, j+hh) into one complex line
  // (registers, or the private shared-memory line for the two-step sizes).
  static FBF_HD void row_fetch(const FftGeom& g, char* smem, int line, LineRegs<N>& regs) {
    if (line >= g.lines1) return;
    const float2* mid = reinterpret_cast<const float2*>(smem + g.off_b);
    const int j = line / T, t = line - j * T;
    const bool has_b = (j + g.hh) < g.he;
    const float2* pa = mid + j * g.pitch2 + t;
    const float2* pb = mid + (j + g.hh) * g.pitch2 + t;
    if constexpr (!kTwoStep) {
#pragma unroll
      for (int k = 0; k <= N / 2; ++k) {
        const float2 a = pa[k * T];
        const float2 b = has_b ? pb[k * T] : make_float2(0.f, 0.f);
        regs.v[k] = tangle_low(a, b);
        if (k > 0 && k < N / 2) regs.v[N - k] = tangle_high(a, b);
      }
    } else {
      float2* ra = reinterpret_cast<float2*>(smem + g.off_a) + line;
      const int pitch = g.pitch1;
#pragma unroll 1
      for (int k = 0; k <= N / 2; ++k) {
        const float2 a = pa[k * T];
        const float2 b = has_b ? pb[k * T] : make_float2(0.f, 0.f);
        ra[k * pitch] = tangle_low(a, b);
        if (k > 0 && k < N / 2) ra[(N - k) * pitch] = tangle_high(a, b);
      }
    }
  }

  // Phase 2b: inverse transform along x, stage the crop columns as real rows.
  static FBF_HD void row_pass(const FftParams& p, const FftGeom& g, char* smem, int line,
                              LineRegs<N>& regs) {
    if (line >= g.lines1) return;
    float* stage = reinterpret_cast<float*>(smem + g.off_b);
    const int j = line / T, t = line - j * T;
    const bool has_b = (j + g.hh) < g.he;
    const int plane_pitch_f = (g.he * g.we) | 1;
    float* sa = stage + t * plane_pitch_f + j * g.we;
    float* sb = stage + t * plane_pitch_f + (j + g.hh) * g.we;
    const int x0 = p.off_x, x1 = p.off_x + g.we;
    if constexpr (!kTwoStep) {
      fft_inreg<N, true>(regs.v);
#pragma unroll
      for (int x = 0; x < N; ++x) {
        if (x >= x0 && x < x1) {
          sa[x - x0] = regs.v[x].x;
          if (has_b) sb[x - x0] = regs.v[x].y;
        }
      }
    } else {
      float2* ra = reinterpret_cast<float2*>(smem + g.off_a) + line;
      const int pitch = g.pitch1;
      fft_two_step_first<N, true>([&](int n) { return ra[n * pitch]; },
                                  [&](int slot, float2 v) { ra[slot * pitch] = v; });
      fft_two_step_second<N, true>([&](int slot) { return ra[slot * pitch]; },
                                   [&](int x, int, float2 v) {
                                     if (x >= x0 && x < x1) {
                                       sa[x - x0] = v.x;
                                       if (has_b) sb[x - x0] = v.y;
                                     }
                                   });
    }
  }

  // Phase 3: staged planes -> global, bias added per plane.
  static FBF_HD void store(const FftParams& p, const FftGeom& g, const char* smem, int tid,
                           int nthreads, int row, int inner0) {
    const float* stage = reinterpret_cast<const float*>(smem + g.off_b);
    const int per_plane = g.he * g.we;
    const int plane_pitch_f = per_plane | 1;
    const int total = per_plane * T;
    for (int i = tid; i < total; i += nthreads) {
      const int t = i / per_plane;
      const int r = i - t * per_plane;
      const int inner = inner0 + t;
      if (inner >= p.n_inner) continue;
      float v = stage[t * plane_pitch_f + r];
      if (p.bias) v += p.bias[inner];
      float* dst = p.real_out +
                   (row * p.real_row_stride + inner * p.real_inner_stride) * (long long)per_plane + r;
      *dst = p.accumulate ? (*dst + v) : v;
    }
  }
};

}  // namespace fbfft
