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
//     spectrum[bin][row][inner]   complex fp32,  bin = ky * (N/2+1) + kx,  kx in [0, N/2]
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

// Asynchronous 4-byte global -> shared copy: no register staging, so a thread keeps as
// many in flight as it issues; async_copy_wait() before the barrier that publishes the
// data.  The host harness copies synchronously.
FBF_HD void async_copy4(float* smem_dst, const float* gmem_src) {
#if defined(__CUDA_ARCH__)
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(smem_dst)),
               "l"(gmem_src)
               : "memory");
#else
  *smem_dst = *gmem_src;
#endif
}
// 16-byte variant: both addresses 16-byte aligned.
FBF_HD void async_copy16(float* smem_dst, const float* gmem_src) {
#if defined(__CUDA_ARCH__)
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(smem_dst)),
               "l"(gmem_src)
               : "memory");
#else
  for (int i = 0; i < 4; ++i) smem_dst[i] = gmem_src[i];
#endif
}
// Four floats moved as one 16-byte access.
struct alignas(16) Quad {
  float a, b, c, d;
};
FBF_HD void async_copy_wait() {
#if defined(__CUDA_ARCH__)
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
#endif
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

// Sizes above 32 are split as N = N1 * N2 (input index n = N2*n1 + n2, output index
// k = k1 + N1*k2): N2 threads each do an N1-point transform and a twiddle, then N1
// threads each do an N2-point transform.
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
constexpr int plane_pitch(int n, int T) {
  if (T >= 16) return (n + 15) / 16 * 16;
  int p = (n + 15) / 16 * 16 + T;
  while (p - 16 >= n) p -= 16;
  return p;
}

struct FftGeom {
  int N, T;
  int he, we;      // forward: extent of the data inside the N x N square (offset included);
                   // inverse: the crop window
  int hh;          // row pairs: rows (j, j + hh) share one complex line
  int hh_magic;    // ceil(2^16 / hh): line / hh == (line * hh_magic) >> 16 for line < 512, hh <= 64
  int pitch1;      // cooperative: line pitch of the row buffer; thread-per-line: pitch of a staged real plane (floats)
  int pitch2;      // row pitch of the column buffer ("mid")
  int lines1;      // hh * T
  int lines2;      // (N/2 + 1) * T
  int chunk;       // cooperative kernels: row lines processed per round
  int threads;
  int off_a, off_b;  // byte offsets of the two shared-memory regions
  int smem_bytes;
};

static inline bool cooperative(int N) { return N > 32; }
#define FBF_COOP_THREADS 256  // measured slower: 288 (whole rounds in the column phases, but a 96-register cap), 384, 512
static_assert(FBF_COOP_THREADS % 32 == 0, "whole warps, and a multiple of every N2");
static inline int coop_threads() { return FBF_COOP_THREADS; }

// Thread-per-line kernels (N <= 32): region A = the T real planes as they lie in global
// memory (pitch1 floats apart), region B = column buffer [y][kx*T + t]; they alias (a thread
// takes its whole line into registers before the barrier that precedes the first write of the
// other region).
// Cooperative kernels (N > 32): region A = one chunk of row lines
// [line][k1*(N2+1) + n2], region B = column buffer [y or slot][t*(N/2+1) + kx].
// Pitch (floats) of one staged real plane of n elements: a multiple of 4 (16-byte copies)
// with room for the 0..3 floats by which a plane is shifted to share the 16-byte phase of
// its global address, and an odd number of 16-byte units so that neighbouring planes start
// in different banks.
static inline int stage_pitch(int n) {
  int p = round_up(n + 3, 4);
  if (((p >> 2) & 1) == 0) p += 4;
  return p;
}

// Row pitch (float2) of the cooperative kernels' column buffer: at least `cols`, and 8 modulo 16, so that
// the eight-element runs that the lanes of neighbouring row lines store in one instruction (row step 2)
// fall into different halves of the banks.  The column phases walk along the rows and do not care.
constexpr int coop_mid_pitch(int cols) { return (cols + 7) / 16 * 16 + 8; }
// Distance (float2) between the planes of a tile inside a row of the column buffer: N/2 + 1 values per
// plane, spaced 4 modulo 16 apart when a tile has several planes, so that the lanes that take the T
// planes of neighbouring bins (column step 2 of the forward, column step 1 of the inverse) use
// different banks.
constexpr int coop_plane_stride(int kx, int T) { return T == 1 ? kx : (kx + 11) / 16 * 16 + 4; }

// `plane_elems`: elements of one real plane as it lies in global memory.
static inline FftGeom make_geom(int N, int T, int he, int we, int plane_elems, bool inverse) {
  FftGeom g;
  g.N = N;
  g.T = T;
  g.he = he;
  g.we = we;
  g.hh = (he + 1) / 2;
  g.hh_magic = (65536 + g.hh - 1) / g.hh;
  g.lines1 = g.hh * T;
  g.lines2 = (N / 2 + 1) * T;
  g.off_a = 0;
  if (!cooperative(N)) {
    g.pitch1 = stage_pitch(plane_elems);
    g.pitch2 = plane_pitch(g.lines2, T);
    g.chunk = g.lines1;
    const int bytes_a = T * g.pitch1 * 4;
    const int bytes_b = he * g.pitch2 * 8;
    g.off_b = 0;
    g.smem_bytes = bytes_a > bytes_b ? bytes_a : bytes_b;
    g.threads = round_up(g.lines2 < 64 ? 64 : g.lines2, 32);
  } else {
    const int n1 = N == 64 ? 8 : 8, n2 = N / n1;
    g.pitch1 = n1 * (n2 + 1);          // = CoopLayout::PITCH1
    g.pitch2 = coop_mid_pitch(T * coop_plane_stride(N / 2 + 1, T));  // = CoopLayout::PITCH2
    g.chunk = N == 64 ? 64 : 32;
    if (g.chunk > g.lines1) g.chunk = g.lines1;
    const int bytes_a = g.chunk * g.pitch1 * 8;
    g.off_b = round_up(bytes_a, 16);
    g.smem_bytes = g.off_b + N * g.pitch2 * 8;
    g.threads = coop_threads();
  }
  return g;
}

static inline FftGeom forward_geom(int N, int T, int h, int w, int pad_u, int pad_l) {
  return make_geom(N, T, h + pad_u, w + pad_l, h * w, false);
}
static inline FftGeom inverse_geom(int N, int T, int oh, int ow) {
  return make_geom(N, T, oh, ow, oh * ow, true);
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
  float2* spec;           // element (bin, row, inner) at bin*spec_bin + row*spec_row + inner*spec_inner:
                          //   bin-major   [bins][n_rows][kc]:      spec_bin = n_rows*kc, spec_row = kc, spec_inner = 1
                          //   plane-major [n_rows][n_inner][bins]: spec_bin = 1, spec_row = n_inner*bins, spec_inner = bins
  long long spec_bin, spec_row, spec_inner;
  const float* bias;      // inverse only: added per inner index (per row when bias_by_row), may be null
  int bias_by_row;
  int h, w;               // extent of the real planes
  int off_y, off_x;       // forward: placement offset; inverse: crop origin
  int n_rows, n_inner;    // valid rows / planes along inner
  int kc;                 // padded inner extent of the spectrum (multiple of 4)
  long long real_row_stride, real_inner_stride;
  int accumulate;         // inverse only: real_out += result
};

// Registers a thread keeps across a barrier (thread-per-line sizes only).
template <int N>
struct LineRegs {
  float2 v[N <= 32 ? N : 1];
};

// ===========================================================================
// Thread-per-line kernels, N <= 32.  Block (tile, row): planes inner0 .. inner0+T-1.
//
// These kernels are bound by instruction issue, not by arithmetic, so the layout is
// chosen for cheap addressing: the real planes are staged in shared memory exactly as
// they lie in global memory (16-byte copies), each plane shifted by the 0..3 floats
// that give it the 16-byte phase of its global address, and every shared-memory pitch
// that an unrolled loop walks is a compile-time constant.
// ===========================================================================
template <int N, int T>
struct TileLayout {
  static constexpr int KX = N / 2 + 1;
  static constexpr int LINES2 = KX * T;
  static constexpr int PITCH2 = plane_pitch(LINES2, T);  // row pitch of mid (float2)
};

// log2 of the lanes that copy one plane of n floats together (3 floats of head and tail
// need at most 3 lanes).
FBF_HD int copy_group_shift(int n) { return n <= 64 ? 3 : n <= 192 ? 4 : 5; }

// 16-byte phase of a float address, in floats.
FBF_HD int phase16(const float* ptr) { return (int)((reinterpret_cast<uintptr_t>(ptr) >> 2) & 3); }

template <int N, int T>
struct Forward {
  using L = TileLayout<N, T>;

  static FBF_HD const float* plane_ptr(const FftParams& p, int row, int inner) {
    return p.real_in + (row * p.real_row_stride + inner * p.real_inner_stride) * ((long long)p.h * p.w);
  }

  // Phase 0: real planes -> stage, plane t at stage + t*pitch1 + phase16(plane); warps take planes.
  static FBF_HD void load(const FftParams& p, const FftGeom& g, char* smem, int tid, int nthreads,
                          int row, int inner0) {
    float* stage = reinterpret_cast<float*>(smem + g.off_a);
    const int hw = p.h * p.w;
    // small planes: a warp splits into groups of 8 or 16 lanes that take one plane each
    const int lp_shift = copy_group_shift(hw);
    const int lanes = 1 << lp_shift, lane = tid & (lanes - 1);
    const int group = tid >> lp_shift, ngroups = nthreads >> lp_shift;
    for (int t = group; t < T; t += ngroups) {
      if (inner0 + t >= p.n_inner) break;
      const float* src = plane_ptr(p, row, inner0 + t);
      const int shift = phase16(src);
      float* dst = stage + t * g.pitch1 + shift;
      int head = (4 - shift) & 3;
      if (head > hw) head = hw;
      const int chunks = (hw - head) >> 2;
      const int tail0 = head + 4 * chunks;
      for (int c = lane; c < chunks; c += lanes) async_copy16(dst + head + 4 * c, src + head + 4 * c);
      if (lane < head) async_copy4(dst + lane, src + lane);
      if (lane < hw - tail0) async_copy4(dst + tail0 + lane, src + tail0 + lane);
    }
    async_copy_wait();
  }

  // Phase 1a: rows (j, j+hh) of plane t into registers as (re, im), zero outside the plane.
  static FBF_HD void row_fetch(const FftParams& p, const FftGeom& g, const char* smem, int line, int row,
                               int inner0, LineRegs<N>& regs) {
    if (line >= g.lines1) return;
    const float* stage = reinterpret_cast<const float*>(smem + g.off_a);
    const int j = line / T, t = line - j * T;
    const bool live = inner0 + t < p.n_inner;
    const float* sp = stage + t * g.pitch1 + phase16(plane_ptr(p, row, inner0 + t));
    const int ya = j - p.off_y, yb = ya + g.hh;
    const bool va = live && (unsigned)ya < (unsigned)p.h, vb = live && (unsigned)yb < (unsigned)p.h;
    const float* pa = sp + ya * p.w - p.off_x;
    const float* pb = pa + g.hh * p.w;
    if constexpr (N >= 4) {
      // Rows that start on 16-byte boundaries of the staged plane (width and offset multiples of four,
      // plane staged without a shift) are read four floats at a time: a quarter of the loads, and the
      // eight planes that neighbouring lanes read lie 16 bytes apart modulo the banks, where scalar
      // loads of rows a multiple of four floats long collide four ways.
      if (((p.w | p.off_x) & 3) == 0 && sp == stage + t * g.pitch1) {
        const Quad zero = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < N / 4; ++c) {
          const bool px = (unsigned)(4 * c - p.off_x) < (unsigned)p.w;
          const Quad a = va && px ? *reinterpret_cast<const Quad*>(pa + 4 * c) : zero;
          const Quad b = vb && px ? *reinterpret_cast<const Quad*>(pb + 4 * c) : zero;
          regs.v[4 * c + 0] = make_float2(a.a, b.a);
          regs.v[4 * c + 1] = make_float2(a.b, b.b);
          regs.v[4 * c + 2] = make_float2(a.c, b.c);
          regs.v[4 * c + 3] = make_float2(a.d, b.d);
        }
        return;
      }
    }
#pragma unroll
    for (int x = 0; x < N; ++x) {
      const bool px = (unsigned)(x - p.off_x) < (unsigned)p.w;
      regs.v[x] = make_float2(va && px ? pa[x] : 0.f, vb && px ? pb[x] : 0.f);
    }
  }

  // Phase 1b: transform along x, split the row pair, write mid[y][kx*T + t].
  static FBF_HD void row_pass(const FftGeom& g, char* smem, int line, LineRegs<N>& regs) {
    if (line >= g.lines1) return;
    float2* mid = reinterpret_cast<float2*>(smem + g.off_b);
    const int j = line / T, t = line - j * T;
    const bool has_b = (j + g.hh) < g.he;
    float2* ma = mid + j * L::PITCH2 + t;
    float2* mb = ma + g.hh * L::PITCH2;
    fft_inreg<N, false>(regs.v);
#pragma unroll
    for (int k = 0; k <= N / 2; ++k) {
      float2 a, b;
      untangle_pair(regs.v[k], regs.v[(N - k) % N], a, b);
      ma[k * T] = a;
      if (has_b) mb[k * T] = b;
    }
  }

  // Phase 2: transform along y for line2 = kx*T + t and write the spectrum.
  static FBF_HD void col_pass(const FftParams& p, const FftGeom& g, char* smem, int line, int row,
                              int inner0) {
    if (line >= L::LINES2) return;
    const float2* mid = reinterpret_cast<const float2*>(smem + g.off_b) + line;
    const int kx = line / T, t = line - kx * T;
    const int inner = inner0 + t;
    if (inner >= p.kc) return;
    const int he = g.he;
    float2 u[N];
#pragma unroll
    for (int y = 0; y < N; ++y) u[y] = y < he ? mid[y * L::PITCH2] : make_float2(0.f, 0.f);
    fft_inreg<N, false>(u);
    // 32-bit offsets inside the row: the launcher refuses spectra of 2^31 elements or more
    float2* dst = p.spec + ((long long)kx * p.spec_bin + row * p.spec_row + inner * p.spec_inner);
    const int step = L::KX * (int)p.spec_bin;
#pragma unroll
    for (int ky = 0; ky < N; ++ky) dst[ky * step] = u[ky];
  }
};

template <int N, int T>
struct Inverse {
  using L = TileLayout<N, T>;

  static FBF_HD float* plane_ptr(const FftParams& p, const FftGeom& g, int row, int inner) {
    return p.real_out + (row * p.real_row_stride + inner * p.real_inner_stride) * ((long long)g.he * g.we);
  }

  // Phase 1: inverse transform along y of line2 = kx*T + t, keep the crop rows.
  static FBF_HD void col_pass(const FftParams& p, const FftGeom& g, char* smem, int line, int row,
                              int inner0) {
    if (line >= L::LINES2) return;
    const int kx = line / T, t = line - kx * T;
    const int inner = inner0 + t;
    const bool live = inner < p.n_inner;
    const float2* src = p.spec + ((long long)kx * p.spec_bin + row * p.spec_row + inner * p.spec_inner);
    const int step = L::KX * (int)p.spec_bin;
    float2 u[N];
#pragma unroll
    for (int ky = 0; ky < N; ++ky) u[ky] = live ? src[ky * step] : make_float2(0.f, 0.f);
    fft_inreg<N, true>(u);
    // row y of the square lands in row y - off_y of mid
    float2* mid = reinterpret_cast<float2*>(smem + g.off_b) + line - p.off_y * L::PITCH2;
    const unsigned he = (unsigned)g.he;
#pragma unroll
    for (int y = 0; y < N; ++y)
      if ((unsigned)(y - p.off_y) < he) mid[y * L::PITCH2] = u[y];
  }

  // Phase 2a: gather the two half spectra of rows (j, j+hh) into one complex line.
  static FBF_HD void row_fetch(const FftGeom& g, char* smem, int line, LineRegs<N>& regs) {
    if (line >= g.lines1) return;
    const float2* mid = reinterpret_cast<const float2*>(smem + g.off_b);
    const int j = line / T, t = line - j * T;
    const bool has_b = (j + g.hh) < g.he;
    const float2* pa = mid + j * L::PITCH2 + t;
    const float2* pb = pa + g.hh * L::PITCH2;
#pragma unroll
    for (int k = 0; k <= N / 2; ++k) {
      const float2 a = pa[k * T];
      const float2 b = has_b ? pb[k * T] : make_float2(0.f, 0.f);
      regs.v[k] = tangle_low(a, b);
      if (k > 0 && k < N / 2) regs.v[N - k] = tangle_high(a, b);
    }
  }

  // Phase 2b: inverse transform along x, stage the crop columns as real rows, plane t at
  // stage + t*pitch1 + phase16(its destination).
  static FBF_HD void row_pass(const FftParams& p, const FftGeom& g, char* smem, int line, int row,
                              int inner0, LineRegs<N>& regs) {
    if (line >= g.lines1) return;
    float* stage = reinterpret_cast<float*>(smem + g.off_a);
    const int j = line / T, t = line - j * T;
    const bool has_b = (j + g.hh) < g.he;
    const int shift = phase16(plane_ptr(p, g, row, inner0 + t));
    float* sa = stage + t * g.pitch1 + shift + j * g.we - p.off_x;
    float* sb = sa + g.hh * g.we;
    const unsigned we = (unsigned)g.we;
    fft_inreg<N, true>(regs.v);
    if constexpr (N >= 4) {
      // rows on 16-byte boundaries of the staged plane: four floats per store (see Forward::row_fetch)
      if (((g.we | p.off_x) & 3) == 0 && shift == 0) {
#pragma unroll
        for (int c = 0; c < N / 4; ++c) {
          if ((unsigned)(4 * c - p.off_x) < we) {
            const Quad a = {regs.v[4 * c].x, regs.v[4 * c + 1].x, regs.v[4 * c + 2].x, regs.v[4 * c + 3].x};
            *reinterpret_cast<Quad*>(sa + 4 * c) = a;
            if (has_b) {
              const Quad b = {regs.v[4 * c].y, regs.v[4 * c + 1].y, regs.v[4 * c + 2].y, regs.v[4 * c + 3].y};
              *reinterpret_cast<Quad*>(sb + 4 * c) = b;
            }
          }
        }
        return;
      }
    }
#pragma unroll
    for (int x = 0; x < N; ++x) {
      if ((unsigned)(x - p.off_x) < we) {
        sa[x] = regs.v[x].x;
        if (has_b) sb[x] = regs.v[x].y;
      }
    }
  }

  static FBF_HD float finish(const FftParams& p, float v, float bias, const float* dst) {
    return p.accumulate ? *dst + (v + bias) : v + bias;
  }

  // Phase 3: staged planes -> global in 16-byte pieces, bias added per plane; warps take planes.
  static FBF_HD void store(const FftParams& p, const FftGeom& g, const char* smem, int tid,
                           int nthreads, int row, int inner0) {
    const float* stage = reinterpret_cast<const float*>(smem + g.off_a);
    const int per_plane = g.he * g.we;
    const int lp_shift = copy_group_shift(per_plane);
    const int lanes = 1 << lp_shift, lane = tid & (lanes - 1);
    const int group = tid >> lp_shift, ngroups = nthreads >> lp_shift;
    for (int t = group; t < T; t += ngroups) {
      const int inner = inner0 + t;
      if (inner >= p.n_inner) break;
      const float bias = p.bias ? p.bias[p.bias_by_row ? row : inner] : 0.f;
      float* dst = plane_ptr(p, g, row, inner);
      const int shift = phase16(dst);
      const float* src = stage + t * g.pitch1 + shift;
      int head = (4 - shift) & 3;
      if (head > per_plane) head = per_plane;
      const int chunks = (per_plane - head) >> 2;
      const int tail0 = head + 4 * chunks;
      for (int c = lane; c < chunks; c += lanes) {
        const Quad s4 = *reinterpret_cast<const Quad*>(src + head + 4 * c);
        float* d4 = dst + head + 4 * c;
        const Quad q{finish(p, s4.a, bias, d4), finish(p, s4.b, bias, d4 + 1), finish(p, s4.c, bias, d4 + 2),
                     finish(p, s4.d, bias, d4 + 3)};
        *reinterpret_cast<Quad*>(d4) = q;
      }
      if (lane < head) dst[lane] = finish(p, src[lane], bias, dst + lane);
      if (lane < per_plane - tail0) dst[tail0 + lane] = finish(p, src[tail0 + lane], bias, dst + tail0 + lane);
    }
  }
};

// ===========================================================================
// Cooperative kernels, N = 64 / 128.  Work is split into items that the threads of
// the block pick up round-robin; barriers separate the phases.  Shared-memory
// pitches are compile-time constants so that every access has an immediate offset.
// ===========================================================================
template <int N, int T>
struct CoopLayout {
  static constexpr int N1 = Split<N>::N1, N2 = Split<N>::N2, KX = N / 2 + 1;
  static constexpr int COLS = T * KX;                 // columns of a tile: (t, kx)
  static constexpr int KXP = coop_plane_stride(KX, T); // column (t, kx) lies at t * KXP + kx of a mid row
  static FBF_HD int col_address(int col) {             // column index t * KX + kx -> its place in a mid row
    if constexpr (T == 1) {
      return col;
    } else {
      const int t = col / KX;
      return col + t * (KXP - KX);
    }
  }
  // Row buffer line pitch (float2): 72 / 136, i.e. 8 modulo 16.  In the second row step the eight lanes of
  // a line read at a stride of N2 + 1 and cover half of the banks; the next line's lanes, 16 banks on, the
  // other half.  (The first row step stores 8 or 16 neighbouring values per line and does not care.)
  static constexpr int PITCH1 = N1 * (N2 + 1);
  static_assert(PITCH1 % 16 == 8, "neighbouring lines of the second row step: different halves of the banks");
  static constexpr int PITCH2 = coop_mid_pitch(T * KXP);  // mid row pitch (float2)
  static_assert(N1 == 8, "the residue pairing below is written for eight residues");
};

// Order of the residues k1 inside a group of eight neighbouring lanes: residues that
// hold each other's mirror image (k1, N1 - k1) sit in lanes that differ in bit 0;
// residues 0 and N1/2 mirror onto themselves.
FBF_HD int coop_residue_of_lane(int p) {
  return p == 0 ? 0 : p == 1 ? 4 : p == 2 ? 1 : p == 3 ? 7 : p == 4 ? 2 : p == 5 ? 6 : p == 6 ? 3 : 5;
}

// line = t * hh + j of a tile of T planes, without an integer division.
template <int T>
FBF_HD void coop_split_line(const FftGeom& g, int line, int& t, int& j) {
  if (T == 1) {
    t = 0;
    j = line;
  } else {
    t = (line * g.hh_magic) >> 16;
    j = line - t * g.hh;
  }
}

template <int N, int T>
struct CoopForward {
  using L = CoopLayout<N, T>;
  static constexpr int N1 = L::N1, N2 = L::N2, KX = L::KX;

  struct RowLoad {
    float2 v[N1];
    int slot;  // ll * PITCH1 + n2, or -1
    int n2;
  };

  static FBF_HD void row_fetch(const FftParams& p, const FftGeom& g, const float* base, long long tstride,
                               int inner0, int line0, int nl, int item, RowLoad& r) {
    r.slot = -1;
    if (item >= nl * N2) return;
    const int ll = item / N2, n2 = item - ll * N2;
    const int line = line0 + ll;
    int t, j;
    coop_split_line<T>(g, line, t, j);
    const bool live = inner0 + t < p.n_inner;
    const float* plane = base + t * tstride;
    const int ya = j - p.off_y, yb = j + g.hh - p.off_y;
    const bool va = live && ya >= 0 && ya < p.h, vb = live && yb >= 0 && yb < p.h;
    const float* pa = plane + ya * p.w + (n2 - p.off_x);
    const float* pb = plane + yb * p.w + (n2 - p.off_x);
#pragma unroll
    for (int n1 = 0; n1 < N1; ++n1) {
      const int x = N2 * n1 + n2 - p.off_x;
      const bool vx = x >= 0 && x < p.w;
      r.v[n1] = make_float2(va && vx ? pa[N2 * n1] : 0.f, vb && vx ? pb[N2 * n1] : 0.f);
    }
    r.slot = ll * L::PITCH1 + n2;
    r.n2 = n2;
  }

  static FBF_HD void row_transform(float2* rb, RowLoad& r, const float2 (&tw)[N1]) {
    if (r.slot < 0) return;
    fft_inreg<N1, false>(r.v);
    float2* dst = rb + r.slot;
    dst[0] = r.v[0];
#pragma unroll
    for (int k1 = 1; k1 < N1; ++k1) dst[k1 * (N2 + 1)] = cmul(r.v[k1], tw[k1]);
  }

  // Row step 1 for lines [line0, line0 + nl): straight from global memory (N2
  // neighbouring floats per row and lane group: whole 32-byte sectors), two items in
  // flight per thread, N1-point transform, twiddle, into the row buffer.
  static FBF_HD void row_step1(const FftParams& p, const FftGeom& g, char* smem, int tid, int nthreads,
                               int row, int inner0, int line0, int nl) {
    float2* rb = reinterpret_cast<float2*>(smem + g.off_a);
    const long long plane_elems = (long long)p.h * p.w;
    const float* base = p.real_in + (row * p.real_row_stride + inner0 * p.real_inner_stride) * plane_elems;
    const long long tstride = p.real_inner_stride * plane_elems;
    // the block size is a multiple of N2, so a thread meets the same n2 in all its items
    float2 tw[N1];
#pragma unroll
    for (int k1 = 0; k1 < N1; ++k1) tw[k1] = tw128_runtime<false>((tid % N2) * k1 * (128 / N));
    for (int item = tid; item < nl * N2; item += 2 * nthreads) {
      RowLoad r0, r1;
      row_fetch(p, g, base, tstride, inner0, line0, nl, item, r0);
      row_fetch(p, g, base, tstride, inner0, line0, nl, item + nthreads, r1);
      row_transform(rb, r0, tw);
      row_transform(rb, r1, tw);
    }
  }

  // Row step 2, first half: item = (line, lane position); the N2-point transform of
  // residue k1 of that line.
  static FBF_HD bool row_step2_fft(const FftGeom& g, const char* smem, int item, int nl, float2 (&u)[N2]) {
    if (item >= nl * N1) return false;
    const float2* rb = reinterpret_cast<const float2*>(smem + g.off_a);
    const int ll = item / N1, k1 = coop_residue_of_lane(item % N1);
    const float2* src = rb + ll * L::PITCH1 + k1 * (N2 + 1);
#pragma unroll
    for (int n2 = 0; n2 < N2; ++n2) u[n2] = src[n2];
    fft_inreg<N2, false>(u);
    return true;
  }

  // Row step 2, second half: Z[k] (own) meets Z[N-k] (own for residues 0 and N1/2, else
  // the odd-indexed outputs of the mirror residue, handed over by the neighbouring
  // lane); the row pair is split and written to mid.  Each lane of a mirror pair takes
  // the even-indexed half of its own outputs, which covers every frequency once.
  static FBF_HD void row_step2_split(const FftGeom& g, char* smem, int item, int line0,
                                     const float2 (&u)[N2], const float2 (&mirror_odd)[N2 / 2]) {
    float2* mid = reinterpret_cast<float2*>(smem + g.off_b);
    const int ll = item / N1, k1 = coop_residue_of_lane(item % N1);
    const int line = line0 + ll;
    int t, j;
    coop_split_line<T>(g, line, t, j);
    const bool has_b = (j + g.hh) < g.he;
    float2* ma = mid + j * L::PITCH2 + t * L::KXP;
    float2* mb = mid + (j + g.hh) * L::PITCH2 + t * L::KXP;
    if (k1 == 0 || k1 == N1 / 2) {
#pragma unroll
      for (int k2 = 0; k2 <= N2 / 2; ++k2) {
        const int k = k1 + N1 * k2;
        if (k > N / 2) continue;
        const float2 znk = (k1 == 0) ? u[(N2 - k2) % N2] : u[N2 - 1 - k2];
        float2 a, b;
        untangle_pair(u[k2], znk, a, b);
        ma[k] = a;
        if (has_b) mb[k] = b;
      }
    } else {
#pragma unroll
      for (int k2 = 0; k2 < N2; k2 += 2) {
        const int k = k1 + N1 * k2;
        const float2 other = mirror_odd[(N2 - 1 - k2) / 2];  // Z[N-k] = mirror[N2-1-k2]
        float2 a, b;
        if (k <= N / 2) {
          untangle_pair(u[k2], other, a, b);
          ma[k] = a;
          if (has_b) mb[k] = b;
        } else {
          untangle_pair(other, u[k2], a, b);
          ma[N - k] = a;
          if (has_b) mb[N - k] = b;
        }
      }
    }
  }

  // Column step 1, in place on mid: item (col, n2) owns rows {N2*n1 + n2}.
  static FBF_HD void col_step1(const FftGeom& g, char* smem, int tid, int nthreads) {
    float2* mid = reinterpret_cast<float2*>(smem + g.off_b);
    for (int item = tid; item < L::COLS * N2; item += nthreads) {
      const int n2 = item / L::COLS, col = item - n2 * L::COLS;
      float2* c = mid + L::col_address(col) + n2 * L::PITCH2;
      float2 v[N1];
#pragma unroll
      for (int n1 = 0; n1 < N1; ++n1)
        v[n1] = (N2 * n1 + n2) < g.he ? c[N2 * n1 * L::PITCH2] : make_float2(0.f, 0.f);
      fft_inreg<N1, false>(v);
      c[0] = v[0];
#pragma unroll
      for (int k1 = 1; k1 < N1; ++k1)
        c[N2 * k1 * L::PITCH2] = cmul(v[k1], tw128_runtime<false>(n2 * k1 * (128 / N)));
    }
  }

  // Column step 2: item (col, k1) reads rows {N2*k1 + n2} and writes bins ky = k1 + N1*k2.
  // PM: the spectrum is plane-major (bins contiguous), every stride a compile-time constant;
  // otherwise offsets are 32-bit (the launcher refuses spectra of 2^31 elements or more).
  template <bool PM>
  static FBF_HD void col_step2(const FftParams& p, const FftGeom& g, const char* smem, int tid,
                               int nthreads, int row, int inner0) {
    const float2* mid = reinterpret_cast<const float2*>(smem + g.off_b);
    const int bin_stride = PM ? 1 : (int)p.spec_bin;
    const int inner_stride = PM ? N * KX : (int)p.spec_inner;
    float2* base = p.spec + row * p.spec_row;
    for (int item = tid; item < L::COLS * N1; item += nthreads) {
      // neighbouring lanes take the T planes of one bin, so that their 8-byte stores share a line
      const int k1 = item / L::COLS, ci = item - k1 * L::COLS;
      const int kx = ci / T, t = ci - kx * T;
      const int col = t * L::KXP + kx;
      const int inner = inner0 + t;
      if (inner >= p.kc) continue;
      const float2* c = mid + col + N2 * k1 * L::PITCH2;
      float2 u[N2];
#pragma unroll
      for (int n2 = 0; n2 < N2; ++n2) u[n2] = c[n2 * L::PITCH2];
      fft_inreg<N2, false>(u);
      float2* dst = base + ((k1 * KX + kx) * bin_stride + inner * inner_stride);
      const int step = (N1 * KX) * bin_stride;
#pragma unroll
      for (int k2 = 0; k2 < N2; ++k2) dst[k2 * step] = u[k2];
    }
  }
};

template <int N, int T>
struct CoopInverse {
  using L = CoopLayout<N, T>;
  static constexpr int N1 = L::N1, N2 = L::N2, KX = L::KX;

  struct ColLoad {
    float2 v[N1];
    int col;  // -1 when idle
    int n2;
  };

  template <bool PM>
  static FBF_HD void col_fetch(const FftParams& p, const float2* base, int inner0, int item, ColLoad& r) {
    r.col = -1;
    if (item >= L::COLS * N2) return;
    // neighbouring lanes take the T planes of one bin: their 8-byte loads share a line
    const int n2 = item / L::COLS, ci = item - n2 * L::COLS;
    const int kx = ci / T, t = ci - kx * T;
    const int col = t * L::KXP + kx;
    const bool live = inner0 + t < p.n_inner;
    const int bin_stride = PM ? 1 : (int)p.spec_bin;
    const int inner_stride = PM ? N * KX : (int)p.spec_inner;
    const float2* src = base + ((n2 * KX + kx) * bin_stride + t * inner_stride);
    const int step = (N2 * KX) * bin_stride;
#pragma unroll
    for (int n1 = 0; n1 < N1; ++n1) r.v[n1] = live ? src[n1 * step] : make_float2(0.f, 0.f);
    r.col = col;
    r.n2 = n2;
  }

  static FBF_HD void col_transform(float2* mid, ColLoad& r) {
    if (r.col < 0) return;
    fft_inreg<N1, true>(r.v);
    float2* c = mid + r.col + N1 * r.n2 * L::PITCH2;
    c[0] = r.v[0];
#pragma unroll
    for (int k1 = 1; k1 < N1; ++k1)
      c[k1 * L::PITCH2] = cmul(r.v[k1], tw128_runtime<true>(r.n2 * k1 * (128 / N)));
  }

  // Column step 1: bins of column (t, kx) from global memory (two items in flight per
  // thread), N1-point inverse transform, twiddle, written to rows k1 + N1*n2 of mid so
  // that step 2 can run in place.
  // PM: plane-major spectrum, compile-time strides; otherwise 32-bit offsets (see CoopForward::col_step2).
  template <bool PM>
  static FBF_HD void col_step1(const FftParams& p, const FftGeom& g, char* smem, int tid, int nthreads,
                               int row, int inner0) {
    float2* mid = reinterpret_cast<float2*>(smem + g.off_b);
    const float2* base = p.spec + (row * p.spec_row + inner0 * p.spec_inner);
    for (int item = tid; item < L::COLS * N2; item += 2 * nthreads) {
      ColLoad r0, r1;
      col_fetch<PM>(p, base, inner0, item, r0);
      col_fetch<PM>(p, base, inner0, item + nthreads, r1);
      col_transform(mid, r0);
      col_transform(mid, r1);
    }
  }

  // Column step 2, in place: item (col, k1) owns rows {k1 + N1*n2}; afterwards row y of
  // mid holds the half spectrum along x of real row y.
  static FBF_HD void col_step2(const FftGeom& g, char* smem, int tid, int nthreads) {
    float2* mid = reinterpret_cast<float2*>(smem + g.off_b);
    for (int item = tid; item < L::COLS * N1; item += nthreads) {
      const int k1 = item / L::COLS, col = item - k1 * L::COLS;
      float2* c = mid + L::col_address(col) + k1 * L::PITCH2;
      float2 u[N2];
#pragma unroll
      for (int n2 = 0; n2 < N2; ++n2) u[n2] = c[N1 * n2 * L::PITCH2];
      fft_inreg<N2, true>(u);
#pragma unroll
      for (int k2 = 0; k2 < N2; ++k2) c[N1 * k2 * L::PITCH2] = u[k2];
    }
  }

  // Row step 1 for lines [line0, line0+nl): rows (y0+j, y0+j+hh) of mid become one complex
  // line (Hermitian extension), N1-point inverse transform, twiddle, into the row buffer.
  static FBF_HD void row_step1(const FftParams& p, const FftGeom& g, char* smem, int tid, int nthreads,
                               int line0, int nl) {
    float2* rb = reinterpret_cast<float2*>(smem + g.off_a);
    const float2* mid = reinterpret_cast<const float2*>(smem + g.off_b);
    // the block size is a multiple of N2, so a thread meets the same n2 in all its items
    float2 tw[N1];
#pragma unroll
    for (int k1 = 0; k1 < N1; ++k1) tw[k1] = tw128_runtime<true>((tid % N2) * k1 * (128 / N));
    for (int item = tid; item < nl * N2; item += nthreads) {
      const int ll = item / N2, n2 = item - ll * N2;
      const int line = line0 + ll;
      int t, j;
    coop_split_line<T>(g, line, t, j);
      const bool has_b = (j + g.hh) < g.he;
      const float2* pa = mid + (p.off_y + j) * L::PITCH2 + t * L::KXP;
      const float2* pb = pa + g.hh * L::PITCH2;
      float2 v[N1];
#pragma unroll
      for (int n1 = 0; n1 < N1; ++n1) {
        const int k = N2 * n1 + n2;
        const int kk = k <= N / 2 ? k : N - k;
        const float2 a = pa[kk];
        const float2 b = has_b ? pb[kk] : make_float2(0.f, 0.f);
        v[n1] = k <= N / 2 ? tangle_low(a, b) : tangle_high(a, b);
      }
      fft_inreg<N1, true>(v);
      float2* dst = rb + ll * L::PITCH1 + n2;
      dst[0] = v[0];
#pragma unroll
      for (int k1 = 1; k1 < N1; ++k1) dst[k1 * (N2 + 1)] = cmul(v[k1], tw[k1]);
    }
  }

  // Row step 2: item (line, k1) produces x = k1 + N1*k2 of both rows of the pair and
  // writes the crop columns straight to global memory (N1 neighbouring floats per row and
  // lane group: whole 32-byte sectors), bias added.
  static FBF_HD void row_step2(const FftParams& p, const FftGeom& g, const char* smem, int tid,
                               int nthreads, int row, int inner0, int line0, int nl) {
    const float2* rb = reinterpret_cast<const float2*>(smem + g.off_a);
    const long long plane_elems = (long long)g.he * g.we;
    float* base = p.real_out + (row * p.real_row_stride + inner0 * p.real_inner_stride) * plane_elems;
    const long long tstride = p.real_inner_stride * plane_elems;
    for (int item = tid; item < nl * N1; item += nthreads) {
      const int ll = item / N1, k1 = item - ll * N1;
      const int line = line0 + ll;
      int t, j;
    coop_split_line<T>(g, line, t, j);
      const int inner = inner0 + t;
      if (inner >= p.n_inner) continue;
      const bool has_b = (j + g.hh) < g.he;
      const float2* src = rb + ll * L::PITCH1 + k1 * (N2 + 1);
      float2 u[N2];
#pragma unroll
      for (int n2 = 0; n2 < N2; ++n2) u[n2] = src[n2];
      fft_inreg<N2, true>(u);
      const float bias = p.bias ? p.bias[p.bias_by_row ? row : inner] : 0.f;
      float* da = base + t * tstride + (long long)j * g.we + (k1 - p.off_x);
      float* db = da + (long long)g.hh * g.we;
#pragma unroll
      for (int k2 = 0; k2 < N2; ++k2) {
        const int x = k1 + N1 * k2 - p.off_x;
        if (x < 0 || x >= g.we) continue;
        const float va = u[k2].x + bias, vb = u[k2].y + bias;
        da[N1 * k2] = p.accumulate ? da[N1 * k2] + va : va;
        if (has_b) db[N1 * k2] = p.accumulate ? db[N1 * k2] + vb : vb;
      }
    }
  }
};

// ===========================================================================
// Batched 1-D transforms up to 32 points: the row half of the 2-D kernels.  A "plane" is a block of up to N
// consecutive rows (p.h of them, p.w floats each); after the row phases the column buffer holds
// the half spectrum of every row, and it is written out / read in as it is:
//     spectrum1d[global row][k],  k in [0, N/2],  global row = inner * p.h + y.
// p.n_rows must be 1; p.spec is the base of the 1-D spectrum.
// ===========================================================================
template <int N, int T>
struct Rows1D {
  static constexpr int KX = N / 2 + 1;

  // element (y, t, k) of the column buffer
  static FBF_HD int mid_index(int y, int t, int k) {
    static_assert(N <= 32, "the 1-D transforms above 32 points have kernels of their own");
    return y * TileLayout<N, T>::PITCH2 + k * T + t;
  }

  static FBF_HD void store_spectrum(const FftParams& p, const FftGeom& g, const char* smem, int tid,
                                    int nthreads, int inner0) {
    const float2* mid = reinterpret_cast<const float2*>(smem + g.off_b);
    const int per_plane = g.he * KX;
    for (int item = tid; item < T * per_plane; item += nthreads) {
      const int t = item / per_plane, r = item - t * per_plane;
      const int y = r / KX, k = r - y * KX;
      const int inner = inner0 + t;
      if (inner >= p.n_inner) break;
      p.spec[((long long)inner * p.h + y) * KX + k] = mid[mid_index(y, t, k)];
    }
  }

  static FBF_HD void load_spectrum(const FftParams& p, const FftGeom& g, char* smem, int tid, int nthreads,
                                   int inner0) {
    float2* mid = reinterpret_cast<float2*>(smem + g.off_b);
    const int per_plane = g.he * KX;
    for (int item = tid; item < T * per_plane; item += nthreads) {
      const int t = item / per_plane, r = item - t * per_plane;
      const int y = r / KX, k = r - y * KX;
      const int inner = inner0 + t;
      mid[mid_index(y, t, k)] =
          inner < p.n_inner ? p.spec[((long long)inner * p.h + y) * KX + k] : make_float2(0.f, 0.f);
    }
  }
};

}  // namespace fbfft
