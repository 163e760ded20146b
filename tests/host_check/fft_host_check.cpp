// Host harness for the FFT kernel phases -- TEST INFRASTRUCTURE ONLY.
// Compiles fbcunn_b200/csrc/fft_core.cuh as plain C++ and runs each thread block as
// loops over thread indices, phase by phase, with shared memory pre-filled with NaN
// so that a read of an unwritten slot shows up in the result.  Checks the index
// arithmetic of the kernels without a GPU; it is never part of the product path.
#include <algorithm>
#include <cstring>
#include <limits>
#include <vector>

#include "../../fbcunn_b200/csrc/fft_core.cuh"

using namespace fbfft;

namespace {

template <int N, int T>
void run_forward(const FftParams& p) {
  const FftGeom g = forward_geom(N, T, p.h, p.w, p.off_y, p.off_x);
  const int tiles = (p.kc + T - 1) / T;
  std::vector<char> smem(g.smem_bytes);
  std::vector<LineRegs<N>> regs(g.threads);
  const int nth = g.threads;
  for (int row = 0; row < p.n_rows; ++row) {
    for (int tile = 0; tile < tiles; ++tile) {
      const int inner0 = tile * T;
      std::memset(smem.data(), 0xFF, smem.size());
      if constexpr (N > 32) {
        for (int line0 = 0; line0 < g.lines1; line0 += g.chunk) {
          const int nl = std::min(g.chunk, g.lines1 - line0);
          std::memset(smem.data() + g.off_a, 0xFF, g.off_b - g.off_a);
          for (int tid = 0; tid < nth; ++tid)
            CoopForward<N, T>::row_step1(p, g, smem.data(), tid, nth, row, inner0, line0, nl);
          {  // the device exchanges the transforms of mirror residues by a lane shuffle
            constexpr int N1 = CoopForward<N, T>::N1, N2 = CoopForward<N, T>::N2;
            const int items = nl * N1;
            std::vector<float2> all(static_cast<size_t>(items) * N2);
            for (int item = 0; item < items; ++item) {
              float2 u[N2];
              CoopForward<N, T>::row_step2_fft(g, smem.data(), item, nl, u);
              std::copy(u, u + N2, all.begin() + static_cast<size_t>(item) * N2);
            }
            for (int item = 0; item < items; ++item) {
              float2 u[N2], mirror_odd[N2 / 2];
              std::copy(all.begin() + static_cast<size_t>(item) * N2,
                        all.begin() + static_cast<size_t>(item + 1) * N2, u);
              const int partner = item ^ 1;
              for (int i = 0; i < N2 / 2; ++i)
                mirror_odd[i] = partner < items ? all[static_cast<size_t>(partner) * N2 + 2 * i + 1]
                                                : make_float2(NAN, NAN);
              CoopForward<N, T>::row_step2_split(g, smem.data(), item, line0, u, mirror_odd);
            }
          }
        }
        for (int tid = 0; tid < nth; ++tid) CoopForward<N, T>::col_step1(g, smem.data(), tid, nth);
        for (int tid = 0; tid < nth; ++tid)
          if (p.spec_bin == 1 && p.spec_inner == (N / 2 + 1) * N)
            CoopForward<N, T>::template col_step2<true>(p, g, smem.data(), tid, nth, row, inner0);
          else
            CoopForward<N, T>::template col_step2<false>(p, g, smem.data(), tid, nth, row, inner0);
      } else {
        for (int tid = 0; tid < g.threads; ++tid)
          Forward<N, T>::load(p, g, smem.data(), tid, g.threads, row, inner0);
        for (int tid = 0; tid < g.threads; ++tid)
          Forward<N, T>::row_fetch(p, g, smem.data(), tid, row, inner0, regs[tid]);
        std::memset(smem.data(), 0xFF, smem.size());  // aliasing: the row buffer is dead now
        for (int tid = 0; tid < g.threads; ++tid)
          Forward<N, T>::row_pass(g, smem.data(), tid, regs[tid]);
        for (int tid = 0; tid < g.threads; ++tid)
          Forward<N, T>::col_pass(p, g, smem.data(), tid, row, inner0);
      }
    }
  }
}

template <int N, int T>
void run_inverse(const FftParams& p, int oh, int ow) {
  const FftGeom g = inverse_geom(N, T, oh, ow);
  const int tiles = (p.n_inner + T - 1) / T;
  std::vector<char> smem(g.smem_bytes);
  std::vector<LineRegs<N>> regs(g.threads);
  for (int row = 0; row < p.n_rows; ++row) {
    for (int tile = 0; tile < tiles; ++tile) {
      const int inner0 = tile * T;
      std::memset(smem.data(), 0xFF, smem.size());
      if constexpr (N > 32) {
        const int nth = g.threads;
        for (int tid = 0; tid < nth; ++tid)
          if (p.spec_bin == 1 && p.spec_inner == (N / 2 + 1) * N)
            CoopInverse<N, T>::template col_step1<true>(p, g, smem.data(), tid, nth, row, inner0);
          else
            CoopInverse<N, T>::template col_step1<false>(p, g, smem.data(), tid, nth, row, inner0);
        for (int tid = 0; tid < nth; ++tid) CoopInverse<N, T>::col_step2(g, smem.data(), tid, nth);
        for (int line0 = 0; line0 < g.lines1; line0 += g.chunk) {
          const int nl = std::min(g.chunk, g.lines1 - line0);
          std::memset(smem.data() + g.off_a, 0xFF, g.off_b - g.off_a);
          for (int tid = 0; tid < nth; ++tid)
            CoopInverse<N, T>::row_step1(p, g, smem.data(), tid, nth, line0, nl);
          for (int tid = 0; tid < nth; ++tid)
            CoopInverse<N, T>::row_step2(p, g, smem.data(), tid, nth, row, inner0, line0, nl);
        }
      } else {
        for (int tid = 0; tid < g.threads; ++tid)
          Inverse<N, T>::col_pass(p, g, smem.data(), tid, row, inner0);
        for (int tid = 0; tid < g.threads; ++tid)
          Inverse<N, T>::row_fetch(g, smem.data(), tid, regs[tid]);
        std::memset(smem.data() + g.off_b, 0xFF, smem.size() - g.off_b);  // mid is dead now
        for (int tid = 0; tid < g.threads; ++tid)
          Inverse<N, T>::row_pass(p, g, smem.data(), tid, row, inner0, regs[tid]);
        for (int tid = 0; tid < g.threads; ++tid)
          Inverse<N, T>::store(p, g, smem.data(), tid, g.threads, row, inner0);
      }
    }
  }
}

// The 1-D kernels up to 32 points: the row phases around Rows1D::store_spectrum / load_spectrum.
template <int N, int T>
void run_1d(bool inverse, const FftParams& p) {
  const FftGeom g = inverse ? inverse_geom(N, T, p.h, p.w) : forward_geom(N, T, p.h, p.w, 0, p.off_x);
  const int tiles = (p.n_inner + T - 1) / T;
  std::vector<char> smem(g.smem_bytes);
  std::vector<LineRegs<N>> regs(g.threads);
  const int nth = g.threads;
  for (int tile = 0; tile < tiles; ++tile) {
    const int inner0 = tile * T;
    std::memset(smem.data(), 0xFF, smem.size());
    if (!inverse) {
      for (int tid = 0; tid < nth; ++tid) Forward<N, T>::load(p, g, smem.data(), tid, nth, 0, inner0);
      for (int tid = 0; tid < nth; ++tid) Forward<N, T>::row_fetch(p, g, smem.data(), tid, 0, inner0, regs[tid]);
      std::memset(smem.data(), 0xFF, smem.size());
      for (int tid = 0; tid < nth; ++tid) Forward<N, T>::row_pass(g, smem.data(), tid, regs[tid]);
      for (int tid = 0; tid < nth; ++tid) Rows1D<N, T>::store_spectrum(p, g, smem.data(), tid, nth, inner0);
    } else {
      for (int tid = 0; tid < nth; ++tid) Rows1D<N, T>::load_spectrum(p, g, smem.data(), tid, nth, inner0);
      for (int tid = 0; tid < nth; ++tid) Inverse<N, T>::row_fetch(g, smem.data(), tid, regs[tid]);
      std::memset(smem.data(), 0xFF, smem.size());
      for (int tid = 0; tid < nth; ++tid) Inverse<N, T>::row_pass(p, g, smem.data(), tid, 0, inner0, regs[tid]);
      for (int tid = 0; tid < nth; ++tid) Inverse<N, T>::store(p, g, smem.data(), tid, nth, 0, inner0);
    }
  }
}

template <int N>
int dispatch_1d_t(bool inverse, const FftParams& p, int T) {
  switch (T) {
    case 1: run_1d<N, 1>(inverse, p); return 0;
    case 2: run_1d<N, 2>(inverse, p); return 0;
    case 4: run_1d<N, 4>(inverse, p); return 0;
    case 8: run_1d<N, 8>(inverse, p); return 0;
    case 16: run_1d<N, 16>(inverse, p); return 0;
  }
  return 2;
}

template <int N>
int dispatch_t(bool inverse, const FftParams& p, int T, int oh, int ow) {
#define FBF_CASE(TT)                                  \
  case TT:                                            \
    if (inverse) run_inverse<N, TT>(p, oh, ow);       \
    else run_forward<N, TT>(p);                       \
    return 0;
  switch (T) {
    FBF_CASE(1) FBF_CASE(2) FBF_CASE(4) FBF_CASE(8) FBF_CASE(16)
  }
#undef FBF_CASE
  return 2;
}

int dispatch(bool inverse, const FftParams& p, int N, int T, int oh, int ow) {
  switch (N) {
    case 2: return dispatch_t<2>(inverse, p, T, oh, ow);
    case 4: return dispatch_t<4>(inverse, p, T, oh, ow);
    case 8: return dispatch_t<8>(inverse, p, T, oh, ow);
    case 16: return dispatch_t<16>(inverse, p, T, oh, ow);
    case 32: return dispatch_t<32>(inverse, p, T, oh, ow);
    case 64: return dispatch_t<64>(inverse, p, T, oh, ow);
    case 128: return dispatch_t<128>(inverse, p, T, oh, ow);
  }
  return 1;
}

}  // namespace

namespace {
void set_layout(FftParams& p, int N, int plane_major) {
  const long long bins = (long long)(N / 2 + 1) * N;
  if (plane_major) {
    p.kc = p.n_inner;
    p.spec_bin = 1;
    p.spec_row = p.n_inner * bins;
    p.spec_inner = bins;
  } else {
    p.spec_bin = (long long)p.n_rows * p.kc;
    p.spec_row = p.kc;
    p.spec_inner = 1;
  }
}
}  // namespace

extern "C" {

// rows of n floats <-> rows of N/2+1 complex values; h rows per block, `planes` blocks
int hostcheck_fft1d(int inverse, float* real, float* spec, int N, int T, int h, int n, int offset, int planes) {
  FftParams p{};
  p.real_in = real;
  p.real_out = real;
  p.spec = reinterpret_cast<float2*>(spec);
  p.h = h; p.w = n; p.off_y = 0; p.off_x = offset;
  p.n_rows = 1; p.n_inner = planes; p.kc = planes;
  p.real_row_stride = 0; p.real_inner_stride = 1;
  switch (N) {
    case 2: return dispatch_1d_t<2>(inverse != 0, p, T);
    case 4: return dispatch_1d_t<4>(inverse != 0, p, T);
    case 8: return dispatch_1d_t<8>(inverse != 0, p, T);
    case 16: return dispatch_1d_t<16>(inverse != 0, p, T);
    case 32: return dispatch_1d_t<32>(inverse != 0, p, T);
  }
  return 1;
}

int hostcheck_fft_forward(const float* real, float* spec, int N, int T, int h, int w, int pad_u,
                          int pad_l, int n_rows, int n_inner, int kc, long long row_stride,
                          long long inner_stride, int plane_major) {
  FftParams p{};
  p.real_in = real;
  p.spec = reinterpret_cast<float2*>(spec);
  p.h = h; p.w = w; p.off_y = pad_u; p.off_x = pad_l;
  p.n_rows = n_rows; p.n_inner = n_inner; p.kc = kc;
  set_layout(p, N, plane_major);
  p.real_row_stride = row_stride; p.real_inner_stride = inner_stride;
  return dispatch(false, p, N, T, 0, 0);
}

int hostcheck_fft_inverse(const float* spec, float* real, const float* bias, int N, int T, int oh,
                          int ow, int off_y, int off_x, int n_rows, int n_inner, int kc,
                          long long row_stride, long long inner_stride, int accumulate, int plane_major) {
  FftParams p{};
  p.real_out = real;
  p.spec = reinterpret_cast<float2*>(const_cast<float*>(spec));
  p.bias = bias;
  p.h = oh; p.w = ow; p.off_y = off_y; p.off_x = off_x;
  p.n_rows = n_rows; p.n_inner = n_inner; p.kc = kc;
  set_layout(p, N, plane_major);
  p.real_row_stride = row_stride; p.real_inner_stride = inner_stride;
  p.accumulate = accumulate;
  return dispatch(true, p, N, T, oh, ow);
}

int hostcheck_forward_smem_bytes(int N, int T, int h, int w, int pad_u, int pad_l) {
  return forward_geom(N, T, h, w, pad_u, pad_l).smem_bytes;
}
int hostcheck_forward_threads(int N, int T, int h, int w, int pad_u, int pad_l) {
  const FftGeom g = forward_geom(N, T, h, w, pad_u, pad_l);
  if (cooperative(N)) return T <= 8 ? g.threads : -1;
  return (g.lines1 > g.threads || g.lines2 > g.threads) ? -1 : g.threads;
}
int hostcheck_inverse_smem_bytes(int N, int T, int oh, int ow) { return inverse_geom(N, T, oh, ow).smem_bytes; }
int hostcheck_inverse_threads(int N, int T, int oh, int ow) {
  const FftGeom g = inverse_geom(N, T, oh, ow);
  if (cooperative(N)) return T <= 8 ? g.threads : -1;
  return (g.lines1 > g.threads || g.lines2 > g.threads) ? -1 : g.threads;
}

}  // extern "C"
