// Batched 2-D R2C / C2R FFT kernels (sm_100a): one thread block transforms a tile
// of T planes that are neighbours in the spectrum's innermost index, entirely in
// shared memory and registers, and writes / reads the bin-major spectrum in runs of
// T complex values.  Phases and index arithmetic live in fft_core.cuh.
//
// Stands where the reference launches fbfft2D / fbifft2D
// (src/fft/FBFFTHost.cpp:84-111); unlike the reference's sizes 64 and 128
// (two launches through a transposed global buffer, :56-104) every size is a
// single launch with no global scratch.
#include <atomic>
#include <cstdlib>
#include <mutex>
#include <vector>

#include "kernels.h"

namespace fbfft {

// The opt-in to a kernel's dynamic shared memory is per device and function and only ever grows:
// it is asked for when a launch needs more than any launch of that kernel on that device before.
cudaError_t ensure_dynamic_smem(const void* kernel, int bytes) {
  struct Entry {
    const void* kernel;
    int device, bytes;
  };
  static std::mutex mutex;
  static std::vector<Entry> seen;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) dev = 0;
  std::lock_guard<std::mutex> lock(mutex);
  for (Entry& e : seen)
    if (e.kernel == kernel && e.device == dev) {
      if (e.bytes >= bytes) return cudaSuccess;
      cudaError_t r = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
      if (r == cudaSuccess) e.bytes = bytes;
      return r;
    }
  cudaError_t r = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (r == cudaSuccess) seen.push_back(Entry{kernel, dev, bytes});
  return r;
}

namespace {

std::atomic<uint64_t> g_launches{0};

template <int N, int T>
constexpr int block_threads() {
  return ((N / 2 + 1) * T + 31) / 32 * 32 < 64 ? 64 : ((N / 2 + 1) * T + 31) / 32 * 32;
}

template <int N, int T>
__global__ void __launch_bounds__(block_threads<N, T>())
fft2d_forward_kernel(const __grid_constant__ FftParams p, const __grid_constant__ FftGeom g) {
  extern __shared__ __align__(16) char smem[];
  const int tid = threadIdx.x;
  const int row = blockIdx.y;
  const int inner0 = blockIdx.x * T;
  Forward<N, T>::load(p, g, smem, tid, blockDim.x, row, inner0);
  __syncthreads();
  LineRegs<N> regs;
  Forward<N, T>::row_fetch(p, g, smem, tid, row, inner0, regs);
  __syncthreads();  // the column buffer aliases the staged planes
  Forward<N, T>::row_pass(g, smem, tid, regs);
  __syncthreads();
  Forward<N, T>::col_pass(p, g, smem, tid, row, inner0);
}

template <int N, int T>
__global__ void __launch_bounds__(block_threads<N, T>())
fft2d_inverse_kernel(const __grid_constant__ FftParams p, const __grid_constant__ FftGeom g) {
  extern __shared__ __align__(16) char smem[];
  const int tid = threadIdx.x;
  const int row = blockIdx.y;
  const int inner0 = blockIdx.x * T;
  Inverse<N, T>::col_pass(p, g, smem, tid, row, inner0);
  __syncthreads();
  LineRegs<N> regs;
  Inverse<N, T>::row_fetch(g, smem, tid, regs);
  __syncthreads();  // the staged output aliases the column buffer
  Inverse<N, T>::row_pass(p, g, smem, tid, row, inner0, regs);
  __syncthreads();
  Inverse<N, T>::store(p, g, smem, tid, blockDim.x, row, inner0);
}

__device__ __forceinline__ void prefetch_l2(const void* p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

template <int N, int T>
__global__ void __launch_bounds__(FBF_COOP_THREADS, 2)
fft2d_forward_coop_kernel(const __grid_constant__ FftParams p, const __grid_constant__ FftGeom g) {
  extern __shared__ __align__(16) char smem[];
  const int tid = threadIdx.x, nth = blockDim.x;
  const int tiles_x = (p.kc + T - 1) / T;
  const int total = tiles_x * p.n_rows;
  // persistent blocks: tile w, then w + gridDim.x, ...; the real planes of the next tile are
  // pulled into L2 while this one is transformed
  for (int w = blockIdx.x; w < total; w += gridDim.x) {
  const int row = w / tiles_x;
  const int inner0 = (w - row * tiles_x) * T;
  if (w + (int)gridDim.x < total) {
    const int wn = w + gridDim.x;
    const int rown = wn / tiles_x, innern = (wn - rown * tiles_x) * T;
    const long long plane_bytes = (long long)p.h * p.w * 4;
    for (int t = 0; t < T; ++t) {
      if (innern + t >= p.n_inner) break;
      const char* src = reinterpret_cast<const char*>(p.real_in) +
                        (rown * p.real_row_stride + (innern + t) * p.real_inner_stride) * plane_bytes;
      for (long long off = (long long)tid * 128; off < plane_bytes; off += (long long)nth * 128) prefetch_l2(src + off);
    }
  }
  for (int line0 = 0; line0 < g.lines1; line0 += g.chunk) {
    const int nl = min(g.chunk, g.lines1 - line0);
    CoopForward<N, T>::row_step1(p, g, smem, tid, nth, row, inner0, line0, nl);
    __syncthreads();
    // groups of eight lanes hold the eight residues of one line; mirror residues are
    // neighbours, so one shuffle hands each lane the partner's odd-indexed outputs
    constexpr int N1 = CoopForward<N, T>::N1, N2 = CoopForward<N, T>::N2;
    const int items = nl * N1;
    for (int base = 0; base < items; base += nth) {
      float2 u[N2], mirror_odd[N2 / 2];
      const bool active = CoopForward<N, T>::row_step2_fft(g, smem, base + tid, nl, u);
#pragma unroll
      for (int i = 0; i < N2 / 2; ++i) {
        mirror_odd[i].x = __shfl_xor_sync(0xffffffffu, u[2 * i + 1].x, 1);
        mirror_odd[i].y = __shfl_xor_sync(0xffffffffu, u[2 * i + 1].y, 1);
      }
      if (active) CoopForward<N, T>::row_step2_split(g, smem, base + tid, line0, u, mirror_odd);
    }
    __syncthreads();
  }
  CoopForward<N, T>::col_step1(g, smem, tid, nth);
  __syncthreads();
  if (p.spec_bin == 1 && p.spec_inner == (N / 2 + 1) * N)
    CoopForward<N, T>::template col_step2<true>(p, g, smem, tid, nth, row, inner0);
  else
    CoopForward<N, T>::template col_step2<false>(p, g, smem, tid, nth, row, inner0);
  __syncthreads();  // the buffers are reused by the next tile
  }
}

template <int N, int T>
__global__ void __launch_bounds__(FBF_COOP_THREADS, 2)
fft2d_inverse_coop_kernel(const __grid_constant__ FftParams p, const __grid_constant__ FftGeom g) {
  extern __shared__ __align__(16) char smem[];
  const int tid = threadIdx.x, nth = blockDim.x;
  const int tiles_x = (p.n_inner + T - 1) / T;
  const int total = tiles_x * p.n_rows;
  for (int w = blockIdx.x; w < total; w += gridDim.x) {
  const int row = w / tiles_x;
  const int inner0 = (w - row * tiles_x) * T;
  if (p.spec_bin == 1 && w + (int)gridDim.x < total) {  // plane-major: the next tile's spectra are contiguous
    const int wn = w + gridDim.x;
    const int rown = wn / tiles_x, innern = (wn - rown * tiles_x) * T;
    const long long plane_bytes = (long long)(N / 2 + 1) * N * 8;
    for (int t = 0; t < T; ++t) {
      if (innern + t >= p.n_inner) break;
      const char* src = reinterpret_cast<const char*>(p.spec + rown * p.spec_row + (innern + t) * p.spec_inner);
      for (long long off = (long long)tid * 128; off < plane_bytes; off += (long long)nth * 128) prefetch_l2(src + off);
    }
  }
  if (p.spec_bin == 1 && p.spec_inner == (N / 2 + 1) * N)
    CoopInverse<N, T>::template col_step1<true>(p, g, smem, tid, nth, row, inner0);
  else
    CoopInverse<N, T>::template col_step1<false>(p, g, smem, tid, nth, row, inner0);
  __syncthreads();
  CoopInverse<N, T>::col_step2(g, smem, tid, nth);
  __syncthreads();
  for (int line0 = 0; line0 < g.lines1; line0 += g.chunk) {
    const int nl = min(g.chunk, g.lines1 - line0);
    CoopInverse<N, T>::row_step1(p, g, smem, tid, nth, line0, nl);
    __syncthreads();
    CoopInverse<N, T>::row_step2(p, g, smem, tid, nth, row, inner0, line0, nl);
    __syncthreads();
  }
  }
}

// ---- batched 1-D transforms up to 32 points: the row phases of the thread-per-line kernels (larger
// ---- sizes have kernels of their own, fft1d_lines.cu)
template <int N, int T>
__global__ void __launch_bounds__(block_threads<N, T>())
fft1d_forward_kernel(const __grid_constant__ FftParams p, const __grid_constant__ FftGeom g) {
  static_assert(N <= 32, "thread-per-line sizes");
  extern __shared__ __align__(16) char smem[];
  const int tid = threadIdx.x, nth = blockDim.x;
  const int inner0 = blockIdx.x * T;
  Forward<N, T>::load(p, g, smem, tid, nth, 0, inner0);
  __syncthreads();
  LineRegs<N> regs;
  Forward<N, T>::row_fetch(p, g, smem, tid, 0, inner0, regs);
  __syncthreads();
  Forward<N, T>::row_pass(g, smem, tid, regs);
  __syncthreads();
  Rows1D<N, T>::store_spectrum(p, g, smem, tid, nth, inner0);
}

template <int N, int T>
__global__ void __launch_bounds__(block_threads<N, T>())
fft1d_inverse_kernel(const __grid_constant__ FftParams p, const __grid_constant__ FftGeom g) {
  static_assert(N <= 32, "thread-per-line sizes");
  extern __shared__ __align__(16) char smem[];
  const int tid = threadIdx.x, nth = blockDim.x;
  const int inner0 = blockIdx.x * T;
  Rows1D<N, T>::load_spectrum(p, g, smem, tid, nth, inner0);
  __syncthreads();
  LineRegs<N> regs;
  Inverse<N, T>::row_fetch(g, smem, tid, regs);
  __syncthreads();
  Inverse<N, T>::row_pass(p, g, smem, tid, 0, inner0, regs);
  __syncthreads();
  Inverse<N, T>::store(p, g, smem, tid, nth, 0, inner0);
}

constexpr int kSmemMax = 227 * 1024;
constexpr int kSmemTwoBlocks = 113 * 1024;

constexpr bool tile_allowed(int N, int T) { return N > 32 ? T <= 8 : (N / 2 + 1) * T <= 512; }

template <class GeomFn>
int pick_tile(int N, GeomFn geom) {
  int best_any = 0;
  // 32-point transforms: 8 planes per block (more blocks per SM at 64-86 registers per thread) measured 5-10 %
  // faster than 16; 8- and 16-point ones are fastest at 16
  for (int T = (N == 32 ? 8 : 16); T >= 1; T >>= 1) {
    if (!tile_allowed(N, T)) continue;
    const int bytes = geom(T).smem_bytes;
    if (bytes <= kSmemTwoBlocks) return T;
    if (bytes <= kSmemMax && best_any == 0) best_any = T;
  }
  return best_any;
}

// Blocks of a persistent cooperative kernel: as many as are resident at once.
int persistent_blocks(long long tiles, int smem_bytes) {
  const int sms = sm_count();
  const int per_sm = smem_bytes <= kSmemTwoBlocks ? 2 : 1;
  const long long resident = (long long)sms * per_sm;
  return (int)(tiles < resident ? tiles : resident);
}

template <int N, int T>
cudaError_t run_forward(const FftParams& p, cudaStream_t stream) {
  if constexpr (!tile_allowed(N, T)) {
    return cudaErrorInvalidConfiguration;
  } else {
    const FftGeom g = forward_geom(N, T, p.h, p.w, p.off_y, p.off_x);
    void (*kernel)(FftParams, FftGeom);
    if constexpr (N > 32) {
      kernel = fft2d_forward_coop_kernel<N, T>;
    } else {
      if (g.threads != block_threads<N, T>()) return cudaErrorInvalidConfiguration;
      kernel = fft2d_forward_kernel<N, T>;
    }
    cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), g.smem_bytes);
    if (e != cudaSuccess) return e;
    dim3 grid((p.kc + T - 1) / T, p.n_rows);
    if constexpr (N > 32) grid = dim3(persistent_blocks((long long)grid.x * grid.y, g.smem_bytes), 1);
    kernel<<<grid, g.threads, g.smem_bytes, stream>>>(p, g);
    count_launch();
    return cudaGetLastError();
  }
}

template <int N, int T>
cudaError_t run_inverse(const FftParams& p, cudaStream_t stream) {
  if constexpr (!tile_allowed(N, T)) {
    return cudaErrorInvalidConfiguration;
  } else {
    const FftGeom g = inverse_geom(N, T, p.h, p.w);
    void (*kernel)(FftParams, FftGeom);
    if constexpr (N > 32) {
      kernel = fft2d_inverse_coop_kernel<N, T>;
    } else {
      if (g.threads != block_threads<N, T>()) return cudaErrorInvalidConfiguration;
      kernel = fft2d_inverse_kernel<N, T>;
    }
    cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), g.smem_bytes);
    if (e != cudaSuccess) return e;
    dim3 grid((p.n_inner + T - 1) / T, p.n_rows);
    if constexpr (N > 32) grid = dim3(persistent_blocks((long long)grid.x * grid.y, g.smem_bytes), 1);
    kernel<<<grid, g.threads, g.smem_bytes, stream>>>(p, g);
    count_launch();
    return cudaGetLastError();
  }
}

template <int N>
cudaError_t dispatch_tile(bool inverse, const FftParams& p, int T, cudaStream_t s) {
  switch (T) {
    case 1: return inverse ? run_inverse<N, 1>(p, s) : run_forward<N, 1>(p, s);
    case 2: return inverse ? run_inverse<N, 2>(p, s) : run_forward<N, 2>(p, s);
    case 4: return inverse ? run_inverse<N, 4>(p, s) : run_forward<N, 4>(p, s);
    case 8: return inverse ? run_inverse<N, 8>(p, s) : run_forward<N, 8>(p, s);
    case 16: return inverse ? run_inverse<N, 16>(p, s) : run_forward<N, 16>(p, s);
  }
  return cudaErrorInvalidConfiguration;
}

cudaError_t dispatch(bool inverse, const FftParams& p, int N, int T, cudaStream_t s) {
  switch (N) {
    case 2: return dispatch_tile<2>(inverse, p, T, s);
    case 4: return dispatch_tile<4>(inverse, p, T, s);
    case 8: return dispatch_tile<8>(inverse, p, T, s);
    case 16: return dispatch_tile<16>(inverse, p, T, s);
    case 32: return dispatch_tile<32>(inverse, p, T, s);
    case 64: return dispatch_tile<64>(inverse, p, T, s);
    case 128: return dispatch_tile<128>(inverse, p, T, s);
  }
  return cudaErrorInvalidValue;
}

}  // namespace

int sm_count() {
  constexpr int kMaxDevices = 64;
  static std::atomic<int> cache[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) dev = 0;
  int n = cache[dev].load(std::memory_order_relaxed);
  if (n > 0) return n;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    return 1;  // not cached: asked again at the next launch
  }
  cache[dev].store(n, std::memory_order_relaxed);
  return n;
}

void count_launch(int n) { g_launches.fetch_add(static_cast<uint64_t>(n), std::memory_order_relaxed); }
uint64_t launch_count() { return g_launches.load(std::memory_order_relaxed); }

int pick_forward_tile(int N, int h, int w, int pad_u, int pad_l) {
  return pick_tile(N, [&](int T) { return forward_geom(N, T, h, w, pad_u, pad_l); });
}
int pick_inverse_tile(int N, int oh, int ow) {
  return pick_tile(N, [&](int T) { return inverse_geom(N, T, oh, ow); });
}

// The kernels address the spectrum with 32-bit element offsets.
bool spectrum_fits(const FftParams& p, int N) {
  const long long bins = (long long)(N / 2 + 1) * N;
  return bins * p.n_rows * p.kc < (1LL << 31);
}

cudaError_t launch_forward(const FftParams& p, int N, cudaStream_t stream) {
  const int T = pick_forward_tile(N, p.h, p.w, p.off_y, p.off_x);
  if (T == 0 || p.n_rows > 65535 || !spectrum_fits(p, N)) return cudaErrorInvalidConfiguration;
  return dispatch(false, p, N, T, stream);
}

cudaError_t launch_inverse(const FftParams& p, int N, cudaStream_t stream) {
  const int T = pick_inverse_tile(N, p.h, p.w);
  if (T == 0 || p.n_rows > 65535 || !spectrum_fits(p, N)) return cudaErrorInvalidConfiguration;
  return dispatch(true, p, N, T, stream);
}

namespace {

template <int N, int T>
cudaError_t run_1d(bool inverse, const FftParams& p, cudaStream_t stream) {
  if constexpr (!tile_allowed(N, T)) {
    return cudaErrorInvalidConfiguration;
  } else {
    const FftGeom g = inverse ? inverse_geom(N, T, p.h, p.w) : forward_geom(N, T, p.h, p.w, 0, p.off_x);
    void (*kernel)(FftParams, FftGeom) = inverse ? fft1d_inverse_kernel<N, T> : fft1d_forward_kernel<N, T>;
    cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), g.smem_bytes);
    if (e != cudaSuccess) return e;
    kernel<<<(p.n_inner + T - 1) / T, g.threads, g.smem_bytes, stream>>>(p, g);
    count_launch();
    return cudaGetLastError();
  }
}

template <int N>
cudaError_t dispatch_1d_tile(bool inverse, const FftParams& p, int T, cudaStream_t s) {
  switch (T) {
    case 1: return run_1d<N, 1>(inverse, p, s);
    case 2: return run_1d<N, 2>(inverse, p, s);
    case 4: return run_1d<N, 4>(inverse, p, s);
    case 8: return run_1d<N, 8>(inverse, p, s);
    case 16: return run_1d<N, 16>(inverse, p, s);
  }
  return cudaErrorInvalidConfiguration;
}

}  // namespace

// Rows [0, rows) of `n` floats each, transform size N: full blocks of N rows, then the rest.
cudaError_t launch_fft1d(bool inverse, const float* real_in, float* real_out, float2* spec, long long rows, int n,
                         int N, int offset, cudaStream_t stream) {
  if (N >= 64) return launch_fft1d_lines(inverse, real_in, real_out, spec, rows, n, N, offset, stream);
  const int KX = N / 2 + 1;
  for (int part = 0; part < 2; ++part) {
    const long long first = part == 0 ? 0 : rows / N * N;
    const int h = part == 0 ? N : (int)(rows % N);
    const long long planes = part == 0 ? rows / N : 1;
    if (h == 0 || planes == 0) continue;
    if (planes > 0x7fffffff) return cudaErrorInvalidValue;
    FftParams p{};
    p.real_in = real_in ? real_in + first * n : nullptr;
    p.real_out = real_out ? real_out + first * n : nullptr;
    p.spec = spec + first * KX;
    p.h = h;
    p.w = n;
    p.off_y = 0;
    p.off_x = offset;
    p.n_rows = 1;
    p.n_inner = (int)planes;
    p.kc = (int)planes;
    p.real_row_stride = 0;
    p.real_inner_stride = 1;
    const int T = inverse ? pick_inverse_tile(N, h, n) : pick_forward_tile(N, h, n, 0, offset);
    if (T == 0) return cudaErrorInvalidConfiguration;
    cudaError_t e;
    switch (N) {
      case 2: e = dispatch_1d_tile<2>(inverse, p, T, stream); break;
      case 4: e = dispatch_1d_tile<4>(inverse, p, T, stream); break;
      case 8: e = dispatch_1d_tile<8>(inverse, p, T, stream); break;
      case 16: e = dispatch_1d_tile<16>(inverse, p, T, stream); break;
      case 32: e = dispatch_1d_tile<32>(inverse, p, T, stream); break;
      default: e = cudaErrorInvalidValue;
    }
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

namespace {

// The reference's 2-D frequency tensor (planes, N/2+1, N, 2) holds, for 8 <= N <= 32, rows ky <= N/2
// of the full spectrum (element [ky][kx] = X[ky][kx] for every kx), and for the other sizes the half
// spectrum along x stored transposed (element [kx][ky] = X[ky][kx], kx <= N/2)
// (test/test_FFTModule.lua:310-342).  The library's half spectrum is [bin = ky*(N/2+1) + kx][plane],
// kx <= N/2; the missing half follows from X[ky][kx] = conj(X[-ky][-kx]).
__global__ void __launch_bounds__(256)
spectrum_to_reference_kernel(const float2* __restrict__ spec, float2* __restrict__ ref, long long planes, int kc,
                             int N, int transposed) {
  const int KX = N / 2 + 1;
  const long long per_plane = (long long)KX * N;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < planes * per_plane;
       i += (long long)gridDim.x * blockDim.x) {
    const long long p = i / per_plane;
    const int r = (int)(i - p * per_plane);
    const int a = r / N, b = r - a * N;  // element [a][b] of the reference tensor, a <= N/2
    int ky, kx;
    bool conj = false;
    if (transposed) {
      kx = a;
      ky = b;
    } else {
      ky = a;
      kx = b;
      if (kx > N / 2) {
        ky = (N - ky) % N;
        kx = N - kx;
        conj = true;
      }
    }
    float2 v = spec[((long long)ky * KX + kx) * kc + p];
    if (conj) v.y = -v.y;
    ref[i] = v;
  }
}

__global__ void __launch_bounds__(256)
reference_to_spectrum_kernel(const float2* __restrict__ ref, float2* __restrict__ spec, long long planes, int kc,
                             int N, int transposed) {
  const int KX = N / 2 + 1;
  const long long bins = (long long)KX * N;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < bins * kc;
       i += (long long)gridDim.x * blockDim.x) {
    const long long bin = i / kc;
    const long long p = i - bin * kc;
    float2 v = make_float2(0.f, 0.f);  // the padding planes of the library's layout are zero
    if (p < planes) {
      const int ky = (int)(bin / KX), kx = (int)(bin - (long long)ky * KX);
      const float2* plane = ref + p * bins;
      if (transposed) {
        v = plane[kx * N + ky];
      } else if (ky <= N / 2) {
        v = plane[ky * N + kx];
      } else {  // X[ky][kx] = conj(X[N-ky][(N-kx) % N])
        v = plane[(N - ky) * N + (N - kx) % N];
        v.y = -v.y;
      }
    }
    spec[i] = v;
  }
}

}  // namespace

cudaError_t launch_spectrum_layout(bool to_reference, const float2* src, float2* dst, long long planes, int kc, int N,
                                   cudaStream_t stream) {
  const bool transposed = N < 8 || N > 32;
  const long long total = to_reference ? planes * (N / 2 + 1) * N : (long long)(N / 2 + 1) * N * kc;
  const long long want = (total + 255) / 256, cap = (long long)sm_count() * 16;
  const int blocks = (int)(want < 1 ? 1 : want < cap ? want : cap);
  if (to_reference)
    spectrum_to_reference_kernel<<<blocks, 256, 0, stream>>>(src, dst, planes, kc, N, transposed);
  else
    reference_to_spectrum_kernel<<<blocks, 256, 0, stream>>>(src, dst, planes, kc, N, transposed);
  count_launch();
  return cudaGetLastError();
}

}  // namespace fbfft

