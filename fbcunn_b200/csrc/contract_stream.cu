// Streaming contraction for layers with at most four input planes (sm_100a).
//
// When one dimension of the per-bin product is that thin (the first layer of a network:
// three colour planes), the contraction is a bandwidth-bound stream over the large
// spectrum, not a matrix product.  The spectra are then kept plane-major,
// [plane][bin] with the bins contiguous, which is also the layout the FFT kernels of the
// large transform sizes read and write with full coalescing; a thread owns two
// neighbouring bins (one 16-byte access) and walks over planes.
//
// Stands where the reference calls transposeMMFFI on its plane-major buffers
// (fbcunn/SpatialConvolutionFBFFT.lua:157-164, :244-251, :337-344; src/MM.cu:54-73).
#include <cstdlib>

#include "kernels.h"

namespace fbfft {

namespace {

constexpr int THREADS = 256;
constexpr int PMAX = 4;

struct C2 {  // two complex values
  float2 a, b;
};
__device__ __forceinline__ C2 ld2(const float2* p) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  return C2{make_float2(v.x, v.y), make_float2(v.z, v.w)};
}
__device__ __forceinline__ void st2(float2* p, const C2& v, float alpha) {
  *reinterpret_cast<float4*>(p) = make_float4(alpha * v.a.x, alpha * v.a.y, alpha * v.b.x, alpha * v.b.y);
}
// acc += x * y, or conj(x) * y, or x * conj(y)
template <int CONJ>  // 0 none, 1 conj x, 2 conj y
__device__ __forceinline__ void mac1(float2& acc, float2 x, float2 y) {
  const float sx = CONJ == 1 ? -1.f : 1.f, sy = CONJ == 2 ? -1.f : 1.f;
  acc.x = fmaf(x.x, y.x, acc.x);
  acc.x = fmaf(-sx * sy * x.y, y.y, acc.x);
  acc.y = fmaf(sy * x.x, y.y, acc.y);
  acc.y = fmaf(sx * x.y, y.x, acc.y);
}
template <int CONJ>
__device__ __forceinline__ void mac2(C2& acc, const C2& x, const C2& y) {
  mac1<CONJ>(acc.a, x.a, y.a);
  mac1<CONJ>(acc.b, x.b, y.b);
}

// 16-byte asynchronous global -> shared copy; a thread only ever reads back its own copies, so
// cp.async.wait_group is all the synchronisation the ring below needs.
__device__ __forceinline__ void copy16_async(float4* smem_dst, const float2* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(smem_dst)),
               "l"(gmem_src)
               : "memory");
}
__device__ __forceinline__ void copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int PENDING>
__device__ __forceinline__ void copy_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory");
}
__device__ __forceinline__ C2 as_c2(float4 v) { return C2{make_float2(v.x, v.y), make_float2(v.z, v.w)}; }

constexpr int RING_STAGES = 3;  // iterations of w in flight per thread (measured best of 2 / 3 / 4 / 6)

// Z[u][v][bin] = alpha * sum_{p<P} X[u][p][bin] * conj(Y[v][p][bin])
// block: TU rows u, a chunk of columns v, 512 bins; the Y planes of the next RING_STAGES - 1
// columns are in flight into the per-thread ring.
template <int TU>
__global__ void __launch_bounds__(THREADS)
stream_expand_kernel(const float2* __restrict__ X, const float2* __restrict__ Y, float2* __restrict__ Z, int U,
                     int V, int P, int v_per_block, long long bins, float alpha) {
  extern __shared__ float4 ring[];  // [RING_STAGES][PMAX][THREADS]
  const long long bin = ((long long)blockIdx.x * THREADS + threadIdx.x) * 2;
  if (bin >= bins) return;
  const int u0 = blockIdx.y * TU;
  const int v0 = blockIdx.z * v_per_block;
  const int v1 = min(V, v0 + v_per_block);
  float4* mine = ring + threadIdx.x;
  auto issue = [&](int v) {
    if (v < v1) {
      float4* st = mine + ((v - v0) % RING_STAGES) * PMAX * THREADS;
#pragma unroll
      for (int p = 0; p < PMAX; ++p)
        if (p < P) copy16_async(st + p * THREADS, Y + ((long long)v * P + p) * bins + bin);
    }
    copy_commit();
  };
#pragma unroll
  for (int i = 0; i < RING_STAGES - 1; ++i) issue(v0 + i);
  const C2 zero{make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
  C2 x[TU][PMAX];
#pragma unroll
  for (int i = 0; i < TU; ++i)
#pragma unroll
    for (int p = 0; p < PMAX; ++p)
      x[i][p] = (u0 + i < U && p < P) ? ld2(X + ((long long)(u0 + i) * P + p) * bins + bin) : zero;
  for (int v = v0; v < v1; ++v) {
    issue(v + RING_STAGES - 1);
    copy_wait<RING_STAGES - 1>();
    const float4* st = mine + ((v - v0) % RING_STAGES) * PMAX * THREADS;
    C2 y[PMAX];
#pragma unroll
    for (int p = 0; p < PMAX; ++p) y[p] = p < P ? as_c2(st[p * THREADS]) : zero;
#pragma unroll
    for (int i = 0; i < TU; ++i) {
      if (u0 + i >= U) break;
      C2 acc = zero;
#pragma unroll
      for (int p = 0; p < PMAX; ++p) mac2<2>(acc, x[i][p], y[p]);
      st2(Z + ((long long)(u0 + i) * V + v) * bins + bin, acc, alpha);
    }
  }
}

// Z[u][p][bin] = alpha * sum_{w<W} opX(X[u*xs_u + w*xs_w][bin]) * Y[w][p][bin],  p < P <= 4
// block: TU rows u, 512 bins; the loop over w is the long one.  The operands of the next
// RING_STAGES - 1 iterations are in flight into a per-thread ring in shared memory: the bytes
// in flight that a bandwidth-bound loop needs do not have to live in registers.
template <int TU, bool CONJX, int NT>
__global__ void __launch_bounds__(NT)
stream_reduce_kernel(const float2* __restrict__ X, const float2* __restrict__ Y, float2* __restrict__ Z, int U,
                     int W, int P, long long xs_u, long long xs_w, long long bins, float alpha) {
  extern __shared__ float4 ring[];  // [RING_STAGES][PMAX + TU][NT]
  constexpr int NLOAD = PMAX + TU;
  const long long bin = ((long long)blockIdx.x * NT + threadIdx.x) * 2;
  if (bin >= bins) return;
  const int u0 = blockIdx.y * TU;
  float4* mine = ring + threadIdx.x;
  auto issue = [&](int w) {
    if (w < W) {
      float4* st = mine + (w % RING_STAGES) * NLOAD * NT;
#pragma unroll
      for (int p = 0; p < PMAX; ++p)
        if (p < P) copy16_async(st + p * NT, Y + ((long long)w * P + p) * bins + bin);
#pragma unroll
      for (int i = 0; i < TU; ++i)
        if (u0 + i < U) copy16_async(st + (PMAX + i) * NT, X + ((u0 + i) * xs_u + w * xs_w) * bins + bin);
    }
    copy_commit();  // one group per iteration, empty or not, keeps the wait count fixed
  };
  C2 acc[TU][PMAX];
#pragma unroll
  for (int i = 0; i < TU; ++i)
#pragma unroll
    for (int p = 0; p < PMAX; ++p) acc[i][p] = C2{make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
  for (int w = 0; w < RING_STAGES - 1; ++w) issue(w);
  const C2 zero{make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
  for (int w = 0; w < W; ++w) {
    issue(w + RING_STAGES - 1);
    copy_wait<RING_STAGES - 1>();
    const float4* st = mine + (w % RING_STAGES) * NLOAD * NT;
    C2 y[PMAX], x[TU];
#pragma unroll
    for (int p = 0; p < PMAX; ++p) y[p] = p < P ? as_c2(st[p * NT]) : zero;
#pragma unroll
    for (int i = 0; i < TU; ++i) x[i] = u0 + i < U ? as_c2(st[(PMAX + i) * NT]) : zero;
#pragma unroll
    for (int i = 0; i < TU; ++i)
#pragma unroll
      for (int p = 0; p < PMAX; ++p) mac2<CONJX ? 1 : 0>(acc[i][p], x[i], y[p]);
  }
#pragma unroll
  for (int i = 0; i < TU; ++i) {
    if (u0 + i >= U) break;
#pragma unroll
    for (int p = 0; p < PMAX; ++p)
      if (p < P) st2(Z + ((long long)(u0 + i) * P + p) * bins + bin, acc[i][p], alpha);
  }
}

}  // namespace

cudaError_t launch_stream_expand(const float2* x, const float2* y, float2* z, int U, int V, int P, long long bins,
                                 float alpha, cudaStream_t stream) {
  if (P < 1 || P > PMAX || (bins & 1)) return cudaErrorInvalidValue;
  constexpr int TU = 4;
  const int bin_blocks = (int)((bins / 2 + THREADS - 1) / THREADS);
  int v_chunks = 1;
  while (v_chunks < 8 && (long long)bin_blocks * ((U + TU - 1) / TU) * v_chunks < sm_count() * 8 && V / (v_chunks * 2) >= 8)
    v_chunks *= 2;
  const int v_per_block = (V + v_chunks - 1) / v_chunks;
  dim3 grid(bin_blocks, (U + TU - 1) / TU, (V + v_per_block - 1) / v_per_block);
  if (grid.y > 65535 || grid.z > 65535) return cudaErrorInvalidValue;
  const int smem = RING_STAGES * PMAX * THREADS * (int)sizeof(float4);
  cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(stream_expand_kernel<TU>), smem);
  if (e != cudaSuccess) return e;
  stream_expand_kernel<TU><<<grid, THREADS, smem, stream>>>(x, y, z, U, V, P, v_per_block, bins, alpha);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_stream_reduce(const float2* x, const float2* y, float2* z, int U, int W, int P, long long xs_u,
                                 long long xs_w, bool conj_x, long long bins, float alpha, cudaStream_t stream) {
  if (P < 1 || P > PMAX || (bins & 1)) return cudaErrorInvalidValue;
  // Four rows per block (128 threads) quarter the re-reads of Y, which come from L2 and would
  // otherwise be twice the DRAM traffic; with few rows (a small batch shard) fewer rows per
  // block keep every SM busy instead.
  auto blocks_for = [&](int nt, int tu) { return (long long)((bins / 2 + nt - 1) / nt) * ((U + tu - 1) / tu); };
  // most rows per block that still gives every SM three blocks; 128-thread blocks below that
  const long long sms = sm_count();
  int tu = 1, nt = 128;
  if (blocks_for(128, 4) >= 3 * sms) {
    tu = 4;
  } else if (blocks_for(256, 2) >= 2 * sms) {
    tu = 2;
    nt = 256;
  } else if (2 * blocks_for(128, 2) >= 3 * sms) {  // measured at 16 rows: 42 us against 51 (one row) and 49 (four)
    tu = 2;
  }
  dim3 grid((unsigned)((bins / 2 + nt - 1) / nt), (U + tu - 1) / tu);
  if (grid.y > 65535) return cudaErrorInvalidValue;
  auto launch = [&](auto kernel) -> cudaError_t {
    const int smem = RING_STAGES * (PMAX + tu) * nt * (int)sizeof(float4);
    cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem);
    if (e != cudaSuccess) return e;
    kernel<<<grid, nt, smem, stream>>>(x, y, z, U, W, P, xs_u, xs_w, bins, alpha);
    return cudaSuccess;
  };
  cudaError_t e;
  if (tu == 4)
    e = conj_x ? launch(stream_reduce_kernel<4, true, 128>) : launch(stream_reduce_kernel<4, false, 128>);
  else if (tu == 2 && nt == 256)
    e = conj_x ? launch(stream_reduce_kernel<2, true, 256>) : launch(stream_reduce_kernel<2, false, 256>);
  else if (tu == 2)
    e = conj_x ? launch(stream_reduce_kernel<2, true, 128>) : launch(stream_reduce_kernel<2, false, 128>);
  else
    e = conj_x ? launch(stream_reduce_kernel<1, true, 128>) : launch(stream_reduce_kernel<1, false, 128>);
  if (e != cudaSuccess) return e;
  count_launch();
  return cudaGetLastError();
}

}  // namespace fbfft
