// Per-bin complex contraction on the CUDA cores in plain fp32 (sm_100a).
//
//   C[bin][m][n] = alpha * sum_k opA(A[bin][m][k]) * opB(B[bin][n][k])
//
// Both operands are read with the contraction index contiguous, which is how the
// FFT kernels lay the spectra out, so no transpose pass exists anywhere.  Stands
// where the reference calls transposeMM (src/MM.cu:14-24, :54-73) or, in its cuBLAS
// variant, cgeam + cgemm(Batched) (src/CuBLASWrapper.cpp:113-125, :266-280, :437-452).
// This is the exact-fp32 path: it serves as the numerical yardstick of the
// tensor-core contraction and as the kernel for shapes that one cannot take.
#include "kernels.h"

namespace fbfft {

namespace {

constexpr int BM = 64, BN = 64, BK = 8, PAD = 2;
constexpr int THREADS = 256;

__device__ __forceinline__ void cmac(float2& acc, const float2 a, const float2 b) {
  acc.x = fmaf(a.x, b.x, acc.x);
  acc.x = fmaf(-a.y, b.y, acc.x);
  acc.y = fmaf(a.x, b.y, acc.y);
  acc.y = fmaf(a.y, b.x, acc.y);
}

__global__ void __launch_bounds__(THREADS)
contract_simt_kernel(const __grid_constant__ ContractParams p) {
  __shared__ __align__(16) float2 As[2][BK][BM + PAD];
  __shared__ __align__(16) float2 Bs[2][BK][BN + PAD];

  const int bin = blockIdx.z;
  const int m0 = blockIdx.y * BM;
  const int n0 = blockIdx.x * BN;
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;

  const float2* A = p.a + (long long)bin * p.m * p.lda;
  const float2* B = p.b + (long long)bin * p.n * p.ldb;
  float2* C = p.c + (long long)bin * p.m * p.ldc;

  // loader mapping: one float4 (two complex) per thread and operand
  const int lr = tid >> 2;        // tile row 0..63
  const int lc = (tid & 3) * 2;   // complex column 0,2,4,6
  const float sa = p.conj_a ? -1.f : 1.f;
  const float sb = p.conj_b ? -1.f : 1.f;

  auto fetch = [&](const float2* base, int rows, int ld, int r0, int k0) -> float4 {
    const int r = r0 + lr, k = k0 + lc;
    if (r < rows && k < ld) return *reinterpret_cast<const float4*>(base + (long long)r * ld + k);
    return make_float4(0.f, 0.f, 0.f, 0.f);
  };

  float2 acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = make_float2(0.f, 0.f);

  const int ksteps = (p.k + BK - 1) / BK;
  float4 ra = fetch(A, p.m, p.lda, m0, 0);
  float4 rb = fetch(B, p.n, p.ldb, n0, 0);

  for (int ks = 0; ks < ksteps; ++ks) {
    const int buf = ks & 1;
    As[buf][lc][lr] = make_float2(ra.x, sa * ra.y);
    As[buf][lc + 1][lr] = make_float2(ra.z, sa * ra.w);
    Bs[buf][lc][lr] = make_float2(rb.x, sb * rb.y);
    Bs[buf][lc + 1][lr] = make_float2(rb.z, sb * rb.w);
    __syncthreads();
    if (ks + 1 < ksteps) {
      ra = fetch(A, p.m, p.lda, m0, (ks + 1) * BK);
      rb = fetch(B, p.n, p.ldb, n0, (ks + 1) * BK);
    }
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float2 a[4], b[4];
      const float4 a01 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
      const float4 a23 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4 + 2]);
      const float4 b01 = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4]);
      const float4 b23 = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4 + 2]);
      a[0] = make_float2(a01.x, a01.y); a[1] = make_float2(a01.z, a01.w);
      a[2] = make_float2(a23.x, a23.y); a[3] = make_float2(a23.z, a23.w);
      b[0] = make_float2(b01.x, b01.y); b[1] = make_float2(b01.z, b01.w);
      b[2] = make_float2(b23.x, b23.y); b[3] = make_float2(b23.z, b23.w);
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) cmac(acc[i][j], a[i], b[j]);
    }
    // the other buffer is rewritten next iteration; one barrier per step suffices
    // because a thread can only get there after everyone left this compute loop
    // of the previous use of that buffer (two steps ago) -- guaranteed by the
    // barrier above of the step in between.
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= p.m) continue;
    const int n = n0 + tx * 4;
    if (n >= p.ldc) continue;  // ldc is a multiple of 4: whole groups of four
    float4* dst = reinterpret_cast<float4*>(C + (long long)m * p.ldc + n);
    dst[0] = make_float4(p.alpha * acc[i][0].x, p.alpha * acc[i][0].y,
                         p.alpha * acc[i][1].x, p.alpha * acc[i][1].y);
    dst[1] = make_float4(p.alpha * acc[i][2].x, p.alpha * acc[i][2].y,
                         p.alpha * acc[i][3].x, p.alpha * acc[i][3].y);
  }
}

}  // namespace

cudaError_t launch_contract_simt(const ContractParams& p, cudaStream_t stream) {
  if (p.bins > 65535 || (p.lda & 3) || (p.ldb & 3) || (p.ldc & 3)) return cudaErrorInvalidValue;
  dim3 grid((p.ldc + BN - 1) / BN, (p.m + BM - 1) / BM, p.bins);
  contract_simt_kernel<<<grid, THREADS, 0, stream>>>(p);
  count_launch();
  return cudaGetLastError();
}

}  // namespace fbfft
