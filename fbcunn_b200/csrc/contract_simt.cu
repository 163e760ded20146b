// Per-bin complex contraction on the CUDA cores in plain fp32 (sm_100a).
//
//   C[bin][m][n] = alpha * sum_k opA(A[bin][m][k]) * opB(B[bin][n][k])
//
// An operand is read either with the contraction index contiguous ([rows][k]) or with it
// as the row index ([k][rows]): the FFT kernels write every spectrum once, plane index
// innermost, and each pass reads it whichever way its sum runs, so no transpose pass
// exists anywhere.  Stands
// where the reference calls transposeMM (src/MM.cu:14-24, :54-73) or, in its cuBLAS
// variant, cgeam + cgemm(Batched) (src/CuBLASWrapper.cpp:113-125, :266-280, :437-452).
// This is the exact-fp32 path: it serves as the numerical yardstick of the
// tensor-core contraction and as the kernel for shapes that one cannot take.
#include "kernels.h"

namespace fbfft {

namespace {

constexpr int THREADS = 256;

__device__ __forceinline__ void cmac(float2& acc, const float2 a, const float2 b) {
  acc.x = fmaf(a.x, b.x, acc.x);
  acc.x = fmaf(-a.y, b.y, acc.x);
  acc.y = fmaf(a.x, b.y, acc.y);
  acc.y = fmaf(a.y, b.x, acc.y);
}

// Block tile BM x BN complex results, thread tile TM x TN, K step of 8 complex.
// (64,64,4,4) is the general shape; (128,4,1,2) serves operands with at most four
// columns (three input planes padded to four), where a wide tile would compute zeros.
template <int BM, int BN, int TM, int TN>
__global__ void __launch_bounds__(THREADS)
contract_simt_kernel(const __grid_constant__ ContractParams p) {
  constexpr int BK = 8, PAD = 2;
  constexpr int TX = BN / TN;  // threads along n
  static_assert((BM / TM) * TX == THREADS, "tile shape must use the whole block");
  static_assert(TM == 1 || TM % 2 == 0, "vector loads need pairs");
  static_assert(TN % 2 == 0, "vector loads need pairs");
  __shared__ __align__(16) float2 As[2][BK][BM + PAD];
  __shared__ __align__(16) float2 Bs[2][BK][BN + PAD];

  const int bin = blockIdx.z;
  const int m0 = blockIdx.y * BM;
  const int n0 = blockIdx.x * BN;
  const int tid = threadIdx.x;
  const int tx = tid % TX, ty = tid / TX;

  const float2* A = p.a + (long long)bin * (p.a_mn ? p.k : p.m) * p.lda;
  const float2* B = p.b + (long long)bin * (p.b_mn ? p.k : p.n) * p.ldb;
  float2* C = p.c + (long long)bin * p.m * p.ldc;

  // loaders: one float4 (two complex) per slot; a tile has rows*4 slots
  const float sa = p.conj_a ? -1.f : 1.f;
  const float sb = p.conj_b ? -1.f : 1.f;
  constexpr int A_SLOTS = BM * 4, B_SLOTS = BN * 4;
  constexpr int A_PER = (A_SLOTS + THREADS - 1) / THREADS, B_PER = (B_SLOTS + THREADS - 1) / THREADS;

  // [rows][k] operand: two neighbouring k of one row.  [k][rows] operand: two neighbouring rows of one k
  // (the leading dimension is a multiple of 4 and its padding is zero, so a pair never straddles it).
  auto fetch = [&](const float2* base, int rows, int ld, int r, int k) -> float4 {
    if (r < rows && k < ld) return *reinterpret_cast<const float4*>(base + (long long)r * ld + k);
    return make_float4(0.f, 0.f, 0.f, 0.f);
  };
  auto fetch_mn = [&](const float2* base, int depth, int ld, int r, int k) -> float4 {
    if (k < depth && r < ld) return *reinterpret_cast<const float4*>(base + (long long)k * ld + r);
    return make_float4(0.f, 0.f, 0.f, 0.f);
  };
  // slot -> (row, k) of its first complex value: [rows][k]: 4 slots per row, each two k;
  // [k][rows]: rows/2 slots per k, each two rows
  constexpr int A_HALF = BM / 2 > 0 ? BM / 2 : 1, B_HALF = BN / 2;

  float2 acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = make_float2(0.f, 0.f);

  float4 ra[A_PER], rb[B_PER];
  auto fetch_tiles = [&](int k0) {
#pragma unroll
    for (int i = 0; i < A_PER; ++i) {
      const int slot = tid + i * THREADS;
      if (slot >= A_SLOTS)
        ra[i] = make_float4(0, 0, 0, 0);
      else if (p.a_mn)
        ra[i] = fetch_mn(A, p.k, p.lda, m0 + (slot % A_HALF) * 2, k0 + slot / A_HALF);
      else
        ra[i] = fetch(A, p.m, p.lda, m0 + (slot >> 2), k0 + (slot & 3) * 2);
    }
#pragma unroll
    for (int i = 0; i < B_PER; ++i) {
      const int slot = tid + i * THREADS;
      if (slot >= B_SLOTS)
        rb[i] = make_float4(0, 0, 0, 0);
      else if (p.b_mn)
        rb[i] = fetch_mn(B, p.k, p.ldb, n0 + (slot % B_HALF) * 2, k0 + slot / B_HALF);
      else
        rb[i] = fetch(B, p.n, p.ldb, n0 + (slot >> 2), k0 + (slot & 3) * 2);
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int i = 0; i < A_PER; ++i) {
      const int slot = tid + i * THREADS;
      if (slot < A_SLOTS) {
        if (p.a_mn) {
          const int r = (slot % A_HALF) * 2, c = slot / A_HALF;
          As[buf][c][r] = make_float2(ra[i].x, sa * ra[i].y);
          As[buf][c][r + 1] = make_float2(ra[i].z, sa * ra[i].w);
        } else {
          const int r = slot >> 2, c = (slot & 3) * 2;
          As[buf][c][r] = make_float2(ra[i].x, sa * ra[i].y);
          As[buf][c + 1][r] = make_float2(ra[i].z, sa * ra[i].w);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < B_PER; ++i) {
      const int slot = tid + i * THREADS;
      if (slot < B_SLOTS) {
        if (p.b_mn) {
          const int r = (slot % B_HALF) * 2, c = slot / B_HALF;
          Bs[buf][c][r] = make_float2(rb[i].x, sb * rb[i].y);
          Bs[buf][c][r + 1] = make_float2(rb[i].z, sb * rb[i].w);
        } else {
          const int r = slot >> 2, c = (slot & 3) * 2;
          Bs[buf][c][r] = make_float2(rb[i].x, sb * rb[i].y);
          Bs[buf][c + 1][r] = make_float2(rb[i].z, sb * rb[i].w);
        }
      }
    }
  };

  const int ksteps = (p.k + BK - 1) / BK;
  fetch_tiles(0);
  for (int ks = 0; ks < ksteps; ++ks) {
    const int buf = ks & 1;
    stash(buf);
    __syncthreads();
    if (ks + 1 < ksteps) fetch_tiles((ks + 1) * BK);
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float2 a[TM], b[TN];
      if constexpr (TM == 1) {
        a[0] = As[buf][k][ty];
      } else {
#pragma unroll
        for (int i = 0; i < TM; i += 2) {
          const float4 v = *reinterpret_cast<const float4*>(&As[buf][k][ty * TM + i]);
          a[i] = make_float2(v.x, v.y);
          a[i + 1] = make_float2(v.z, v.w);
        }
      }
#pragma unroll
      for (int j = 0; j < TN; j += 2) {
        const float4 v = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * TN + j]);
        b[j] = make_float2(v.x, v.y);
        b[j + 1] = make_float2(v.z, v.w);
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) cmac(acc[i][j], a[i], b[j]);
    }
    // One barrier per step is enough with two buffers: nobody can overwrite buffer
    // `buf` (two steps from now) before passing the barrier of the step in between,
    // which every thread reaches only after leaving this loop.
  }

#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= p.m) continue;
#pragma unroll
    for (int j = 0; j < TN; j += 2) {
      const int n = n0 + tx * TN + j;
      if (n >= p.ldc) continue;  // ldc is a multiple of 4: pairs never straddle it
      *reinterpret_cast<float4*>(C + (long long)m * p.ldc + n) =
          make_float4(p.alpha * acc[i][j].x, p.alpha * acc[i][j].y, p.alpha * acc[i][j + 1].x,
                      p.alpha * acc[i][j + 1].y);
    }
  }
}

}  // namespace

cudaError_t launch_contract_simt(const ContractParams& p, cudaStream_t stream) {
  if (p.bins > 65535 || (p.lda & 3) || (p.ldb & 3) || (p.ldc & 3)) return cudaErrorInvalidValue;
  if (p.ldc <= 4) {
    dim3 grid(1, (p.m + 127) / 128, p.bins);
    contract_simt_kernel<128, 4, 1, 2><<<grid, THREADS, 0, stream>>>(p);
  } else {
    dim3 grid((p.ldc + 63) / 64, (p.m + 63) / 64, p.bins);
    contract_simt_kernel<64, 64, 4, 4><<<grid, THREADS, 0, stream>>>(p);
  }
  count_launch();
  return cudaGetLastError();
}

}  // namespace fbfft
