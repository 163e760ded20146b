// Per-bin complex contraction on the 5th-generation tensor cores (sm_100a):
// tcgen05.mma kind::tf32 with the accumulator in tensor memory, operands staged by
// TMA, fp32-level accuracy by the 3xTF32 split.
//
//   C[bin][m][n] = alpha * sum_k opA(A[bin][m][k]) * opB(B[bin][n][k])      (complex)
//
// Stands where the reference calls transposeMM / cublasCgemm(Batched)
// (src/MM.cu:54-73, src/CuBLASWrapper.cpp:266-280, :437-452).
//
// Formulation.  A row of A, read as 2K interleaved floats (ar, ai, ...), is used as it
// is.  From each row n of B two real rows are made,
//     B1[n] = ( br, -sa*sb*bi, ...)      B2[n] = ( sb*bi, sa*br, ...)
// (sa, sb = -1 where the operand is conjugated), and interleaved as rows 2n, 2n+1 of
// the MMA's B operand, so that accumulator column 2n is Re C[m][n] and column 2n+1 is
// Im C[m][n]: the accumulator row IS the interleaved complex row of C.
// 3xTF32: x = hi + lo with hi = x truncated to the 10-bit TF32 mantissa and
// lo = x - hi (exact), and  A*B ~= Ahi*Bhi + Alo*Bhi + Ahi*Blo.
//
// One thread block computes a 128 x 64 (complex) tile of one bin.  Warp roles:
//   warp 0      TMA producer: raw fp32 tiles of A (128 rows) and B (64 rows), 32 floats
//               (16 complex k) per stage
//   warp 1      allocates tensor memory; one lane issues the MMAs
//   warps 2..9  converters (split, rotate, write the 128-byte-swizzled K-major operand
//               tiles), then the epilogue (tcgen05.ld, scale, store)
// Every wait on an mbarrier is bounded; on a time-out the block raises a flag, stops
// issuing work, waits (bounded) for copies in flight, frees its tensor memory and
// returns, and the host sees the error code.
#include <cuda.h>

#include <cstdint>
#include <cstdlib>

#include "kernels.h"

namespace fbfft {

namespace {

constexpr int BM = 128;            // rows of A per tile
constexpr int BNC = 64;            // complex columns (rows of B) per tile
constexpr int UMMA_N = 2 * BNC;    // real accumulator columns
constexpr int KB_FLOATS = 32;      // floats of K per stage: one 128-byte swizzle row
constexpr int RAW_STAGES = 3;
constexpr int CONV_STAGES = 2;
constexpr int CONVERTER_WARPS = 8;
constexpr int CONVERTER_THREADS = 32 * CONVERTER_WARPS;
constexpr int THREADS = 64 + CONVERTER_THREADS;

constexpr int RAW_A_BYTES = BM * KB_FLOATS * 4;     // 16 KB
constexpr int RAW_B_BYTES = BNC * KB_FLOATS * 4;    //  8 KB
constexpr int RAW_STAGE_BYTES = RAW_A_BYTES + RAW_B_BYTES;
constexpr int OP_A_BYTES = BM * KB_FLOATS * 4;      // 16 KB per hi / lo
constexpr int OP_B_BYTES = UMMA_N * KB_FLOATS * 4;  // 16 KB per hi / lo
constexpr int CONV_STAGE_BYTES = 2 * OP_A_BYTES + 2 * OP_B_BYTES;  // 64 KB
constexpr int SMEM_TILES = CONV_STAGES * CONV_STAGE_BYTES + RAW_STAGES * RAW_STAGE_BYTES;
constexpr int SMEM_BYTES = SMEM_TILES + 1024 /*alignment slack*/ + 256 /*barriers*/;

constexpr uint32_t kSpinLimit = 1u << 21;  // polls of ~0.1 us each: a fraction of a second
constexpr uint32_t kWaitHintNs = 2000;     // one suspended wait
constexpr uint32_t kWaitLimit = 1u << 18;  // suspended waits before giving up: about half a second

__device__ int g_tc_error = 0;  // sticky: first non-zero code of any block

// ---- PTX wrappers ------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// One bounded hardware wait: the thread is suspended until the phase completes or about
// `hint_ns` have passed, whichever comes first (no issue slots are spent meanwhile).
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (and raises the block's abort flag) on a time-out or
// when another role has already given up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int code) {
  if (mbar_test(bar, parity)) return true;
  for (uint32_t spin = 0; spin < kWaitLimit; ++spin) {
    if (mbar_try_wait(bar, parity, kWaitHintNs)) return true;
    if (*abort_flag) return false;
  }
  *abort_flag = code;
  atomicCAS(&g_tc_error, 0, code);
  return false;
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1,
                                            int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void fence_generic_to_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(columns)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_load_32cols(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void tmem_load_16cols_nowait(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// 16 complex values of one accumulator row whose real parts sit in columns [re_col, re_col+16)
// and imaginary parts in [im_col, im_col+16): interleaved (re, im) as they lie in C.
__device__ __forceinline__ void tmem_load_16complex(uint32_t re_addr, uint32_t im_addr, float (&v)[32]) {
  uint32_t re[16], im[16];
  tmem_load_16cols_nowait(re_addr, re);
  tmem_load_16cols_nowait(im_addr, im);
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    v[2 * i] = __uint_as_float(re[i]);
    v[2 * i + 1] = __uint_as_float(im[i]);
  }
}

// K-major operand tile with 128-byte rows, 128-byte swizzle, 8-row groups 1024 bytes
// apart: start address, LBO = 1, SBO = 64 (both in 16-byte units), version 1, layout 2.
__device__ __forceinline__ uint64_t operand_desc(uint32_t smem_addr) {
  uint64_t d = (smem_addr >> 4) & 0x3FFFu;
  d |= uint64_t(1) << 16;
  d |= uint64_t(1024 >> 4) << 32;
  d |= uint64_t(1) << 46;
  d |= uint64_t(2) << 61;
  return d;
}
// fp32 accumulator, TF32 operands, both K-major, M = 128, N = UMMA_N
constexpr uint32_t kInstrDesc = (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(UMMA_N >> 3) << 17) |
                                (uint32_t(BM >> 4) << 24);

__device__ __forceinline__ float tf32_hi(float x) { return __uint_as_float(__float_as_uint(x) & 0xFFFFE000u); }

__device__ __forceinline__ void split4(const float4 x, float4& hi, float4& lo) {
  hi = make_float4(tf32_hi(x.x), tf32_hi(x.y), tf32_hi(x.z), tf32_hi(x.w));
  lo = make_float4(tf32_hi(x.x - hi.x), tf32_hi(x.y - hi.y), tf32_hi(x.z - hi.z), tf32_hi(x.w - hi.w));
}
// byte offset of 16-byte chunk `c` of row `r` in a 128-byte-swizzled tile
__device__ __forceinline__ int swizzled(int r, int c) { return r * 128 + ((c ^ (r & 7)) << 4); }

struct TcParams {
  float2* c;
  int m, n, ldc;        // complex sizes
  int k_floats;         // 2 * lda
  float alpha;
  float s_b1_im;        // -sa*sb
  float s_b2_re, s_b2_im;  // sb, sa
};

// One accumulator block -- 32 rows (one per lane) x 32 floats in registers -- to global memory
// through a 4 KB shared staging tile, so that a store instruction writes four 128-byte row
// segments instead of 32 scattered 16-byte pieces.  Chunks are XOR-swizzled by the row:
// both the row-per-lane writes and the row-segment reads are free of bank conflicts.
// `c_block` = C + element (first row, first complex column) of the block.
__device__ __forceinline__ void store_block_coalesced(char* stage, const float (&v)[32], float alpha, int lane,
                                                      float2* c_block, int ldc, int rows_valid, int cols_valid) {
#pragma unroll
  for (int j = 0; j < 8; ++j)
    *reinterpret_cast<float4*>(stage + lane * 128 + ((j ^ (lane & 7)) << 4)) =
        make_float4(alpha * v[4 * j], alpha * v[4 * j + 1], alpha * v[4 * j + 2], alpha * v[4 * j + 3]);
  __syncwarp();
  const int ch = lane & 7, rsub = lane >> 3;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = i * 4 + rsub;
    const float4 x = *reinterpret_cast<const float4*>(stage + r * 128 + ((ch ^ (r & 7)) << 4));
    if (r < rows_valid && ch * 2 < cols_valid) *reinterpret_cast<float4*>(c_block + (long long)r * ldc + ch * 2) = x;
  }
  __syncwarp();
}

__global__ void __launch_bounds__(THREADS, 1)
contract_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   const __grid_constant__ TcParams p) {
  extern __shared__ char smem_raw[];
  char* smem = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  char* conv = smem;                                  // CONV_STAGES x {Ahi, Alo, Bhi, Blo}
  char* raw = smem + CONV_STAGES * CONV_STAGE_BYTES;  // RAW_STAGES x {A, B}
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SMEM_TILES);
  uint64_t* full_raw = bars;                    // [RAW_STAGES]
  uint64_t* empty_raw = bars + RAW_STAGES;      // [RAW_STAGES]
  uint64_t* full_conv = bars + 2 * RAW_STAGES;  // [CONV_STAGES]
  uint64_t* empty_conv = full_conv + CONV_STAGES;
  uint64_t* accum_full = empty_conv + CONV_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bin = blockIdx.z;
  const int m0 = blockIdx.y * BM;
  const int n0 = blockIdx.x * BNC;
  const int kblocks = (p.k_floats + KB_FLOATS - 1) / KB_FLOATS;

  if (threadIdx.x == 0) {
    for (int i = 0; i < RAW_STAGES; ++i) {
      mbar_init(&full_raw[i], 1);
      mbar_init(&empty_raw[i], CONVERTER_WARPS);
    }
    for (int i = 0; i < CONV_STAGES; ++i) {
      mbar_init(&full_conv[i], CONVERTER_WARPS);
      mbar_init(&empty_conv[i], 1);
    }
    mbar_init(accum_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, UMMA_N);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int issued = 0;
      for (int kb = 0; kb < kblocks; ++kb) {
        const int s = kb % RAW_STAGES;
        if (kb >= RAW_STAGES && !mbar_wait(&empty_raw[s], ((kb / RAW_STAGES) - 1) & 1, abort_flag, 1)) break;
        char* dst = raw + s * RAW_STAGE_BYTES;
        mbar_arrive_expect_tx(&full_raw[s], RAW_STAGE_BYTES);
        tma_load_3d(dst, &map_a, &full_raw[s], kb * KB_FLOATS, m0, bin);
        tma_load_3d(dst + RAW_A_BYTES, &map_b, &full_raw[s], kb * KB_FLOATS, n0, bin);
        issued = kb + 1;
      }
      if (*abort_flag) {
        // copies already issued must land before this block's shared memory goes away
        for (int kb = (issued > RAW_STAGES ? issued - RAW_STAGES : 0); kb < issued; ++kb) {
          const int s = kb % RAW_STAGES;
          for (uint32_t spin = 0; spin < kSpinLimit; ++spin)
            if (mbar_test(&full_raw[s], (kb / RAW_STAGES) & 1)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      bool ok = true;
      for (int kb = 0; kb < kblocks && ok; ++kb) {
        const int cs = kb % CONV_STAGES;
        ok = mbar_wait(&full_conv[cs], (kb / CONV_STAGES) & 1, abort_flag, 2);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t base = smem_u32(conv + cs * CONV_STAGE_BYTES);
        const uint32_t a_hi = base, a_lo = base + OP_A_BYTES;
        const uint32_t b_hi = base + 2 * OP_A_BYTES, b_lo = b_hi + OP_B_BYTES;
#pragma unroll
        for (int kk = 0; kk < KB_FLOATS / 8; ++kk) {
          const uint32_t off = kk * 32;  // 8 TF32 values = 32 bytes along K inside the swizzle row
          umma_tf32(tmem_base, operand_desc(a_hi + off), operand_desc(b_hi + off), kInstrDesc, (kb | kk) != 0);
          umma_tf32(tmem_base, operand_desc(a_lo + off), operand_desc(b_hi + off), kInstrDesc, 1);
          umma_tf32(tmem_base, operand_desc(a_hi + off), operand_desc(b_lo + off), kInstrDesc, 1);
        }
        umma_commit(&empty_conv[cs]);  // arrives when the MMAs above have read their operands
      }
      if (ok) umma_commit(accum_full);
    }
  } else {
    // ---------------- converters, then epilogue ----------------
    const int ct = threadIdx.x - 64;  // 0..CONVERTER_THREADS-1
    bool ok = true;
    for (int kb = 0; kb < kblocks && ok; ++kb) {
      const int s = kb % RAW_STAGES, cs = kb % CONV_STAGES;
      ok = mbar_wait(&full_raw[s], (kb / RAW_STAGES) & 1, abort_flag, 3);
      if (ok && kb >= CONV_STAGES) ok = mbar_wait(&empty_conv[cs], ((kb / CONV_STAGES) - 1) & 1, abort_flag, 4);
      if (!ok) break;
      const char* ra = raw + s * RAW_STAGE_BYTES;
      const char* rbt = ra + RAW_A_BYTES;
      char* a_hi = conv + cs * CONV_STAGE_BYTES;
      char* a_lo = a_hi + OP_A_BYTES;
      char* b_hi = a_lo + OP_A_BYTES;
      char* b_lo = b_hi + OP_B_BYTES;
      // A: 128 rows x 8 chunks of 16 bytes; consecutive threads take consecutive chunks
#pragma unroll
      for (int i = 0; i < (BM * 8) / CONVERTER_THREADS; ++i) {
        const int idx = ct + i * CONVERTER_THREADS;
        const int r = idx >> 3, c = idx & 7;
        const float4 x = *reinterpret_cast<const float4*>(ra + r * 128 + c * 16);
        float4 hi, lo;
        split4(x, hi, lo);
        const int o = swizzled(r, c);
        *reinterpret_cast<float4*>(a_hi + o) = hi;
        *reinterpret_cast<float4*>(a_lo + o) = lo;
      }
      // B: 64 rows x 8 chunks; each chunk (re0, im0, re1, im1) makes one chunk of row 2n and of row 2n+1
#pragma unroll
      for (int i = 0; i < (BNC * 8) / CONVERTER_THREADS; ++i) {
        const int idx = ct + i * CONVERTER_THREADS;
        const int r = idx >> 3, c = idx & 7;
        const float4 x = *reinterpret_cast<const float4*>(rbt + r * 128 + c * 16);
        const float4 b1 = make_float4(x.x, p.s_b1_im * x.y, x.z, p.s_b1_im * x.w);
        const float4 b2 = make_float4(p.s_b2_re * x.y, p.s_b2_im * x.x, p.s_b2_re * x.w, p.s_b2_im * x.z);
        float4 hi, lo;
        split4(b1, hi, lo);
        int o = swizzled(2 * r, c);
        *reinterpret_cast<float4*>(b_hi + o) = hi;
        *reinterpret_cast<float4*>(b_lo + o) = lo;
        split4(b2, hi, lo);
        o = swizzled(2 * r + 1, c);
        *reinterpret_cast<float4*>(b_hi + o) = hi;
        *reinterpret_cast<float4*>(b_lo + o) = lo;
      }
      fence_generic_to_async_smem();  // operand tiles become visible to the tensor core
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&full_conv[cs]);
        mbar_arrive(&empty_raw[s]);
      }
    }
    if (ok) ok = mbar_wait(accum_full, 0, abort_flag, 5);
    ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld below needs the whole warp
    if (ok) {
      tc_fence_after_sync();
      // tensor-memory lanes 32*(warp%4) .. +31 belong to this warp; lane = tile row.  The
      // warps that share a quarter split the accumulator columns between them.
      const int quarter = warp & 3;
      const int share = (warp - 2) >> 2;
      constexpr int kColBlocks = UMMA_N / 32, kShares = CONVERTER_WARPS / 4;
      const int row0 = m0 + quarter * 32;
      float2* cblock = p.c + ((long long)bin * p.m + row0) * p.ldc + n0;
      // every load has landed and every MMA has read its operands: the raw stages are free
      char* stage = raw + (warp - 2) * 4096;
#pragma unroll 1
      for (int cb = share * (kColBlocks / kShares); cb < (share + 1) * (kColBlocks / kShares); ++cb) {
        float v[32];
        tmem_load_32cols(tmem_base + (uint32_t(quarter * 32) << 16) + cb * 32, v);
        store_block_coalesced(stage, v, p.alpha, lane, cblock + cb * 16, p.ldc, p.m - row0, p.ldc - (n0 + cb * 16));
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, UMMA_N);
  }
}

#include "contract_tc_wide.inc"

// ---- host side -----------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// [bins][rows][k_floats] fp32, box {32 floats, box_rows, 1}; out-of-range elements read as zero.
bool make_map(CUtensorMap* map, const void* base, int k_floats, int rows, int bins, int box_rows,
              int box_floats = KB_FLOATS) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[3] = {(cuuint64_t)k_floats, (cuuint64_t)rows, (cuuint64_t)bins};
  const cuuint64_t strides[2] = {(cuuint64_t)k_floats * 4, (cuuint64_t)k_floats * 4 * (cuuint64_t)rows};
  const cuuint32_t box[3] = {(cuuint32_t)box_floats, (cuuint32_t)box_rows, 1};
  const cuuint32_t elem[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

bool contract_tc_supported(const ContractParams& p) {
  return encode_fn() != nullptr && p.bins <= 65535 && (reinterpret_cast<uintptr_t>(p.a) & 15) == 0 &&
         (reinterpret_cast<uintptr_t>(p.b) & 15) == 0 && (reinterpret_cast<uintptr_t>(p.c) & 15) == 0 &&
         (p.lda & 3) == 0 && (p.ldb & 3) == 0 && (p.ldc & 3) == 0;
}

// Wide persistent kernel for shapes with at least 96 complex columns.
cudaError_t launch_contract_tc_wide(const ContractParams& p, cudaStream_t stream) {
  using namespace wide;
  CUtensorMap map_a, map_b;
  if (!make_map(&map_a, p.a, 2 * p.lda, p.m, p.bins, WBM, WKB) ||
      !make_map(&map_b, p.b, 2 * p.ldb, p.n, p.bins, WBNC, WKB))
    return cudaErrorInvalidValue;
  WideParams t;
  t.c = p.c;
  t.m = p.m;
  t.n = p.n;
  t.ldc = p.ldc;
  t.k_floats = 2 * p.lda;
  t.m_tiles = (p.m + WBM - 1) / WBM;
  t.n_tiles = (p.ldc + WBNC - 1) / WBNC;
  const long long total = (long long)t.m_tiles * t.n_tiles * p.bins;
  if (total > 0x7fffffff) return cudaErrorInvalidValue;
  t.total_tiles = (int)total;
  t.alpha = p.alpha;
  const float sa = p.conj_a ? -1.f : 1.f, sb = p.conj_b ? -1.f : 1.f;
  t.s_b1_im = -sa * sb;
  t.s_b2_re = sb;
  t.s_b2_im = sa;
  cudaError_t e = cudaFuncSetAttribute(contract_tc_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, W_SMEM_BYTES);
  if (e != cudaSuccess) return e;
  const int sms = sm_count();
  const int grid = (int)(total < sms ? total : sms);
  contract_tc_wide_kernel<<<grid, W_THREADS, W_SMEM_BYTES, stream>>>(map_a, map_b, t);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_contract_tc(const ContractParams& p, cudaStream_t stream) {
  if (!contract_tc_supported(p)) return cudaErrorInvalidValue;
  if (p.ldc >= 96) return launch_contract_tc_wide(p, stream);
  CUtensorMap map_a, map_b;
  if (!make_map(&map_a, p.a, 2 * p.lda, p.m, p.bins, BM) || !make_map(&map_b, p.b, 2 * p.ldb, p.n, p.bins, BNC))
    return cudaErrorInvalidValue;
  TcParams t;
  t.c = p.c;
  t.m = p.m;
  t.n = p.n;
  t.ldc = p.ldc;
  t.k_floats = 2 * p.lda;
  t.alpha = p.alpha;
  const float sa = p.conj_a ? -1.f : 1.f, sb = p.conj_b ? -1.f : 1.f;
  t.s_b1_im = -sa * sb;
  t.s_b2_re = sb;
  t.s_b2_im = sa;
  cudaError_t e = cudaFuncSetAttribute(contract_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return e;
  dim3 grid((p.ldc + BNC - 1) / BNC, (p.m + BM - 1) / BM, p.bins);
  contract_tc_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(map_a, map_b, t);
  count_launch();
  return cudaGetLastError();
}

int contract_tc_error(bool reset) {
  int code = 0;
  if (cudaMemcpyFromSymbol(&code, g_tc_error, sizeof(int)) != cudaSuccess) return -1;
  if (reset && code != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int));
  }
  return code;
}

}  // namespace fbfft
