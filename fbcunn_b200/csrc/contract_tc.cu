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
// The kernel itself (persistent blocks, tiles of 128 rows x 16 / 32 / 64 / 128 complex
// columns, TMA producer / MMA issuer / converter / epilogue warps) is in
// contract_tc_wide.inc; this file holds the PTX wrappers it is written in and the host
// side.  Every wait on an mbarrier is bounded; on a time-out the block raises a flag,
// stops issuing work, waits (bounded) for copies in flight, frees its tensor memory and
// returns, and the host sees the error code.
#include <cuda.h>

#include <cstdint>
#include <cstdlib>
#include <mutex>

#include "kernels.h"

namespace fbfft {

namespace {

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
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int code,
                                          uint32_t limit = kWaitLimit) {
  if (mbar_test(bar, parity)) return true;
  for (uint32_t spin = 0; spin < limit; ++spin) {
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

__device__ __forceinline__ float tf32_hi(float x) { return __uint_as_float(__float_as_uint(x) & 0xFFFFE000u); }

__device__ __forceinline__ void split4(const float4 x, float4& hi, float4& lo) {
  hi = make_float4(tf32_hi(x.x), tf32_hi(x.y), tf32_hi(x.z), tf32_hi(x.w));
  lo = make_float4(tf32_hi(x.x - hi.x), tf32_hi(x.y - hi.y), tf32_hi(x.z - hi.z), tf32_hi(x.w - hi.w));
}
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

#include "contract_tc_wide.inc"

// Exercises the give-up path of mbar_wait without TMA or tensor memory: one thread waits on a
// barrier that nothing will ever complete, with a limit of a few suspended waits (microseconds),
// and the kernel returns normally with the sticky code set.
constexpr int kWaitProbeCode = 99;
__global__ void wait_probe_kernel(int* gave_up) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const bool done = mbar_wait(&bar, 0, &abort_flag, kWaitProbeCode, 4);
    *gave_up = (!done && abort_flag == kWaitProbeCode) ? 1 : 0;
  }
}

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

// [bins][rows][inner_floats] fp32, box {box_floats, box_rows, 1}; out-of-range elements read as zero.
bool make_map(CUtensorMap* map, const void* base, int inner_floats, int rows, int bins, int box_rows,
              int box_floats) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[3] = {(cuuint64_t)inner_floats, (cuuint64_t)rows, (cuuint64_t)bins};
  const cuuint64_t strides[2] = {(cuuint64_t)inner_floats * 4, (cuuint64_t)inner_floats * 4 * (cuuint64_t)rows};
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

namespace {

// Tensor maps are encoded once per (base, sizes) and kept: the passes of a layer call with the same
// buffers step after step, and an encode plus a copy of 128 bytes per operand would otherwise sit in
// front of every launch of a launch-bound layer.
struct MapKey {
  const void* base;
  int inner_floats, rows, bins, box_rows, box_floats;
  bool operator==(const MapKey& o) const {
    return base == o.base && inner_floats == o.inner_floats && rows == o.rows && bins == o.bins &&
           box_rows == o.box_rows && box_floats == o.box_floats;
  }
};
// Map of one operand with `rows` rows of the tile dimension (tile of `tile_rows`) and depth k:
// stored [bins][rows][ld] (ld >= k) or, transposed, [bins][k][ld] (ld >= rows).
MapKey operand_key(const void* base, int rows, int k, int ld, int bins, int tile_rows, int kb_floats, bool mn) {
  if (mn) return MapKey{base, 2 * ld, k, bins, kb_floats / 2, 2 * tile_rows};
  return MapKey{base, 2 * ld, rows, bins, tile_rows, kb_floats};
}
struct MapCache {
  static constexpr int kSlots = 32;
  std::mutex mutex;
  MapKey keys[kSlots] = {};
  CUtensorMap maps[kSlots];
  bool used[kSlots] = {};
  int next = 0;
  bool get(const MapKey& key, CUtensorMap* out) {
    std::lock_guard<std::mutex> lock(mutex);
    for (int i = 0; i < kSlots; ++i)
      if (used[i] && keys[i] == key) {
        *out = maps[i];
        return true;
      }
    CUtensorMap m;
    if (!make_map(&m, key.base, key.inner_floats, key.rows, key.bins, key.box_rows, key.box_floats)) return false;
    const int slot = next;
    next = (next + 1) % kSlots;
    keys[slot] = key;
    maps[slot] = m;
    used[slot] = true;
    *out = m;
    return true;
  }
};
MapCache g_maps;

template <int WBNC, bool A_MN, bool B_MN>
cudaError_t launch_wide_as(const ContractParams& p, cudaStream_t stream) {
  using namespace wide;
  using TL = WideTile<WBNC>;
  CUtensorMap map_a, map_b;
  if (!g_maps.get(operand_key(p.a, p.m, p.k, p.lda, p.bins, WBM, TL::KB, p.a_mn != 0), &map_a) ||
      !g_maps.get(operand_key(p.b, p.n, p.k, p.ldb, p.bins, WBNC, TL::KB, p.b_mn != 0), &map_b))
    return cudaErrorInvalidValue;
  WideParams t;
  t.c = p.c;
  t.m = p.m;
  t.n = p.n;
  t.ldc = p.ldc;
  // depth in floats: the padded row length of a [rows][k] operand (its padding is zero), 2k otherwise
  t.k_floats = !p.a_mn ? 2 * p.lda : (!p.b_mn ? 2 * p.ldb : 2 * p.k);
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
  cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(contract_tc_wide_kernel<WBNC, A_MN, B_MN>), TL::SMEM_BYTES);
  if (e != cudaSuccess) return e;
  const int sms = sm_count();
  const int grid = (int)(total < sms ? total : sms);
  contract_tc_wide_kernel<WBNC, A_MN, B_MN><<<grid, W_THREADS, TL::SMEM_BYTES, stream>>>(map_a, map_b, t);
  count_launch();
  return cudaGetLastError();
}

template <int WBNC>
cudaError_t launch_wide(const ContractParams& p, cudaStream_t stream) {
  if (p.a_mn) return p.b_mn ? launch_wide_as<WBNC, true, true>(p, stream) : launch_wide_as<WBNC, true, false>(p, stream);
  return p.b_mn ? launch_wide_as<WBNC, false, true>(p, stream) : launch_wide_as<WBNC, false, false>(p, stream);
}

}  // namespace

// The tile's column count follows the problem's: the smallest of 16 / 32 / 64 / 128 complex columns
// that covers it, 128 beyond.
cudaError_t launch_contract_tc(const ContractParams& p, cudaStream_t stream) {
  if (!contract_tc_supported(p)) return cudaErrorInvalidValue;
  if (p.ldc <= 16) return launch_wide<16>(p, stream);
  if (p.ldc <= 32) return launch_wide<32>(p, stream);
  if (p.ldc <= 64) return launch_wide<64>(p, stream);
  return launch_wide<128>(p, stream);
}

// Runs wait_probe_kernel and returns 1 when the wait gave up as designed, 0 when it did not,
// negative on a CUDA error.  Leaves the sticky code (kWaitProbeCode) for contract_tc_error.
int contract_tc_wait_probe(cudaStream_t stream) {
  int* flag = nullptr;
  if (cudaMalloc(&flag, sizeof(int)) != cudaSuccess) return -1;
  int result = -1;
  if (cudaMemsetAsync(flag, 0xFF, sizeof(int), stream) == cudaSuccess) {
    wait_probe_kernel<<<1, 32, 0, stream>>>(flag);
    count_launch();
    if (cudaGetLastError() == cudaSuccess && cudaStreamSynchronize(stream) == cudaSuccess &&
        cudaMemcpy(&result, flag, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
      result = -1;
  }
  cudaFree(flag);
  return result;
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
