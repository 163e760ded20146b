// Bias kernels (sm_100a).  The forward bias add is normally fused into the inverse
// FFT's store; the stand-alone kernels here back the entry points that mirror the
// reference's updateOutputBiasFFI / accGradParametersBiasFFI
// (src/ConvolutionBias.cu:39-51, :61-97).
#include <mutex>
#include <string>

#include "../../include/fbfftconv.h"
#include "kernels.h"

namespace fbfft {

namespace {

__global__ void bias_add_kernel(float* out, const float* __restrict__ bias, int planes, int hw,
                                long long total) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int f = (int)((i / hw) % planes);
    out[i] += bias[f];
  }
}

__device__ __forceinline__ float block_sum(float v) {
  __shared__ float warp_part[32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) warp_part[warp] = v;
  __syncthreads();
  const int nwarps = (blockDim.x + 31) >> 5;
  v = (threadIdx.x < nwarps) ? warp_part[threadIdx.x] : 0.f;
  if (warp == 0) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  }
  return v;  // valid in thread 0
}

// scratch[f * batch + b] = sum of plane (b, f)
__global__ void __launch_bounds__(256)
plane_sum_kernel(const float* __restrict__ grad_out, float* scratch, int batch, int planes, int hw) {
  const int f = blockIdx.x, b = blockIdx.y;
  const float* src = grad_out + ((long long)b * planes + f) * hw;
  float v = 0.f;
  for (int i = threadIdx.x; i < hw; i += blockDim.x) v += src[i];
  v = block_sum(v);
  if (threadIdx.x == 0) scratch[(long long)f * batch + b] = v;
}

// grad_bias[f] (=|+=) scale * sum_b src[f * ld + b * step]
__global__ void __launch_bounds__(128)
row_sum_kernel(const float* __restrict__ src, float* grad_bias, int batch, long long ld, long long step,
               float scale, int accumulate) {
  const int f = blockIdx.x;
  float v = 0.f;
  for (int b = threadIdx.x; b < batch; b += blockDim.x) v += src[(long long)f * ld + (long long)b * step];
  v = block_sum(v);
  if (threadIdx.x == 0) grad_bias[f] = accumulate ? grad_bias[f] + scale * v : scale * v;
}

__global__ void __launch_bounds__(256)
copy_or_add_kernel(const float* __restrict__ src, float* dst, long long n, int accumulate) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dst[i] = accumulate ? dst[i] + src[i] : src[i];
}

}  // namespace

cudaError_t launch_copy_or_add(const float* src, float* dst, long long n, int accumulate, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  const long long want = (n + 255) / 256;
  const int blocks = (int)(want < sm_count() * 8 ? want : sm_count() * 8);
  copy_or_add_kernel<<<blocks, 256, 0, stream>>>(src, dst, n, accumulate);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_bias_add(float* out, const float* bias, int batch, int planes, int hw,
                            cudaStream_t stream) {
  const long long total = (long long)batch * planes * hw;
  const int blocks = (int)((total + 255) / 256 < sm_count() * 16 ? (total + 255) / 256 : sm_count() * 16);
  bias_add_kernel<<<blocks > 0 ? blocks : 1, 256, 0, stream>>>(out, bias, planes, hw, total);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_bias_grad(const float* grad_out, float* grad_bias, float* scratch, int batch,
                             int planes, int hw, float scale, int accumulate, cudaStream_t stream) {
  if (batch > 65535) return cudaErrorInvalidValue;
  plane_sum_kernel<<<dim3(planes, batch), 256, 0, stream>>>(grad_out, scratch, batch, planes, hw);
  row_sum_kernel<<<planes, 128, 0, stream>>>(scratch, grad_bias, batch, batch, 1, scale, accumulate);
  count_launch(2);
  return cudaGetLastError();
}

cudaError_t launch_row_sum(const float* src, float* dst, int rows, int count, long long ld, long long step,
                           float scale, int accumulate, cudaStream_t stream) {
  row_sum_kernel<<<rows, 128, 0, stream>>>(src, dst, count, ld, step, scale, accumulate);
  count_launch();
  return cudaGetLastError();
}

}  // namespace fbfft

// ---------------------------------------------------------------------------
// Bias gradient without any allocation
// ---------------------------------------------------------------------------
// Some callers must not (or cannot) obtain device memory at the moment they need a
// bias gradient: a framework whose caching allocator already owns all of the GPU's
// memory, so that a raw cudaMalloc fails or fragments its pool; a serving or
// training loop under a fixed memory budget; code running where an allocation's
// implicit device synchronisation is not acceptable.  For them the per-plane partial
// sums of the two-stage reduction live in a fixed array inside the library image
// instead of in caller-provided scratch.
namespace {

constexpr int kNoAllocMaxPartials = 65536;  // batch * planes; 256 KiB of device memory
constexpr int kNoAllocMaxDevices = 64;

// One copy per GPU that loads this library, held until the process exits.  In host
// code this name is only a stand-in for the symbol: the device address has to be
// asked for (below), it must never be passed to a kernel as it is.
static __device__ __align__(256) float g_noalloc_partials[kNoAllocMaxPartials];

std::mutex g_noalloc_mutex;
float* g_noalloc_address[kNoAllocMaxDevices] = {};

// Device address of the array on the current device, resolved on first use.
cudaError_t noalloc_scratch(float** out) {
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return e;
  if (device < 0 || device >= kNoAllocMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_address[device]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_partials);
    if (e != cudaSuccess) return e;
    g_noalloc_address[device] = p;
  }
  *out = g_noalloc_address[device];
  return cudaSuccess;
}

}  // namespace

extern "C" int fbfftconv_acc_grad_parameters_bias_noalloc(const float* grad_output, float* grad_bias,
                                                          int batch, int planes, int h, int w,
                                                          float scale, int accumulate,
                                                          fbfftconv_stream stream) {
  using fbfft::report_error;
  if (!grad_output || !grad_bias || batch <= 0 || planes <= 0 || h <= 0 || w <= 0 || batch > 65535)
    return report_error(FBFFTCONV_ERR_INVALID_ARGUMENT, "bad bias-gradient arguments");
  if ((long long)batch * planes > kNoAllocMaxPartials) {
    const std::string msg = "batch * planes = " + std::to_string((long long)batch * planes) +
                            " exceeds the " + std::to_string(kNoAllocMaxPartials) +
                            " partial sums of the allocation-free bias gradient; use "
                            "fbfftconv_acc_grad_parameters_bias with caller scratch";
    return report_error(FBFFTCONV_ERR_UNSUPPORTED_SIZE, msg.c_str());
  }
  float* partials = nullptr;
  cudaError_t e = noalloc_scratch(&partials);
  if (e != cudaSuccess)
    return report_error(FBFFTCONV_ERR_CUDA, (std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e)).c_str());
  // Stage one writes every partial that stage two reads (planes * batch of them), so
  // nothing left in the array by an earlier call is ever consumed and nothing needs
  // clearing.
  e = fbfft::launch_bias_grad(grad_output, grad_bias, partials, batch, planes, h * w, scale,
                              accumulate != 0, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess)
    return report_error(FBFFTCONV_ERR_CUDA, (std::string("bias gradient launch: ") + cudaGetErrorString(e)).c_str());
  return FBFFTCONV_OK;
}
