// Internal launch interface between the C ABI (api.cu) and the kernel files.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "fft_core.cuh"

namespace fbfft {

// Counts every kernel this library launches (reported through the C ABI).
void count_launch(int n = 1);
uint64_t launch_count();

// Streaming multiprocessors of the current device (queried once per device); grids of the
// persistent kernels and the "does this launch fill the GPU" decisions are sized from it.
int sm_count();

// Opts `kernel` in to `bytes` of dynamic shared memory on the current device unless an earlier call
// already did (the attribute is per device and function; asking on every launch costs a driver call).
cudaError_t ensure_dynamic_smem(const void* kernel, int bytes);

// Largest plane tile (planes per block) whose shared memory fits, preferring two
// resident blocks per SM; 0 when even one plane does not fit.
int pick_forward_tile(int N, int h, int w, int pad_u, int pad_l);
int pick_inverse_tile(int N, int oh, int ow);

cudaError_t launch_forward(const FftParams& p, int N, cudaStream_t stream);
// batched 1-D real <-> half-complex transforms of contiguous rows (the row phases of the 2-D kernels)
cudaError_t launch_fft1d(bool inverse, const float* real_in, float* real_out, float2* spec, long long rows, int n,
                         int N, int offset, cudaStream_t stream);
// The 1-D transforms of 64, 128 and 256 points (fft1d_lines.cu), same arguments.
cudaError_t launch_fft1d_lines(bool inverse, const float* real_in, float* real_out, float2* spec, long long rows,
                               int n, int N, int offset, cudaStream_t stream);
cudaError_t launch_inverse(const FftParams& p, int N, cudaStream_t stream);
// Between the library's half spectrum [bin][plane (padded to kc)] and the reference's 2-D frequency
// tensor (planes, N/2+1, N, 2) (nn.FFTWrapper, test/test_FFTModule.lua:310-342).
cudaError_t launch_spectrum_layout(bool to_reference, const float2* src, float2* dst, long long planes, int kc, int N,
                                   cudaStream_t stream);

struct ContractParams {
  const float2* a;   // [bins][m][lda], lda >= k;  with a_mn: [bins][k][lda], lda >= m
  const float2* b;   // [bins][n][ldb], ldb >= k;  with b_mn: [bins][k][ldb], ldb >= n
  float2* c;         // [bins][m][ldc]
  int bins, m, n, k; // complex sizes; padding up to the leading dimensions is zero
  int lda, ldb, ldc; // multiples of 4
  float alpha;
  int conj_a, conj_b;
  int a_mn, b_mn;    // operand stored with the contraction index as the row ("MN-major")
};
cudaError_t launch_contract_simt(const ContractParams& p, cudaStream_t stream);
// Tensor-core (tcgen05, 3xTF32) contraction.  contract_tc_error returns the first
// non-zero code a block of that kernel has raised (a bounded wait that ran out) since the
// last reset; it synchronises with the device.
bool contract_tc_supported(const ContractParams& p);
cudaError_t launch_contract_tc(const ContractParams& p, cudaStream_t stream);
int contract_tc_error(bool reset);
// Makes one bounded wait run out on purpose (a barrier nothing completes, a limit of microseconds):
// 1 = the wait gave up and left its code (99) for contract_tc_error, 0 = it did not, < 0 = CUDA error.
int contract_tc_wait_probe(cudaStream_t stream);

// Plane-major ([plane][bin]) streaming contractions for <= 4 input planes (contract_stream.cu):
//   expand: z[u][v] = alpha * sum_p x[u][p] * conj(y[v][p])
//   reduce: z[u][p] = alpha * sum_w op(x[u*xs_u + w*xs_w]) * y[w][p]
cudaError_t launch_stream_expand(const float2* x, const float2* y, float2* z, int U, int V, int P, long long bins,
                                 float alpha, cudaStream_t stream);
cudaError_t launch_stream_reduce(const float2* x, const float2* y, float2* z, int U, int W, int P, long long xs_u,
                                 long long xs_w, bool conj_x, long long bins, float alpha, cudaStream_t stream);

cudaError_t launch_bias_add(float* out, const float* bias, int batch, int planes, int hw,
                            cudaStream_t stream);
cudaError_t launch_bias_grad(const float* grad_out, float* grad_bias, float* scratch, int batch,
                             int planes, int hw, float scale, int accumulate, cudaStream_t stream);
// dst[r] (=|+=) scale * sum_{i<count} src[r*ld + i*step]
// dst[i] = src[i], or dst[i] += src[i]
cudaError_t launch_copy_or_add(const float* src, float* dst, long long n, int accumulate, cudaStream_t stream);
cudaError_t launch_row_sum(const float* src, float* dst, int rows, int count, long long ld, long long step,
                           float scale, int accumulate, cudaStream_t stream);

// ---- sums across ranks over peer memory (peer.cu) ------------------------------------------
constexpr int kMaxPeers = 8;  // the GPUs of one NVSwitch box
// What one rank knows of all ranks (index = rank; the own entries are local addresses, the others
// CUDA IPC mappings): the weight-gradient spectrum, the vector that is summed after the inverse
// transform and the block the sum is delivered to, and the flag array of the barriers.
struct PeerTable {
  char* spec[kMaxPeers];
  char* vec_in[kMaxPeers];
  char* vec_out[kMaxPeers];
  unsigned* flags[kMaxPeers];  // kMaxPeers slots each: slot r = last epoch rank r has signalled
  unsigned* counter;           // local, zero: counts the blocks that reached a kernel's end barrier
  int rank, nranks;
  unsigned spin_limit;         // polls before a wait gives up; 0 = the default (about ten seconds)
};
// Each launch is a collective: every rank calls it with the same epoch (which then advances by 2).
// reduce: this rank's share [first4, first4 + count4) of spec (float4 units) becomes the sum over ranks.
// allreduce: vec_out[i] = sum over ranks of vec_in[i], i < n4 float4s, on every rank.
cudaError_t launch_peer_reduce(const PeerTable& t, unsigned epoch, size_t first4, size_t count4, cudaStream_t stream);
cudaError_t launch_peer_allreduce(const PeerTable& t, unsigned epoch, size_t n4, cudaStream_t stream);
// First non-zero code since the last reset: 1 + the rank a bounded wait gave up on.  Waits for the device.
int peer_error(bool reset);
// Makes one bounded wait on a peer flag run out on purpose: 1 = it gave up (code 1 left for
// peer_error), 0 = it did not, < 0 = CUDA error.
int peer_wait_probe(cudaStream_t stream);

// Records `message` as the calling thread's last error (what fbfftconv_last_error
// returns) and hands `code` back, for entry points that live outside api.cu.
int report_error(int code, const char* message);
// FBFFTCONV_OK when `ptr` is null or device (or managed) memory of `device`; otherwise records a
// message naming `name` and returns FBFFTCONV_ERR_INVALID_ARGUMENT (or FBFFTCONV_ERR_CUDA).
int validate_device_pointer(int device, const void* ptr, const char* name);

}  // namespace fbfft
