/*
 * fbfftconv -- C ABI of the B200 (sm_100a) FFT spatial convolution.
 *
 * A plain-C boundary (raw device pointers, sizes, a CUDA stream, an int status)
 * that stands where the reference's Torch7 bindings for nn.SpatialConvolutionFBFFT
 * stand.  Each entry point names the reference interface it replaces (paths are
 * relative to the reference checkout).
 *
 * Conventions
 *   - all tensors are fp32, contiguous, NCHW, on the handle's device, 4-byte aligned
 *       input       (batch, nInputPlane,  iH, iW)
 *       weight      (nOutputPlane, nInputPlane, kH, kW)
 *       bias        (nOutputPlane)
 *       output      (batch, nOutputPlane, oH, oW),  oH = iH + 2*padH - kH + 1
 *   - stride is 1 and padding symmetric, as the reference module requires
 *     (fbcunn/SpatialConvolutionFBFFT.lua:60-61, fbcunn/SpatialConvolutionFFT.lua:171-174)
 *   - every call returns FBFFTCONV_OK or an error code; nothing throws or aborts.
 *     fbfftconv_last_error() gives the message of the calling thread's last failure.
 *   - work is enqueued on the caller's stream and is asynchronous to the host.
 *   - a handle is used by one host thread at a time.
 *   - there is no CPU or library fallback: without a CUDA device every compute entry
 *     point returns FBFFTCONV_ERR_CUDA.
 */
#ifndef FBFFTCONV_H_
#define FBFFTCONV_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct fbfftconv_handle fbfftconv_handle;
typedef void* fbfftconv_stream; /* cudaStream_t */

enum {
  FBFFTCONV_OK = 0,
  FBFFTCONV_ERR_INVALID_ARGUMENT = 1,
  FBFFTCONV_ERR_UNSUPPORTED_SIZE = 2, /* transform larger than 128 (reference: src/fft/FBFFTHost.cpp:96-98,115) */
  FBFFTCONV_ERR_NOMEM = 3,
  FBFFTCONV_ERR_CUDA = 4,
  FBFFTCONV_ERR_COMM = 5
};

/* flags of fbfftconv_desc */
enum {
  /* accGradParameters adds into gradWeight / gradBias (the nn.Module contract).
   * Default (flag clear) overwrites them, which is what the reference does:
   * fbcunn/SpatialConvolutionFBFFT.lua:337-349, src/ConvolutionBias.cu:95. */
  FBFFTCONV_ACCUMULATE_GRADS = 1,
  /* contraction on the CUDA cores in plain fp32 instead of the tensor cores */
  FBFFTCONV_CONTRACT_SIMT = 2,
  /* keep the bin-major frequency layout even for layers with <= 4 input planes, which by
   * default use plane-major buffers and a streaming contraction at transform sizes 64/128 */
  FBFFTCONV_BIN_MAJOR_ONLY = 4,
  /* with a communicator attached, sum gradWeight across ranks after the inverse transform
   * (F*P*kH*kW floats) instead of summing its spectrum before it (F*P*bins complex
   * values).  The transform is linear, so both orders give the same gradient; the
   * default is the frequency-domain sum. */
  FBFFTCONV_ALLREDUCE_SPATIAL = 8,
  /* Spectrum reuse across the passes of one training step, the memoryReusePolicy of the
   * reference module (fbcunn/SpatialConvolutionFFT.lua:59-63, :405-416;
   * fbcunn/SpatialConvolutionFBFFT.lua:226-237, :305-330).  The caller promises that the
   * tensor in question has not changed since the pass that transformed it:
   *   REUSE_WEIGHT  updateGradInput takes the weight spectrum of the last updateOutput,
   *   REUSE_INPUT   accGradParameters takes the input spectrum of the last updateOutput,
   *   REUSE_OUTPUT  accGradParameters takes the gradOutput spectrum of the last updateGradInput.
   * Every tensor's spectrum is written once, in one layout, and each pass reads it whichever way
   * its sum runs, so a spectrum can be taken over by any later pass of the step.  With REUSE_INPUT
   * the gradInput spectrum gets a buffer of its own (the input spectrum must survive
   * updateGradInput). */
  FBFFTCONV_REUSE_INPUT = 16,
  FBFFTCONV_REUSE_OUTPUT = 32,
  FBFFTCONV_REUSE_WEIGHT = 64,
  /* with a communicator attached, keep the whole weight-gradient exchange on NCCL instead of the
   * sums over peer memory described at fbfftconv_comm_init (must be the same on every rank) */
  FBFFTCONV_EXCHANGE_NCCL = 128
};

/* Constructor arguments of nn.SpatialConvolutionFBFFT
 * (fbcunn/SpatialConvolutionFBFFT.lua:26-35) plus the sizes the Lua module reads
 * from its first input. */
typedef struct fbfftconv_desc {
  int32_t batch;
  int32_t n_input_plane;
  int32_t n_output_plane;
  int32_t input_h, input_w;
  int32_t kernel_h, kernel_w;
  int32_t stride_h, stride_w; /* must be 1 */
  int32_t pad_h, pad_w;       /* padUp, padLeft; must be smaller than the kernel */
  int32_t device;             /* CUDA device ordinal, -1 = current device */
  uint32_t flags;
} fbfftconv_desc;

/* ---- lifetime ------------------------------------------------------------ */

/* Replaces nn.SpatialConvolutionFBFFT:__init plus prepareFBFFTSizeAndBuffers
 * (fbcunn/SpatialConvolutionFBFFT.lua:26-100, fbcunn/SpatialConvolutionFFT.lua:947-964):
 * validates the arguments, picks the square power-of-two transform size and sizes
 * the three frequency buffers.  Allocates no device memory yet. */
int fbfftconv_create(const fbfftconv_desc* desc, fbfftconv_handle** out);
/* Replaces cleanupBuffers (fbcunn/SpatialConvolutionFFT.lua:852-870). */
int fbfftconv_destroy(fbfftconv_handle* h);

/* Transform size N chosen for the layer (fbcunn/SpatialConvolutionFFT.lua:875-882). */
int fbfftconv_fft_size(const fbfftconv_handle* h);
/* Bytes of device scratch the three passes need (the reference's inputBuffer /
 * outputBuffer / weightBuffer, fbcunn/SpatialConvolutionFFT.lua:652-688). */
size_t fbfftconv_workspace_bytes(const fbfftconv_handle* h);
/* Optional: hand the library a caller-owned scratch block of at least
 * fbfftconv_workspace_bytes(); otherwise it is allocated with cudaMalloc on the
 * first pass and freed by fbfftconv_destroy. */
int fbfftconv_set_workspace(fbfftconv_handle* h, void* device_ptr, size_t bytes);

/* ---- the three nn passes, device pointers -----------------------------------
 * Every tensor argument is checked before anything is launched: a host pointer or memory of
 * another GPU than the handle's returns FBFFTCONV_ERR_INVALID_ARGUMENT (what
 * THCudaTensor_checkGPU does for the reference's bindings,
 * src/fft/SpatialConvolutionCuFFTHost.cpp:33-66).  Managed memory is accepted. */

/* Replaces SpatialConvolutionFBFFT:updateOutputFFTImpl
 * (fbcunn/SpatialConvolutionFBFFT.lua:102-183): FFT(input), FFT(weight),
 * transposeMMFFI(.., conjB), inverse FFT, updateOutputBiasFFI.  bias may be NULL
 * (the reference's metaData.skipBias, :172). */
int fbfftconv_update_output(fbfftconv_handle* h, const float* input, const float* weight,
                            const float* bias, float* output, fbfftconv_stream stream);
/* Replaces updateGradInputFFTImpl (fbcunn/SpatialConvolutionFBFFT.lua:189-263). */
int fbfftconv_update_grad_input(fbfftconv_handle* h, const float* grad_output, const float* weight,
                                float* grad_input, fbfftconv_stream stream);
/* Replaces accGradParametersFFTImpl (fbcunn/SpatialConvolutionFBFFT.lua:269-354),
 * including accGradParametersBiasFFI.  grad_bias may be NULL (skipBias, :298).
 * With a communicator attached the frequency-domain weight gradient is summed over
 * all ranks before the inverse transform, and so is grad_bias. */
int fbfftconv_acc_grad_parameters(fbfftconv_handle* h, const float* input, const float* grad_output,
                                  float* grad_weight, float* grad_bias, float scale,
                                  fbfftconv_stream stream);

/* ---- the same passes on tiles of the image -----------------------------------
 * Replaces nn.SpatialConvolutionFFTTiled (fbcunn/SpatialConvolutionFFTTiled.lua:265-365, :489-563,
 * :601-683, :724-802): the output is cut into disjoint tiles of (tile - k + 1) pixels, each computed
 * from an input tile of `tile` pixels (overlap-save), so the transform size follows the tile, not the
 * image -- images beyond 128 pixels become possible, small kernels on large images transform less
 * padding.  The tiles of an image are extra batch entries of one untiled pass (batch x tiles per image
 * must not exceed 65535); cutting, assembling (with the bias, added once) and the overlap-add of
 * updateGradInput are kernels of the library, and accGradParameters' sum over the batch is also the
 * sum over tiles.  desc describes the whole layer (its flags apply to the untiled layer of the
 * tiles); tile_h / tile_w are clipped to the padded image.  The tile buffers are allocated with
 * cudaMalloc at the first pass.  fbfftconv_tiled_inner gives the untiled layer's handle (owned by the
 * tiled one) for fbfftconv_comm_init, the profile and status queries. */
typedef struct fbfftconv_tiled fbfftconv_tiled;
int fbfftconv_tiled_create(const fbfftconv_desc* desc, int tile_h, int tile_w, fbfftconv_tiled** out);
int fbfftconv_tiled_destroy(fbfftconv_tiled* t);
fbfftconv_handle* fbfftconv_tiled_inner(fbfftconv_tiled* t);
/* Device bytes the tiled passes need: the untiled layer's scratch plus the two tile buffers. */
size_t fbfftconv_tiled_workspace_bytes(const fbfftconv_tiled* t);
/* out = { input tile h, w; output tile (= step of the input tiles) h, w; tiles per image along h, w }
 * (the geometry of fbcunn/SpatialConvolutionFFTTiled.lua:55-221 for disjoint output tiles). */
int fbfftconv_tiled_geometry(const fbfftconv_tiled* t, int32_t out[6]);
int fbfftconv_tiled_update_output(fbfftconv_tiled* t, const float* input, const float* weight, const float* bias,
                                  float* output, fbfftconv_stream stream);
int fbfftconv_tiled_update_grad_input(fbfftconv_tiled* t, const float* grad_output, const float* weight,
                                      float* grad_input, fbfftconv_stream stream);
int fbfftconv_tiled_acc_grad_parameters(fbfftconv_tiled* t, const float* input, const float* grad_output,
                                        float* grad_weight, float* grad_bias, float scale, fbfftconv_stream stream);

/* ---- the same passes with HOST buffers --------------------------------------
 * Copies the operands to the device, runs the pass and copies the result back on
 * `stream`, then waits for it.  Pinned host memory makes the copies asynchronous;
 * pageable memory works too.  These stand for a Torch7 caller that keeps its
 * tensors on the host and moves them per call. */
int fbfftconv_update_output_host(fbfftconv_handle* h, const float* input, const float* weight,
                                 const float* bias, float* output, fbfftconv_stream stream);
int fbfftconv_update_grad_input_host(fbfftconv_handle* h, const float* grad_output,
                                     const float* weight, float* grad_input, fbfftconv_stream stream);
int fbfftconv_acc_grad_parameters_host(fbfftconv_handle* h, const float* input,
                                       const float* grad_output, float* grad_weight,
                                       float* grad_bias, float scale, fbfftconv_stream stream);

/* Asynchronous forms of the three calls above for callers that pipeline a training step: each
 * returns as soon as its work is enqueued, and the host outputs of every call issued so far are
 * valid after fbfftconv_host_sync().  Uploads, kernels and downloads run on three streams (the
 * caller's for the kernels) linked by events, and each pass has staging buffers of its own, so
 * the download of one pass overlaps the upload of the next: PCIe carries both directions at once.
 * Host buffers must stay untouched until the sync and should be pinned (pageable memory makes
 * the copies synchronous). */
int fbfftconv_update_output_host_async(fbfftconv_handle* h, const float* input, const float* weight,
                                       const float* bias, float* output, fbfftconv_stream stream);
int fbfftconv_update_grad_input_host_async(fbfftconv_handle* h, const float* grad_output,
                                           const float* weight, float* grad_input,
                                           fbfftconv_stream stream);
int fbfftconv_acc_grad_parameters_host_async(fbfftconv_handle* h, const float* input,
                                             const float* grad_output, float* grad_weight,
                                             float* grad_bias, float scale, fbfftconv_stream stream);
/* nn.Module:backward(input, gradOutput, scale) for host buffers: updateGradInput and
 * accGradParameters (fbcunn/SpatialConvolutionFFT.lua:405-416) with input, gradOutput and weight
 * uploaded once for both, and gradOutput, which both passes see unchanged, transformed once. */
int fbfftconv_backward_host_async(fbfftconv_handle* h, const float* input, const float* grad_output,
                                  const float* weight, float* grad_input, float* grad_weight,
                                  float* grad_bias, float scale, fbfftconv_stream stream);
int fbfftconv_host_sync(fbfftconv_handle* h);

/* ---- the sub-steps, for callers and tests that drive them one by one --------- */

/* Frequency buffers are complex fp32 laid out [bin][row][inner_padded] with
 * bin = ky*(N/2+1) + kx, kx in [0, N/2], ky in [0, N): bin-major, plane index innermost,
 * inner_padded = inner rounded up to a multiple of 4 (padding is written as zero). */
size_t fbfftconv_spectrum_bytes(int fft_size, int rows, int inner);

/* Replaces FFTWrapper_fft for the 2-D batched case (src/fft/FFTWrapperLua.cpp:209-272,
 * src/fft/FBFFTHost.cpp:39-116): real (d1, d2, h, w) placed at (pad_u, pad_l) of an
 * N x N zero square -> half spectrum.  transposed == 0 writes [bin][d1][d2],
 * 1 writes [bin][d2][d1], 2 writes plane-major [d1][d2][bin] (no padding of d2). */
int fbfftconv_fft2d(const float* real, void* spectrum, int d1, int d2, int h, int w, int fft_size,
                    int pad_u, int pad_l, int transposed, fbfftconv_stream stream);
/* Replaces FFTWrapper_ffti (src/fft/FFTWrapperLua.cpp:209-272): un-normalised inverse
 * of spectrum [bin][d1][d2], cropped to the h x w window whose corner is (off_y, off_x).
 * bias (d2 values, may be NULL) is added to every element of plane (., j);
 * accumulate != 0 adds into `real` instead of overwriting; plane_major != 0 reads
 * [d1][d2][bin] instead of [bin][d1][d2]. */
int fbfftconv_ifft2d(const void* spectrum, float* real, const float* bias, int d1, int d2, int h,
                     int w, int fft_size, int off_y, int off_x, int accumulate, int plane_major,
                     fbfftconv_stream stream);
/* The same 2-D transforms on the reference's frequency tensor (planes, N/2+1, N, 2) complex fp32
 * (nn.FFTWrapper with two FFT dimensions, fbcunn/FFTWrapper.lua:53-132): for 8 <= N <= 32 element
 * [ky][kx] = X[ky][kx], ky <= N/2, every kx; for the other sizes the half spectrum along x stored
 * transposed, element [kx][ky] = X[ky][kx], kx <= N/2 (test/test_FFTModule.lua:310-342).  `planes`
 * real planes of h x w (at most 65535); `scratch` holds fbfftconv_spectrum_bytes(fft_size, 1, planes)
 * bytes for the library's own layout; a kernel converts between the two. */
int fbfftconv_fft2d_reference_layout(const float* real, void* frequency, void* scratch, int planes, int h, int w,
                                     int fft_size, int pad_u, int pad_l, fbfftconv_stream stream);
int fbfftconv_ifft2d_reference_layout(const void* frequency, float* real, void* scratch, int planes, int h, int w,
                                      int fft_size, int off_y, int off_x, fbfftconv_stream stream);
/* Replaces FFTWrapper_fft / FFTWrapper_ffti for the 1-D batched case
 * (src/fft/FFTWrapperLua.cpp:209-272, fbfft1dHost in src/fft/FBFFTHost.cpp:119-160): `rows`
 * contiguous rows of n floats, each placed at `pad_left` of a zero line of fft_size, ->
 * spectrum[row][k], k in [0, fft_size/2], complex fp32: the reference's (batch, N/2+1, 2)
 * tensor.  The inverse is un-normalised and keeps columns [offset, offset + n).
 * fft_size in {2, 4, 8, 16, 32, 64, 128, 256}: 256 is the reference's largest 1-D size
 * (test/test_FFTModule.lua:170-260) and exists for these two calls only; the 2-D stand-alone
 * transforms take 2 ... 128, and a convolution handle never picks less than 8. */
int fbfftconv_fft1d(const float* real, void* spectrum, long long rows, int n, int fft_size,
                    int pad_left, fbfftconv_stream stream);
int fbfftconv_ifft1d(const void* spectrum, float* real, long long rows, int n, int fft_size,
                     int offset, fbfftconv_stream stream);

/* Replaces transposeMMFFI (fbcunn/FFTCDefs.lua:7-14, src/MM.cu:54-73) on bin-major
 * operands: for every bin  C[m][n] = alpha * sum_k opA(A[m][k]) * opB(B[n][k]),
 * C [bins][m][n_padded].  conj_a / conj_b are flag sets per operand: bit 0 = use the complex
 * conjugate; bit 1 = the operand is stored with the contraction index as the row index,
 * A as [bins][k][m_padded] (B as [bins][k][n_padded]) instead of [bins][m][k_padded]
 * ([bins][n][k_padded]) -- the reference's 't' / 'c' operand forms on plane-major data.
 * Padding (up to a multiple of 4) must be zero.  use_simt != 0 forces the fp32 CUDA-core kernel. */
int fbfftconv_transpose_mm(const void* a, const void* b, void* c, int bins, int m, int n, int k,
                           float alpha, int conj_a, int conj_b, int use_simt,
                           fbfftconv_stream stream);
/* The tensor-core contraction bounds every wait on the device; a block whose wait runs out
 * stops, frees its tensor memory and records a non-zero code.  This call waits for the
 * device and returns the first such code since the last reset (0 = none, -1 = the query
 * itself failed).  The host-buffer entry points and fbfftconv_host_sync, which wait for the
 * device anyway, check it themselves and return FBFFTCONV_ERR_CUDA; callers of the
 * device-pointer passes, which never wait, poll it where they synchronise. */
int fbfftconv_tensor_core_status(int reset);
/* Self-test of that give-up path (no counterpart in the reference, whose kernels never wait on
 * one another): launches one thread that waits on a barrier nothing will ever complete, with a
 * limit of a few microseconds.  Returns FBFFTCONV_OK when the wait gave up as designed; the
 * device code 99 is then what fbfftconv_tensor_core_status reports until it is reset, and the
 * context stays usable. */
int fbfftconv_tensor_core_wait_selftest(fbfftconv_stream stream);
/* Replaces updateOutputBiasFFI (fbcunn/FFTCDefs.lua:4, src/ConvolutionBias.cu:39-51). */
int fbfftconv_update_output_bias(float* output, const float* bias, int batch, int planes, int h,
                                 int w, fbfftconv_stream stream);
/* Replaces accGradParametersBiasFFI (fbcunn/FFTCDefs.lua:5-6, src/ConvolutionBias.cu:61-97):
 * grad_bias[f] (=, or += when accumulate != 0) scale * sum grad_output[:, f, :, :].
 * scratch must hold batch*planes floats. */
int fbfftconv_acc_grad_parameters_bias(const float* grad_output, float* grad_bias, float* scratch,
                                       int batch, int planes, int h, int w, float scale,
                                       int accumulate, fbfftconv_stream stream);

/* The same bias gradient for callers that cannot allocate device memory when they
 * need it -- a framework allocator that already owns the whole GPU so that a raw
 * cudaMalloc fails or fragments its pool, a loop under a fixed memory budget, or code
 * that cannot afford the implicit synchronisation of an allocation.  It has no
 * counterpart in the reference.  The per-plane partial sums live in a fixed
 * 256 KiB array inside the library (one copy on every GPU that loads it, held until
 * the process exits), so batch * planes must not exceed 65536; larger problems get
 * FBFFTCONV_ERR_UNSUPPORTED_SIZE and should use the variant above.  The call makes no
 * cudaMalloc / cudaFree and calls no allocating routine.  The first call on each
 * device looks the array's device address up once (with that device current); make
 * that first call before any stream capture begins.  All calls on one device share the
 * array: two calls whose kernels can overlap on the GPU (different streams) race;
 * calls ordered on one stream do not.  Nothing needs clearing between calls. */
int fbfftconv_acc_grad_parameters_bias_noalloc(const float* grad_output, float* grad_bias, int batch,
                                               int planes, int h, int w, float scale,
                                               int accumulate, fbfftconv_stream stream);

/* ---- multi-GPU: one process per GPU ------------------------------------------
 * Replaces the gather / add / broadcast of nn.DataParallel
 * (fbcunn/DataParallel.lua:105-131) by one NCCL all-reduce over NVLink.  Rank 0
 * makes an id, every rank gets the same 128 bytes (by any side channel) and calls
 * fbfftconv_comm_init.  Handles that name the same id share one communicator; it stays
 * alive (an id cannot be used twice) until fbfftconv_comm_shutdown, which destroys every
 * communicator no handle is attached to.  fbfftconv_comm_destroy detaches one handle.
 * libnccl is loaded at run time on the first call: the copy the process already holds, else
 * libnccl.so.2; FBFFTCONV_NCCL_LIB in the environment names another file.
 *
 * How the weight gradient is summed.  Up to 8 ranks (the GPUs of one NVSwitch box) whose scratch the
 * library allocated itself map one another's scratch (CUDA IPC) at the first accGradParameters -- a
 * collective step that waits for the stream once, so make that first call before any stream capture
 * -- and the sum is then done by the library's own kernels over peer memory: every rank reads its
 * share of the gradient spectrum from all ranks over NVLink, sums it in rank order, inverts it, and
 * the small spatial parts are summed and delivered the same way; ranks meet at flag barriers in peer
 * memory whose waits are bounded (about ten seconds), after which the kernel gives up and
 * fbfftconv_peer_exchange_status reports it.  NCCL carries the exchange instead when the ranks do not
 * divide the filters (plane-major layers) or the bins (bin-major layers), when a rank could not map a
 * peer (all ranks then agree on NCCL), with caller-owned scratch (fbfftconv_set_workspace), with
 * FBFFTCONV_EXCHANGE_NCCL, or with FBFFTCONV_PEER_EXCHANGE=0 in the environment of every rank. */
int fbfftconv_comm_unique_id(void* id128);
int fbfftconv_comm_init(fbfftconv_handle* h, const void* id128, int rank, int nranks);
int fbfftconv_comm_destroy(fbfftconv_handle* h);
int fbfftconv_comm_shutdown(void);
/* 1 = this handle sums over peer memory, 0 = it uses NCCL (or has no communicator, or has not run
 * accGradParameters yet); 100 + c = a bounded wait of the exchange gave up on rank c - 1 since the
 * last reset (results of that call are incomplete); -1 = the query failed.  Waits for the device. */
int fbfftconv_peer_exchange_status(fbfftconv_handle* h, int reset);
/* Self-test of that give-up path without a second rank: one block waits for a flag nothing sets,
 * with a limit of a few polls.  FBFFTCONV_OK when the wait gave up as designed. */
int fbfftconv_peer_exchange_wait_selftest(fbfftconv_stream stream);
/* Which sum accGradParameters would use over `nranks` ranks and which share of it is `rank`'s:
 * arithmetic on the handle's sizes only (no device, no communicator needed; nranks = 0: no
 * communicator).  out[0] = one of the FBFFTCONV_SUM_* below; [1] floats of the whole gradient
 * spectrum; [2], [3] floats and first float of this rank's share of it (BY_FILTERS, BY_BINS);
 * [4], [5] floats before / after the share that are cleared before the inverse transform (BY_BINS);
 * [6] floats of gradWeight; [7], [8] floats and first float of this rank's filters in gradWeight
 * (BY_FILTERS); [9] 16-byte units of the vector [gradWeight | gradBias] that is summed after the
 * transform.  The shares of all ranks tile the spectrum, and every share starts on and spans whole
 * 16-byte units.  The layer falls back from a share-wise sum to SPECTRUM_WHOLE when the ranks do
 * not divide the filters (plane-major layers) or the bins (bin-major layers). */
enum {
  FBFFTCONV_SUM_NONE = 0,                /* one process: nothing to sum */
  FBFFTCONV_SUM_SPECTRUM_BY_FILTERS = 1, /* reduce-scatter of the spectrum by filters, inverse of the own filters, gather */
  FBFFTCONV_SUM_SPECTRUM_BY_BINS = 2,    /* reduce-scatter by bin range, inverse of the own bins, sum of the partial results */
  FBFFTCONV_SUM_SPECTRUM_WHOLE = 3,      /* one all-reduce of the whole spectrum */
  FBFFTCONV_SUM_SPATIAL = 4              /* FBFFTCONV_ALLREDUCE_SPATIAL: all-reduce of gradWeight after the transform */
};
int fbfftconv_exchange_plan(const fbfftconv_handle* h, int rank, int nranks, long long out[10]);

/* ---- per-kernel timing ---------------------------------------------------------
 * With profiling enabled every kernel (and collective) a pass enqueues is bracketed
 * by a pair of CUDA events on the caller's stream; fbfftconv_profile_read waits for
 * them and returns the summed device time and the number of launches of one stage of
 * one pass since the last reset.  Stands where the reference wraps its FFT and GEMM
 * calls in cuda::KernelTimer (src/fft/FFTWrapperLua.cpp:52-66,
 * src/CuBLASWrapperLua.cpp:90-108). */
enum { FBFFTCONV_PASS_UPDATE_OUTPUT = 0, FBFFTCONV_PASS_UPDATE_GRAD_INPUT = 1, FBFFTCONV_PASS_ACC_GRAD_PARAMETERS = 2 };
enum {
  FBFFTCONV_STAGE_FFT_A = 0,     /* first forward transform: input / gradOutput / gradOutput */
  FBFFTCONV_STAGE_FFT_B = 1,     /* second forward transform: weight / weight / input */
  FBFFTCONV_STAGE_CONTRACT = 2,  /* per-bin complex contraction */
  FBFFTCONV_STAGE_ALLREDUCE = 3, /* NCCL sum of the weight-gradient spectrum */
  FBFFTCONV_STAGE_IFFT = 4,      /* inverse transform + crop (+ bias) */
  FBFFTCONV_STAGE_BIAS = 5,      /* bias-gradient reduction */
  FBFFTCONV_STAGE_COUNT = 6
};
int fbfftconv_profile_enable(fbfftconv_handle* h, int enable);
int fbfftconv_profile_reset(fbfftconv_handle* h);
int fbfftconv_profile_read(fbfftconv_handle* h, int pass, int stage, double* total_ms, int* launches);
/* 1 if launches of this stage since the last reset ran next to another stage of the pass on the
 * handle's second stream (a small second forward transform): its time then overlaps the other
 * stage's and is not its cost alone.  0 otherwise, negative on a bad query. */
int fbfftconv_profile_overlapped(const fbfftconv_handle* h, int pass, int stage);

/* ---- diagnostics ------------------------------------------------------------ */
const char* fbfftconv_last_error(void);
const char* fbfftconv_status_string(int status);
/* Number of kernels this library has launched from the calling process so far. */
uint64_t fbfftconv_kernel_launches(void);

#ifdef __cplusplus
}
#endif
#endif /* FBFFTCONV_H_ */
