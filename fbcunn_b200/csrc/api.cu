// C ABI of the library (declared in include/fbfftconv.h): handle, scratch
// management, the three passes, their host-buffer variants, the sub-steps and the
// NCCL hook.  Plays the part of the reference's pass driver
// (fbcunn/SpatialConvolutionFBFFT.lua:102-354) and buffer cache
// (fbcunn/SpatialConvolutionFFT.lua:652-870) on the native side of the boundary.
#include <dlfcn.h>
#include <nccl.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/fbfftconv.h"
#include "kernels.h"

using namespace fbfft;

namespace {

thread_local std::string t_error;

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  t_error = buf;
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  return fail(FBFFTCONV_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

#define FBF_CUDA(expr)                                   \
  do {                                                   \
    cudaError_t e_ = (expr);                             \
    if (e_ != cudaSuccess) return cuda_fail(e_, #expr);  \
  } while (0)
#define FBF_TRY(expr)                    \
  do {                                   \
    int rc_ = (expr);                    \
    if (rc_ != FBFFTCONV_OK) return rc_; \
  } while (0)

int pad4(int v) { return (v + 3) & ~3; }

int next_pow2(int v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}

// ---- NCCL, resolved at run time so that single-GPU users need no libnccl -----
struct NcclApi {
  void* lib = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                            cudaStream_t) = nullptr;
  ncclResult_t (*ReduceScatter)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                                cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

NcclApi* nccl_api() {
  static NcclApi api;
  static bool tried = false;
  if (tried) return api.lib ? &api : nullptr;
  tried = true;
  const char* env = getenv("FBFFTCONV_NCCL_LIB");
  void* lib = nullptr;
  if (env && *env) lib = dlopen(env, RTLD_NOW | RTLD_GLOBAL);
  if (!lib) lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
  if (!lib) lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) return nullptr;
  api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(lib, "ncclGetUniqueId"));
  api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(lib, "ncclCommInitRank"));
  api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(dlsym(lib, "ncclAllReduce"));
  api.ReduceScatter = reinterpret_cast<decltype(api.ReduceScatter)>(dlsym(lib, "ncclReduceScatter"));
  api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(lib, "ncclAllGather"));
  api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(dlsym(lib, "ncclGroupStart"));
  api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(dlsym(lib, "ncclGroupEnd"));
  api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(lib, "ncclCommDestroy"));
  api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(lib, "ncclGetErrorString"));
  if (!api.GetUniqueId || !api.CommInitRank || !api.AllReduce || !api.CommDestroy) return nullptr;
  api.lib = lib;
  return &api;
}

// One NCCL communicator per unique id and process, shared by every handle that names
// that id (a model has many layers but needs one communicator).
struct SharedComm {
  ncclComm_t comm = nullptr;
  int refs = 0;
  int rank = 0, nranks = 0, device = -1;  // what the communicator was initialised with
};
std::mutex g_comm_mutex;
std::map<std::string, SharedComm> g_comms;

int nccl_fail(NcclApi* api, ncclResult_t r, const char* what) {
  return fail(FBFFTCONV_ERR_COMM, "%s: %s", what,
              api && api->GetErrorString ? api->GetErrorString(r) : "nccl error");
}

}  // namespace

struct EventPair {
  cudaEvent_t start, stop;
};

struct fbfftconv_handle {
  fbfftconv_desc d;
  // per-kernel timing: event pairs per (pass, stage), reused after a reset
  bool profiling = false;
  std::vector<EventPair> events[3][FBFFTCONV_STAGE_COUNT];
  int events_used[3][FBFFTCONV_STAGE_COUNT] = {};
  bool overlapped[3][FBFFTCONV_STAGE_COUNT] = {};  // stage ran on the second stream since the last reset
  int device;
  int N, bins;
  int oH, oW;
  bool plane_major = false;  // <= 4 input planes at a cooperative transform size: see contract_stream.cu
  // frequency buffers, each sized for the largest use among the three passes
  size_t bytes_in, bytes_out, bytes_w, bytes_small, bytes_gi, bytes_total;
  // spectrum reuse (plane-major layers only): which tensor's forward spectrum a buffer holds
  bool have_input_spec = false, have_grad_output_spec = false, have_weight_spec = false;
  // set by a backward call between its two passes: the second one is handed the gradOutput whose spectrum
  // the first has just left in buf_out
  bool same_grad_output = false;
  char* ws = nullptr;
  bool ws_owned = false;
  // device copies for the host-buffer entry points
  char* stage = nullptr;
  size_t stage_bytes = 0;
  // asynchronous host-buffer passes: staging per pass, an upload and a download stream, and per
  // pass the events 'kernels done' (its input staging may be overwritten) and 'download done'
  // (its output staging may be overwritten)
  char* astage[3] = {nullptr, nullptr, nullptr};
  cudaStream_t up = nullptr, down = nullptr;
  cudaEvent_t ev_up = nullptr, ev_kernels[3] = {nullptr, nullptr, nullptr}, ev_down[3] = {nullptr, nullptr, nullptr};
  bool async_used[3] = {false, false, false};
  // second stream for the second forward transform of a pass, when the two together fit the GPU
  cudaStream_t aux = nullptr;
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
  // communicator
  ncclComm_t comm = nullptr;
  std::string comm_key;
  int rank = 0, nranks = 1;
  // sums over peer memory (peer.cu): set up at the first accGradParameters with a communicator
  bool peer_tried = false, peer_ready = false;
  PeerTable peers{};
  unsigned char* peer_block = nullptr;  // flag slots, block counter, staging of the handle exchange
  void* peer_mapped[2 * kMaxPeers] = {};  // cudaIpcOpenMemHandle results, to be closed
  int n_peer_mapped = 0;
  unsigned peer_epoch = 0;

  float2* buf_in() const { return reinterpret_cast<float2*>(ws); }
  float2* buf_out() const { return reinterpret_cast<float2*>(ws + bytes_in); }
  float2* buf_w() const { return reinterpret_cast<float2*>(ws + bytes_in + bytes_out); }
  float* small() const { return reinterpret_cast<float*>(ws + bytes_in + bytes_out + bytes_w); }
  // gradInput spectrum when the input spectrum has to survive updateGradInput
  // vector summed across ranks after the inverse transform: gradWeight (or this rank's part of it)
  // followed by the bias gradient; and the block the sum over peers is delivered to
  float* vec_in() const { return small() + align_floats(((size_t)d.batch * d.n_output_plane + d.n_output_plane)); }
  float* vec_out() const {
    return vec_in() + align_floats((size_t)d.n_output_plane * d.n_input_plane * d.kernel_h * d.kernel_w + d.n_output_plane);
  }
  static size_t align_floats(size_t n) { return ((n * sizeof(float) + 255) & ~size_t(255)) / sizeof(float); }
  float2* buf_gi() const {
    return bytes_gi ? reinterpret_cast<float2*>(ws + bytes_in + bytes_out + bytes_w + bytes_small) : buf_in();
  }
};

namespace {

size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

int ensure_workspace(fbfftconv_handle* h) {
  if (h->ws) return FBFFTCONV_OK;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, h->bytes_total);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(e == cudaErrorMemoryAllocation ? FBFFTCONV_ERR_NOMEM : FBFFTCONV_ERR_CUDA,
                "workspace of %zu bytes: %s", h->bytes_total, cudaGetErrorString(e));
  }
  h->ws = static_cast<char*>(p);
  h->ws_owned = true;
  return FBFFTCONV_OK;
}

// Brackets the work enqueued during its lifetime with an event pair of (pass, stage).
struct StageTimer {
  fbfftconv_handle* h;
  cudaStream_t s;
  EventPair* ev = nullptr;
  StageTimer(fbfftconv_handle* h_, int pass, int stage, cudaStream_t s_) : h(h_), s(s_) {
    if (!h->profiling) return;
    auto& pool = h->events[pass][stage];
    int& used = h->events_used[pass][stage];
    if (used == (int)pool.size()) {
      EventPair p;
      if (cudaEventCreate(&p.start) != cudaSuccess || cudaEventCreate(&p.stop) != cudaSuccess) return;
      pool.push_back(p);
    }
    ev = &pool[used++];
    cudaEventRecord(ev->start, s);
  }
  ~StageTimer() {
    if (ev) cudaEventRecord(ev->stop, s);
  }
};

// The two forward transforms of a pass are independent.  Where at least one of them is too
// small to fill the GPU by itself (small layers, small batch shards) the second runs on the
// handle's own stream between an event fork and join, so the two overlap; the pattern is
// capturable in a CUDA graph.  Large transforms stay in order on the caller's stream.
struct Fork {
  fbfftconv_handle* h;
  cudaStream_t main;
  bool active = false;
  Fork(fbfftconv_handle* h_, cudaStream_t s, long long tiles_a, long long tiles_b) : h(h_), main(s) {
    const long long fills_the_gpu = 4LL * sm_count();
    if (tiles_a >= fills_the_gpu && tiles_b >= fills_the_gpu) return;
    if (!h->aux) {
      if (cudaStreamCreateWithFlags(&h->aux, cudaStreamNonBlocking) != cudaSuccess ||
          cudaEventCreateWithFlags(&h->ev_fork, cudaEventDisableTiming) != cudaSuccess ||
          cudaEventCreateWithFlags(&h->ev_join, cudaEventDisableTiming) != cudaSuccess) {
        cudaGetLastError();
        return;  // stay on one stream
      }
    }
    if (cudaEventRecord(h->ev_fork, main) != cudaSuccess || cudaStreamWaitEvent(h->aux, h->ev_fork, 0) != cudaSuccess) {
      cudaGetLastError();
      return;
    }
    active = true;
  }
  cudaStream_t second() const { return active ? h->aux : main; }
  cudaError_t join() {
    if (!active) return cudaSuccess;
    active = false;
    cudaError_t e = cudaEventRecord(h->ev_join, h->aux);
    if (e != cudaSuccess) return e;
    return cudaStreamWaitEvent(main, h->ev_join, 0);
  }
  ~Fork() { join(); }  // an early return between fork and join must not leave the streams apart
};

// Tiles (blocks of work) of a forward transform of d1 x d2 planes.
long long forward_tiles(int N, int d1, int d2, int h, int w, int pad_u, int pad_l, bool transposed) {
  const int T = pick_forward_tile(N, h, w, pad_u, pad_l);
  if (T <= 0) return 1LL << 40;
  const long long rows = transposed ? d2 : d1, inner = transposed ? d1 : d2;
  return rows * ((inner + T - 1) / T);
}

struct DeviceGuard {
  int prev = -1;
  bool switched = false;
  cudaError_t enter(int dev) {
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return e;
    if (prev != dev) {
      e = cudaSetDevice(dev);
      switched = (e == cudaSuccess);
    }
    return e;
  }
  ~DeviceGuard() {
    if (switched) cudaSetDevice(prev);
  }
};

// layout: 0 = [bin][d1][d2], 1 = [bin][d2][d1], 2 = plane-major [d1][d2][bin]
void set_spectrum_layout(FftParams& p, int fft_size, bool plane_major) {
  const long long bins = (long long)(fft_size / 2 + 1) * fft_size;
  if (plane_major) {
    p.kc = p.n_inner;
    p.spec_bin = 1;
    p.spec_row = (long long)p.n_inner * bins;
    p.spec_inner = bins;
  } else {
    p.kc = pad4(p.n_inner);
    p.spec_bin = (long long)p.n_rows * p.kc;
    p.spec_row = p.kc;
    p.spec_inner = 1;
  }
}

FftParams forward_params(const float* real, float2* spec, int d1, int d2, int h, int w, int pad_u,
                         int pad_l, int layout, int fft_size) {
  const bool transposed = layout == 1;
  FftParams p{};
  p.real_in = real;
  p.spec = spec;
  p.h = h;
  p.w = w;
  p.off_y = pad_u;
  p.off_x = pad_l;
  if (!transposed) {  // [bin][d1][d2]
    p.n_rows = d1;
    p.n_inner = d2;
    p.real_row_stride = d2;
    p.real_inner_stride = 1;
  } else {  // [bin][d2][d1]
    p.n_rows = d2;
    p.n_inner = d1;
    p.real_row_stride = 1;
    p.real_inner_stride = d2;
  }
  set_spectrum_layout(p, fft_size, layout == 2);
  return p;
}

// layout as in forward_params: 0 = spectrum [bin][d1][d2], 1 = [bin][d2][d1], 2 = plane-major [d1][d2][bin];
// the real tensor is (d1, d2, h, w) and bias has d2 entries in every case.
FftParams inverse_params(const float2* spec, float* real, const float* bias, int d1, int d2, int h,
                         int w, int off_y, int off_x, int accumulate, int layout, int fft_size) {
  FftParams p{};
  p.real_out = real;
  p.spec = const_cast<float2*>(spec);
  p.bias = bias;
  p.h = h;
  p.w = w;
  p.off_y = off_y;
  p.off_x = off_x;
  if (layout != 1) {
    p.n_rows = d1;
    p.n_inner = d2;
    p.real_row_stride = d2;
    p.real_inner_stride = 1;
  } else {
    p.n_rows = d2;
    p.n_inner = d1;
    p.real_row_stride = 1;
    p.real_inner_stride = d2;
    p.bias_by_row = 1;
  }
  p.accumulate = accumulate;
  set_spectrum_layout(p, fft_size, layout == 2);
  return p;
}

// With a small batch (a shard of a data-parallel step) the batch goes on the column side of the
// tensor-core contraction, whose tile narrows to 16 / 32 / 64 columns, and the filters or input
// planes fill the 128 rows of the MMA; the product then comes out transposed ([bin][f][b] instead of
// [bin][b][f]) and the inverse transform reads it that way.  At 128 images nothing changes.
bool batch_on_columns(int batch, int other) { return batch <= 64 && other > batch; }

// An operand is [bins][rows][pad4(k)], or -- `mn` set -- [bins][k][pad4(rows)]: the spectra are written
// once, plane index innermost, and a pass whose sum runs over the outer plane index reads them that way.
int contract(const float2* a, const float2* b, float2* c, int bins, int m, int n, int k, float alpha,
             int conj_a, int conj_b, bool simt, cudaStream_t s, bool a_mn = false, bool b_mn = false) {
  ContractParams p{};
  p.a = a;
  p.b = b;
  p.c = c;
  p.bins = bins;
  p.m = m;
  p.n = n;
  p.k = k;
  p.lda = a_mn ? pad4(m) : pad4(k);
  p.ldb = b_mn ? pad4(n) : pad4(k);
  p.ldc = pad4(n);
  p.alpha = alpha;
  p.conj_a = conj_a;
  p.conj_b = conj_b;
  p.a_mn = a_mn;
  p.b_mn = b_mn;
  if (!simt && contract_tc_supported(p)) {
    FBF_CUDA(launch_contract_tc(p, s));
  } else {
    FBF_CUDA(launch_contract_simt(p, s));
  }
  return FBFFTCONV_OK;
}

// Contractions with a tiny column count or depth are bandwidth-bound streams: the CUDA-core
// kernels (one of them shaped for <= 4 columns) serve them; everything else goes to the
// tensor cores.
bool thin_contraction(int m, int n, int k) {
  (void)m;
  return n <= 4 || k < 8;
}

// sizes of the stand-alone transforms (nn.FFTWrapper, test/test_FFTModule.lua:170-260); a convolution never
// picks less than 8
bool valid_fft_size(int n) { return n == 2 || n == 4 || n == 8 || n == 16 || n == 32 || n == 64 || n == 128; }
// the 1-D stand-alone transforms also have the reference's largest 1-D size
bool valid_fft1d_size(int n) { return valid_fft_size(n) || n == 256; }

// What the reference's bindings check before they launch (THCudaTensor_checkGPU over all tensors,
// src/fft/SpatialConvolutionCuFFTHost.cpp:33-66): every tensor lives in device memory of the
// module's GPU.  A host pointer, or memory of another GPU, is refused instead of launched on.
int check_device_pointer(int device, const void* ptr, const char* name) {
  if (!ptr) return FBFFTCONV_OK;  // optional arguments; the required ones were checked for null
  cudaPointerAttributes attr{};
  cudaError_t e = cudaPointerGetAttributes(&attr, ptr);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return cuda_fail(e, "cudaPointerGetAttributes");
  }
  if (attr.type == cudaMemoryTypeManaged) return FBFFTCONV_OK;
  if (attr.type != cudaMemoryTypeDevice)
    return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "%s is not a device pointer (use the *_host entry points for host buffers)", name);
  if (attr.device != device)
    return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "%s lives on device %d, the handle on device %d", name, attr.device, device);
  return FBFFTCONV_OK;
}

// A bounded wait of the tensor-core contraction that ran out leaves its tile unwritten and a
// sticky device code; entry points that have just synchronised report it.
int check_tensor_core_status() {
  const int code = contract_tc_error(false);
  if (code > 0)
    return fail(FBFFTCONV_ERR_CUDA, "tensor-core contraction gave up a bounded wait (device code %d); results are incomplete", code);
  return FBFFTCONV_OK;
}

void close_peers(fbfftconv_handle* h) {
  for (int i = 0; i < h->n_peer_mapped; ++i) cudaIpcCloseMemHandle(h->peer_mapped[i]);
  h->n_peer_mapped = 0;
  if (h->peer_block) cudaFree(h->peer_block);
  h->peer_block = nullptr;
  h->peer_tried = h->peer_ready = false;
  cudaGetLastError();
}

// What a rank publishes to the others: how to map its scratch and its flag block, and where in the
// scratch the blocks of the exchange lie (a rank's layout follows its own batch share).
struct PeerEntry {
  cudaIpcMemHandle_t ws, block;
  unsigned long long off_spec, off_in, off_out;
  int ok;
  int pad[9];
};
static_assert(sizeof(PeerEntry) == 192, "entry size is part of the exchange");
constexpr size_t kPeerBlockBytes = 8192;  // [0, 1024): flags, counter; [1024, ...): exchange staging
constexpr size_t kPeerStaging = 1024;
constexpr size_t kPeerVerdict = 4096;

// Collective over the communicator: every rank with a communicator calls it at the same point (the
// first accGradParameters).  Afterwards peer_ready is the same on all ranks: true only if every rank
// could export its blocks and map everybody else's; otherwise the NCCL exchange is used.  Waits for
// the stream once.
int ensure_peers(fbfftconv_handle* h, NcclApi* api, cudaStream_t s) {
  if (h->peer_tried) return FBFFTCONV_OK;
  h->peer_tried = true;
  h->peer_ready = false;
  if (!h->comm || h->nranks < 2) return FBFFTCONV_OK;
  const char* env = getenv("FBFFTCONV_PEER_EXCHANGE");
  bool mine = h->nranks <= kMaxPeers && h->ws_owned && api->AllGather && !(h->d.flags & FBFFTCONV_EXCHANGE_NCCL) &&
              !(env && env[0] == '0');
  void* block = nullptr;
  cudaError_t e = cudaMalloc(&block, kPeerBlockBytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(FBFFTCONV_ERR_NOMEM, "flag block of the peer exchange: %s", cudaGetErrorString(e));
  }
  h->peer_block = static_cast<unsigned char*>(block);
  FBF_CUDA(cudaMemsetAsync(block, 0, kPeerBlockBytes, s));
  if (!api->AllGather || h->nranks * sizeof(PeerEntry) > kPeerVerdict - kPeerStaging) {
    // no way to agree: every rank sees the same condition and stays on NCCL
    return FBFFTCONV_OK;
  }
  PeerEntry me{};
  if (mine) {
    mine = cudaIpcGetMemHandle(&me.ws, h->ws) == cudaSuccess && cudaIpcGetMemHandle(&me.block, block) == cudaSuccess;
    cudaGetLastError();
  }
  me.ok = mine ? 1 : 0;
  me.off_spec = reinterpret_cast<char*>(h->buf_w()) - h->ws;
  me.off_in = reinterpret_cast<char*>(h->vec_in()) - h->ws;
  me.off_out = reinterpret_cast<char*>(h->vec_out()) - h->ws;
  unsigned char* staging = h->peer_block + kPeerStaging;
  FBF_CUDA(cudaMemcpyAsync(staging + h->rank * sizeof(PeerEntry), &me, sizeof(me), cudaMemcpyHostToDevice, s));
  ncclResult_t r = api->AllGather(staging + h->rank * sizeof(PeerEntry), staging, sizeof(PeerEntry), ncclChar, h->comm, s);
  if (r != ncclSuccess) return nccl_fail(api, r, "ncclAllGather(peer handles)");
  std::vector<PeerEntry> all(h->nranks);
  FBF_CUDA(cudaMemcpyAsync(all.data(), staging, h->nranks * sizeof(PeerEntry), cudaMemcpyDeviceToHost, s));
  FBF_CUDA(cudaStreamSynchronize(s));
  bool everyone = true;
  for (const PeerEntry& p : all) everyone = everyone && p.ok == 1;
  // map the peers (every rank tries only if every rank exported), then agree on the outcome
  int mapped_ok = everyone ? 1 : 0;
  PeerTable t{};
  t.rank = h->rank;
  t.nranks = h->nranks;
  t.spin_limit = 0;  // default
  t.counter = reinterpret_cast<unsigned*>(h->peer_block + 512);
  for (int q = 0; q < h->nranks && mapped_ok; ++q) {
    char* base;
    unsigned char* blk;
    if (q == h->rank) {
      base = h->ws;
      blk = h->peer_block;
    } else {
      void* pw = nullptr;
      void* pb = nullptr;
      if (cudaIpcOpenMemHandle(&pw, all[q].ws, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        cudaGetLastError();
        mapped_ok = 0;
        break;
      }
      h->peer_mapped[h->n_peer_mapped++] = pw;
      if (cudaIpcOpenMemHandle(&pb, all[q].block, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        cudaGetLastError();
        mapped_ok = 0;
        break;
      }
      h->peer_mapped[h->n_peer_mapped++] = pb;
      base = static_cast<char*>(pw);
      blk = static_cast<unsigned char*>(pb);
    }
    t.spec[q] = base + all[q].off_spec;
    t.vec_in[q] = base + all[q].off_in;
    t.vec_out[q] = base + all[q].off_out;
    t.flags[q] = reinterpret_cast<unsigned*>(blk);
  }
  int* verdict = reinterpret_cast<int*>(h->peer_block + kPeerVerdict);
  FBF_CUDA(cudaMemcpyAsync(verdict, &mapped_ok, sizeof(int), cudaMemcpyHostToDevice, s));
  r = api->AllReduce(verdict, verdict, 1, ncclInt, ncclMin, h->comm, s);
  if (r != ncclSuccess) return nccl_fail(api, r, "ncclAllReduce(peer mapping)");
  int agreed = 0;
  FBF_CUDA(cudaMemcpyAsync(&agreed, verdict, sizeof(int), cudaMemcpyDeviceToHost, s));
  FBF_CUDA(cudaStreamSynchronize(s));
  if (agreed == 1) {
    h->peers = t;
    h->peer_ready = true;
    h->peer_epoch = 1;  // the flag slots start at 0: the first barrier must wait for a real signal
  } else {
    for (int i = 0; i < h->n_peer_mapped; ++i) cudaIpcCloseMemHandle(h->peer_mapped[i]);
    h->n_peer_mapped = 0;
    cudaGetLastError();
  }
  return FBFFTCONV_OK;
}

void release_comm(fbfftconv_handle* h) {
  close_peers(h);
  if (!h->comm) return;
  std::lock_guard<std::mutex> lock(g_comm_mutex);
  auto it = g_comms.find(h->comm_key);
  if (it != g_comms.end()) --it->second.refs;  // the communicator itself stays: an id cannot be used twice
  h->comm = nullptr;
  h->comm_key.clear();
  h->rank = 0;
  h->nranks = 1;
}

}  // namespace

namespace fbfft {
int report_error(int code, const char* message) { return fail(code, "%s", message); }
int validate_device_pointer(int device, const void* ptr, const char* name) {
  return check_device_pointer(device, ptr, name);
}
}  // namespace fbfft

extern "C" {

const char* fbfftconv_last_error(void) { return t_error.c_str(); }

const char* fbfftconv_status_string(int status) {
  switch (status) {
    case FBFFTCONV_OK: return "ok";
    case FBFFTCONV_ERR_INVALID_ARGUMENT: return "invalid argument";
    case FBFFTCONV_ERR_UNSUPPORTED_SIZE: return "unsupported transform size";
    case FBFFTCONV_ERR_NOMEM: return "out of device memory";
    case FBFFTCONV_ERR_CUDA: return "CUDA error";
    case FBFFTCONV_ERR_COMM: return "communicator error";
  }
  return "unknown status";
}

uint64_t fbfftconv_kernel_launches(void) { return launch_count(); }

size_t fbfftconv_spectrum_bytes(int fft_size, int rows, int inner) {
  if (!valid_fft_size(fft_size) || rows <= 0 || inner <= 0) return 0;
  return (size_t)(fft_size / 2 + 1) * fft_size * rows * pad4(inner) * sizeof(float2);
}

int fbfftconv_create(const fbfftconv_desc* desc, fbfftconv_handle** out) {
  if (!desc || !out) return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null argument");
  *out = nullptr;
  const fbfftconv_desc& d = *desc;
  if (d.batch <= 0 || d.n_input_plane <= 0 || d.n_output_plane <= 0 || d.input_h <= 0 ||
      d.input_w <= 0 || d.kernel_h <= 0 || d.kernel_w <= 0)
    return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "sizes must be positive");
  if (d.stride_h != 1 || d.stride_w != 1)
    return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "fft only supports stride-1 convolutions");
  if (d.pad_h < 0 || d.pad_w < 0 || d.pad_h >= d.kernel_h || d.pad_w >= d.kernel_w)
    return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "padding must be non-negative and smaller than the kernel");
  const int oH = d.input_h + 2 * d.pad_h - d.kernel_h + 1;
  const int oW = d.input_w + 2 * d.pad_w - d.kernel_w + 1;
  if (oH <= 0 || oW <= 0)
    return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "kernel larger than the padded input");
  int need = d.input_h + 2 * d.pad_h;
  if (d.input_w + 2 * d.pad_w > need) need = d.input_w + 2 * d.pad_w;
  if (d.kernel_h > need) need = d.kernel_h;
  if (d.kernel_w > need) need = d.kernel_w;
  int N = next_pow2(need);
  if (N < 8) N = 8;
  if (N > 128)
    return fail(FBFFTCONV_ERR_UNSUPPORTED_SIZE, "transform size %d exceeds 128", N);
  if ((long long)d.batch > 65535 || d.n_input_plane > 65535 || d.n_output_plane > 65535)
    return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "batch / plane counts above 65535 are not supported");

  int device = d.device;
  if (device < 0) {
    if (cudaGetDevice(&device) != cudaSuccess) {
      cudaGetLastError();
      device = 0;  // resolved again, with an error, at the first pass
    }
  }
  fbfftconv_handle* h = new fbfftconv_handle();
  h->d = d;
  h->device = device;
  h->N = N;
  h->bins = (N / 2 + 1) * N;
  h->plane_major = d.n_input_plane <= 4 && N >= 64 && !(d.flags & FBFFTCONV_BIN_MAJOR_ONLY);
  h->oH = oH;
  h->oW = oW;
  const size_t B = d.batch, P = d.n_input_plane, F = d.n_output_plane, bins = h->bins;
  auto mx = [](size_t a, size_t b) { return a > b ? a : b; };
  h->bytes_in = align256(bins * mx(B * pad4(P), P * pad4(B)) * sizeof(float2));
  h->bytes_out = align256(bins * mx(B * pad4(F), F * pad4(B)) * sizeof(float2));
  // (+ F floats behind the gradWeight spectrum: the bias gradient rides in the same all-reduce)
  h->bytes_w = align256(bins * mx(F * pad4(P), P * pad4(F)) * sizeof(float2) + F * sizeof(float));
  h->bytes_small = align256((B * F + F) * sizeof(float));
  // local gradWeight + gradBias where they are summed or gathered across ranks in the spatial domain
  h->bytes_small += 2 * align256((F * P * d.kernel_h * d.kernel_w + F) * sizeof(float));  // vec_in, vec_out
  h->bytes_gi = (d.flags & FBFFTCONV_REUSE_INPUT) ? h->bytes_in : 0;
  h->bytes_total = h->bytes_in + h->bytes_out + h->bytes_w + h->bytes_small + h->bytes_gi;
  *out = h;
  return FBFFTCONV_OK;
}

int fbfftconv_destroy(fbfftconv_handle* h) {
  if (!h) return FBFFTCONV_OK;
  DeviceGuard g;
  g.enter(h->device);
  release_comm(h);
  if (h->ws && h->ws_owned) cudaFree(h->ws);
  if (h->stage) cudaFree(h->stage);
  for (int i = 0; i < 3; ++i) {
    if (h->astage[i]) cudaFree(h->astage[i]);
    if (h->ev_kernels[i]) cudaEventDestroy(h->ev_kernels[i]);
    if (h->ev_down[i]) cudaEventDestroy(h->ev_down[i]);
  }
  if (h->ev_up) cudaEventDestroy(h->ev_up);
  if (h->up) cudaStreamDestroy(h->up);
  if (h->down) cudaStreamDestroy(h->down);
  if (h->aux) cudaStreamDestroy(h->aux);
  if (h->ev_fork) cudaEventDestroy(h->ev_fork);
  if (h->ev_join) cudaEventDestroy(h->ev_join);
  for (auto& per_pass : h->events)
    for (auto& pool : per_pass)
      for (auto& p : pool) {
        cudaEventDestroy(p.start);
        cudaEventDestroy(p.stop);
      }
  delete h;
  return FBFFTCONV_OK;
}

int fbfftconv_fft_size(const fbfftconv_handle* h) { return h ? h->N : 0; }
size_t fbfftconv_workspace_bytes(const fbfftconv_handle* h) { return h ? h->bytes_total : 0; }

int fbfftconv_set_workspace(fbfftconv_handle* h, void* device_ptr, size_t bytes) {
  if (!h) return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null handle");
  if (!device_ptr || bytes < h->bytes_total || (reinterpret_cast<uintptr_t>(device_ptr) & 255))
    return fail(FBFFTCONV_ERR_INVALID_ARGUMENT,
                "workspace must be 256-byte aligned and hold %zu bytes", h->bytes_total);
  if (h->ws && h->ws_owned) {
    DeviceGuard g;
    g.enter(h->device);
    cudaFree(h->ws);
  }
  h->ws = static_cast<char*>(device_ptr);
  h->ws_owned = false;
  {
    DeviceGuard g;
    g.enter(h->device);
    close_peers(h);  // mappings of the old block are stale; the exchange goes back to NCCL for this handle
  }
  // the new block holds no spectra yet: nothing of an earlier pass can be taken over
  h->have_input_spec = h->have_grad_output_spec = h->have_weight_spec = false;
  return FBFFTCONV_OK;
}

// ---- passes ----------------------------------------------------------------

int fbfftconv_update_output(fbfftconv_handle* h, const float* input, const float* weight,
                            const float* bias, float* output, fbfftconv_stream stream) {
  if (!h || !input || !weight || !output) return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null argument");
  DeviceGuard g;
  FBF_CUDA(g.enter(h->device));
  FBF_TRY(check_device_pointer(h->device, input, "input"));
  FBF_TRY(check_device_pointer(h->device, weight, "weight"));
  FBF_TRY(check_device_pointer(h->device, bias, "bias"));
  FBF_TRY(check_device_pointer(h->device, output, "output"));
  FBF_TRY(ensure_workspace(h));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const fbfftconv_desc& d = h->d;
  const int B = d.batch, P = d.n_input_plane, F = d.n_output_plane;
  const bool simt = (d.flags & FBFFTCONV_CONTRACT_SIMT) || thin_contraction(B, F, P);
  const int pass = FBFFTCONV_PASS_UPDATE_OUTPUT;
  const bool pm = h->plane_major;
  const bool flip = !pm && !simt && batch_on_columns(B, F);
  const float norm = 1.0f / (float)(h->N * h->N);
  // I^[bin][b][p], W^[bin][f][p]   (plane-major: I^[b][p][bin], W^[f][p][bin])
  {
    Fork fork(h, s, forward_tiles(h->N, B, P, d.input_h, d.input_w, d.pad_h, d.pad_w, false),
              forward_tiles(h->N, F, P, d.kernel_h, d.kernel_w, 0, 0, false));
    {
      StageTimer t(h, pass, FBFFTCONV_STAGE_FFT_A, s);
      FBF_CUDA(launch_forward(forward_params(input, h->buf_in(), B, P, d.input_h, d.input_w, d.pad_h, d.pad_w, pm ? 2 : 0, h->N), h->N, s));
    }
    {
      StageTimer t(h, pass, FBFFTCONV_STAGE_FFT_B, fork.second());
      if (fork.active) h->overlapped[pass][FBFFTCONV_STAGE_FFT_B] = true;
      FBF_CUDA(launch_forward(forward_params(weight, h->buf_w(), F, P, d.kernel_h, d.kernel_w, 0, 0, pm ? 2 : 0, h->N), h->N, fork.second()));
    }
    FBF_CUDA(fork.join());
  }
  // O^[b][f] = 1/N^2 sum_p I^[b][p] conj(W^[f][p]) per bin
  {
    StageTimer t(h, pass, FBFFTCONV_STAGE_CONTRACT, s);
    if (pm) {
      FBF_CUDA(launch_stream_expand(h->buf_in(), h->buf_w(), h->buf_out(), B, F, P, h->bins, norm, s));
    } else if (flip) {  // O^[f][b] = 1/N^2 sum_p conj(W^[f][p]) I^[b][p]
      FBF_TRY(contract(h->buf_w(), h->buf_in(), h->buf_out(), h->bins, F, B, P, norm, 1, 0, simt, s));
    } else {
      FBF_TRY(contract(h->buf_in(), h->buf_w(), h->buf_out(), h->bins, B, F, P, norm, 0, 1, simt, s));
    }
  }
  {
    StageTimer t(h, pass, FBFFTCONV_STAGE_IFFT, s);
    FBF_CUDA(launch_inverse(inverse_params(h->buf_out(), output, bias, B, F, h->oH, h->oW, 0, 0, 0,
                                           pm ? 2 : (flip ? 1 : 0), h->N), h->N, s));
  }
  // what the buffers hold now (every pass reads a tensor's spectrum in the one layout it is written in)
  h->have_input_spec = true;
  h->have_weight_spec = true;
  h->have_grad_output_spec = false;  // buf_out holds the output spectrum
  return FBFFTCONV_OK;
}

int fbfftconv_update_grad_input(fbfftconv_handle* h, const float* grad_output, const float* weight,
                                float* grad_input, fbfftconv_stream stream) {
  if (!h || !grad_output || !weight || !grad_input)
    return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null argument");
  DeviceGuard g;
  FBF_CUDA(g.enter(h->device));
  FBF_TRY(check_device_pointer(h->device, grad_output, "gradOutput"));
  FBF_TRY(check_device_pointer(h->device, weight, "weight"));
  FBF_TRY(check_device_pointer(h->device, grad_input, "gradInput"));
  FBF_TRY(ensure_workspace(h));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const fbfftconv_desc& d = h->d;
  const int B = d.batch, P = d.n_input_plane, F = d.n_output_plane;
  const bool simt = (d.flags & FBFFTCONV_CONTRACT_SIMT) || thin_contraction(B, P, F);
  const int pass = FBFFTCONV_PASS_UPDATE_GRAD_INPUT;
  const bool pm = h->plane_major;
  const bool flip = !pm && !simt && batch_on_columns(B, P);
  const float norm = 1.0f / (float)(h->N * h->N);
  // O'^[bin][b][f], W^[bin][f][p] (the sum over f reads W^ with f as the row index)
  {
    Fork fork(h, s, forward_tiles(h->N, B, F, h->oH, h->oW, 0, 0, false),
              forward_tiles(h->N, F, P, d.kernel_h, d.kernel_w, 0, 0, false));
    {
      StageTimer t(h, pass, FBFFTCONV_STAGE_FFT_A, s);
      FBF_CUDA(launch_forward(forward_params(grad_output, h->buf_out(), B, F, h->oH, h->oW, 0, 0, pm ? 2 : 0, h->N), h->N, s));
    }
    h->have_grad_output_spec = true;
    if (!((d.flags & FBFFTCONV_REUSE_WEIGHT) && h->have_weight_spec)) {
      StageTimer t(h, pass, FBFFTCONV_STAGE_FFT_B, fork.second());
      if (fork.active) h->overlapped[pass][FBFFTCONV_STAGE_FFT_B] = true;
      FBF_CUDA(launch_forward(forward_params(weight, h->buf_w(), F, P, d.kernel_h, d.kernel_w, 0, 0, pm ? 2 : 0, h->N), h->N, fork.second()));
      h->have_weight_spec = true;
    }
    FBF_CUDA(fork.join());
  }
  // with REUSE_INPUT the input spectrum stays in its buffer for accGradParameters
  float2* gi = h->buf_gi();
  if (gi == h->buf_in()) h->have_input_spec = false;
  // I'^[bin][b][p] = 1/N^2 sum_f O'^[b][f] W^[f][p]
  {
    StageTimer t(h, pass, FBFFTCONV_STAGE_CONTRACT, s);
    if (pm) {  // I'^[b][p] = sum_f O'^[b][f] W^[f][p]
      FBF_CUDA(launch_stream_reduce(h->buf_out(), h->buf_w(), gi, B, F, P, F, 1, false, h->bins, norm, s));
    } else if (flip) {  // I'^[p][b] = 1/N^2 sum_f W^[f][p] O'^[b][f]
      FBF_TRY(contract(h->buf_w(), h->buf_out(), gi, h->bins, P, B, F, norm, 0, 0, simt, s, true, false));
    } else {
      FBF_TRY(contract(h->buf_out(), h->buf_w(), gi, h->bins, B, P, F, norm, 0, 0, simt, s, false, true));
    }
  }
  {
    StageTimer t(h, pass, FBFFTCONV_STAGE_IFFT, s);
    FBF_CUDA(launch_inverse(inverse_params(gi, grad_input, nullptr, B, P, d.input_h, d.input_w,
                                           d.pad_h, d.pad_w, 0, pm ? 2 : (flip ? 1 : 0), h->N), h->N, s));
  }
  return FBFFTCONV_OK;
}

namespace {

// How accGradParameters sums the weight gradient over `nranks` ranks, as `rank` sees it: arithmetic
// on the handle's sizes only (no device), used by the pass and reported by fbfftconv_exchange_plan.
struct ExchangePlan {
  int mode;                          // FBFFTCONV_SUM_*
  size_t spec_floats;                // the whole gradient spectrum
  size_t chunk_floats, first_float;  // this rank's share of it (by filters / by bins)
  size_t zero_before, zero_after;    // by bins: the other ranks' bins, cleared before the inverse transform
  size_t n_weight;                   // gradWeight
  size_t slice_floats, slice_first;  // by filters: this rank's filters inside gradWeight
  size_t vec4;                       // float4s of [gradWeight | gradBias], the vector summed after the transform
};

ExchangePlan exchange_plan(const fbfftconv_handle* h, int rank, int nranks) {
  const fbfftconv_desc& d = h->d;
  const size_t F = d.n_output_plane, P = d.n_input_plane;
  const bool pm = h->plane_major;
  ExchangePlan x{};
  x.spec_floats = (size_t)h->bins * F * (pm ? P : (size_t)pad4((int)P)) * 2;
  x.n_weight = F * P * d.kernel_h * d.kernel_w;
  x.vec4 = (x.n_weight + F + 3) / 4;
  if (nranks < 1) {
    x.mode = FBFFTCONV_SUM_NONE;
  } else if (d.flags & FBFFTCONV_ALLREDUCE_SPATIAL) {
    x.mode = FBFFTCONV_SUM_SPATIAL;
  } else if (pm && F % nranks == 0) {
    // plane-major spectra are contiguous per filter: every rank sums and inverts its own filters
    x.mode = FBFFTCONV_SUM_SPECTRUM_BY_FILTERS;
    x.chunk_floats = x.spec_floats / nranks;
    x.first_float = (size_t)rank * x.chunk_floats;
    x.slice_floats = x.n_weight / nranks;
    x.slice_first = (size_t)rank * x.slice_floats;
  } else if (!pm && nranks > 1 && h->bins % nranks == 0) {
    // bin-major spectra are contiguous per bin: every rank sums a range of bins and inverts the
    // spectrum that is zero outside it (the transform is linear in the bins)
    x.mode = FBFFTCONV_SUM_SPECTRUM_BY_BINS;
    x.chunk_floats = x.spec_floats / nranks;
    x.first_float = (size_t)rank * x.chunk_floats;
    x.zero_before = x.first_float;
    x.zero_after = x.spec_floats - x.first_float - x.chunk_floats;
  } else {
    x.mode = FBFFTCONV_SUM_SPECTRUM_WHOLE;
  }
  return x;
}

}  // namespace

int fbfftconv_exchange_plan(const fbfftconv_handle* h, int rank, int nranks, long long out[10]) {
  if (!h || !out) return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null argument");
  if (nranks < 0 || (nranks > 0 && (rank < 0 || rank >= nranks)))
    return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "rank %d of %d", rank, nranks);
  const ExchangePlan x = exchange_plan(h, rank, nranks);
  const long long v[10] = {x.mode, (long long)x.spec_floats, (long long)x.chunk_floats, (long long)x.first_float,
                           (long long)x.zero_before, (long long)x.zero_after, (long long)x.n_weight,
                           (long long)x.slice_floats, (long long)x.slice_first, (long long)x.vec4};
  for (int i = 0; i < 10; ++i) out[i] = v[i];
  return FBFFTCONV_OK;
}

int fbfftconv_acc_grad_parameters(fbfftconv_handle* h, const float* input, const float* grad_output,
                                  float* grad_weight, float* grad_bias, float scale,
                                  fbfftconv_stream stream) {
  if (!h || !input || !grad_output || !grad_weight)
    return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null argument");
  DeviceGuard g;
  FBF_CUDA(g.enter(h->device));
  FBF_TRY(check_device_pointer(h->device, input, "input"));
  FBF_TRY(check_device_pointer(h->device, grad_output, "gradOutput"));
  FBF_TRY(check_device_pointer(h->device, grad_weight, "gradWeight"));
  FBF_TRY(check_device_pointer(h->device, grad_bias, "gradBias"));
  FBF_TRY(ensure_workspace(h));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const fbfftconv_desc& d = h->d;
  const int B = d.batch, P = d.n_input_plane, F = d.n_output_plane;
  const bool simt = (d.flags & FBFFTCONV_CONTRACT_SIMT) || thin_contraction(F, P, B);
  const int accumulate = (d.flags & FBFFTCONV_ACCUMULATE_GRADS) ? 1 : 0;
  const int pass = FBFFTCONV_PASS_ACC_GRAD_PARAMETERS;
  const bool pm = h->plane_major;
  // O'^[bin][b][f], I^[bin][b][p]: the batch, the row index of both, is the contraction index here
  {
    Fork fork(h, s, forward_tiles(h->N, B, F, h->oH, h->oW, 0, 0, false),
              forward_tiles(h->N, B, P, d.input_h, d.input_w, d.pad_h, d.pad_w, false));
    if (!(((d.flags & FBFFTCONV_REUSE_OUTPUT) || h->same_grad_output) && h->have_grad_output_spec)) {
      StageTimer t(h, pass, FBFFTCONV_STAGE_FFT_A, s);
      FBF_CUDA(launch_forward(forward_params(grad_output, h->buf_out(), B, F, h->oH, h->oW, 0, 0, pm ? 2 : 0, h->N), h->N, s));
      h->have_grad_output_spec = true;
    }
    if (!((d.flags & FBFFTCONV_REUSE_INPUT) && h->have_input_spec)) {
      StageTimer t(h, pass, FBFFTCONV_STAGE_FFT_B, fork.second());
      if (fork.active) h->overlapped[pass][FBFFTCONV_STAGE_FFT_B] = true;
      FBF_CUDA(launch_forward(forward_params(input, h->buf_in(), B, P, d.input_h, d.input_w, d.pad_h, d.pad_w, pm ? 2 : 0, h->N), h->N, fork.second()));
      h->have_input_spec = true;
    }
    FBF_CUDA(fork.join());
  }
  h->have_weight_spec = false;  // the weight buffer receives the gradient spectrum below
  NcclApi* api = h->comm ? nccl_api() : nullptr;
  if (h->comm && !api) return fail(FBFFTCONV_ERR_COMM, "libnccl is not loadable");
  if (h->comm) FBF_TRY(ensure_peers(h, api, s));
  // Sums over peer memory replace the NCCL calls below wherever the exchange is a reduce-scatter plus a
  // small sum (and for the spatial sum); the same choice is made on every rank.
  const bool peer = h->comm && h->peer_ready;
  // The same arithmetic on every rank: which sum, and which share of it is this rank's.
  ExchangePlan x = exchange_plan(h, h->comm ? h->rank : 0, h->comm ? h->nranks : 0);
  // without peer memory the shares travel by NCCL calls this libnccl may not have
  if (!peer && x.mode == FBFFTCONV_SUM_SPECTRUM_BY_FILTERS &&
      !(api->ReduceScatter && api->AllGather && api->GroupStart && api->GroupEnd))
    x.mode = FBFFTCONV_SUM_SPECTRUM_WHOLE;
  if (!peer && x.mode == FBFFTCONV_SUM_SPECTRUM_BY_BINS && !api->ReduceScatter) x.mode = FBFFTCONV_SUM_SPECTRUM_WHOLE;
  const size_t vec4 = x.vec4, spec_floats = x.spec_floats, n_weight = x.n_weight;
  const bool spatial = x.mode == FBFFTCONV_SUM_SPATIAL;
  const bool scatter = x.mode == FBFFTCONV_SUM_SPECTRUM_BY_FILTERS;
  const bool scatter_bins = x.mode == FBFFTCONV_SUM_SPECTRUM_BY_BINS;
  // Across ranks the bias gradient travels behind whatever the weight gradient is summed
  // as: behind its spectrum, or behind the local spatial gradient.
  float* local_w = h->vec_in();
  float* bias_part =
      (spatial || scatter || scatter_bins) ? local_w + n_weight : reinterpret_cast<float*>(h->buf_w()) + spec_floats;
  // W'^[bin][f][p] = scale/N^2 sum_b conj(O'^[b][f]) I^[b][p]
  {
    StageTimer t(h, pass, FBFFTCONV_STAGE_CONTRACT, s);
    const float norm = scale / (float)(h->N * h->N);
    if (pm) {  // W'^[f][p] = sum_b conj(O'^[b][f]) I^[b][p]
      FBF_CUDA(launch_stream_reduce(h->buf_out(), h->buf_in(), h->buf_w(), F, B, P, 1, F, true, h->bins, norm, s));
    } else {
      FBF_TRY(contract(h->buf_out(), h->buf_in(), h->buf_w(), h->bins, F, P, B, norm, 1, 0, simt, s, true, true));
    }
  }
  if (grad_bias) {
    StageTimer t(h, pass, FBFFTCONV_STAGE_BIAS, s);
    // bin (0,0) of O'^[bin][b][f] is the plain sum of gradOutput plane (b, f): its real
    // parts, summed over b, are the bias gradient (src/ConvolutionBias.cu:61-97).
    // (plane-major: element (b, f, bin 0) sits at ((b*F + f) * bins) complex values)
    const float* dc = reinterpret_cast<const float*>(h->buf_out());
    const long long ld = pm ? 2LL * h->bins : 2;
    const long long dc_step = pm ? 2LL * F * h->bins : 2LL * pad4(F);
    if (h->comm)
      FBF_CUDA(launch_row_sum(dc, bias_part, F, B, ld, dc_step, scale, 0, s));
    else
      FBF_CUDA(launch_row_sum(dc, grad_bias, F, B, ld, dc_step, scale, accumulate, s));
  }
  const size_t bias_floats = grad_bias ? (size_t)F : 0;
  if (scatter) {
    const size_t chunk = x.chunk_floats, slice = x.slice_floats;
    float* mine = reinterpret_cast<float*>(h->buf_w()) + x.first_float;
    {
      StageTimer t(h, pass, FBFFTCONV_STAGE_ALLREDUCE, s);
      if (peer) {
        FBF_CUDA(launch_peer_reduce(h->peers, h->peer_epoch, x.first_float / 4, chunk / 4, s));
        h->peer_epoch += 2;
        // this rank's filters will be the only non-zero part of the vector summed below
        FBF_CUDA(cudaMemsetAsync(local_w, 0, n_weight * sizeof(float), s));
      } else {
        ncclResult_t r = api->ReduceScatter(h->buf_w(), mine, chunk, ncclFloat, ncclSum, h->comm, s);
        if (r != ncclSuccess) return nccl_fail(api, r, "ncclReduceScatter(gradWeight spectrum)");
      }
    }
    {
      StageTimer t(h, pass, FBFFTCONV_STAGE_IFFT, s);
      FBF_CUDA(launch_inverse(inverse_params(reinterpret_cast<const float2*>(mine), local_w + x.slice_first,
                                             nullptr, F / h->nranks, P, d.kernel_h, d.kernel_w, 0, 0, 0, 2, h->N),
                              h->N, s));
    }
    if (peer) {
      StageTimer t(h, pass, FBFFTCONV_STAGE_ALLREDUCE, s);
      if (!grad_bias) FBF_CUDA(cudaMemsetAsync(bias_part, 0, F * sizeof(float), s));
      FBF_CUDA(launch_peer_allreduce(h->peers, h->peer_epoch, vec4, s));
      h->peer_epoch += 2;
      FBF_CUDA(launch_copy_or_add(h->vec_out(), grad_weight, (long long)n_weight, accumulate, s));
    } else {
      StageTimer t(h, pass, FBFFTCONV_STAGE_ALLREDUCE, s);
      ncclResult_t r = api->GroupStart();
      if (r == ncclSuccess)
        r = api->AllGather(local_w + x.slice_first, local_w, slice, ncclFloat, h->comm, s);
      if (r == ncclSuccess && bias_floats)
        r = api->AllReduce(bias_part, bias_part, bias_floats, ncclFloat, ncclSum, h->comm, s);
      const ncclResult_t r2 = api->GroupEnd();
      if (r != ncclSuccess || r2 != ncclSuccess)
        return nccl_fail(api, r != ncclSuccess ? r : r2, "ncclAllGather(gradWeight) / ncclAllReduce(gradBias)");
      FBF_CUDA(launch_copy_or_add(local_w, grad_weight, (long long)n_weight, accumulate, s));
    }
  } else if (scatter_bins) {
    const size_t chunk = x.chunk_floats;
    float* all = reinterpret_cast<float*>(h->buf_w());
    float* mine = all + x.first_float;
    {
      StageTimer t(h, pass, FBFFTCONV_STAGE_ALLREDUCE, s);
      if (peer) {
        FBF_CUDA(launch_peer_reduce(h->peers, h->peer_epoch, x.first_float / 4, chunk / 4, s));
        h->peer_epoch += 2;
      } else {
        ncclResult_t r = api->ReduceScatter(all, mine, chunk, ncclFloat, ncclSum, h->comm, s);
        if (r != ncclSuccess) return nccl_fail(api, r, "ncclReduceScatter(gradWeight spectrum)");
      }
    }
    // the other ranks' bins still hold this rank's partial products
    if (x.zero_before) FBF_CUDA(cudaMemsetAsync(all, 0, x.zero_before * sizeof(float), s));
    if (x.zero_after) FBF_CUDA(cudaMemsetAsync(mine + chunk, 0, x.zero_after * sizeof(float), s));
    {
      StageTimer t(h, pass, FBFFTCONV_STAGE_IFFT, s);
      FBF_CUDA(launch_inverse(inverse_params(h->buf_w(), local_w, nullptr, F, P, d.kernel_h, d.kernel_w, 0, 0, 0, 0,
                                             h->N), h->N, s));
    }
    {
      StageTimer t(h, pass, FBFFTCONV_STAGE_ALLREDUCE, s);
      if (peer) {
        if (!grad_bias) FBF_CUDA(cudaMemsetAsync(bias_part, 0, F * sizeof(float), s));
        FBF_CUDA(launch_peer_allreduce(h->peers, h->peer_epoch, vec4, s));
        h->peer_epoch += 2;
        FBF_CUDA(launch_copy_or_add(h->vec_out(), grad_weight, (long long)n_weight, accumulate, s));
      } else {
        ncclResult_t r = api->AllReduce(local_w, local_w, n_weight + bias_floats, ncclFloat, ncclSum, h->comm, s);
        if (r != ncclSuccess) return nccl_fail(api, r, "ncclAllReduce(gradWeight partial transforms)");
        FBF_CUDA(launch_copy_or_add(local_w, grad_weight, (long long)n_weight, accumulate, s));
      }
    }
  } else if (x.mode == FBFFTCONV_SUM_SPECTRUM_WHOLE) {
    StageTimer t(h, pass, FBFFTCONV_STAGE_ALLREDUCE, s);
    ncclResult_t r = api->AllReduce(h->buf_w(), h->buf_w(), spec_floats + bias_floats, ncclFloat, ncclSum, h->comm, s);
    if (r != ncclSuccess) return nccl_fail(api, r, "ncclAllReduce(gradWeight spectrum)");
  }
  if (!scatter && !scatter_bins) {
    StageTimer t(h, pass, FBFFTCONV_STAGE_IFFT, s);
    FBF_CUDA(launch_inverse(inverse_params(h->buf_w(), spatial ? local_w : grad_weight, nullptr, F, P, d.kernel_h,
                                           d.kernel_w, 0, 0, spatial ? 0 : accumulate, pm ? 2 : 0, h->N), h->N, s));
  }
  const bool summed_by_peers = peer && (scatter || scatter_bins || spatial);
  if (spatial) {
    StageTimer t(h, pass, FBFFTCONV_STAGE_ALLREDUCE, s);
    if (peer) {
      if (!grad_bias) FBF_CUDA(cudaMemsetAsync(bias_part, 0, F * sizeof(float), s));
      FBF_CUDA(launch_peer_allreduce(h->peers, h->peer_epoch, vec4, s));
      h->peer_epoch += 2;
      FBF_CUDA(launch_copy_or_add(h->vec_out(), grad_weight, (long long)n_weight, accumulate, s));
    } else {
      ncclResult_t r = api->AllReduce(local_w, local_w, n_weight + bias_floats, ncclFloat, ncclSum, h->comm, s);
      if (r != ncclSuccess) return nccl_fail(api, r, "ncclAllReduce(gradWeight)");
      FBF_CUDA(launch_copy_or_add(local_w, grad_weight, (long long)n_weight, accumulate, s));
    }
  }
  if (h->comm && grad_bias) {
    StageTimer t(h, pass, FBFFTCONV_STAGE_BIAS, s);
    // summed over peers the bias gradient arrives behind gradWeight in the delivered vector
    FBF_CUDA(launch_copy_or_add(summed_by_peers ? h->vec_out() + n_weight : bias_part, grad_bias, F, accumulate, s));
  }
  return FBFFTCONV_OK;
}

// ---- host-buffer variants ----------------------------------------------------

namespace {

struct StageLayout {
  size_t input, weight, bias, output, grad_bias, total;
};

StageLayout stage_layout(const fbfftconv_handle* h) {
  const fbfftconv_desc& d = h->d;
  StageLayout l;
  const size_t in = align256((size_t)d.batch * d.n_input_plane * d.input_h * d.input_w * 4);
  const size_t w = align256((size_t)d.n_output_plane * d.n_input_plane * d.kernel_h * d.kernel_w * 4);
  const size_t b = align256((size_t)d.n_output_plane * 4);
  const size_t o = align256((size_t)d.batch * d.n_output_plane * h->oH * h->oW * 4);
  l.input = 0;
  l.weight = in;
  l.bias = in + w;
  l.output = in + w + b;
  l.grad_bias = in + w + b + o;
  l.total = in + w + b + o + b;
  return l;
}

int ensure_stage(fbfftconv_handle* h) {
  if (h->stage) return FBFFTCONV_OK;
  const StageLayout l = stage_layout(h);
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, l.total);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(FBFFTCONV_ERR_NOMEM, "staging of %zu bytes: %s", l.total, cudaGetErrorString(e));
  }
  h->stage = static_cast<char*>(p);
  h->stage_bytes = l.total;
  return FBFFTCONV_OK;
}

}  // namespace

int fbfftconv_update_output_host(fbfftconv_handle* h, const float* input, const float* weight,
                                 const float* bias, float* output, fbfftconv_stream stream) {
  if (!h || !input || !weight || !output) return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null argument");
  DeviceGuard g;
  FBF_CUDA(g.enter(h->device));
  FBF_TRY(ensure_stage(h));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const fbfftconv_desc& d = h->d;
  const StageLayout l = stage_layout(h);
  float* din = reinterpret_cast<float*>(h->stage + l.input);
  float* dw = reinterpret_cast<float*>(h->stage + l.weight);
  float* db = reinterpret_cast<float*>(h->stage + l.bias);
  float* dout = reinterpret_cast<float*>(h->stage + l.output);
  const size_t n_in = (size_t)d.batch * d.n_input_plane * d.input_h * d.input_w;
  const size_t n_w = (size_t)d.n_output_plane * d.n_input_plane * d.kernel_h * d.kernel_w;
  const size_t n_out = (size_t)d.batch * d.n_output_plane * h->oH * h->oW;
  FBF_CUDA(cudaMemcpyAsync(din, input, n_in * 4, cudaMemcpyHostToDevice, s));
  FBF_CUDA(cudaMemcpyAsync(dw, weight, n_w * 4, cudaMemcpyHostToDevice, s));
  if (bias) FBF_CUDA(cudaMemcpyAsync(db, bias, (size_t)d.n_output_plane * 4, cudaMemcpyHostToDevice, s));
  FBF_TRY(fbfftconv_update_output(h, din, dw, bias ? db : nullptr, dout, stream));
  FBF_CUDA(cudaMemcpyAsync(output, dout, n_out * 4, cudaMemcpyDeviceToHost, s));
  FBF_CUDA(cudaStreamSynchronize(s));
  return check_tensor_core_status();
}

int fbfftconv_update_grad_input_host(fbfftconv_handle* h, const float* grad_output,
                                     const float* weight, float* grad_input, fbfftconv_stream stream) {
  if (!h || !grad_output || !weight || !grad_input)
    return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null argument");
  DeviceGuard g;
  FBF_CUDA(g.enter(h->device));
  FBF_TRY(ensure_stage(h));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const fbfftconv_desc& d = h->d;
  const StageLayout l = stage_layout(h);
  float* din = reinterpret_cast<float*>(h->stage + l.input);
  float* dw = reinterpret_cast<float*>(h->stage + l.weight);
  float* dout = reinterpret_cast<float*>(h->stage + l.output);
  const size_t n_in = (size_t)d.batch * d.n_input_plane * d.input_h * d.input_w;
  const size_t n_w = (size_t)d.n_output_plane * d.n_input_plane * d.kernel_h * d.kernel_w;
  const size_t n_out = (size_t)d.batch * d.n_output_plane * h->oH * h->oW;
  FBF_CUDA(cudaMemcpyAsync(dout, grad_output, n_out * 4, cudaMemcpyHostToDevice, s));
  FBF_CUDA(cudaMemcpyAsync(dw, weight, n_w * 4, cudaMemcpyHostToDevice, s));
  FBF_TRY(fbfftconv_update_grad_input(h, dout, dw, din, stream));
  FBF_CUDA(cudaMemcpyAsync(grad_input, din, n_in * 4, cudaMemcpyDeviceToHost, s));
  FBF_CUDA(cudaStreamSynchronize(s));
  return check_tensor_core_status();
}

int fbfftconv_acc_grad_parameters_host(fbfftconv_handle* h, const float* input,
                                       const float* grad_output, float* grad_weight,
                                       float* grad_bias, float scale, fbfftconv_stream stream) {
  if (!h || !input || !grad_output || !grad_weight)
    return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null argument");
  DeviceGuard g;
  FBF_CUDA(g.enter(h->device));
  FBF_TRY(ensure_stage(h));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const fbfftconv_desc& d = h->d;
  const StageLayout l = stage_layout(h);
  float* din = reinterpret_cast<float*>(h->stage + l.input);
  float* dw = reinterpret_cast<float*>(h->stage + l.weight);
  float* dgb = reinterpret_cast<float*>(h->stage + l.grad_bias);
  float* dout = reinterpret_cast<float*>(h->stage + l.output);
  const size_t n_in = (size_t)d.batch * d.n_input_plane * d.input_h * d.input_w;
  const size_t n_w = (size_t)d.n_output_plane * d.n_input_plane * d.kernel_h * d.kernel_w;
  const size_t n_out = (size_t)d.batch * d.n_output_plane * h->oH * h->oW;
  const bool accumulate = d.flags & FBFFTCONV_ACCUMULATE_GRADS;
  FBF_CUDA(cudaMemcpyAsync(din, input, n_in * 4, cudaMemcpyHostToDevice, s));
  FBF_CUDA(cudaMemcpyAsync(dout, grad_output, n_out * 4, cudaMemcpyHostToDevice, s));
  if (accumulate) {
    FBF_CUDA(cudaMemcpyAsync(dw, grad_weight, n_w * 4, cudaMemcpyHostToDevice, s));
    if (grad_bias) FBF_CUDA(cudaMemcpyAsync(dgb, grad_bias, (size_t)d.n_output_plane * 4, cudaMemcpyHostToDevice, s));
  }
  FBF_TRY(fbfftconv_acc_grad_parameters(h, din, dout, dw, grad_bias ? dgb : nullptr, scale, stream));
  FBF_CUDA(cudaMemcpyAsync(grad_weight, dw, n_w * 4, cudaMemcpyDeviceToHost, s));
  if (grad_bias) FBF_CUDA(cudaMemcpyAsync(grad_bias, dgb, (size_t)d.n_output_plane * 4, cudaMemcpyDeviceToHost, s));
  FBF_CUDA(cudaStreamSynchronize(s));
  return check_tensor_core_status();
}

// ---- asynchronous host-buffer variants ----------------------------------------

namespace {

int ensure_async(fbfftconv_handle* h, int pass) {
  if (!h->up) {
    FBF_CUDA(cudaStreamCreateWithFlags(&h->up, cudaStreamNonBlocking));
    FBF_CUDA(cudaStreamCreateWithFlags(&h->down, cudaStreamNonBlocking));
    FBF_CUDA(cudaEventCreateWithFlags(&h->ev_up, cudaEventDisableTiming));
    for (int i = 0; i < 3; ++i) {
      FBF_CUDA(cudaEventCreateWithFlags(&h->ev_kernels[i], cudaEventDisableTiming));
      FBF_CUDA(cudaEventCreateWithFlags(&h->ev_down[i], cudaEventDisableTiming));
    }
  }
  if (!h->astage[pass]) {
    void* p = nullptr;
    const size_t bytes = stage_layout(h).total;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(FBFFTCONV_ERR_NOMEM, "staging of %zu bytes: %s", bytes, cudaGetErrorString(e));
    }
    h->astage[pass] = static_cast<char*>(p);
  }
  return FBFFTCONV_OK;
}

// Order of one asynchronous pass: uploads (after the kernels of this pass's previous use have
// read the staging) -> kernels on the caller's stream (after the previous download has read the
// output staging) -> downloads.
struct AsyncPass {
  fbfftconv_handle* h;
  int pass;
  cudaStream_t s;
  int begin_uploads() {
    if (h->async_used[pass]) FBF_CUDA(cudaStreamWaitEvent(h->up, h->ev_kernels[pass], 0));
    return FBFFTCONV_OK;
  }
  int begin_kernels() {
    FBF_CUDA(cudaEventRecord(h->ev_up, h->up));
    FBF_CUDA(cudaStreamWaitEvent(s, h->ev_up, 0));
    if (h->async_used[pass]) FBF_CUDA(cudaStreamWaitEvent(s, h->ev_down[pass], 0));
    return FBFFTCONV_OK;
  }
  int begin_downloads() {
    FBF_CUDA(cudaEventRecord(h->ev_kernels[pass], s));
    FBF_CUDA(cudaStreamWaitEvent(h->down, h->ev_kernels[pass], 0));
    return FBFFTCONV_OK;
  }
  int finish() {
    FBF_CUDA(cudaEventRecord(h->ev_down[pass], h->down));
    h->async_used[pass] = true;
    return FBFFTCONV_OK;
  }
};

}  // namespace

int fbfftconv_update_output_host_async(fbfftconv_handle* h, const float* input, const float* weight,
                                       const float* bias, float* output, fbfftconv_stream stream) {
  if (!h || !input || !weight || !output) return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null argument");
  DeviceGuard g;
  FBF_CUDA(g.enter(h->device));
  FBF_TRY(ensure_async(h, 0));
  const fbfftconv_desc& d = h->d;
  const StageLayout l = stage_layout(h);
  char* st = h->astage[0];
  float* din = reinterpret_cast<float*>(st + l.input);
  float* dw = reinterpret_cast<float*>(st + l.weight);
  float* db = reinterpret_cast<float*>(st + l.bias);
  float* dout = reinterpret_cast<float*>(st + l.output);
  const size_t n_in = (size_t)d.batch * d.n_input_plane * d.input_h * d.input_w;
  const size_t n_w = (size_t)d.n_output_plane * d.n_input_plane * d.kernel_h * d.kernel_w;
  const size_t n_out = (size_t)d.batch * d.n_output_plane * h->oH * h->oW;
  AsyncPass a{h, 0, static_cast<cudaStream_t>(stream)};
  FBF_TRY(a.begin_uploads());
  FBF_CUDA(cudaMemcpyAsync(din, input, n_in * 4, cudaMemcpyHostToDevice, h->up));
  FBF_CUDA(cudaMemcpyAsync(dw, weight, n_w * 4, cudaMemcpyHostToDevice, h->up));
  if (bias) FBF_CUDA(cudaMemcpyAsync(db, bias, (size_t)d.n_output_plane * 4, cudaMemcpyHostToDevice, h->up));
  FBF_TRY(a.begin_kernels());
  FBF_TRY(fbfftconv_update_output(h, din, dw, bias ? db : nullptr, dout, stream));
  FBF_TRY(a.begin_downloads());
  FBF_CUDA(cudaMemcpyAsync(output, dout, n_out * 4, cudaMemcpyDeviceToHost, h->down));
  return a.finish();
}

int fbfftconv_update_grad_input_host_async(fbfftconv_handle* h, const float* grad_output,
                                           const float* weight, float* grad_input,
                                           fbfftconv_stream stream) {
  if (!h || !grad_output || !weight || !grad_input)
    return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null argument");
  DeviceGuard g;
  FBF_CUDA(g.enter(h->device));
  FBF_TRY(ensure_async(h, 1));
  const fbfftconv_desc& d = h->d;
  const StageLayout l = stage_layout(h);
  char* st = h->astage[1];
  float* din = reinterpret_cast<float*>(st + l.input);
  float* dw = reinterpret_cast<float*>(st + l.weight);
  float* dout = reinterpret_cast<float*>(st + l.output);
  const size_t n_in = (size_t)d.batch * d.n_input_plane * d.input_h * d.input_w;
  const size_t n_w = (size_t)d.n_output_plane * d.n_input_plane * d.kernel_h * d.kernel_w;
  const size_t n_out = (size_t)d.batch * d.n_output_plane * h->oH * h->oW;
  AsyncPass a{h, 1, static_cast<cudaStream_t>(stream)};
  FBF_TRY(a.begin_uploads());
  FBF_CUDA(cudaMemcpyAsync(dout, grad_output, n_out * 4, cudaMemcpyHostToDevice, h->up));
  FBF_CUDA(cudaMemcpyAsync(dw, weight, n_w * 4, cudaMemcpyHostToDevice, h->up));
  FBF_TRY(a.begin_kernels());
  FBF_TRY(fbfftconv_update_grad_input(h, dout, dw, din, stream));
  FBF_TRY(a.begin_downloads());
  FBF_CUDA(cudaMemcpyAsync(grad_input, din, n_in * 4, cudaMemcpyDeviceToHost, h->down));
  return a.finish();
}

int fbfftconv_acc_grad_parameters_host_async(fbfftconv_handle* h, const float* input,
                                             const float* grad_output, float* grad_weight,
                                             float* grad_bias, float scale, fbfftconv_stream stream) {
  if (!h || !input || !grad_output || !grad_weight)
    return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null argument");
  DeviceGuard g;
  FBF_CUDA(g.enter(h->device));
  FBF_TRY(ensure_async(h, 2));
  const fbfftconv_desc& d = h->d;
  const StageLayout l = stage_layout(h);
  char* st = h->astage[2];
  float* din = reinterpret_cast<float*>(st + l.input);
  float* dw = reinterpret_cast<float*>(st + l.weight);
  float* dgb = reinterpret_cast<float*>(st + l.grad_bias);
  float* dout = reinterpret_cast<float*>(st + l.output);
  const size_t n_in = (size_t)d.batch * d.n_input_plane * d.input_h * d.input_w;
  const size_t n_w = (size_t)d.n_output_plane * d.n_input_plane * d.kernel_h * d.kernel_w;
  const size_t n_out = (size_t)d.batch * d.n_output_plane * h->oH * h->oW;
  const bool accumulate = d.flags & FBFFTCONV_ACCUMULATE_GRADS;
  AsyncPass a{h, 2, static_cast<cudaStream_t>(stream)};
  FBF_TRY(a.begin_uploads());
  // the gradient staging is both output of the kernels and input of the download: with
  // accumulation it is also uploaded, which must wait for the previous download of it
  if (accumulate && h->async_used[2]) FBF_CUDA(cudaStreamWaitEvent(h->up, h->ev_down[2], 0));
  FBF_CUDA(cudaMemcpyAsync(din, input, n_in * 4, cudaMemcpyHostToDevice, h->up));
  FBF_CUDA(cudaMemcpyAsync(dout, grad_output, n_out * 4, cudaMemcpyHostToDevice, h->up));
  if (accumulate) {
    FBF_CUDA(cudaMemcpyAsync(dw, grad_weight, n_w * 4, cudaMemcpyHostToDevice, h->up));
    if (grad_bias) FBF_CUDA(cudaMemcpyAsync(dgb, grad_bias, (size_t)d.n_output_plane * 4, cudaMemcpyHostToDevice, h->up));
  }
  FBF_TRY(a.begin_kernels());
  FBF_TRY(fbfftconv_acc_grad_parameters(h, din, dout, dw, grad_bias ? dgb : nullptr, scale, stream));
  FBF_TRY(a.begin_downloads());
  FBF_CUDA(cudaMemcpyAsync(grad_weight, dw, n_w * 4, cudaMemcpyDeviceToHost, h->down));
  if (grad_bias) FBF_CUDA(cudaMemcpyAsync(grad_bias, dgb, (size_t)d.n_output_plane * 4, cudaMemcpyDeviceToHost, h->down));
  return a.finish();
}

int fbfftconv_backward_host_async(fbfftconv_handle* h, const float* input, const float* grad_output,
                                  const float* weight, float* grad_input, float* grad_weight,
                                  float* grad_bias, float scale, fbfftconv_stream stream) {
  if (!h || !input || !grad_output || !weight || !grad_input || !grad_weight)
    return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null argument");
  DeviceGuard g;
  FBF_CUDA(g.enter(h->device));
  FBF_TRY(ensure_async(h, 1));
  FBF_TRY(ensure_async(h, 2));
  const fbfftconv_desc& d = h->d;
  const StageLayout l = stage_layout(h);
  // staging of pass 1: gradOutput, weight, gradInput; of pass 2: input, gradWeight, gradBias
  float* dgo = reinterpret_cast<float*>(h->astage[1] + l.output);
  float* dw = reinterpret_cast<float*>(h->astage[1] + l.weight);
  float* dgi = reinterpret_cast<float*>(h->astage[1] + l.input);
  float* din = reinterpret_cast<float*>(h->astage[2] + l.input);
  float* dgw = reinterpret_cast<float*>(h->astage[2] + l.weight);
  float* dgb = reinterpret_cast<float*>(h->astage[2] + l.grad_bias);
  const size_t n_in = (size_t)d.batch * d.n_input_plane * d.input_h * d.input_w;
  const size_t n_w = (size_t)d.n_output_plane * d.n_input_plane * d.kernel_h * d.kernel_w;
  const size_t n_out = (size_t)d.batch * d.n_output_plane * h->oH * h->oW;
  const bool accumulate = d.flags & FBFFTCONV_ACCUMULATE_GRADS;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  AsyncPass a1{h, 1, s}, a2{h, 2, s};
  FBF_TRY(a1.begin_uploads());
  FBF_TRY(a2.begin_uploads());
  if (accumulate && h->async_used[2]) FBF_CUDA(cudaStreamWaitEvent(h->up, h->ev_down[2], 0));
  FBF_CUDA(cudaMemcpyAsync(dw, weight, n_w * 4, cudaMemcpyHostToDevice, h->up));
  FBF_CUDA(cudaMemcpyAsync(din, input, n_in * 4, cudaMemcpyHostToDevice, h->up));
  FBF_CUDA(cudaMemcpyAsync(dgo, grad_output, n_out * 4, cudaMemcpyHostToDevice, h->up));
  if (accumulate) {
    FBF_CUDA(cudaMemcpyAsync(dgw, grad_weight, n_w * 4, cudaMemcpyHostToDevice, h->up));
    if (grad_bias) FBF_CUDA(cudaMemcpyAsync(dgb, grad_bias, (size_t)d.n_output_plane * 4, cudaMemcpyHostToDevice, h->up));
  }
  FBF_TRY(a1.begin_kernels());
  if (h->async_used[2]) FBF_CUDA(cudaStreamWaitEvent(s, h->ev_down[2], 0));
  FBF_TRY(fbfftconv_update_grad_input(h, dgo, dw, dgi, stream));
  FBF_TRY(a1.begin_downloads());  // gradInput can leave while the weight gradient is computed
  FBF_CUDA(cudaMemcpyAsync(grad_input, dgi, n_in * 4, cudaMemcpyDeviceToHost, h->down));
  // both passes of a backward call see the same gradOutput: its spectrum is transformed once
  h->same_grad_output = true;
  const int rc_acc = fbfftconv_acc_grad_parameters(h, din, dgo, dgw, grad_bias ? dgb : nullptr, scale, stream);
  h->same_grad_output = false;
  FBF_TRY(rc_acc);
  // gradOutput's staging belongs to pass 1 but is read until here: its 'kernels done' moves
  FBF_CUDA(cudaEventRecord(h->ev_kernels[1], s));
  FBF_TRY(a2.begin_downloads());
  FBF_CUDA(cudaMemcpyAsync(grad_weight, dgw, n_w * 4, cudaMemcpyDeviceToHost, h->down));
  if (grad_bias) FBF_CUDA(cudaMemcpyAsync(grad_bias, dgb, (size_t)d.n_output_plane * 4, cudaMemcpyDeviceToHost, h->down));
  FBF_TRY(a1.finish());
  return a2.finish();
}

int fbfftconv_host_sync(fbfftconv_handle* h) {
  if (!h) return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null handle");
  if (!h->down) return FBFFTCONV_OK;
  DeviceGuard g;
  FBF_CUDA(g.enter(h->device));
  FBF_CUDA(cudaStreamSynchronize(h->down));
  return check_tensor_core_status();
}

// ---- sub-steps ---------------------------------------------------------------

int fbfftconv_fft2d(const float* real, void* spectrum, int d1, int d2, int h, int w, int fft_size,
                    int pad_u, int pad_l, int transposed, fbfftconv_stream stream) {
  if (!real || !spectrum) return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null argument");
  if (!valid_fft_size(fft_size)) return fail(FBFFTCONV_ERR_UNSUPPORTED_SIZE, "transform size %d not in {2,4,8,16,32,64,128}", fft_size);
  if (d1 <= 0 || d2 <= 0 || h <= 0 || w <= 0 || pad_u < 0 || pad_l < 0 || h + pad_u > fft_size ||
      w + pad_l > fft_size || d1 > 65535 || d2 > 65535)
    return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "plane of %dx%d at (%d,%d) does not fit %d", h, w, pad_u, pad_l, fft_size);
  FBF_CUDA(launch_forward(forward_params(real, static_cast<float2*>(spectrum), d1, d2, h, w, pad_u, pad_l, transposed, fft_size),
                          fft_size, static_cast<cudaStream_t>(stream)));
  return FBFFTCONV_OK;
}

int fbfftconv_ifft2d(const void* spectrum, float* real, const float* bias, int d1, int d2, int h,
                     int w, int fft_size, int off_y, int off_x, int accumulate, int plane_major,
                     fbfftconv_stream stream) {
  if (!real || !spectrum) return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null argument");
  if (!valid_fft_size(fft_size)) return fail(FBFFTCONV_ERR_UNSUPPORTED_SIZE, "transform size %d not in {2,4,8,16,32,64,128}", fft_size);
  if (d1 <= 0 || d2 <= 0 || h <= 0 || w <= 0 || off_y < 0 || off_x < 0 || h + off_y > fft_size ||
      w + off_x > fft_size || d1 > 65535 || d2 > 65535)
    return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "window of %dx%d at (%d,%d) does not fit %d", h, w, off_y, off_x, fft_size);
  FBF_CUDA(launch_inverse(inverse_params(static_cast<const float2*>(spectrum), real, bias, d1, d2, h, w, off_y, off_x, accumulate != 0, plane_major != 0 ? 2 : 0, fft_size),
                          fft_size, static_cast<cudaStream_t>(stream)));
  return FBFFTCONV_OK;
}

int fbfftconv_fft2d_reference_layout(const float* real, void* frequency, void* scratch, int planes, int h, int w,
                                     int fft_size, int pad_u, int pad_l, fbfftconv_stream stream) {
  if (!scratch || !frequency) return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null argument");
  FBF_TRY(fbfftconv_fft2d(real, scratch, 1, planes, h, w, fft_size, pad_u, pad_l, 0, stream));
  FBF_CUDA(launch_spectrum_layout(true, static_cast<const float2*>(scratch), static_cast<float2*>(frequency), planes,
                                  pad4(planes), fft_size, static_cast<cudaStream_t>(stream)));
  return FBFFTCONV_OK;
}

int fbfftconv_ifft2d_reference_layout(const void* frequency, float* real, void* scratch, int planes, int h, int w,
                                      int fft_size, int off_y, int off_x, fbfftconv_stream stream) {
  if (!scratch || !frequency || !real) return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null argument");
  if (!valid_fft_size(fft_size)) return fail(FBFFTCONV_ERR_UNSUPPORTED_SIZE, "transform size %d not in {2,4,8,16,32,64,128}", fft_size);
  if (planes <= 0 || planes > 65535) return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "between 1 and 65535 planes");
  FBF_CUDA(launch_spectrum_layout(false, static_cast<const float2*>(frequency), static_cast<float2*>(scratch), planes,
                                  pad4(planes), fft_size, static_cast<cudaStream_t>(stream)));
  return fbfftconv_ifft2d(scratch, real, nullptr, 1, planes, h, w, fft_size, off_y, off_x, 0, 0, stream);
}

int fbfftconv_fft1d(const float* real, void* spectrum, long long rows, int n, int fft_size,
                    int pad_left, fbfftconv_stream stream) {
  if (!real || !spectrum) return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null argument");
  if (!valid_fft1d_size(fft_size)) return fail(FBFFTCONV_ERR_UNSUPPORTED_SIZE, "transform size %d not in {2,4,8,16,32,64,128,256}", fft_size);
  if (rows <= 0 || n <= 0 || pad_left < 0 || n + pad_left > fft_size)
    return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "row of %d floats at %d does not fit %d", n, pad_left, fft_size);
  FBF_CUDA(launch_fft1d(false, real, nullptr, static_cast<float2*>(spectrum), rows, n, fft_size, pad_left,
                        static_cast<cudaStream_t>(stream)));
  return FBFFTCONV_OK;
}

int fbfftconv_ifft1d(const void* spectrum, float* real, long long rows, int n, int fft_size,
                     int offset, fbfftconv_stream stream) {
  if (!real || !spectrum) return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null argument");
  if (!valid_fft1d_size(fft_size)) return fail(FBFFTCONV_ERR_UNSUPPORTED_SIZE, "transform size %d not in {2,4,8,16,32,64,128,256}", fft_size);
  if (rows <= 0 || n <= 0 || offset < 0 || n + offset > fft_size)
    return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "window of %d floats at %d does not fit %d", n, offset, fft_size);
  FBF_CUDA(launch_fft1d(true, nullptr, real, static_cast<float2*>(const_cast<void*>(spectrum)), rows, n, fft_size,
                        offset, static_cast<cudaStream_t>(stream)));
  return FBFFTCONV_OK;
}

int fbfftconv_transpose_mm(const void* a, const void* b, void* c, int bins, int m, int n, int k,
                           float alpha, int conj_a, int conj_b, int use_simt,
                           fbfftconv_stream stream) {
  if (!a || !b || !c) return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null argument");
  if (bins <= 0 || m <= 0 || n <= 0 || k <= 0 || bins > 65535)
    return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "bad contraction sizes");
  if ((conj_a & ~3) || (conj_b & ~3)) return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "operand flags are 0..3");
  return contract(static_cast<const float2*>(a), static_cast<const float2*>(b), static_cast<float2*>(c),
                  bins, m, n, k, alpha, conj_a & 1, conj_b & 1, use_simt != 0,
                  static_cast<cudaStream_t>(stream), (conj_a & 2) != 0, (conj_b & 2) != 0);
}

int fbfftconv_update_output_bias(float* output, const float* bias, int batch, int planes, int h,
                                 int w, fbfftconv_stream stream) {
  if (!output || !bias || batch <= 0 || planes <= 0 || h <= 0 || w <= 0)
    return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "bad bias arguments");
  FBF_CUDA(launch_bias_add(output, bias, batch, planes, h * w, static_cast<cudaStream_t>(stream)));
  return FBFFTCONV_OK;
}

int fbfftconv_acc_grad_parameters_bias(const float* grad_output, float* grad_bias, float* scratch,
                                       int batch, int planes, int h, int w, float scale,
                                       int accumulate, fbfftconv_stream stream) {
  if (!grad_output || !grad_bias || !scratch || batch <= 0 || planes <= 0 || h <= 0 || w <= 0 || batch > 65535)
    return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "bad bias-gradient arguments");
  FBF_CUDA(launch_bias_grad(grad_output, grad_bias, scratch, batch, planes, h * w, scale, accumulate != 0,
                            static_cast<cudaStream_t>(stream)));
  return FBFFTCONV_OK;
}

int fbfftconv_tensor_core_status(int reset) { return contract_tc_error(reset != 0); }

int fbfftconv_peer_exchange_status(fbfftconv_handle* h, int reset) {
  if (!h) return -1;
  DeviceGuard g;
  if (g.enter(h->device) != cudaSuccess) return -1;
  const int code = peer_error(reset != 0);
  if (code != 0) return code < 0 ? -1 : 100 + code;  // 100 + (1 + rank that did not arrive)
  return h->peer_ready ? 1 : 0;
}

int fbfftconv_peer_exchange_wait_selftest(fbfftconv_stream stream) {
  const int r = peer_wait_probe(static_cast<cudaStream_t>(stream));
  if (r < 0) return fail(FBFFTCONV_ERR_CUDA, "wait self-test could not run: %s", cudaGetErrorString(cudaGetLastError()));
  if (r != 1) return fail(FBFFTCONV_ERR_CUDA, "wait self-test: the bounded wait did not give up");
  peer_error(true);  // the code it leaves (1) belongs to the test, not to an exchange
  return FBFFTCONV_OK;
}

int fbfftconv_tensor_core_wait_selftest(fbfftconv_stream stream) {
  const int r = contract_tc_wait_probe(static_cast<cudaStream_t>(stream));
  if (r < 0) return fail(FBFFTCONV_ERR_CUDA, "wait self-test could not run: %s", cudaGetErrorString(cudaGetLastError()));
  if (r != 1) return fail(FBFFTCONV_ERR_CUDA, "wait self-test: the bounded wait did not give up");
  return FBFFTCONV_OK;
}

// ---- per-kernel timing ---------------------------------------------------------

int fbfftconv_profile_enable(fbfftconv_handle* h, int enable) {
  if (!h) return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null handle");
  h->profiling = enable != 0;
  return FBFFTCONV_OK;
}

int fbfftconv_profile_reset(fbfftconv_handle* h) {
  if (!h) return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null handle");
  memset(h->events_used, 0, sizeof(h->events_used));
  memset(h->overlapped, 0, sizeof(h->overlapped));
  return FBFFTCONV_OK;
}

int fbfftconv_profile_overlapped(const fbfftconv_handle* h, int pass, int stage) {
  if (!h || pass < 0 || pass > 2 || stage < 0 || stage >= FBFFTCONV_STAGE_COUNT) return -1;
  return h->overlapped[pass][stage] ? 1 : 0;
}

int fbfftconv_profile_read(fbfftconv_handle* h, int pass, int stage, double* total_ms, int* launches) {
  if (!h || pass < 0 || pass > 2 || stage < 0 || stage >= FBFFTCONV_STAGE_COUNT || !total_ms || !launches)
    return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "bad profile query");
  DeviceGuard g;
  FBF_CUDA(g.enter(h->device));
  double sum = 0.0;
  const int n = h->events_used[pass][stage];
  for (int i = 0; i < n; ++i) {
    const EventPair& p = h->events[pass][stage][i];
    FBF_CUDA(cudaEventSynchronize(p.stop));
    float ms = 0.f;
    FBF_CUDA(cudaEventElapsedTime(&ms, p.start, p.stop));
    sum += ms;
  }
  *total_ms = sum;
  *launches = n;
  return FBFFTCONV_OK;
}

// ---- communicator ------------------------------------------------------------

int fbfftconv_comm_unique_id(void* id128) {
  if (!id128) return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null id");
  NcclApi* api = nccl_api();
  if (!api) return fail(FBFFTCONV_ERR_COMM, "libnccl is not loadable: %s", dlerror());
  static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
  ncclUniqueId id;
  ncclResult_t r = api->GetUniqueId(&id);
  if (r != ncclSuccess) return nccl_fail(api, r, "ncclGetUniqueId");
  memcpy(id128, &id, sizeof(id));
  return FBFFTCONV_OK;
}

int fbfftconv_comm_init(fbfftconv_handle* h, const void* id128, int rank, int nranks) {
  if (!h || !id128 || nranks <= 0 || rank < 0 || rank >= nranks)
    return fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "bad communicator arguments");
  NcclApi* api = nccl_api();
  if (!api) return fail(FBFFTCONV_ERR_COMM, "libnccl is not loadable: %s", dlerror());
  DeviceGuard g;
  FBF_CUDA(g.enter(h->device));
  release_comm(h);
  const std::string key(static_cast<const char*>(id128), sizeof(ncclUniqueId));
  std::lock_guard<std::mutex> lock(g_comm_mutex);
  SharedComm& shared = g_comms[key];
  if (!shared.comm) {
    ncclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    ncclResult_t r = api->CommInitRank(&shared.comm, nranks, id, rank);
    if (r != ncclSuccess) {
      g_comms.erase(key);
      return nccl_fail(api, r, "ncclCommInitRank");
    }
    shared.rank = rank;
    shared.nranks = nranks;
    shared.device = h->device;
  } else if (shared.rank != rank || shared.nranks != nranks || shared.device != h->device) {
    return fail(FBFFTCONV_ERR_INVALID_ARGUMENT,
                "this id already names a communicator of rank %d/%d on device %d; asked for rank %d/%d on device %d",
                shared.rank, shared.nranks, shared.device, rank, nranks, h->device);
  }
  ++shared.refs;
  h->comm = shared.comm;
  h->comm_key = key;
  h->rank = rank;
  h->nranks = nranks;
  return FBFFTCONV_OK;
}

int fbfftconv_comm_shutdown(void) {
  std::lock_guard<std::mutex> lock(g_comm_mutex);
  NcclApi* api = nccl_api();
  for (auto it = g_comms.begin(); it != g_comms.end();) {
    if (it->second.refs > 0) {
      ++it;
      continue;
    }
    if (api) api->CommDestroy(it->second.comm);
    it = g_comms.erase(it);
  }
  return g_comms.empty() ? FBFFTCONV_OK
                         : fail(FBFFTCONV_ERR_COMM, "%zu communicator(s) still attached to handles", g_comms.size());
}

int fbfftconv_comm_destroy(fbfftconv_handle* h) {
  if (!h || !h->comm) return FBFFTCONV_OK;
  DeviceGuard g;
  g.enter(h->device);
  release_comm(h);
  return FBFFTCONV_OK;
}

}  // extern "C"
