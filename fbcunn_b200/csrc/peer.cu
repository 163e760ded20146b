// Sums across ranks over peer memory (NVLink loads and stores between the GPUs of one box),
// for the weight-gradient exchange of accGradParameters.
//
// Stands where nn.DataParallel gathers, adds and broadcasts gradients
// (fbcunn/DataParallel.lua:105-131).  Every rank maps the scratch block of every other rank
// (CUDA IPC); a collective is then one kernel per rank that reads its share from all peers,
// sums it in rank order (the result does not depend on timing) and writes it where it is
// needed -- no staging copies, no ring.  Each rank's blocks sit at its own addresses (a rank's
// scratch layout follows its batch share), so the table carries one pointer per rank and block.
// Ranks meet at flag barriers: a rank stores an epoch number into its slot of every peer's flag
// array and then polls its own, local array.
//
// Every wait is bounded.  A rank whose peers do not show up within the limit skips its part,
// records a code (peer_error) and returns; nothing spins forever.  Peer memory is only ever touched
// by plain loads and stores on peer pointers: no NVSwitch reduction object, no TMA.
#include "kernels.h"

namespace fbfft {

namespace {

__device__ int g_peer_error = 0;  // sticky: first non-zero code (1 + rank that did not arrive)

// about ten seconds: a peer may reach its launch much later than this rank (host-side skew)
constexpr unsigned kPeerSleepNs = 1000;
constexpr unsigned kPeerSpinLimit = 10u * 1000u * 1000u;

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// peer data: never through the (incoherent) L1
__device__ __forceinline__ float4 ld_peer(const float4* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Threads 0 .. nranks-1 of the calling block store `epoch` into this rank's slot on every peer.
__device__ __forceinline__ void peer_signal(const PeerTable& t, unsigned epoch) {
  if ((int)threadIdx.x < t.nranks) st_release_sys(t.flags[threadIdx.x] + t.rank, epoch);
}
// Threads 0 .. nranks-1 wait, each for one rank's slot of the local array; true for the whole
// block when every rank has arrived.
__device__ __forceinline__ bool peer_wait(const PeerTable& t, unsigned epoch) {
  bool ok = true;
  if ((int)threadIdx.x < t.nranks) {
    const unsigned* slot = t.flags[t.rank] + threadIdx.x;
    unsigned spins = 0;
    // epochs only grow; the signed difference tolerates the 32-bit wrap
    while ((int)(ld_acquire_sys(slot) - epoch) < 0) {
      // ranks of a running job arrive within microseconds of one another: poll fast at first
      __nanosleep(spins < 256 ? 64 : kPeerSleepNs);
      if (++spins > (t.spin_limit ? t.spin_limit : kPeerSpinLimit)) {
        ok = false;
        atomicCAS(&g_peer_error, 0, 1 + (int)threadIdx.x);
        break;
      }
    }
  }
  return __syncthreads_and(ok) != 0;
}
// After the body: the last block of the grid to get here signals `epoch` and waits for every
// rank, so the kernel -- and with it everything later on this stream -- ends only when all
// ranks have passed.  `counter` is a zero-initialised word of local memory; it is zero again
// afterwards.
__device__ __forceinline__ void peer_end_barrier(const PeerTable& t, unsigned epoch, unsigned* counter, bool ok) {
  __shared__ int is_last;
  __threadfence_system();  // this block's peer stores (and loads) are done before the count moves
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned done = atomicAdd(counter, 1u) + 1u;
    is_last = done == gridDim.x;
    if (is_last) *counter = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence_system();
  peer_signal(t, epoch);
  if (ok) peer_wait(t, epoch);  // after a time-out the peers are told, not waited for again
}

// Sum over ranks, in rank order, of element i of every rank's block.  All NR loads are issued
// before the first add: a load over NVLink takes microseconds, and what keeps the links busy is the
// number of loads in flight, not the number of threads.
template <int NR>
__device__ __forceinline__ float4 peer_sum(char* const (&block)[kMaxPeers], size_t i) {
  float4 v[NR];
#pragma unroll
  for (int r = 0; r < NR; ++r) v[r] = ld_peer(reinterpret_cast<const float4*>(block[r]) + i);
  float4 acc = v[0];
#pragma unroll
  for (int r = 1; r < NR; ++r) {
    acc.x += v[r].x;
    acc.y += v[r].y;
    acc.z += v[r].z;
    acc.w += v[r].w;
  }
  return acc;
}

// In place, on this rank's share [first4, first4 + count4) (units of float4) of the spectrum
// block every rank holds (t.spec): share = sum over ranks.  Barrier before (every rank has
// produced its block) and after (every rank has read what it needs, so the blocks may be
// overwritten).  NR = t.nranks.
template <int NR>
__global__ void __launch_bounds__(256)
peer_reduce_kernel(const __grid_constant__ PeerTable t, unsigned epoch, size_t first4, size_t count4) {
  if (blockIdx.x == 0) peer_signal(t, epoch);
  const bool ok = peer_wait(t, epoch);
  if (ok) {
    float4* mine = reinterpret_cast<float4*>(t.spec[t.rank]) + first4;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    // two elements per round while both exist: 2 * NR loads in flight per thread
    for (; i + stride < count4; i += 2 * stride) {
      const float4 a = peer_sum<NR>(t.spec, first4 + i);
      const float4 b = peer_sum<NR>(t.spec, first4 + i + stride);
      mine[i] = a;
      mine[i + stride] = b;
    }
    if (i < count4) mine[i] = peer_sum<NR>(t.spec, first4 + i);
  }
  peer_end_barrier(t, epoch + 1, t.counter, ok);
}

// out[i] = sum over ranks of in[i] for all i < n4 (float4 units), on every rank: this rank sums
// its share of t.vec_in and stores it into every rank's t.vec_out.  Barrier before (inputs
// complete, output blocks free) and after (all shares have landed here).  NR = t.nranks.
template <int NR>
__global__ void __launch_bounds__(256)
peer_allreduce_kernel(const __grid_constant__ PeerTable t, unsigned epoch, size_t n4) {
  if (blockIdx.x == 0) peer_signal(t, epoch);
  const bool ok = peer_wait(t, epoch);
  if (ok) {
    const size_t per = (n4 + NR - 1) / NR;
    const size_t first = per * t.rank;
    const size_t last = first + per < n4 ? first + per : n4;
    for (size_t i = first + blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < last; i += (size_t)gridDim.x * blockDim.x) {
      const float4 acc = peer_sum<NR>(t.vec_in, i);
#pragma unroll
      for (int r = 0; r < NR; ++r) reinterpret_cast<float4*>(t.vec_out[r])[i] = acc;
    }
  }
  peer_end_barrier(t, epoch + 1, t.counter, ok);
}

// One block waits for an epoch nobody signals, with the table's (small) spin limit.
__global__ void peer_wait_probe_kernel(const __grid_constant__ PeerTable t, unsigned epoch, int* gave_up) {
  const bool ok = peer_wait(t, epoch);
  if (threadIdx.x == 0) *gave_up = ok ? 0 : 1;
}

}  // namespace

// Makes one bounded wait on a peer flag run out on purpose (a one-rank table, an epoch nothing
// signals, a limit of a few polls): 1 = it gave up and left code 1 for peer_error, 0 = it did not,
// < 0 = CUDA error.
int peer_wait_probe(cudaStream_t stream) {
  unsigned* flags = nullptr;
  if (cudaMalloc(&flags, 64 * sizeof(unsigned)) != cudaSuccess) return -1;
  int result = -1;
  if (cudaMemsetAsync(flags, 0, 64 * sizeof(unsigned), stream) == cudaSuccess) {
    PeerTable t{};
    t.rank = 0;
    t.nranks = 1;
    t.flags[0] = flags;
    t.counter = flags + 32;
    t.spin_limit = 4;
    int* gave_up = reinterpret_cast<int*>(flags + 48);
    peer_wait_probe_kernel<<<1, 32, 0, stream>>>(t, 7u, gave_up);
    count_launch();
    if (cudaGetLastError() == cudaSuccess && cudaStreamSynchronize(stream) == cudaSuccess &&
        cudaMemcpy(&result, gave_up, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
      result = -1;
  }
  cudaFree(flags);
  return result;
}

cudaError_t launch_peer_reduce(const PeerTable& t, unsigned epoch, size_t first4, size_t count4, cudaStream_t stream) {
  if (t.nranks < 1 || t.nranks > kMaxPeers) return cudaErrorInvalidValue;
  const size_t want = (count4 + 255) / 256;
  const size_t cap = (size_t)sm_count() * 4;
  const int blocks = (int)(want < 1 ? 1 : want < cap ? want : cap);
  switch (t.nranks) {
#define FBF_PEER_CASE(NR) \
  case NR: peer_reduce_kernel<NR><<<blocks, 256, 0, stream>>>(t, epoch, first4, count4); break;
    FBF_PEER_CASE(1) FBF_PEER_CASE(2) FBF_PEER_CASE(3) FBF_PEER_CASE(4)
    FBF_PEER_CASE(5) FBF_PEER_CASE(6) FBF_PEER_CASE(7) FBF_PEER_CASE(8)
#undef FBF_PEER_CASE
  }
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_peer_allreduce(const PeerTable& t, unsigned epoch, size_t n4, cudaStream_t stream) {
  if (t.nranks < 1 || t.nranks > kMaxPeers) return cudaErrorInvalidValue;
  const size_t per = (n4 + t.nranks - 1) / t.nranks;
  const size_t want = (per + 255) / 256;
  const size_t cap = (size_t)sm_count() * 2;
  const int blocks = (int)(want < 1 ? 1 : want < cap ? want : cap);
  switch (t.nranks) {
#define FBF_PEER_CASE(NR) \
  case NR: peer_allreduce_kernel<NR><<<blocks, 256, 0, stream>>>(t, epoch, n4); break;
    FBF_PEER_CASE(1) FBF_PEER_CASE(2) FBF_PEER_CASE(3) FBF_PEER_CASE(4)
    FBF_PEER_CASE(5) FBF_PEER_CASE(6) FBF_PEER_CASE(7) FBF_PEER_CASE(8)
#undef FBF_PEER_CASE
  }
  count_launch();
  return cudaGetLastError();
}

int peer_error(bool reset) {
  int code = 0;
  if (cudaMemcpyFromSymbol(&code, g_peer_error, sizeof(int)) != cudaSuccess) return -1;
  if (reset && code != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_peer_error, &zero, sizeof(int));
  }
  return code;
}

}  // namespace fbfft
