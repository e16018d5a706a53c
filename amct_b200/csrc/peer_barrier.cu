// Barrier between the ranks of one node over peer-mapped flag words, for collectives made of copy-engine
// transfers: it orders "everything this rank's stream did before" against "everything the peers' streams do
// after" without a communication library kernel, in one tiny block that fits beside resident GEMM blocks.
//
// Every rank owns a flag array of `world` 32-bit words in memory that all ranks have mapped.  Barrier number
// `seq` (1, 2, 3 ... counted by the callers, the same on every rank): lane t stores `seq` into word [rank] of
// rank t's array (release, system scope), then waits until word [t] of its own array has reached `seq`
// (acquire, system scope).  Sequence numbers only grow, so nothing has to be reset between barriers and a
// rank that runs ahead by one barrier cannot be mistaken for the current one.  The wait is bounded: after
// kBarrierLimitNs the lane sets bit 1 of the status word and the kernel returns, so a peer that never arrives
// costs a wrong result that the host can see, not a hung device.  Once that bit is set, later barriers with the
// same status word still signal (so that the peers, whose data is wrong already, do not each wait out their own
// limit at every barrier that follows) but no longer wait.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/amct_b200.h"

namespace amct {

constexpr int kMaxPeers = 16;
constexpr uint64_t kBarrierLimitNs = 2000000000ull;

struct PeerFlags {
  uint32_t* ptr[kMaxPeers];
};

__device__ __forceinline__ uint64_t barrier_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__global__ void __launch_bounds__(32) peer_barrier_kernel(PeerFlags flags, int world, int rank, uint32_t seq, int* status) {
  const int t = threadIdx.x;
  if (t >= world || t == rank) return;
  __threadfence_system();                                            // earlier kernels' writes, before the signal
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags.ptr[t] + rank), "r"(seq) : "memory");
  // a barrier that has given up once stays open: the data is already wrong, and every later barrier of a rank
  // that lost its peers would otherwise wait its full limit again
  if (status && (*reinterpret_cast<volatile int*>(status) & 2)) return;
  const uint32_t* mine = flags.ptr[rank] + t;
  const uint64_t t0 = barrier_timer_ns();
  for (;;) {
    uint32_t seen;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
    if ((int32_t)(seen - seq) >= 0) break;
    if (barrier_timer_ns() - t0 > kBarrierLimitNs) {
      if (status) atomicOr(status, 2);
      break;
    }
    __nanosleep(200);
  }
}

}  // namespace amct

extern "C" int amct_peer_barrier(void* const* flag_arrays, int world, int rank, uint32_t seq, int* status, void* stream) {
  if (!flag_arrays || world < 1 || world > amct::kMaxPeers || rank < 0 || rank >= world) return AMCT_ERR_ARG;
  amct::PeerFlags f{};
  for (int r = 0; r < world; ++r) {
    if (!flag_arrays[r]) return AMCT_ERR_ARG;
    f.ptr[r] = static_cast<uint32_t*>(flag_arrays[r]);
  }
  if (world == 1) return 0;
  amct::peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(f, world, rank, seq, status);
  return cudaGetLastError() == cudaSuccess ? AMCT_OK : AMCT_ERR_CUDA;
}
