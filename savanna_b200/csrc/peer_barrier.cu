// Stream-ordered barrier between the GPUs of one NVSwitch domain, through symmetric memory.
// Every rank owns a signal array sig[world] (int32) mapped into all peers.  A barrier with sequence number `epoch`:
//   thread r:  st.release.sys  peer_r.sig[me] = epoch          (tell rank r that `me` has arrived)
//              spin on ld.acquire.sys own.sig[r] >= epoch       (wait until rank r has arrived)
// Epochs increase monotonically, so no reset is needed and a late reader can never miss a signal.  The spin is
// bounded (WAIT_BUDGET_NS): on expiry the kernel records ST_TIMEOUT_PEER with the missing rank in the status word
// and returns, the host raises at its next status check.  One tiny kernel per GPU — about 5 us instead of a
// collective-library launch.
#include "sm100.cuh"

namespace sb {
struct SigPtrs { int* p[16]; };

__global__ void peer_barrier_kernel(SigPtrs sig, int me, int world, int epoch, uint32_t* status,
                                    unsigned long long budget_ns) {
  const int r = threadIdx.x;
  if (r >= world) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(sig.p[r] + me), "r"(epoch) : "memory");
  const int* mine = sig.p[me] + r;
  const unsigned long long t0 = globaltimer();
  uint32_t it = 0;
  while (true) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (v >= epoch) break;
    if ((++it & 127u) == 0u && globaltimer() - t0 > budget_ns) {
      if (status) atomicCAS(status, 0u, (uint32_t(ST_TIMEOUT_PEER) << 24) | 0x800000u | uint32_t(r));
      break;
    }
  }
  __threadfence_system();
}
}  // namespace sb

// sig[r]: rank r's signal array (int32[world], zero-initialised once) as mapped in this process.  `budget_ns` bounds the
// wait for each peer (0 = the library default of 1.5 s); when it runs out the kernel records ST_TIMEOUT_PEER and returns.
extern "C" int sb_peer_barrier_budget(int* const* sig, int me, int world, int epoch, unsigned int* status,
                                      unsigned long long budget_ns, cudaStream_t st) {
  if (world < 1 || world > 16) return -1;
  sb::SigPtrs s;
  for (int r = 0; r < 16; ++r) s.p[r] = r < world ? sig[r] : nullptr;
  sb::peer_barrier_kernel<<<1, 32, 0, st>>>(s, me, world, epoch, status, budget_ns ? budget_ns : sb::WAIT_BUDGET_NS);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int sb_peer_barrier(int* const* sig, int me, int world, int epoch, unsigned int* status, cudaStream_t st) {
  return sb_peer_barrier_budget(sig, me, world, epoch, status, 0ull, st);
}
