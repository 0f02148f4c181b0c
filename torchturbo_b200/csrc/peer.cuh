// Peer-memory primitives shared by the communication kernels and by the GEMM kernels that fuse a token exchange:
// the table of every rank's symmetric-buffer base address, system-scope release / acquire accesses for the epoch
// flags, and the bounded flag wait.  Protocol:
//   writer : data stores -> __threadfence_system() -> st.release.sys flag = epoch
//   reader : ld.acquire.sys flag until it is >= epoch (bounded by a time budget) -> data loads
// Epochs of one flag only grow, so a flag is never reset and a stale value can never satisfy a later wait.
#pragma once
#include "common.cuh"

namespace ttb {

constexpr unsigned KID_COMM = 3;
constexpr int MAX_RANKS = 16;

struct PeerTable {
  unsigned long long base[MAX_RANKS];  // device-visible base address of every rank's symmetric buffer
};

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Orders generic-proxy accesses (the acquire above, peers' plain stores) before later async-proxy reads (TMA loads)
// of the same global memory by this thread.
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Wait until *flag >= epoch.  Returns false after `budget_ns`; the failure is recorded in the unit's status word and,
// when `status` is given, in the workspace status word that later kernels of the same workspace check before they
// touch remote memory (so the total stall of a broken exchange stays within one budget).
__device__ __forceinline__ bool wait_flag(const int* flag, int epoch, unsigned long long budget_ns, unsigned site,
                                          unsigned peer, int* status) {
  if (ld_acquire_sys(flag) >= epoch) return true;
  if (status && *reinterpret_cast<volatile int*>(status) != 0) return false;
  const uint64_t t0 = globaltimer_ns();
  while (ld_acquire_sys(flag) < epoch) {
    if (globaltimer_ns() - t0 > budget_ns) {
      set_status(KID_COMM, site, peer);
      if (status) atomicExch(status, static_cast<int>((site << 8) | peer | 0x10000));
      return false;
    }
    __nanosleep(64);
  }
  return true;
}

// Rows of an expert-parallel exchange carry a tag that names where their result goes back to:
// (source rank << EP_TAG_SHIFT) | entry index on the source (token * k + slot); negative = padding row.
constexpr int EP_TAG_SHIFT = 26;
constexpr int EP_TAG_MASK = (1 << EP_TAG_SHIFT) - 1;

}  // namespace ttb
