// Device-side primitives for kernels that talk to peer GPUs over NVLink / NVSwitch:
// system-scope release/acquire signals with bounded waits, and NVLS multimem loads, stores
// and reductions.  Peer memory is reached through plain pointers (symmetric buffers mapped
// into this process); nothing here issues a TMA multicast load.
//
// Signals are monotonically increasing 32-bit epochs, so they never need to be reset
// between launches: a waiter waits for `value >= epoch`.
#pragma once
#include "../common/ptx.cuh"

namespace st {

constexpr int kMaxRanks = 8;

// Plain system-scope store: for flags written after one fence_sys() (the fence orders everything
// before it; W release stores would each pay their own fence and serialise ~3 us apiece).
__device__ __forceinline__ void st_relaxed_sys(unsigned* p, unsigned v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_relaxed_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(unsigned* p, unsigned v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_relaxed_sys_add(unsigned* p, unsigned v) {
  asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_global() {
  asm volatile("fence.proxy.async.global;" ::: "memory");
}

// Bounded wait for *flag >= epoch (wrap-safe comparison).  Returns false after
// wait_limit_ns(); the caller reports the failure and unwinds.
__device__ __forceinline__ bool wait_flag_ge(const unsigned* flag, unsigned epoch) {
  if (static_cast<int>(ld_acquire_sys(flag) - epoch) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  unsigned it = 0;
  while (static_cast<int>(ld_acquire_sys(flag) - epoch) < 0) {
    if (((++it) & 0xFF) == 0 && globaltimer_ns() - t0 > wait_limit_ns()) return false;
  }
  return true;
}

// ---- NVLS multimem (addresses come from the multicast mapping of a symmetric buffer) ----
__device__ __forceinline__ void multimem_st_v4(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}
__device__ __forceinline__ void multimem_st_u32(void* mc_addr, unsigned v) {
  asm volatile("multimem.st.relaxed.sys.global.u32 [%0], %1;" ::"l"(mc_addr), "r"(v) : "memory");
}
// Sum of four fp32 values over every rank's copy (reduced in the switch).
__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const void* mc_addr) {
  float4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w)
               : "l"(mc_addr)
               : "memory");
  return r;
}
// Sum of eight bf16 values (four bf16x2 words) over every rank's copy, fp32 accumulation.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(mc_addr)
               : "memory");
  return r;
}

// Per-launch description of the peer group, passed by value to kernels.
struct PeerGroup {
  int world;
  int rank;
  unsigned epoch;               // this launch's signal value
  unsigned* signals[kMaxRanks]; // signals[p] = base of rank p's signal area (peer pointers)
  unsigned* signals_mc;         // multicast alias of the signal area (null without NVLS)
};

// Rendezvous at a signal slot: rank r writes `epoch` into slot[r] of every peer, then waits
// until every slot[p] of its own area has reached `epoch`.  Executed by ONE thread (others
// synchronise with it through a CTA barrier).  `slot_base` is an index into the signal area
// with room for `world` words.
__device__ __forceinline__ bool peer_barrier(const PeerGroup& g, int slot_base) {
  fence_sys();
  for (int p = 0; p < g.world; ++p) st_relaxed_sys(g.signals[p] + slot_base + g.rank, g.epoch);
  for (int p = 0; p < g.world; ++p)
    if (!wait_flag_ge(g.signals[g.rank] + slot_base + p, g.epoch)) return false;
  return true;
}

}  // namespace st
