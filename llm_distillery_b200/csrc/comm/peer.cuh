// Pieces shared by the kernels that touch other GPUs' memory: the table of per-rank pointers into symmetric
// buffers, system-scope release/acquire accesses for flag words, and bounded waits on such words.
#pragma once
#include "../common/ptx.cuh"

namespace b200 {
namespace comm {

constexpr int MAX_RANKS = 16;
struct Peers { void* p[MAX_RANKS]; };

__device__ __forceinline__ void st_release_sys(unsigned int* addr, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* addr) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* addr) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(unsigned int* addr, unsigned int v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}

// Wait until *addr (a counter or epoch that only grows) has reached `target`. SYS selects system scope (a word
// that another GPU writes) or device scope (a word that other CTAs of this kernel write). Bounded: after
// kWaitTimeoutNs the CTA's abort flag is set, `code` goes to the error word and the wait returns false.
template <bool SYS>
__device__ __forceinline__ bool wait_reached_bounded(const unsigned int* addr, unsigned int target,
                                                     volatile int* abort_flag, unsigned int* err_word,
                                                     unsigned int code) {
  const unsigned long long t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    const unsigned int v = SYS ? ld_acquire_sys(addr) : ld_acquire_gpu(addr);
    if (static_cast<int>(v - target) >= 0) return true;
    if (((++spins) & 0x3fu) == 0u) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > kWaitTimeoutNs) {
        *abort_flag = 1;
        if (err_word) atomicCAS(err_word, 0u, code);
        return false;
      }
    }
    __nanosleep(40);
  }
}

}  // namespace comm
}  // namespace b200
