// Grid-wide barrier for kernels launched cooperatively (every CTA resident), with a bounded wait.
//
// `counter` is a device word that holds zero when the kernel starts (the host clears it in stream order before the
// launch).  Barrier number k (1, 2, ...) is passed once the counter has reached k * gridDim.x.  Every thread of the CTA
// calls grid_sync(); thread 0 publishes the CTA's earlier global writes (fence), arrives and polls.  A wait that exceeds
// `limit_ns` sets `*status` to 1 and makes grid_sync() return false for the whole CTA: the caller then returns, and the
// other CTAs run into their own limit at their next barrier -- nothing spins forever.
#pragma once

#include <cstdint>

namespace sb {

struct GridBarrier {
  unsigned *counter;
  unsigned long long limit_ns;
  int32_t *status;
  unsigned passed;      // barriers this CTA has passed so far
};

__device__ __forceinline__ unsigned long long grid_sync_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool grid_sync(GridBarrier &gb) {
  __shared__ int s_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(gb.counter, 1u);
    const unsigned target = (gb.passed + 1u) * gridDim.x;
    const unsigned long long t0 = grid_sync_timer_ns();
    int ok = 1, polls = 0;
    while (static_cast<int>(*reinterpret_cast<volatile unsigned *>(gb.counter) - target) < 0) {
      if ((++polls & 31) == 0 && grid_sync_timer_ns() - t0 > gb.limit_ns) {     // (the timer is read now and then: it is slow)
        ok = 0;
        if (gb.status) atomicExch(gb.status, 1);
        break;
      }
    }
    __threadfence();
    s_ok = ok;
  }
  __syncthreads();
  gb.passed += 1u;
  return s_ok != 0;
}

}  // namespace sb
