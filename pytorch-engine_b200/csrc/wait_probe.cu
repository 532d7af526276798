// How long the library's bounded waits can last: one thread polls, `polls` times, an mbarrier on which nothing ever
// arrives, with the very poll that every wait of the library uses (tma::mbar_try_wait), and reports the time.  The
// kernel always ends by itself: it counts its polls, it waits for nothing.  With the time of one poll the limit of
// tma::mbar_wait (kWaitLimit polls) turns into seconds; tests check that product.
#include "api.h"
#include "common.cuh"
#include "tma.cuh"

namespace pe {

__global__ void wait_probe_kernel(unsigned long long* out, int polls) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    tma::mbar_init(&bar, 1);
    tma::fence_barrier_init();
    unsigned long long t0, t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    unsigned long long passed = 0;
    for (int i = 0; i < polls; ++i) passed += tma::mbar_try_wait(&bar, 0) ? 1u : 0u;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    out[0] = t1 - t0;      // nanoseconds for all polls
    out[1] = passed;       // polls that found the phase complete: none
  }
}

}  // namespace pe

// out: two 64-bit integers on the device (nanoseconds for all polls; polls that passed).  polls: 1 .. 1,000,000.
extern "C" int pe_wait_probe(unsigned long long* out, int polls, cudaStream_t stream) {
  if (out == nullptr || polls < 1 || polls > 1000000) return PE_ERR_BAD_ARGUMENT;
  pe::wait_probe_kernel<<<1, 32, 0, stream>>>(out, polls);
  PE_LAUNCH_CHECK();
  return PE_OK;
}

// The poll limit of every bounded wait in the library.
extern "C" long long pe_wait_limit_polls() { return (long long)pe::tma::kWaitLimit; }
