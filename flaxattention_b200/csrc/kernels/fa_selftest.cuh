// Self test of the bounded wait that every mbarrier wait of the tcgen05 kernels goes through.
// One warp waits on a barrier that nobody arrives at; the wait must give up after
// FA_WAIT_LIMIT_NS (set short by the host for this kernel), raise the abort flag, and the kernel
// must report FA_STATUS_WAIT_TIMEOUT in the status word and return normally: no trap, the
// context stays usable.  The second warp's wait must end through the abort flag of the first
// (lane 0 of warp 0 starts first, the others follow the flag or their own clock).
#pragma once
#include "fa_sm100.cuh"

struct FaSelftestParams {
  int* status;          // bit FA_STATUS_WAIT_TIMEOUT is ORed in when the wait ran out
  int* gave_up;         // [0] threads whose wait returned false, [1] threads whose wait returned true
  unsigned long long* waited_ns;  // globaltimer span thread 0 spent in the wait
};

extern "C" __global__ void __launch_bounds__(64, 1) fa_wait_selftest_kernel(const __grid_constant__ FaSelftestParams p) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int abort_word;
  const fa_u32 b = fa_smem_u32(&bar);
  if (threadIdx.x == 0) {
    fa_mbar_init(b, 1);
    fa_mbar_init_fence();
    abort_word = 0;
  }
  __syncthreads();
  volatile int* abort_flag = &abort_word;
  const fa_u64 t0 = fa_globaltimer();
  // phase 0 of a fresh barrier completes only with an arrival, and there is none
  const bool ok = (threadIdx.x < 32) ? fa_mbar_wait_warp(b, 0, abort_flag) : fa_mbar_wait_all(b, 0, abort_flag);
  const fa_u64 t1 = fa_globaltimer();
  atomicAdd(p.gave_up + (ok ? 1 : 0), 1);
  if (threadIdx.x == 0) *p.waited_ns = t1 - t0;
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag != 0) atomicOr(p.status, FA_STATUS_WAIT_TIMEOUT);
}
