// Self-test of the bounded waits that the tcgen05 kernels rely on (tc_common.cuh: mbar_wait).
//
// Those kernels hand shared-memory slots between warp roles through mbarriers, and every wait has an iteration limit:
// when it runs out the role sets an abort flag, the CTA winds down (frees its tensor memory) and the host gets error
// code 5 instead of a hung GPU.  That path cannot be reached with healthy kernels, so this entry point exercises the
// primitive itself: one CTA waits, with a short limit, on a barrier that nothing will ever arrive at, and reports what
// the wait returned.  Nothing traps and nothing spins for ever.
#include "tc_common.cuh"

#include <cstdio>

namespace cb200 {

__global__ void __launch_bounds__(64)
bounded_wait_selftest_kernel(uint32_t limit, int* result) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // warp 1 is the consumer of a slot that no producer ever fills; warp 0 just goes on to the wind-down
    bool ok = true;
    if (threadIdx.x == 32) ok = mbar_wait(&bar, 0, &abort_flag, limit);
    __syncthreads();                                   // the wind-down every role reaches, also after a wait gave up
    if (threadIdx.x == 32) {
        result[0] = ok ? 0 : 5;                        // 5: the code the tensor-core entry points return for this
        result[1] = abort_flag;
    }
}

static __device__ int g_selftest_result[2];

}  // namespace cb200

// Returns 5 when the wait ran out by its limit (the expected outcome), 0 if the barrier completed, 3/4 on launch
// problems.  spin_limit is the number of polls (tens of nanoseconds each).
extern "C" int cb200_selftest_bounded_wait(unsigned spin_limit, char* errbuf, size_t errlen) {
    using namespace cb200;
    char local[8];
    if (!errbuf || errlen == 0) { errbuf = local; errlen = sizeof local; }
    errbuf[0] = 0;
    int* dev = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&dev), g_selftest_result);
    if (e != cudaSuccess) { snprintf(errbuf, errlen, "cudaGetSymbolAddress: %s", cudaGetErrorString(e)); return 3; }
    cudaStream_t st = current_stream();
    cudaMemsetAsync(dev, 0xff, 2 * sizeof(int), st);
    bounded_wait_selftest_kernel<<<1, 64, 0, st>>>(spin_limit, dev);
    count_launch();
    int host[2] = {-1, -1};
    e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaMemcpyAsync(host, dev, sizeof host, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) { snprintf(errbuf, errlen, "bounded-wait self-test: %s", cudaGetErrorString(e)); return 4; }
    if (host[0] == 5) snprintf(errbuf, errlen, "the wait ran out after %u polls and returned (abort flag %d)", spin_limit, host[1]);
    return host[0];
}

// The multiplier and shifts that `a / s` and `a % s` use for a host scalar (divmod_scalar.cuh), for callers and tests
// that want to check them without a GPU: |divisor| -> (multiplier, first shift, second shift), 32- and 64-bit.
#include "divmod_scalar.cuh"

extern "C" void cb200_invariant_divisor_u32(uint32_t d, uint32_t* m, int* sh1, int* sh2) {
    const cb200::InvariantDivisor<uint32_t> k = cb200::make_invariant_divisor<uint32_t>(d, false);
    *m = k.m; *sh1 = k.sh1; *sh2 = k.sh2;
}
extern "C" void cb200_invariant_divisor_u64(uint64_t d, uint64_t* m, int* sh1, int* sh2) {
    const cb200::InvariantDivisor<uint64_t> k = cb200::make_invariant_divisor<uint64_t>(d, false);
    *m = k.m; *sh1 = k.sh1; *sh2 = k.sh2;
}
