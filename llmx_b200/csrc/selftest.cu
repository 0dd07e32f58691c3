// A self-test of the kernels' bounded waits: a wait that nothing will ever satisfy runs out after the limit it is
// given, records its code in the error word, and the block goes on to its end.
//
// Every wait on an mbarrier in the tensor-core and attention kernels goes through tc::mbar_wait_limit (two seconds
// there).  This kernel makes that path run on purpose and harmlessly: one block initialises a barrier that expects one
// arrival, nobody arrives, and thread 0 waits on it with a limit of the caller's choosing (a millisecond in the
// tests).  Nothing hangs and nothing faults: the wait gives up, `error_word` holds ERR_SELFTEST_WAIT, `out[0]`
// says what the wait returned (1: completed, which would be a fault of the wait; 2: gave up) and the kernel returns.
#include "tc_common.cuh"

namespace {
constexpr int ERR_SELFTEST_WAIT = 105;

__global__ void wait_selftest_kernel(unsigned long long limit_ns, int* error_word, int* out) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        tc::mbar_init(&bar, 1);
        tc::fence_barrier_init();
        abort_flag = 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const bool completed = tc::mbar_wait_limit(&bar, 0, &abort_flag, error_word, ERR_SELFTEST_WAIT, limit_ns);
        out[0] = completed ? 1 : 2;
    }
    __syncthreads();
    // What a kernel's other warps do after a failed wait: every later wait returns at once.
    if (threadIdx.x == 32) out[1] = tc::mbar_wait_limit(&bar, 0, &abort_flag, error_word, ERR_SELFTEST_WAIT, limit_ns) ? 1 : 2;
}
}  // namespace

// limit_ns: 1,000 .. 100,000,000 (a tenth of a second at most).  out: two device ints.
LLMX_EXPORT int llmx_wait_selftest(unsigned long long limit_ns, int* error_word, int* out, cudaStream_t stream) {
    if (!error_word || !out || limit_ns < 1000ull || limit_ns > 100000000ull) return LLMX_ERR_BAD_ARGUMENT;
    wait_selftest_kernel<<<1, 64, 0, stream>>>(limit_ns, error_word, out);
    return launch_status();
}
