// Self-test of the bounded mbarrier wait every tensor-core kernel relies on.
//
// One CTA initialises an mbarrier that nothing ever arrives on and waits for it
// with the same wait routine the kernels use, but with a caller-chosen limit.
// The wait must give up after the limit, raise the abort flag, record its code in
// *status and return, leaving the context usable.  Nothing here faults or hangs.
#include "tc_common.cuh"

namespace chebykan {
namespace {
using namespace tc;

__global__ void bounded_wait_selftest_kernel(int32_t* status, uint64_t limit_ns, int code) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // warp 0 waits until the limit expires; warp 1 waits too and must leave through the abort flag
    if (!mbar_try_wait(smem_u32(&bar), 0))
        mbar_wait_slow(smem_u32(&bar), 0, &abort_flag, status, code,
                       threadIdx.x < 32 ? limit_ns : (uint64_t)4000000000ull);
    __syncthreads();
}
}  // namespace
}  // namespace chebykan

extern "C" int chebykan_selftest_bounded_wait(int32_t* status, int64_t limit_ns, int code, void* stream) {
    using namespace chebykan;
    if (!status || limit_ns <= 0 || limit_ns > 1000000000ll || code == 0) return CHEBYKAN_EINVAL;
    bounded_wait_selftest_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(status, (uint64_t)limit_ns, code);
    return check_cuda(cudaGetLastError());
}
