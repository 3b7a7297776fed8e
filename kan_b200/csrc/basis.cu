// The basis object's own methods, for callers outside the fused layer path (symbolic export, plots):
//   normalize_input  t = tanh(x)                         reference kan/basis/chebyshev.py:68-78
//   basis_functions  Phi[b,i,d] = T_d(t[b,i]), d = 0..deg  reference kan/basis/chebyshev.py:103-172
// The layer's forward never builds Phi; these two kernels exist so that the stand-in basis object offers the
// whole BasisFunction surface (kan/basis/base.py:28-94) on the GPU.  fp32, HBM-bound: one read of x and one
// write of (deg+1) values per element.
#include "common.cuh"

namespace chebykan {

__global__ void __launch_bounds__(256)
tanh_kernel(const float* __restrict__ x, float* __restrict__ t, int64_t n) {
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x)
        t[e] = tanh_exact(x[e]);
}

// one thread per element; the dp1 values of an element are contiguous, so a warp writes 32*dp1 consecutive floats
__global__ void __launch_bounds__(256)
basis_kernel(const float* __restrict__ t_in, float* __restrict__ phi, int64_t n, int dp1) {
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x) {
        // the reference clamps to [-1, 1] before acos (chebyshev.py:136)
        const float t = fminf(fmaxf(t_in[e], -1.f), 1.f);
        float* dst = phi + e * dp1;
        float tm1 = 1.f, tm2 = t;          // T_0 = 1, T_{-1} = T_1 = t
        dst[0] = 1.f;
        const float t2 = 2.f * t;
        for (int d = 1; d < dp1; ++d) {
            const float v = fmaf(t2, tm1, -tm2);
            dst[d] = v; tm2 = tm1; tm1 = v;
        }
    }
}

static unsigned blocks_for(int64_t n) {
    int64_t b = ceil_div(n, 256);
    if (b > 148 * 16) b = 148 * 16;
    return (unsigned)(b < 1 ? 1 : b);
}

}  // namespace chebykan

using namespace chebykan;

extern "C" int chebykan_normalize_input(const float* x, float* t, int64_t n, void* stream) {
    if (n < 0 || (n > 0 && (!x || !t))) return CHEBYKAN_EINVAL;
    if (n == 0) return CHEBYKAN_OK;
    int rc = check_device();
    if (rc) return rc;
    tanh_kernel<<<blocks_for(n), 256, 0, (cudaStream_t)stream>>>(x, t, n);
    return check_cuda(cudaGetLastError());
}

extern "C" int chebykan_basis_functions(const float* t, float* phi, int64_t n, int64_t deg, void* stream) {
    if (n < 0 || deg < 0 || deg > 127 || (n > 0 && (!t || !phi))) return CHEBYKAN_EINVAL;
    if (n == 0) return CHEBYKAN_OK;
    int rc = check_device();
    if (rc) return rc;
    basis_kernel<<<blocks_for(n), 256, 0, (cudaStream_t)stream>>>(t, phi, n, (int)deg + 1);
    return check_cuda(cudaGetLastError());
}
