// True Jacobian of the layer, J[b,o,i] = d y[b,o] / d x[b,i]
//   = (1 - t^2) * sum_d d U_{d-1}(t) C[i,o,d],   t = tanh x[b,i]   (T_d' = d U_{d-1}).
// The reference offers KANLayer.jacobian (kan/layers/base.py:116-141) on top of
// ChebyshevBasis.derivative (kan/basis/chebyshev.py:174-267), which does not return this
// derivative (its coefficient rule doubles the T_1 term and it re-applies tanh); this kernel
// returns the derivative autograd gives.  fp32 FFMA, correctly rounded tanh; meant for the small
// layers such an API is used on (the output has B*out*in elements).
#include "common.cuh"

namespace chebykan {

__global__ void __launch_bounds__(256)
jacobian_kernel(const float* __restrict__ x, const float* __restrict__ coeffs, float* __restrict__ jac,
                int64_t B, int in, int out, int dp1) {
    const int64_t b = (int64_t)blockIdx.x * 8 + threadIdx.y;
    const int i = blockIdx.y * 32 + threadIdx.x;      // lanes run along the inputs: coalesced stores
    if (b >= B || i >= in) return;
    const float t = tanh_exact(x[b * in + i]);
    const float s = fmaf(-t, t, 1.f);
    const float t2 = 2.f * t;
    const float* ci = coeffs + (int64_t)i * out * dp1;
    float* jrow = jac + b * out * in + i;
    for (int o = 0; o < out; ++o) {
        const float* c = ci + (int64_t)o * dp1;
        float um1 = 1.f, um2 = 0.f, acc = 0.f;        // U_0 = 1, U_{-1} = 0
        for (int d = 1; d < dp1; ++d) {
            acc = fmaf((float)d * um1, c[d], acc);
            const float u = fmaf(t2, um1, -um2);
            um2 = um1; um1 = u;
        }
        jrow[(int64_t)o * in] = s * acc;
    }
}

int launch_jacobian(const float* x, const float* coeffs, float* jac, int64_t B, int64_t in, int64_t out,
                    int64_t deg, cudaStream_t s) {
    const int64_t gx = ceil_div(B, 8), gy = ceil_div(in, 32);
    if (gx > 0x7fffffffLL || gy > 65535) return CHEBYKAN_EUNSUPPORTED;
    jacobian_kernel<<<dim3((unsigned)gx, (unsigned)gy), dim3(32, 8), 0, s>>>(x, coeffs, jac, B, (int)in, (int)out,
                                                                            (int)deg + 1);
    return check_cuda(cudaGetLastError());
}

}  // namespace chebykan
