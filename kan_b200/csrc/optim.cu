// Vectorised SGD and Adam updates on a flat fp32 parameter.
//
// Stand in for torch.optim.SGD(lr) and torch.optim.Adam(lr, betas, eps) as the
// reference's training loop calls them (README.md:59-66): plain SGD without
// momentum; Adam with bias correction, no weight decay, no amsgrad.  The update
// is elementwise, so only rounding (fused multiply-adds) can differ from torch.
#include "common.cuh"

namespace chebykan {

__global__ void __launch_bounds__(256)
sgd_kernel(float* __restrict__ p, const float* __restrict__ g, int64_t n, float lr, float gs) {
    const int64_t n4 = n >> 2;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t t0 = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    const float a = -lr * gs;
    for (int64_t e = t0; e < n4; e += stride) {
        float4 pv = reinterpret_cast<float4*>(p)[e];
        const float4 gv = reinterpret_cast<const float4*>(g)[e];
        pv.x = fmaf(a, gv.x, pv.x); pv.y = fmaf(a, gv.y, pv.y);
        pv.z = fmaf(a, gv.z, pv.z); pv.w = fmaf(a, gv.w, pv.w);
        reinterpret_cast<float4*>(p)[e] = pv;
    }
    for (int64_t e = (n4 << 2) + t0; e < n; e += stride) p[e] = fmaf(a, g[e], p[e]);
}

struct AdamConst { float b1, b2, omb1, omb2, step_size, inv_sqrt_bc2, eps, gs; };

__device__ __forceinline__ void adam_one(float& p, float g, float& m, float& v, const AdamConst& c) {
    g *= c.gs;
    m = fmaf(c.b1, m, c.omb1 * g);
    v = fmaf(c.b2, v, c.omb2 * g * g);
    const float denom = sqrtf(v) * c.inv_sqrt_bc2 + c.eps;
    p -= c.step_size * (m / denom);
}

__global__ void __launch_bounds__(256)
adam_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
            float* __restrict__ v, int64_t n, AdamConst c) {
    const int64_t n4 = n >> 2;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t t0 = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    for (int64_t e = t0; e < n4; e += stride) {
        float4 pv = reinterpret_cast<float4*>(p)[e];
        const float4 gv = reinterpret_cast<const float4*>(g)[e];
        float4 mv = reinterpret_cast<float4*>(m)[e];
        float4 vv = reinterpret_cast<float4*>(v)[e];
        adam_one(pv.x, gv.x, mv.x, vv.x, c); adam_one(pv.y, gv.y, mv.y, vv.y, c);
        adam_one(pv.z, gv.z, mv.z, vv.z, c); adam_one(pv.w, gv.w, mv.w, vv.w, c);
        reinterpret_cast<float4*>(p)[e] = pv;
        reinterpret_cast<float4*>(m)[e] = mv;
        reinterpret_cast<float4*>(v)[e] = vv;
    }
    for (int64_t e = (n4 << 2) + t0; e < n; e += stride) adam_one(p[e], g[e], m[e], v[e], c);
}

// Adam with the step count kept in device memory, so that a captured CUDA graph can be replayed:
// every thread derives the bias corrections from *step_dev + 1 (double precision, as torch does on
// the host); adam_step_inc_kernel then advances the counter.
__global__ void __launch_bounds__(256)
adam_dev_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                float* __restrict__ v, int64_t n, float lr, float b1, float b2, float eps, float gs,
                const int64_t* __restrict__ step_dev) {
    const double t = (double)(*step_dev + 1);
    const double bc1 = 1.0 - pow((double)b1, t);
    const double bc2 = 1.0 - pow((double)b2, t);
    AdamConst c;
    c.b1 = b1; c.b2 = b2; c.omb1 = 1.f - b1; c.omb2 = 1.f - b2;
    c.step_size = (float)((double)lr / bc1);
    c.inv_sqrt_bc2 = (float)(1.0 / sqrt(bc2));
    c.eps = eps; c.gs = gs;
    const int64_t n4 = n >> 2;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t t0 = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    for (int64_t e = t0; e < n4; e += stride) {
        float4 pv = reinterpret_cast<float4*>(p)[e];
        const float4 gv = reinterpret_cast<const float4*>(g)[e];
        float4 mv = reinterpret_cast<float4*>(m)[e];
        float4 vv = reinterpret_cast<float4*>(v)[e];
        adam_one(pv.x, gv.x, mv.x, vv.x, c); adam_one(pv.y, gv.y, mv.y, vv.y, c);
        adam_one(pv.z, gv.z, mv.z, vv.z, c); adam_one(pv.w, gv.w, mv.w, vv.w, c);
        reinterpret_cast<float4*>(p)[e] = pv;
        reinterpret_cast<float4*>(m)[e] = mv;
        reinterpret_cast<float4*>(v)[e] = vv;
    }
    for (int64_t e = (n4 << 2) + t0; e < n; e += stride) adam_one(p[e], g[e], m[e], v[e], c);
}

__global__ void adam_step_inc_kernel(int64_t* step_dev) { *step_dev += 1; }

static unsigned flat_grid(int64_t n) {
    int64_t blocks = ceil_div(ceil_div(n, 4), 256);
    if (blocks < 1) blocks = 1;
    if (blocks > 148 * 8) blocks = 148 * 8;
    return (unsigned)blocks;
}

int launch_sgd(float* p, const float* g, int64_t n, float lr, float gs, cudaStream_t s) {
    sgd_kernel<<<flat_grid(n), 256, 0, s>>>(p, g, n, lr, gs);
    return check_cuda(cudaGetLastError());
}

int launch_adam(float* p, const float* g, float* m, float* v, int64_t n, float lr, float b1,
                float b2, float eps, int64_t step, float gs, cudaStream_t s) {
    // same scalar arithmetic as torch's single-tensor Adam: double on the host
    const double bc1 = 1.0 - pow((double)b1, (double)step);
    const double bc2 = 1.0 - pow((double)b2, (double)step);
    AdamConst c;
    c.b1 = b1; c.b2 = b2; c.omb1 = 1.f - b1; c.omb2 = 1.f - b2;
    c.step_size = (float)((double)lr / bc1);
    c.inv_sqrt_bc2 = (float)(1.0 / sqrt(bc2));
    c.eps = eps; c.gs = gs;
    adam_kernel<<<flat_grid(n), 256, 0, s>>>(p, g, m, v, n, c);
    return check_cuda(cudaGetLastError());
}

int launch_adam_dev(float* p, const float* g, float* m, float* v, int64_t n, float lr, float b1,
                    float b2, float eps, int64_t* step_dev, float gs, cudaStream_t s) {
    adam_dev_kernel<<<flat_grid(n), 256, 0, s>>>(p, g, m, v, n, lr, b1, b2, eps, gs, step_dev);
    int rc = check_cuda(cudaGetLastError());
    if (rc) return rc;
    adam_step_inc_kernel<<<1, 1, 0, s>>>(step_dev);
    return check_cuda(cudaGetLastError());
}

}  // namespace chebykan
