// Mean-squared-error loss and its gradient in one pass over the layer's output.
//
// The reference's training loop calls torch's MSE loss on the last layer's output (README.md:57-69):
// forward squares and averages (two passes), backward re-reads y and the target to form dY.  On the
// basis-bound narrow stacks those passes cost as much as a third of a layer kernel.  Here one kernel
// reads y and the target once, writes dY = 2 (y - t) * inv_n and leaves per-block partial sums of
// (y - t)^2; a second, single-block kernel adds the partials in a fixed order, so the loss is
// repeatable bit for bit.  HBM-bound: 12 bytes per element.
#include "common.cuh"

namespace chebykan {

constexpr int MSE_BLOCKS = 148 * 4;
constexpr int MSE_THREADS = 256;

__global__ void __launch_bounds__(MSE_THREADS)
mse_grad_kernel(const float* __restrict__ y, const float* __restrict__ t, float* __restrict__ dy,
                float* __restrict__ partial, int64_t n, float scale) {
    float acc = 0.f;
    const int64_t n4 = n >> 2;
    const float4* y4 = reinterpret_cast<const float4*>(y);
    const float4* t4 = reinterpret_cast<const float4*>(t);
    float4* d4 = reinterpret_cast<float4*>(dy);
    for (int64_t e = blockIdx.x * (int64_t)MSE_THREADS + threadIdx.x; e < n4; e += (int64_t)gridDim.x * MSE_THREADS) {
        const float4 a = y4[e], b = t4[e];
        const float4 d = make_float4(a.x - b.x, a.y - b.y, a.z - b.z, a.w - b.w);
        acc = fmaf(d.x, d.x, acc); acc = fmaf(d.y, d.y, acc); acc = fmaf(d.z, d.z, acc); acc = fmaf(d.w, d.w, acc);
        d4[e] = make_float4(d.x * scale, d.y * scale, d.z * scale, d.w * scale);
    }
    if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {        // scalar tail
        const int64_t e = (n4 << 2) + threadIdx.x;
        const float d = y[e] - t[e];
        acc = fmaf(d, d, acc);
        dy[e] = d * scale;
    }
    __shared__ float red[MSE_THREADS / 32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < MSE_THREADS / 32; ++w) s += red[w];
        partial[blockIdx.x] = s;
    }
}

__global__ void __launch_bounds__(256)
mse_final_kernel(const float* __restrict__ partial, int nblocks, float* __restrict__ loss, float inv_n) {
    // fixed order: thread k adds partials k, k+256, ...; then a tree over the 256 threads
    __shared__ double red[256];
    double s = 0.0;
    for (int k = threadIdx.x; k < nblocks; k += 256) s += (double)partial[k];
    red[threadIdx.x] = s;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) *loss = (float)(red[0] * (double)inv_n);
}

// dy *= *g unless *g == 1 (the usual case: backward() of the loss itself), in which case nothing is touched
__global__ void __launch_bounds__(256)
scale_by_device_scalar_kernel(float* __restrict__ dy, const float* __restrict__ g, int64_t n) {
    const float s = *g;
    if (s == 1.0f) return;
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x)
        dy[e] *= s;
}

}  // namespace chebykan

using namespace chebykan;

extern "C" int64_t chebykan_mse_workspace_bytes(void) { return (int64_t)MSE_BLOCKS * 4; }

extern "C" int chebykan_mse_loss_grad(const float* y, const float* target, float* dy, float* loss, void* workspace,
                                      int64_t workspace_bytes, int64_t n, int64_t n_mean, float grad_scale,
                                      void* stream) {
    if (n < 1 || n_mean < 1 || !y || !target || !dy || !loss || !workspace) return CHEBYKAN_EINVAL;
    if (!aligned16(y) || !aligned16(target) || !aligned16(dy) || !aligned16(workspace)) return CHEBYKAN_EALIGN;
    if (workspace_bytes < chebykan_mse_workspace_bytes()) return CHEBYKAN_EWORKSPACE;
    int rc = check_device();
    if (rc) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    int64_t blocks = ceil_div(ceil_div(n, 4), MSE_THREADS);
    if (blocks > MSE_BLOCKS) blocks = MSE_BLOCKS;
    if (blocks < 1) blocks = 1;
    const float inv_n = 1.0f / (float)n_mean;
    mse_grad_kernel<<<(unsigned)blocks, MSE_THREADS, 0, s>>>(y, target, dy, reinterpret_cast<float*>(workspace), n,
                                                             2.0f * inv_n * grad_scale);
    if ((rc = check_cuda(cudaGetLastError()))) return rc;
    mse_final_kernel<<<1, 256, 0, s>>>(reinterpret_cast<const float*>(workspace), (int)blocks, loss, inv_n);
    return check_cuda(cudaGetLastError());
}

extern "C" int chebykan_scale_by_device_scalar(float* dy, const float* scalar, int64_t n, void* stream) {
    if (n < 0 || !dy || !scalar) return CHEBYKAN_EINVAL;
    if (n == 0) return CHEBYKAN_OK;
    int rc = check_device();
    if (rc) return rc;
    int64_t blocks = ceil_div(n, 256 * 4);
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (blocks < 1) blocks = 1;
    scale_by_device_scalar_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(dy, scalar, n);
    return check_cuda(cudaGetLastError());
}
