// One-launch training step for a single small ChebyKAN layer: forward, mean-squared-error loss, backward and the
// optimizer update in one kernel of one CTA.
//
// The reference's own example (README.md:57-69: a 1 -> 1 layer of degree 8 fitted to 100 points with Adam) is a
// dozen microsecond-scale kernels per step when every stage is its own launch; launch and host overhead, not
// arithmetic, set its time.  Here the whole step
//     y = layer(x); loss = mse(y, target); loss.backward(); optimizer.step()
// (kan/layers/chebykan.py:53-67, kan/basis/chebyshev.py:80-145 and their autograd backward) runs as one CTA:
//   phase A  a thread per row: t = tanh x, the three-term recurrence, y, the residual, dY = 2 (y - target) / n;
//            t and dY stay in shared memory, the squared residuals are summed in a fixed order;
//   phase B  dC[i,o,d] = sum_b T_d(t[b,i]) dY[b,o] in an order that depends on the shape only (bitwise
//            repeatable): a thread per coefficient, or several row slices per coefficient when there are few;
//            then the Adam (or SGD) update of that coefficient in place.
// fp32 throughout, tanh correctly rounded as in the fp32 layer kernels.  Limits: at most 2048 coefficients, 16
// outputs, and rows * (in + out) <= 49152 values of shared memory.
#include <math.h>
#include "common.cuh"

namespace chebykan {

constexpr int SMALL_MAX_PARAMS = 2048;
constexpr int SMALL_MAX_OUT = 16;
constexpr int64_t SMALL_MAX_ROW_VALUES = 49152;

__global__ void __launch_bounds__(256, 1)
small_step_kernel(const float* __restrict__ x, const float* __restrict__ target, float* __restrict__ coeffs,
                  float* __restrict__ exp_avg, float* __restrict__ exp_avg_sq, int64_t* __restrict__ step_dev,
                  float* __restrict__ loss_out, float* __restrict__ dcoeffs_out, int B, int in, int out, int dp1,
                  int adam, float lr, float b1, float b2, float eps) {
    extern __shared__ float sm[];
    const int P = in * out * dp1;
    float* c_s = sm;                       // [in][out][dp1]
    float* t_s = c_s + P;                  // [B][in]
    float* dy_s = t_s + (size_t)B * in;    // [B][out]
    float* red = dy_s + (size_t)B * out;   // [256]
    const int tid = threadIdx.x;
    for (int e = tid; e < P; e += 256) c_s[e] = coeffs[e];
    __syncthreads();

    // ---- phase A: forward, residual, dY
    const float inv_n = 1.f / ((float)B * (float)out);
    float loss_part = 0.f;
    for (int b = tid; b < B; b += 256) {
        float y[SMALL_MAX_OUT];
#pragma unroll
        for (int o = 0; o < SMALL_MAX_OUT; ++o) y[o] = 0.f;
        for (int i = 0; i < in; ++i) {
            const float t = tanh_exact(x[(size_t)b * in + i]);
            t_s[(size_t)b * in + i] = t;
            const float t2 = 2.f * t;
            float tm1 = 1.f, tm2 = t;          // T_0 = 1, T_{-1} = T_1 = t
            const float* ci = c_s + (size_t)i * out * dp1;
            for (int d = 0; d < dp1; ++d) {
                const float phi = d == 0 ? 1.f : fmaf(t2, tm1, -tm2);
                if (d > 0) { tm2 = tm1; tm1 = phi; }
#pragma unroll
                for (int o = 0; o < SMALL_MAX_OUT; ++o)
                    if (o < out) y[o] = fmaf(ci[o * dp1 + d], phi, y[o]);
            }
        }
#pragma unroll
        for (int o = 0; o < SMALL_MAX_OUT; ++o)
            if (o < out) {
                const float r = y[o] - target[(size_t)b * out + o];
                loss_part = fmaf(r, r, loss_part);
                dy_s[(size_t)b * out + o] = 2.f * r * inv_n;
            }
    }
    red[tid] = loss_part;
    __syncthreads();
    if (tid == 0) {
        float s = 0.f;
        for (int k = 0; k < 256; ++k) s += red[k];      // fixed order
        *loss_out = s * inv_n;
    }

    // ---- phase B: coefficient gradients (rows in order) and the update
    double bc1 = 1.0, bc2 = 1.0;
    if (adam) {
        const double step = (double)(*step_dev + 1);
        bc1 = 1.0 - pow((double)b1, step);
        bc2 = 1.0 - pow((double)b2, step);
    }
    const float step_size = (float)((double)lr / bc1);
    const float inv_sqrt_bc2 = (float)(1.0 / sqrt(bc2));
    // Few coefficients: S row slices per coefficient, one thread each (rows b = s, s + S, ...), partial sums added in
    // slice order.  Many coefficients: one thread per coefficient walks all rows.  Either way the order of the
    // additions depends on the shape only.
    const int S = P < 256 ? min(256 / P, 32) : 1;
    __syncthreads();                                     // thread 0 has read the loss partials: `red` is free
    for (int p0 = 0; p0 < P; p0 += 256) {
        const int p = S > 1 ? tid / S : p0 + tid;
        const int sl = S > 1 ? tid % S : 0;
        const bool active = p < P && (S == 1 || tid < P * S);
        float g = 0.f;
        if (active) {
            const int d = p % dp1, o = (p / dp1) % out, i = p / (dp1 * out);
            for (int b = sl; b < B; b += S) {
                const float t = t_s[(size_t)b * in + i];
                const float t2 = 2.f * t;
                float tm1 = 1.f, tm2 = t, phi = 1.f;
                for (int k = 1; k <= d; ++k) { phi = fmaf(t2, tm1, -tm2); tm2 = tm1; tm1 = phi; }
                g = fmaf(phi, dy_s[(size_t)b * out + o], g);
            }
        }
        if (S > 1) {
            red[tid] = g;
            __syncthreads();
            if (active && sl == 0) {
                g = 0.f;
                for (int k = 0; k < S; ++k) g += red[p * S + k];
            }
        }
        if (active && sl == 0) {
            if (dcoeffs_out) dcoeffs_out[p] = g;
            float w = c_s[p];
            if (adam) {
                float m = exp_avg[p], v = exp_avg_sq[p];
                m = fmaf(b1, m, (1.f - b1) * g);
                v = fmaf(b2, v, (1.f - b2) * g * g);
                const float denom = sqrtf(v) * inv_sqrt_bc2 + eps;
                w -= step_size * (m / denom);
                exp_avg[p] = m; exp_avg_sq[p] = v;
            } else {
                w = fmaf(-lr, g, w);
            }
            coeffs[p] = w;
        }
        if (S > 1) break;                                // all P coefficients were covered in this pass
    }
    __syncthreads();                                     // every thread has read the step count
    if (adam && tid == 0) *step_dev += 1;
}

}  // namespace chebykan

using namespace chebykan;

extern "C" int chebykan_small_train_step_supported(int64_t B, int64_t in, int64_t out, int64_t deg) {
    return B >= 1 && in >= 1 && out >= 1 && out <= SMALL_MAX_OUT && deg >= 0 && deg <= 127 &&
           in * out * (deg + 1) <= SMALL_MAX_PARAMS && B * (in + out) <= SMALL_MAX_ROW_VALUES;
}

extern "C" int chebykan_small_train_step(const float* x, const float* target, float* coeffs, float* exp_avg,
                                         float* exp_avg_sq, int64_t* step_dev, float* loss, float* dcoeffs_out,
                                         int64_t B, int64_t in, int64_t out, int64_t deg, int optimizer, float lr,
                                         float beta1, float beta2, float eps, void* stream) {
    if (!x || !target || !coeffs || !loss || (optimizer != 0 && optimizer != 1)) return CHEBYKAN_EINVAL;
    if (optimizer == 1 && (!exp_avg || !exp_avg_sq || !step_dev)) return CHEBYKAN_EINVAL;
    if (B < 1 || in < 1 || out < 1 || deg < 0 || deg > 127) return CHEBYKAN_EINVAL;
    if (!chebykan_small_train_step_supported(B, in, out, deg)) return CHEBYKAN_EUNSUPPORTED;
    int rc = check_device();
    if (rc) return rc;
    const size_t smem = (size_t)(in * out * (deg + 1) + B * (in + out) + 256) * sizeof(float);
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        rc = check_cuda(cudaFuncSetAttribute(small_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        if (rc) return rc;
        attr_set[dev] = true;
    }
    small_step_kernel<<<1, 256, smem, (cudaStream_t)stream>>>(x, target, coeffs, exp_avg, exp_avg_sq, step_dev, loss,
                                                              dcoeffs_out, (int)B, (int)in, (int)out, (int)deg + 1,
                                                              optimizer, lr, beta1, beta2, eps);
    return check_cuda(cudaGetLastError());
}
