// Coefficient packing: cheby_coeffs[in][out][deg+1] fp32 -> the per-mode GEMM
// operand layouts described in common.cuh.  Takes the place of the permute +
// copy torch.einsum does before its bmm (reference kan/basis/chebyshev.py:101).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "common.cuh"

namespace chebykan {

template <int MODE>
__global__ void __launch_bounds__(256)
pack_kernel(const float* __restrict__ c, void* __restrict__ packed, int in, int out, int dp1,
            int ib, int64_t k_pad, int64_t n_pad, int nd, int64_t k_main, const float* __restrict__ bias) {
    const int64_t total = k_pad * n_pad;
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total;
         e += (int64_t)gridDim.x * blockDim.x) {
        int64_t k, n;
        if (MODE == CHEBYKAN_MODE_FP32) { k = e / n_pad; n = e % n_pad; }
        else                            { n = e / k_pad; k = e % k_pad; }
        float v = 0.f;
        if (k >= k_main) {
            // the bias block (tensor-core layouts): slot 0 holds the bias as the mode rounds it, slot 1 what that
            // rounding dropped, so the kernel's block of ones adds the bias to about twice the mode's precision
            if (n < out && k <= k_main + 1) {
                const float b = bias[n];
                float head = b;
                if (MODE == CHEBYKAN_MODE_BF16) head = __bfloat162float(__float2bfloat16_rn(b));
                else if (MODE == CHEBYKAN_MODE_TF32) { uint32_t r; asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(b)); head = __uint_as_float(r); }
                v = (k == k_main) ? b : b - head;
            }
        } else {
            // nd degrees take K slots: all dp1 of them, or degrees 1..deg when degree 0 travels as the bias
            const int64_t blk = k / ((int64_t)ib * nd);
            const int64_t rem = k % ((int64_t)ib * nd);
            const int d = (int)(rem / ib) + (dp1 - nd);
            const int64_t i = blk * ib + rem % ib;
            if (i < in && n < out) v = c[(i * out + n) * dp1 + d];
        }
        if (MODE == CHEBYKAN_MODE_FP32) {
            reinterpret_cast<float*>(packed)[e] = v;
        } else if (MODE == CHEBYKAN_MODE_FP32X3) {
            // head = the value truncated to tf32, tail = what is left (exact in fp32; the tensor pipe
            // reads its top 11 bits): head + tail carries 22 bits of the coefficient
            const uint32_t hi = __float_as_uint(v) & 0xFFFFE000u;
            reinterpret_cast<uint32_t*>(packed)[e] = hi;
            reinterpret_cast<float*>(packed)[total + e] = v - __uint_as_float(hi);
        } else if (MODE == CHEBYKAN_MODE_TF32) {
            uint32_t r;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
            reinterpret_cast<uint32_t*>(packed)[e] = r;
        } else {
            reinterpret_cast<__nv_bfloat16*>(packed)[e] = __float2bfloat16_rn(v);
        }
    }
}

// ---- the fp16 plane of the TF32 mode's narrow layers (layout in common.cuh) ----------------------------------
__global__ void __launch_bounds__(256)
coeff_absmax_kernel(const float* __restrict__ c, int64_t n, uint32_t* __restrict__ header) {
    uint32_t m = 0u;
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x)
        m = max(m, __float_as_uint(fabsf(c[e])));      // a NaN's bit pattern beats every finite value: scaling is off then
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0 && m != 0u) atomicMax(header, m);
}

__global__ void __launch_bounds__(256)
pack_half_kernel(const float* __restrict__ c, uint32_t* __restrict__ header, __half* __restrict__ plane, int in, int out,
                 int dp1, int ib, int64_t k_pad, int64_t n_pad, int nd, int64_t k_main) {
    const float scale = half_scale_for(header[0]);
    if (blockIdx.x == 0 && threadIdx.x == 0) reinterpret_cast<float*>(header)[1] = 1.f / scale;
    const int64_t total = k_pad * n_pad;
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = e / k_pad, k = e % k_pad;
        float v = 0.f;
        if (k < k_main) {      // (the bias block stays zero: the narrow kernel adds the fp32 bias vector)
            const int64_t blk = k / ((int64_t)ib * nd);
            const int64_t rem = k % ((int64_t)ib * nd);
            const int d = (int)(rem / ib) + (dp1 - nd);
            const int64_t i = blk * ib + rem % ib;
            if (i < in && n < out) v = c[(i * out + n) * dp1 + d] * scale;
        }
        plane[e] = __float2half_rn(v);
    }
}

// bias[n] = sum_i C[i][n][0], each term rounded as the mode stores coefficients (bf16 / tf32; exact in the
// three-product mode); one warp per output, lanes stride over the inputs, fixed-order tree: bitwise repeatable.
template <int MODE>
__global__ void __launch_bounds__(256)
pack_bias_kernel(const float* __restrict__ c, float* __restrict__ bias, int in, int out, int dp1, int64_t n_pad) {
    const int64_t n = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (n >= n_pad) return;
    float s = 0.f;
    if (n < out) {
        for (int i = lane; i < in; i += 32) {
            float v = c[((int64_t)i * out + n) * dp1];
            if (MODE == CHEBYKAN_MODE_BF16) v = __bfloat162float(__float2bfloat16_rn(v));
            else if (MODE == CHEBYKAN_MODE_TF32) { uint32_t r; asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v)); v = __uint_as_float(r); }
            s += v;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) bias[n] = s;
}

static int launch_pack_half_plane(const float* coeffs, void* packed, int64_t in, int64_t out, int64_t deg, cudaStream_t s) {
    const PackedDims p = packed_dims(in, out, deg, CHEBYKAN_MODE_BF16);
    char* base = reinterpret_cast<char*>(packed) + tf32_half_plane_offset(in, out, deg);
    uint32_t* header = reinterpret_cast<uint32_t*>(base);
    int rc = check_cuda(cudaMemsetAsync(header, 0, HALF_PLANE_HEADER, s));
    if (rc) return rc;
    const int64_t n = in * out * (deg + 1);
    int64_t blocks = ceil_div(n, 256);
    if (blocks > 148 * 4) blocks = 148 * 4;
    coeff_absmax_kernel<<<(unsigned)blocks, 256, 0, s>>>(coeffs, n, header);
    if ((rc = check_cuda(cudaGetLastError()))) return rc;
    const int64_t total = p.k_pad * p.n_pad;
    blocks = ceil_div(total, 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    pack_half_kernel<<<(unsigned)blocks, 256, 0, s>>>(coeffs, header, reinterpret_cast<__half*>(base + HALF_PLANE_HEADER),
                                                    (int)in, (int)out, (int)deg + 1, (int)p.ib, p.k_pad, p.n_pad, (int)p.nd, p.in_pad * p.nd);
    return check_cuda(cudaGetLastError());
}

int launch_pack(const float* coeffs, void* packed, int64_t in, int64_t out, int64_t deg, int mode,
                cudaStream_t s) {
    const PackedDims p = packed_dims(in, out, deg, mode);
    const int64_t total = p.k_pad * p.n_pad;
    const int64_t k_main = p.in_pad * p.nd;        // K slots of the inputs; the bias block (if any) follows
    int64_t blocks = ceil_div(total, 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    const int dp1 = (int)deg + 1;
    int rc = CHEBYKAN_OK;
    float* bias = nullptr;
    if (packed_has_bias(deg, mode)) {
        // the bias vector first: the matrices' bias block is filled from it
        bias = reinterpret_cast<float*>(reinterpret_cast<char*>(packed) + packed_bias_offset(in, out, deg, mode));
        const unsigned bb = (unsigned)ceil_div(p.n_pad * 32, 256);
        if (mode == CHEBYKAN_MODE_BF16) pack_bias_kernel<CHEBYKAN_MODE_BF16><<<bb, 256, 0, s>>>(coeffs, bias, (int)in, (int)out, dp1, p.n_pad);
        else if (mode == CHEBYKAN_MODE_TF32) pack_bias_kernel<CHEBYKAN_MODE_TF32><<<bb, 256, 0, s>>>(coeffs, bias, (int)in, (int)out, dp1, p.n_pad);
        else pack_bias_kernel<CHEBYKAN_MODE_FP32X3><<<bb, 256, 0, s>>>(coeffs, bias, (int)in, (int)out, dp1, p.n_pad);
        if ((rc = check_cuda(cudaGetLastError()))) return rc;
    }
    if (mode == CHEBYKAN_MODE_FP32)
        pack_kernel<CHEBYKAN_MODE_FP32><<<(unsigned)blocks, 256, 0, s>>>(coeffs, packed, (int)in, (int)out, dp1, (int)p.ib, p.k_pad, p.n_pad, (int)p.nd, k_main, bias);
    else if (mode == CHEBYKAN_MODE_FP32X3)
        pack_kernel<CHEBYKAN_MODE_FP32X3><<<(unsigned)blocks, 256, 0, s>>>(coeffs, packed, (int)in, (int)out, dp1, (int)p.ib, p.k_pad, p.n_pad, (int)p.nd, k_main, bias);
    else if (mode == CHEBYKAN_MODE_TF32)
        pack_kernel<CHEBYKAN_MODE_TF32><<<(unsigned)blocks, 256, 0, s>>>(coeffs, packed, (int)in, (int)out, dp1, (int)p.ib, p.k_pad, p.n_pad, (int)p.nd, k_main, bias);
    else
        pack_kernel<CHEBYKAN_MODE_BF16><<<(unsigned)blocks, 256, 0, s>>>(coeffs, packed, (int)in, (int)out, dp1, (int)p.ib, p.k_pad, p.n_pad, (int)p.nd, k_main, bias);
    if ((rc = check_cuda(cudaGetLastError()))) return rc;
    if (deg >= 1 && mode == CHEBYKAN_MODE_TF32 && tf32_has_half_plane(in, out))
        rc = launch_pack_half_plane(coeffs, packed, in, out, deg, s);
    return rc;
}

__global__ void __launch_bounds__(256)
bias_rows_kernel(const float* __restrict__ bias, float* __restrict__ y, int64_t B, int out) {
    const int64_t n = B * out;
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x)
        y[e] = bias[e % out];
}

int launch_bias_rows(const void* packed, float* y, int64_t B, int64_t in, int64_t out, int mode, cudaStream_t s) {
    const float* bias = reinterpret_cast<const float*>(reinterpret_cast<const char*>(packed) + packed_bias_offset(in, out, 0, mode));
    int64_t blocks = ceil_div(B * out, 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    bias_rows_kernel<<<(unsigned)blocks, 256, 0, s>>>(bias, y, B, (int)out);
    return check_cuda(cudaGetLastError());
}

}  // namespace chebykan
