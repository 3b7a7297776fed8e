// Shared helpers for the ChebyKAN sm_100a kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "../../include/chebykan_b200.h"

namespace chebykan {

__host__ __device__ constexpr int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
__host__ __device__ constexpr int64_t round_up(int64_t a, int64_t b) { return ceil_div(a, b) * b; }

// ---- packed coefficient layouts ------------------------------------------
// FP32 mode:  Wf[K_pad][N_pad] fp32, N contiguous.
//   k = (i / 8) * (deg+1) * 8 + d * 8 + (i % 8)           (degree-major inside
//   blocks of 8 inputs), in padded to a multiple of 8, out to a multiple of 64.
// BF16 mode:  Wt[N_pad][K_pad] bf16, K contiguous (K-major B operand).
//   k = (i / 64) * (deg+1) * 64 + d * 64 + (i % 64), in padded to a multiple of
//   64, out to a multiple of 128.  One 64-wide K block (= one 128-byte swizzle
//   row) holds one degree of 64 consecutive inputs.
// TF32 mode:  Wt[N_pad][K_pad] fp32 (rounded to tf32), blocks of 32 inputs; narrow layers carry a second,
//   fp16 plane behind it (see tf32_has_half_plane below).
constexpr int FP32_IB = 8;
constexpr int BF16_IB = 64;
constexpr int TF32_IB = 32;
constexpr int FP32_NPAD = 64;
constexpr int TC_NPAD = 128;

struct PackedDims {
    int64_t ib;      // inputs per K block
    int64_t in_pad;  // inputs padded to a multiple of ib
    int64_t nd;      // degrees that take K slots (see below)
    int64_t k_pad;   // in_pad * nd
    int64_t n_pad;   // padded outputs
    int64_t elem;    // bytes per element
    bool    k_major; // true: [N_pad][K_pad]; false: [K_pad][N_pad]
    int64_t planes;  // matrices stored back to back (FP32X3: tf32 head, then tf32 tail)
};

// Degree 0 of every basis here is the constant 1, so its part of y, sum_i C[i][o][0], does not depend on x.  The
// tensor-core layouts leave it out of the GEMM (K covers degrees 1..deg: a ninth fewer MMAs at degree 8, a fifth
// fewer at degree 4) and carry it as a bias vector bias[N_pad] behind the matrices, which the forward kernels'
// epilogues add.  A layer of degree 0 is its bias alone (no matrix); the FP32 (FFMA) layout keeps all deg+1 degrees.
inline __host__ __device__ bool packed_has_bias(int64_t deg, int mode) { (void)deg; return mode != CHEBYKAN_MODE_FP32; }
inline __host__ __device__ int64_t packed_degrees(int64_t deg, int mode) { return packed_has_bias(deg, mode) ? deg : deg + 1; }

inline __host__ __device__ PackedDims packed_dims(int64_t in, int64_t out, int64_t deg, int mode) {
    PackedDims p{};
    if (mode == CHEBYKAN_MODE_FP32) {
        p.ib = FP32_IB; p.elem = 4; p.k_major = false; p.n_pad = round_up(out, FP32_NPAD);
    } else if (mode == CHEBYKAN_MODE_BF16) {
        p.ib = BF16_IB; p.elem = 2; p.k_major = true; p.n_pad = round_up(out, TC_NPAD);
    } else {
        p.ib = TF32_IB; p.elem = 4; p.k_major = true; p.n_pad = round_up(out, TC_NPAD);
    }
    p.planes = (mode == CHEBYKAN_MODE_FP32X3) ? 2 : 1;
    p.in_pad = round_up(in, p.ib);
    p.nd = packed_degrees(deg, mode);
    // tensor-core layouts: one more K block behind the last input block, whose first slot holds the bias (the wide
    // forward multiplies it with a block of ones, which costs one K block per tile and no epilogue work)
    p.k_pad = p.in_pad * p.nd + (packed_has_bias(deg, mode) ? p.ib : 0);
    return p;
}

// TF32 mode, narrow layers (at most 128 outputs, in % 4 == 0): behind the tf32 matrix the packed buffer carries a
// second plane for the tensor-memory forward kernel: a 256-byte header {bit pattern of max |C|, 1 / scale} and
// the coefficients times a power-of-two scale as fp16 in the BF16 layout.
constexpr int64_t HALF_PLANE_HEADER = 256;
inline __host__ __device__ bool tf32_has_half_plane(int64_t in, int64_t out) { return out <= 128 && (in % 4) == 0; }
inline __host__ __device__ int64_t tf32_half_plane_offset(int64_t in, int64_t out, int64_t deg) {
    const PackedDims p = packed_dims(in, out, deg, CHEBYKAN_MODE_TF32);
    return round_up(p.k_pad * p.n_pad * p.elem, 256);
}
inline __host__ __device__ int64_t tf32_half_plane_bytes(int64_t in, int64_t out, int64_t deg) {
    const PackedDims p = packed_dims(in, out, deg, CHEBYKAN_MODE_BF16);
    return HALF_PLANE_HEADER + p.k_pad * p.n_pad * 2;
}
// whole packed buffer: matrices (TF32 narrow layers: tf32 matrix, then the fp16 plane), then the bias vector
inline __host__ __device__ int64_t packed_matrix_bytes(int64_t in, int64_t out, int64_t deg, int mode) {
    const PackedDims p = packed_dims(in, out, deg, mode);
    if (mode == CHEBYKAN_MODE_TF32 && tf32_has_half_plane(in, out))
        return tf32_half_plane_offset(in, out, deg) + tf32_half_plane_bytes(in, out, deg);
    return p.k_pad * p.n_pad * p.elem * p.planes;
}
inline __host__ __device__ int64_t packed_bias_offset(int64_t in, int64_t out, int64_t deg, int mode) {
    return round_up(packed_matrix_bytes(in, out, deg, mode), 256);
}
inline __host__ __device__ int64_t packed_total_bytes(int64_t in, int64_t out, int64_t deg, int mode) {
    if (!packed_has_bias(deg, mode)) return packed_matrix_bytes(in, out, deg, mode);
    return packed_bias_offset(in, out, deg, mode) + packed_dims(in, out, deg, mode).n_pad * 4;
}
// power of two that puts `maxbits` (a non-negative float's bit pattern) into [2^14, 2^15); 1 for zero, inf and NaN
__device__ __forceinline__ float half_scale_for(uint32_t maxbits) {
    const int e = (int)(maxbits >> 23);            // biased exponent; 0 = zero / subnormal, 255 = inf / NaN
    if (e == 0 || e == 255) return 1.f;
    int k = 14 - (e - 127);
    if (k > 126) k = 126;                           // keep the scale a normal float
    if (k < -126) k = -126;
    return __uint_as_float((uint32_t)(k + 127) << 23);
}

// ---- tanh ------------------------------------------------------------------
// FP32 mode: tanh evaluated in double and rounded once, i.e. the correctly
// rounded fp32 value (high-degree T_d amplifies an error in t by up to d^2, so
// a 2-ulp tanh alone would spend the whole 1e-5 tolerance at degree 32).
__device__ __forceinline__ float tanh_exact(float x) { return (float)tanh((double)x); }

// Tensor-core modes: 1 - 2/(1+2^(2x log2 e)) with the approximate ex2 and rcp
// units; absolute error about 2e-7, far below bf16/tf32 operand rounding.
__device__ __forceinline__ float tanh_fast(float x) {
    float e, r;
    float z = x * 2.885390081777927f;  // 2*log2(e)
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(z));
    float den = e + 1.0f;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(den));
    return fmaf(-2.0f, r, 1.0f);
}

// ---- polynomial families ------------------------------------------------------
// Every layer of the reference that is "normalise, three-term recurrence, einsum('bid,iod->bo')" fits
//   u = scale * tanh(x)            (or the affine map u = scale * (x - shift) + offset)
//   P_0 = 1,  P_d = (A[d] u + B[d]) P_{d-1} - C[d] P_{d-2}   for d >= 1, with P_{-1} = 0
// (kan/basis/jacobi.py:136-188, kan/basis/hermite.py:163-233).  The fp32 kernels take the recurrence as a
// policy: ChebyshevRec is the compile-time special case (A = 2, C = 1, P_1 = u), TableRec reads the
// coefficients from a table passed by value as a __grid_constant__ kernel parameter.
struct RecurrenceTable {
    float scale, shift, offset;
    int32_t affine;               // 0: u = scale * tanh(x);  1: u = scale * (x - shift) + offset
    float A[128], B[128], C[128]; // entry 0 unused; entry 1 holds P_1 = A[1] u + B[1], C[1] = 0
};

struct ChebyshevRec {
    static constexpr bool kChebyshev = true;
    __device__ __forceinline__ float normalize(float x) const { return tanh_exact(x); }
    // value carried per point between degrees (2u), and the stand-in for P_{-1} that makes degree 1 come out as u
    __device__ __forceinline__ float carry(float u) const { return 2.f * u; }
    __device__ __forceinline__ float before_first(float u) const { return u; }
    __device__ __forceinline__ float next(int, float c, float pm1, float pm2) const { return fmaf(c, pm1, -pm2); }
};

struct TableRec {
    static constexpr bool kChebyshev = false;
    RecurrenceTable t;
    __device__ __forceinline__ float normalize(float x) const {
        return t.affine ? fmaf(t.scale, x - t.shift, t.offset) : t.scale * tanh_exact(x);
    }
    // du/dx at a point whose normalised value is u
    __device__ __forceinline__ float dnormalize(float u) const {
        if (t.affine) return t.scale;
        const float th = u / t.scale;
        return t.scale * fmaf(-th, th, 1.f);
    }
    __device__ __forceinline__ float carry(float u) const { return u; }
    __device__ __forceinline__ float before_first(float) const { return 0.f; }
    __device__ __forceinline__ float next(int d, float u, float pm1, float pm2) const {
        return fmaf(fmaf(t.A[d], u, t.B[d]), pm1, -(t.C[d] * pm2));
    }
    // derivative with respect to u of the same recurrence
    __device__ __forceinline__ float dnext(int d, float u, float pm1, float dpm1, float dpm2) const {
        return fmaf(t.A[d], pm1, fmaf(fmaf(t.A[d], u, t.B[d]), dpm1, -(t.C[d] * dpm2)));
    }
};

// thread-local record of the last CUDA error seen by an entry point
void set_last_cuda_error(int e);
inline int check_cuda(cudaError_t e) {
    if (e == cudaSuccess) return CHEBYKAN_OK;
    set_last_cuda_error((int)e);
    return CHEBYKAN_ECUDA;
}

// CHEBYKAN_OK when the current device is compute capability 10.x (also binds the device's primary context to the
// calling thread); every entry point that launches a kernel calls it first
int check_device();

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Optional LayerNorm fusion of the tensor-core forward.  stats_* hold two floats per row (sum and
// sum of squares over the row's features).  With stats_in the kernel normalises its input rows,
// x' = (x - mean) * rstd * gamma + beta, before tanh; with stats_out it adds the sums of the rows
// of y it produces (the caller zeroes the buffer), which the next layer consumes as its stats_in.
struct LnFusion {
    const float* stats_in = nullptr;
    const float* gamma = nullptr;
    const float* beta = nullptr;
    float eps = 1e-5f;
    float* stats_out = nullptr;
};

// ---- launchers implemented in the .cu files ------------------------------------
int launch_pack(const float* coeffs, void* packed, int64_t in, int64_t out, int64_t deg, int mode,
                cudaStream_t s);
// fp32 launchers: `rec` == nullptr is the Chebyshev layer, otherwise the family described by the table
int launch_fwd_ffma(const float* x, const float* wf, float* y, int64_t B, int64_t in, int64_t out,
                    int64_t deg, cudaStream_t s, const RecurrenceTable* rec = nullptr);
// `rec` != nullptr: another polynomial family (bf16 / tf32 modes, no LayerNorm fusion)
// y[b][o] = bias[o] for every row: the whole forward of a degree-0 layer in the tensor-core modes
int launch_bias_rows(const void* packed, float* y, int64_t B, int64_t in, int64_t out, int mode, cudaStream_t s);
int launch_fwd_tc(const float* x, const void* wt, float* y, int64_t B, int64_t in, int64_t out,
                  int64_t deg, int mode, int32_t* status, cudaStream_t s, const LnFusion& ln = LnFusion(),
                  const RecurrenceTable* rec = nullptr);
// narrow layers (<= 128 outputs): the basis tile lives in tensor memory (fwd_ts.cu)
bool fwd_ts_supported(int64_t B, int64_t in, int64_t out, int64_t deg, int mode);
int launch_fwd_ts(const float* x, const void* wt, float* y, int64_t B, int64_t in, int64_t out, int64_t deg, int mode,
                  int32_t* status, cudaStream_t s);
int64_t dcoeff_workspace_bytes(int64_t B, int64_t in, int64_t out, int64_t deg, int mode);
int launch_dcoeff_ffma(const float* x, const float* dy, float* dc, void* ws, int64_t ws_bytes,
                       int64_t B, int64_t in, int64_t out, int64_t deg, int accumulate,
                       cudaStream_t s, const RecurrenceTable* rec = nullptr);
int launch_dcoeff_reduce(const float* ws, float* dc, int64_t n, int splits, int accumulate, cudaStream_t s);
// FP32X3 backward: the tf32 tensor-core kernels run three times on head/tail operands.  Worth it only for
// large products (three launches and two operand splits against one FFMA launch), and the dx kernel keeps a whole
// row of outputs in one accumulator, whose truncating accumulation stays inside the tolerance up to 2048 outputs.
inline bool x3_backward_on_tensor_cores(int64_t B, int64_t in, int64_t out, int64_t deg) {
    return B * in * (deg + 1) * out >= ((int64_t)1 << 30);
}
inline bool x3_dx_on_tensor_cores(int64_t B, int64_t in, int64_t out, int64_t deg) {
    return out <= 2048 && x3_backward_on_tensor_cores(B, in, out, deg);
}
bool dcoeff_tc_supported(int64_t B, int64_t in, int64_t out, int64_t deg);
// narrow layers (<= 128 outputs): fp16 operands (11 significant bits, like tf32) with a scaled, transposed copy of dY
bool dcoeff_f16_supported(int64_t B, int64_t in, int64_t out, int64_t deg);
int64_t dcoeff_f16_workspace_bytes(int64_t B, int64_t in, int64_t out, int64_t deg);
int launch_dcoeff_f16(const float* x, const float* dy, float* dc, void* ws, int64_t ws_bytes, int64_t B, int64_t in,
                      int64_t out, int64_t deg, int accumulate, int32_t* status, cudaStream_t s);
// `family` / `rec`: another polynomial family (tf32 kernel with the table recurrence; never the fp16-operand one)
int64_t dcoeff_tc_workspace_bytes(int64_t B, int64_t in, int64_t out, int64_t deg, int x3 = 0, int family = 0);
int launch_dcoeff_tc(const float* x, const float* dy, float* dc, void* ws, int64_t ws_bytes, int64_t B,
                     int64_t in, int64_t out, int64_t deg, int accumulate, int32_t* status, cudaStream_t s, int x3 = 0,
                     const RecurrenceTable* rec = nullptr);
int launch_dx_ffma(const float* x, const float* dy, const float* coeffs, float* dx, int64_t B,
                   int64_t in, int64_t out, int64_t deg, cudaStream_t s, const RecurrenceTable* rec = nullptr);
bool dx_tc_supported(int64_t B, int64_t in, int64_t out, int64_t deg);
int64_t dx_tc_workspace_bytes(int64_t B, int64_t in, int64_t out, int64_t deg, int x3);
int launch_dx_tc(const float* x, const float* dy, const float* coeffs, float* dx, void* ws, int64_t ws_bytes,
                 int64_t B, int64_t in, int64_t out, int64_t deg, int32_t* status, cudaStream_t s, int x3,
                 const RecurrenceTable* rec = nullptr);
int launch_sgd(float* p, const float* g, int64_t n, float lr, float gs, cudaStream_t s);
int launch_adam(float* p, const float* g, float* m, float* v, int64_t n, float lr, float b1,
                float b2, float eps, int64_t step, float gs, cudaStream_t s);

int launch_jacobian(const float* x, const float* coeffs, float* jac, int64_t B, int64_t in, int64_t out,
                    int64_t deg, cudaStream_t s);
int launch_adam_dev(float* p, const float* g, float* m, float* v, int64_t n, float lr, float b1,
                    float b2, float eps, int64_t* step_dev, float gs, cudaStream_t s);

}  // namespace chebykan
