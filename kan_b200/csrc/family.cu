// Polynomial families other than Chebyshev: Jacobi and Hermite layers of the reference
// (kan/layers/jacobikan.py:20-68, kan/layers/hermitekan.py:22-83) share the Chebyshev layer's structure, so the
// fp32 forward, dC and dx kernels and the tcgen05 forward take the family's three-term recurrence as a table and are
// otherwise unchanged.  This file builds the table on the host from the family's description and holds the entry
// points.
#include <math.h>
#include "common.cuh"

namespace chebykan {

// Recurrence of the family in the form  P_d = (A[d] u + B[d]) P_{d-1} - C[d] P_{d-2},  evaluated in double
// and rounded once to fp32.
static int build_table(const chebykan_family* f, int64_t deg, RecurrenceTable* t) {
    if (f == nullptr || deg < 0 || deg > 127) return CHEBYKAN_EINVAL;
    const bool hermite = f->kind == CHEBYKAN_FAMILY_HERMITE || f->kind == CHEBYKAN_FAMILY_HERMITE_PROB;
    if (f->kind != CHEBYKAN_FAMILY_CHEBYSHEV && f->kind != CHEBYKAN_FAMILY_JACOBI && !hermite) return CHEBYKAN_EINVAL;
    if (f->affine != 0 && f->affine != 1) return CHEBYKAN_EINVAL;
    if (!isfinite(f->scale) || !isfinite(f->shift) || !isfinite(f->offset)) return CHEBYKAN_EINVAL;
    t->affine = f->affine;
    t->scale = f->scale != 0.f ? f->scale : (hermite ? 3.f : 1.f);
    t->shift = f->shift;
    t->offset = f->offset;
    for (int d = 0; d < 128; ++d) { t->A[d] = 0.f; t->B[d] = 0.f; t->C[d] = 0.f; }
    t->B[0] = 1.f;      // entry 0: P_0 = (0 u + 1) P_{-1} with P_{-1} = 1, for kernels that treat degree 0 as a step
    switch (f->kind) {
        case CHEBYKAN_FAMILY_CHEBYSHEV:
            t->A[1] = 1.f;
            for (int d = 2; d <= deg; ++d) { t->A[d] = 2.f; t->C[d] = 1.f; }
            break;
        case CHEBYKAN_FAMILY_HERMITE:            // H_1 = 2u, H_d = 2u H_{d-1} - 2(d-1) H_{d-2}   (hermite.py:163-196)
            for (int d = 1; d <= deg; ++d) { t->A[d] = 2.f; t->C[d] = 2.f * (float)(d - 1); }
            break;
        case CHEBYKAN_FAMILY_HERMITE_PROB:       // He_1 = u, He_d = u He_{d-1} - (d-1) He_{d-2}  (hermite.py:198-233)
            for (int d = 1; d <= deg; ++d) { t->A[d] = 1.f; t->C[d] = (float)(d - 1); }
            break;
        default: {                               // Jacobi (jacobi.py:136-188)
            const double al = f->alpha, be = f->beta;
            if (!(al > -1.0) || !(be > -1.0) || !isfinite(al) || !isfinite(be)) return CHEBYKAN_EINVAL;
            const double ab = al + be;
            t->A[1] = (float)((ab + 2.0) / 2.0);
            t->B[1] = (float)((al - be) / 2.0);
            for (int d = 2; d <= deg; ++d) {
                const double n = d;
                const double common = 2.0 * n + ab - 1.0;
                const double lin = (2.0 * n + ab) * (2.0 * n + ab - 2.0);
                const double denom = 2.0 * n * (n + ab) * (2.0 * n + ab - 2.0);
                t->A[d] = (float)(common * lin / denom);
                t->B[d] = (float)(common * (al * al - be * be) / denom);
                t->C[d] = (float)(2.0 * (n + al - 1.0) * (n + be - 1.0) * (2.0 * n + ab) / denom);
            }
        }
    }
    return CHEBYKAN_OK;
}

__global__ void __launch_bounds__(256)
family_normalize_kernel(const float* __restrict__ x, float* __restrict__ u, int64_t n, const __grid_constant__ TableRec rec) {
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x)
        u[e] = rec.normalize(x[e]);
}

// one thread per point; the deg+1 values of a point are contiguous
__global__ void __launch_bounds__(256)
family_basis_kernel(const float* __restrict__ u_in, float* __restrict__ phi, int64_t n, int dp1,
                    const __grid_constant__ TableRec rec) {
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x) {
        const float u = u_in[e];
        float* dst = phi + e * dp1;
        float pm1 = 1.f, pm2 = 0.f;
        dst[0] = 1.f;
        for (int d = 1; d < dp1; ++d) {
            const float v = rec.next(d, u, pm1, pm2);
            dst[d] = v; pm2 = pm1; pm1 = v;
        }
    }
}

static unsigned family_blocks_for(int64_t n) {
    int64_t b = ceil_div(n, 256);
    if (b > 148 * 16) b = 148 * 16;
    return (unsigned)(b < 1 ? 1 : b);
}

static bool family_shape_ok(int64_t B, int64_t in, int64_t out, int64_t deg) {
    return B >= 0 && in >= 1 && out >= 1 && deg >= 0 && deg <= 127 && in <= (1 << 20) && out <= (1 << 20) &&
           B <= (int64_t)1 << 31 && in * (deg + 1) <= (int64_t)1 << 24;
}

}  // namespace chebykan

using namespace chebykan;

extern "C" {

int chebykan_family_table(const chebykan_family* family, int64_t deg, float* a_host, float* b_host, float* c_host) {
    RecurrenceTable t;
    int rc = build_table(family, deg, &t);
    if (rc) return rc;
    if (!a_host || !b_host || !c_host) return CHEBYKAN_EINVAL;
    for (int d = 0; d <= deg; ++d) { a_host[d] = t.A[d]; b_host[d] = t.B[d]; c_host[d] = t.C[d]; }
    return CHEBYKAN_OK;
}

int chebykan_family_fwd(const chebykan_family* family, const float* x, const void* packed, float* y, int64_t B,
                        int64_t in, int64_t out, int64_t deg, int mode, int32_t* status, void* stream) {
    RecurrenceTable t;
    if (!family_shape_ok(B, in, out, deg) || !packed) return CHEBYKAN_EINVAL;
    if (mode != CHEBYKAN_MODE_FP32 && mode != CHEBYKAN_MODE_TF32 && mode != CHEBYKAN_MODE_BF16)
        return mode == CHEBYKAN_MODE_FP32X3 ? CHEBYKAN_EUNSUPPORTED : CHEBYKAN_EINVAL;
    int rc = build_table(family, deg, &t);
    if (rc) return rc;
    if (B == 0) return CHEBYKAN_OK;
    if (!x || !y) return CHEBYKAN_EINVAL;
    if (!aligned16(x) || !aligned16(y) || !aligned16(packed)) return CHEBYKAN_EALIGN;
    if ((rc = check_device())) return rc;
    if (mode == CHEBYKAN_MODE_FP32)
        return launch_fwd_ffma(x, reinterpret_cast<const float*>(packed), y, B, in, out, deg, (cudaStream_t)stream, &t);
    // bf16 / tf32: the tcgen05 kernel of the Chebyshev layer with the table-driven recurrence in its producer warps
    if (!status) return CHEBYKAN_EINVAL;
    if (deg == 0) return launch_bias_rows(packed, y, B, in, out, mode, (cudaStream_t)stream);     // P_0 = 1 in every family
    return launch_fwd_tc(x, packed, y, B, in, out, deg, mode, status, (cudaStream_t)stream, LnFusion(), &t);
}

static bool family_mode_ok(int mode) {
    return mode == CHEBYKAN_MODE_FP32 || mode == CHEBYKAN_MODE_TF32 || mode == CHEBYKAN_MODE_BF16;
}
// tf32 / bf16 modes: the tcgen05 kind::tf32 kernels of the Chebyshev layer's backward with the table recurrence,
// on the shapes those kernels cover; fp32 mode and every other shape: the FFMA kernels
static bool family_dcoeff_on_tensor_cores(int64_t B, int64_t in, int64_t out, int64_t deg, int mode) {
    return mode != CHEBYKAN_MODE_FP32 && B > 0 && dcoeff_tc_supported(B, in, out, deg);
}
static bool family_dx_on_tensor_cores(int64_t B, int64_t in, int64_t out, int64_t deg, int mode) {
    return mode != CHEBYKAN_MODE_FP32 && B > 0 && dx_tc_supported(B, in, out, deg);
}

int64_t chebykan_family_workspace_bytes(int op, int64_t B, int64_t in, int64_t out, int64_t deg, int mode) {
    if (!family_shape_ok(B, in, out, deg)) return CHEBYKAN_EINVAL;
    if (!family_mode_ok(mode)) return mode == CHEBYKAN_MODE_FP32X3 ? CHEBYKAN_EUNSUPPORTED : CHEBYKAN_EINVAL;
    switch (op) {
        case CHEBYKAN_OP_FWD: return 0;
        case CHEBYKAN_OP_BWD_DCOEFF:
            if (B == 0) return 0;
            return family_dcoeff_on_tensor_cores(B, in, out, deg, mode)
                       ? dcoeff_tc_workspace_bytes(B, in, out, deg, 0, 1)
                       : dcoeff_workspace_bytes(B, in, out, deg, CHEBYKAN_MODE_FP32);
        case CHEBYKAN_OP_BWD_DX:
            return family_dx_on_tensor_cores(B, in, out, deg, mode) ? dx_tc_workspace_bytes(B, in, out, deg, 0) : 0;
        default: return CHEBYKAN_EINVAL;
    }
}

int chebykan_family_bwd_dcoeff(const chebykan_family* family, const float* x, const float* dy, float* dcoeffs,
                               void* workspace, int64_t workspace_bytes, int64_t B, int64_t in, int64_t out,
                               int64_t deg, int mode, int accumulate, int32_t* status, void* stream) {
    RecurrenceTable t;
    if (!family_shape_ok(B, in, out, deg) || !dcoeffs) return CHEBYKAN_EINVAL;
    if (!family_mode_ok(mode)) return mode == CHEBYKAN_MODE_FP32X3 ? CHEBYKAN_EUNSUPPORTED : CHEBYKAN_EINVAL;
    int rc = build_table(family, deg, &t);
    if (rc) return rc;
    if (!aligned16(dcoeffs) || !aligned16(workspace)) return CHEBYKAN_EALIGN;
    if ((rc = check_device())) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    if (B == 0) {
        if (!accumulate) return check_cuda(cudaMemsetAsync(dcoeffs, 0, in * out * (deg + 1) * 4, s));
        return CHEBYKAN_OK;
    }
    if (!x || !dy) return CHEBYKAN_EINVAL;
    if (!aligned16(x) || !aligned16(dy)) return CHEBYKAN_EALIGN;
    if (family_dcoeff_on_tensor_cores(B, in, out, deg, mode)) {
        if (!status) return CHEBYKAN_EINVAL;
        return launch_dcoeff_tc(x, dy, dcoeffs, workspace, workspace_bytes, B, in, out, deg, accumulate, status, s, 0, &t);
    }
    return launch_dcoeff_ffma(x, dy, dcoeffs, workspace, workspace_bytes, B, in, out, deg, accumulate, s, &t);
}

int chebykan_family_bwd_dx(const chebykan_family* family, const float* x, const float* dy, const float* coeffs,
                           float* dx, void* workspace, int64_t workspace_bytes, int64_t B, int64_t in, int64_t out,
                           int64_t deg, int mode, int32_t* status, void* stream) {
    RecurrenceTable t;
    if (!family_shape_ok(B, in, out, deg) || !coeffs) return CHEBYKAN_EINVAL;
    if (!family_mode_ok(mode)) return mode == CHEBYKAN_MODE_FP32X3 ? CHEBYKAN_EUNSUPPORTED : CHEBYKAN_EINVAL;
    int rc = build_table(family, deg, &t);
    if (rc) return rc;
    if (B == 0) return CHEBYKAN_OK;
    if (!x || !dy || !dx) return CHEBYKAN_EINVAL;
    if (!aligned16(x) || !aligned16(dy) || !aligned16(dx) || !aligned16(coeffs) || !aligned16(workspace)) return CHEBYKAN_EALIGN;
    if ((rc = check_device())) return rc;
    if (family_dx_on_tensor_cores(B, in, out, deg, mode)) {
        if (!status) return CHEBYKAN_EINVAL;
        return launch_dx_tc(x, dy, coeffs, dx, workspace, workspace_bytes, B, in, out, deg, status, (cudaStream_t)stream, 0, &t);
    }
    return launch_dx_ffma(x, dy, coeffs, dx, B, in, out, deg, (cudaStream_t)stream, &t);
}

int chebykan_family_normalize(const chebykan_family* family, const float* x, float* u, int64_t n, void* stream) {
    TableRec rec;
    int rc = build_table(family, 0, &rec.t);
    if (rc) return rc;
    if (n < 0 || (n > 0 && (!x || !u))) return CHEBYKAN_EINVAL;
    if (n == 0) return CHEBYKAN_OK;
    if ((rc = check_device())) return rc;
    family_normalize_kernel<<<family_blocks_for(n), 256, 0, (cudaStream_t)stream>>>(x, u, n, rec);
    return check_cuda(cudaGetLastError());
}

int chebykan_family_basis(const chebykan_family* family, const float* u, float* phi, int64_t n, int64_t deg,
                          void* stream) {
    TableRec rec;
    int rc = build_table(family, deg, &rec.t);
    if (rc) return rc;
    if (n < 0 || (n > 0 && (!u || !phi))) return CHEBYKAN_EINVAL;
    if (n == 0) return CHEBYKAN_OK;
    if ((rc = check_device())) return rc;
    family_basis_kernel<<<family_blocks_for(n), 256, 0, (cudaStream_t)stream>>>(u, phi, n, (int)deg + 1, rec);
    return check_cuda(cudaGetLastError());
}

}  // extern "C"
