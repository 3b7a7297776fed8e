// C ABI of the library: argument validation and dispatch to the kernels.
#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <mutex>
#include "common.cuh"

namespace chebykan {
static thread_local int g_last_cuda_error = 0;
void set_last_cuda_error(int e) { g_last_cuda_error = e; }

// 0 = unknown, 1 = compute capability 10.x, -1 = anything else (per device ordinal)
static int g_cc_ok[64] = {0};

int check_device() {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { set_last_cuda_error((int)e); return CHEBYKAN_ECUDA; }
    // Tensor maps are encoded through the driver API, which needs the device's primary context
    // bound to the CALLING thread.  A thread that has only ever selected a device (autograd's
    // backward threads, for instance) has none until its first runtime call that touches the
    // device: cudaFree(0) is that call.  Once per thread and device.
    static thread_local int bound_dev = -1;
    if (bound_dev != dev) {
        e = cudaFree(nullptr);
        if (e != cudaSuccess) { set_last_cuda_error((int)e); return CHEBYKAN_ECUDA; }
        bound_dev = dev;
    }
    if (dev < 0 || dev >= 64) return CHEBYKAN_EDEVICE;
    if (g_cc_ok[dev] == 0) {
        int major = 0;
        e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        if (e != cudaSuccess) { set_last_cuda_error((int)e); return CHEBYKAN_ECUDA; }
        g_cc_ok[dev] = (major == 10) ? 1 : -1;
    }
    return g_cc_ok[dev] == 1 ? CHEBYKAN_OK : CHEBYKAN_EDEVICE;
}

static bool shape_ok(int64_t B, int64_t in, int64_t out, int64_t deg) {
    // 32-bit tile arithmetic inside the kernels; deg+1 <= 128 slots per tile
    return B >= 0 && in >= 1 && out >= 1 && deg >= 0 && deg <= 127 &&
           in <= (1 << 20) && out <= (1 << 20) && B <= (int64_t)1 << 31 &&
           in * (deg + 1) <= (int64_t)1 << 24;
}
static bool mode_ok(int mode) {
    return mode == CHEBYKAN_MODE_FP32 || mode == CHEBYKAN_MODE_TF32 || mode == CHEBYKAN_MODE_BF16 ||
           mode == CHEBYKAN_MODE_FP32X3;
}
// CHEBYKAN_DX_WIDE=tf32 in the environment keeps the bf16 mode's wide layers on tf32 operands (A/B timing; read once)
static bool wide_dx_in_tf32() {
    static const bool v = [] {
        const char* e = getenv("CHEBYKAN_DX_WIDE");
        return e != nullptr && strcmp(e, "tf32") == 0;
    }();
    return v;
}
// operand variant of the tensor-core dx kernel: 1 = three tf32 products (FP32X3), 2 = fp16 operands (the bf16 mode on
// wide layers, where the kernel is bound by the tensor pipe: half the MMAs at tf32's 11 significant bits; narrow
// layers are bound by the fold, and the scaled fp16 copy of dY would only cost), 0 = tf32 operands
static int dx_variant(int64_t out, int64_t deg, int mode) {
    if (mode == CHEBYKAN_MODE_FP32X3) return 1;
    if (mode == CHEBYKAN_MODE_BF16 && out >= 512 && deg >= 1 && !wide_dx_in_tf32()) return 2;
    return 0;
}
static bool dx_on_tensor_cores(int64_t B, int64_t in, int64_t out, int64_t deg, int mode) {
    if (mode == CHEBYKAN_MODE_FP32 || !dx_tc_supported(B, in, out, deg)) return false;
    return mode != CHEBYKAN_MODE_FP32X3 || x3_dx_on_tensor_cores(B, in, out, deg);
}
// CHEBYKAN_NARROW_FWD=smem in the environment keeps narrow layers on the shared-memory-operand kernel (A/B timing
// of the two forward kernels; read once)
static bool narrow_forward_in_shared_memory() {
    static const bool v = [] {
        const char* e = getenv("CHEBYKAN_NARROW_FWD");
        return e != nullptr && strcmp(e, "smem") == 0;
    }();
    return v;
}
// modes whose backward kernels are the fp32 ones
static bool fp32_backward(int mode) {
    return mode == CHEBYKAN_MODE_FP32 || mode == CHEBYKAN_MODE_FP32X3;
}
}  // namespace chebykan

using namespace chebykan;

extern "C" {

int chebykan_abi_version(void) { return CHEBYKAN_ABI_VERSION; }

const char* chebykan_strerror(int code) {
    switch (code) {
        case CHEBYKAN_OK: return "ok";
        case CHEBYKAN_EINVAL: return "invalid argument (shape, null pointer or enum)";
        case CHEBYKAN_EALIGN: return "pointer is not 16-byte aligned";
        case CHEBYKAN_EUNSUPPORTED: return "shape not supported in this mode";
        case CHEBYKAN_ECUDA: return "CUDA runtime error";
        case CHEBYKAN_ETIMEOUT: return "a bounded device-side wait gave up";
        case CHEBYKAN_EWORKSPACE: return "workspace or packed buffer too small";
        case CHEBYKAN_EDEVICE: return "current device is not compute capability 10.x (B200)";
        case CHEBYKAN_ESTATIC: return "shape needs more scratch than the library's built-in 16 MiB array; use the workspace variant";
        default: return "unknown error code";
    }
}

int chebykan_last_cuda_error(void) { return g_last_cuda_error; }

int64_t chebykan_packed_bytes(int64_t in, int64_t out, int64_t deg, int mode) {
    if (!shape_ok(0, in, out, deg) || !mode_ok(mode)) return CHEBYKAN_EINVAL;
    return packed_total_bytes(in, out, deg, mode);
}

int chebykan_pack_coeffs(const float* coeffs, void* packed, int64_t in, int64_t out, int64_t deg,
                         int mode, void* stream) {
    if (!shape_ok(0, in, out, deg) || !mode_ok(mode) || !coeffs || !packed) return CHEBYKAN_EINVAL;
    if (!aligned16(coeffs) || !aligned16(packed)) return CHEBYKAN_EALIGN;
    int rc = check_device();
    if (rc) return rc;
    return launch_pack(coeffs, packed, in, out, deg, mode, (cudaStream_t)stream);
}

int64_t chebykan_workspace_bytes(int op, int64_t B, int64_t in, int64_t out, int64_t deg, int mode) {
    if (!shape_ok(B, in, out, deg) || !mode_ok(mode)) return CHEBYKAN_EINVAL;
    switch (op) {
        case CHEBYKAN_OP_FWD: return 0;
        case CHEBYKAN_OP_BWD_DCOEFF: return B == 0 ? 0 : dcoeff_workspace_bytes(B, in, out, deg, mode);
        case CHEBYKAN_OP_BWD_DX:
            return dx_on_tensor_cores(B, in, out, deg, mode)
                       ? dx_tc_workspace_bytes(B, in, out, deg, dx_variant(out, deg, mode)) : 0;
        default: return CHEBYKAN_EINVAL;
    }
}

int chebykan_fwd(const float* x, const void* packed, float* y, int64_t B, int64_t in, int64_t out,
                 int64_t deg, int mode, int32_t* status, void* stream) {
    if (!shape_ok(B, in, out, deg) || !mode_ok(mode) || !packed) return CHEBYKAN_EINVAL;
    if (B == 0) return CHEBYKAN_OK;
    if (!x || !y) return CHEBYKAN_EINVAL;
    if (!aligned16(x) || !aligned16(y) || !aligned16(packed)) return CHEBYKAN_EALIGN;
    int rc = check_device();
    if (rc) return rc;
    if (mode == CHEBYKAN_MODE_FP32)
        return launch_fwd_ffma(x, reinterpret_cast<const float*>(packed), y, B, in, out, deg,
                               (cudaStream_t)stream);
    if (!status) return CHEBYKAN_EINVAL;
    // degree 0 in a tensor-core mode: y is the bias vector of the packed buffer in every row
    if (deg == 0) return launch_bias_rows(packed, y, B, in, out, mode, (cudaStream_t)stream);
    if (fwd_ts_supported(B, in, out, deg, mode) && !narrow_forward_in_shared_memory())
        return launch_fwd_ts(x, reinterpret_cast<const void*>(packed), y, B, in, out, deg, mode, status, (cudaStream_t)stream);
    return launch_fwd_tc(x, packed, y, B, in, out, deg, mode, status, (cudaStream_t)stream);
}

int chebykan_fwd_ln(const float* x, const void* packed, float* y, int64_t B, int64_t in, int64_t out,
                    int64_t deg, int mode, const float* ln_stats_in, const float* ln_gamma,
                    const float* ln_beta, float ln_eps, float* ln_stats_out, int32_t* status, void* stream) {
    if (!shape_ok(B, in, out, deg) || !mode_ok(mode) || !packed || !status) return CHEBYKAN_EINVAL;
    if (fp32_backward(mode)) return CHEBYKAN_EUNSUPPORTED;   // fusion lives in the bf16 / tf32 tensor-core kernels
    if (deg == 0) return CHEBYKAN_EUNSUPPORTED;               // a degree-0 layer is a constant: nothing to fuse into
    if (ln_stats_in && (!ln_gamma || !ln_beta)) return CHEBYKAN_EINVAL;
    if (B == 0) return CHEBYKAN_OK;
    if (!x || !y) return CHEBYKAN_EINVAL;
    if (!aligned16(x) || !aligned16(y) || !aligned16(packed)) return CHEBYKAN_EALIGN;
    int rc = check_device();
    if (rc) return rc;
    LnFusion ln;
    ln.stats_in = ln_stats_in; ln.gamma = ln_gamma; ln.beta = ln_beta; ln.eps = ln_eps; ln.stats_out = ln_stats_out;
    return launch_fwd_tc(x, packed, y, B, in, out, deg, mode, status, (cudaStream_t)stream, ln);
}

int chebykan_bwd_dcoeff(const float* x, const float* dy, float* dcoeffs, void* workspace,
                        int64_t workspace_bytes, int64_t B, int64_t in, int64_t out, int64_t deg,
                        int mode, int accumulate, int32_t* status, void* stream) {
    if (!shape_ok(B, in, out, deg) || !mode_ok(mode) || !dcoeffs) return CHEBYKAN_EINVAL;
    if (!aligned16(dcoeffs) || !aligned16(workspace)) return CHEBYKAN_EALIGN;
    int rc = check_device();
    if (rc) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    if (B == 0) {
        if (!accumulate) return check_cuda(cudaMemsetAsync(dcoeffs, 0, in * out * (deg + 1) * 4, s));
        return CHEBYKAN_OK;
    }
    if (!x || !dy) return CHEBYKAN_EINVAL;
    if (!aligned16(x) || !aligned16(dy)) return CHEBYKAN_EALIGN;
    // tf32 and bf16 modes: tcgen05 kind::tf32 (bf16 operands would miss the 2e-3 tolerance for this
    // product); shapes it does not cover, and fp32 mode, accumulate in fp32 on the FFMA pipe
    if (!fp32_backward(mode) && dcoeff_tc_supported(B, in, out, deg)) {
        if (!status) return CHEBYKAN_EINVAL;
        return launch_dcoeff_tc(x, dy, dcoeffs, workspace, workspace_bytes, B, in, out, deg, accumulate,
                                status, s);
    }
    // FP32X3, large products: the same kernel three times on tf32 heads and tails, short batch slices
    if (mode == CHEBYKAN_MODE_FP32X3 && dcoeff_tc_supported(B, in, out, deg) &&
        x3_backward_on_tensor_cores(B, in, out, deg)) {
        if (!status) return CHEBYKAN_EINVAL;
        return launch_dcoeff_tc(x, dy, dcoeffs, workspace, workspace_bytes, B, in, out, deg, accumulate,
                                status, s, 1);
    }
    return launch_dcoeff_ffma(x, dy, dcoeffs, workspace, workspace_bytes, B, in, out, deg,
                              accumulate, s);
}

int chebykan_bwd_dx(const float* x, const float* dy, const float* coeffs, float* dx, void* workspace,
                    int64_t workspace_bytes, int64_t B, int64_t in, int64_t out, int64_t deg, int mode,
                    int32_t* status, void* stream) {
    if (!shape_ok(B, in, out, deg) || !mode_ok(mode) || !coeffs) return CHEBYKAN_EINVAL;
    if (B == 0) return CHEBYKAN_OK;
    if (!x || !dy || !dx) return CHEBYKAN_EINVAL;
    if (!aligned16(x) || !aligned16(dy) || !aligned16(dx) || !aligned16(coeffs) || !aligned16(workspace))
        return CHEBYKAN_EALIGN;
    int rc = check_device();
    if (rc) return rc;
    // tf32 mode (and narrow layers in the bf16 mode): tcgen05 kind::tf32 with the coefficients repacked into the
    // workspace; bf16 mode on wide layers: kind::f16 on scaled fp16 copies of dY and the coefficients
    // FP32X3: the same kernel three times on tf32 heads and tails of dY and of the coefficients
    if (dx_on_tensor_cores(B, in, out, deg, mode)) {
        if (!status) return CHEBYKAN_EINVAL;
        return launch_dx_tc(x, dy, coeffs, dx, workspace, workspace_bytes, B, in, out, deg, status,
                            (cudaStream_t)stream, dx_variant(out, deg, mode));
    }
    return launch_dx_ffma(x, dy, coeffs, dx, B, in, out, deg, (cudaStream_t)stream);
}

int chebykan_jacobian(const float* x, const float* coeffs, float* jac, int64_t B, int64_t in, int64_t out,
                      int64_t deg, void* stream) {
    if (!shape_ok(B, in, out, deg) || !coeffs) return CHEBYKAN_EINVAL;
    if (B == 0) return CHEBYKAN_OK;
    if (!x || !jac) return CHEBYKAN_EINVAL;
    int rc = check_device();
    if (rc) return rc;
    return launch_jacobian(x, coeffs, jac, B, in, out, deg, (cudaStream_t)stream);
}

int chebykan_sgd_step(float* param, const float* grad, int64_t n, float lr, float grad_scale,
                      void* stream) {
    if (n < 0 || !param || !grad) return CHEBYKAN_EINVAL;
    if (!aligned16(param) || !aligned16(grad)) return CHEBYKAN_EALIGN;
    if (n == 0) return CHEBYKAN_OK;
    int rc = check_device();
    if (rc) return rc;
    return launch_sgd(param, grad, n, lr, grad_scale, (cudaStream_t)stream);
}

int chebykan_adam_step(float* param, const float* grad, float* exp_avg, float* exp_avg_sq,
                       int64_t n, float lr, float beta1, float beta2, float eps, int64_t step,
                       float grad_scale, void* stream) {
    if (n < 0 || step < 1 || !param || !grad || !exp_avg || !exp_avg_sq) return CHEBYKAN_EINVAL;
    if (!aligned16(param) || !aligned16(grad) || !aligned16(exp_avg) || !aligned16(exp_avg_sq))
        return CHEBYKAN_EALIGN;
    if (n == 0) return CHEBYKAN_OK;
    int rc = check_device();
    if (rc) return rc;
    return launch_adam(param, grad, exp_avg, exp_avg_sq, n, lr, beta1, beta2, eps, step,
                       grad_scale, (cudaStream_t)stream);
}

int chebykan_adam_step_graph(float* param, const float* grad, float* exp_avg, float* exp_avg_sq,
                             int64_t n, float lr, float beta1, float beta2, float eps,
                             int64_t* step_dev, float grad_scale, void* stream) {
    if (n < 0 || !param || !grad || !exp_avg || !exp_avg_sq || !step_dev) return CHEBYKAN_EINVAL;
    if (!aligned16(param) || !aligned16(grad) || !aligned16(exp_avg) || !aligned16(exp_avg_sq))
        return CHEBYKAN_EALIGN;
    if (n == 0) return CHEBYKAN_OK;
    int rc = check_device();
    if (rc) return rc;
    return launch_adam_dev(param, grad, exp_avg, exp_avg_sq, n, lr, beta1, beta2, eps, step_dev,
                           grad_scale, (cudaStream_t)stream);
}

// ---- host-buffer forward ------------------------------------------------------------
static int64_t a256(int64_t v) { return round_up(v, 256); }

int64_t chebykan_fwd_host_scratch_bytes(int64_t B, int64_t in, int64_t out, int64_t deg, int mode) {
    if (!shape_ok(B, in, out, deg) || !mode_ok(mode)) return CHEBYKAN_EINVAL;
    return a256(B * in * 4) + a256(in * out * (deg + 1) * 4) +
           a256(chebykan_packed_bytes(in, out, deg, mode)) + a256(B * out * 4) + 256;
}

int chebykan_fwd_host(const float* x_host, const float* coeffs_host, float* y_host,
                      void* device_scratch, int64_t scratch_bytes, int64_t B, int64_t in,
                      int64_t out, int64_t deg, int mode, void* stream) {
    if (!shape_ok(B, in, out, deg) || !mode_ok(mode) || !coeffs_host || !device_scratch)
        return CHEBYKAN_EINVAL;
    if (B == 0) return CHEBYKAN_OK;
    if (!x_host || !y_host) return CHEBYKAN_EINVAL;
    if (!aligned16(device_scratch)) return CHEBYKAN_EALIGN;
    if (scratch_bytes < chebykan_fwd_host_scratch_bytes(B, in, out, deg, mode)) return CHEBYKAN_EWORKSPACE;
    cudaStream_t s = (cudaStream_t)stream;
    char* base = reinterpret_cast<char*>(device_scratch);
    float* xd = reinterpret_cast<float*>(base);            base += a256(B * in * 4);
    float* cd = reinterpret_cast<float*>(base);            base += a256(in * out * (deg + 1) * 4);
    void* pk = base;                                       base += a256(chebykan_packed_bytes(in, out, deg, mode));
    float* yd = reinterpret_cast<float*>(base);            base += a256(B * out * 4);
    int32_t* st = reinterpret_cast<int32_t*>(base);
    int rc;
    if ((rc = check_cuda(cudaMemcpyAsync(xd, x_host, B * in * 4, cudaMemcpyHostToDevice, s)))) return rc;
    if ((rc = check_cuda(cudaMemcpyAsync(cd, coeffs_host, in * out * (deg + 1) * 4, cudaMemcpyHostToDevice, s)))) return rc;
    if ((rc = check_cuda(cudaMemsetAsync(st, 0, 4, s)))) return rc;
    if ((rc = chebykan_pack_coeffs(cd, pk, in, out, deg, mode, stream))) return rc;
    if ((rc = chebykan_fwd(xd, pk, yd, B, in, out, deg, mode, st, stream))) return rc;
    if ((rc = check_cuda(cudaMemcpyAsync(y_host, yd, B * out * 4, cudaMemcpyDeviceToHost, s)))) return rc;
    int32_t st_host = 0;
    if ((rc = check_cuda(cudaMemcpyAsync(&st_host, st, 4, cudaMemcpyDeviceToHost, s)))) return rc;
    if ((rc = check_cuda(cudaStreamSynchronize(s)))) return rc;
    return st_host ? CHEBYKAN_ETIMEOUT : CHEBYKAN_OK;
}

// ---- pipelined host-buffer forward ----------------------------------------------------
namespace {
// device buffers per direction in the pipelined host forward (a third one, which lets either copy stream run
// further ahead of the other, measured no faster: 6.51 against 6.34-6.40 ms for 65536 x 1024 -> 1024)
constexpr int HOST_SLOTS = 2;
struct HostPipe {
    bool ready = false;
    cudaStream_t s_in = nullptr, s_out = nullptr;
    cudaEvent_t e_start = nullptr, e_in[HOST_SLOTS] = {}, e_cmp[HOST_SLOTS] = {}, e_free_x[HOST_SLOTS] = {}, e_free_y[HOST_SLOTS] = {};
};
HostPipe g_pipes[64];
std::mutex g_pipe_mutex;

int pipe_for_device(int dev, HostPipe** out) {
    if (dev < 0 || dev >= 64) return CHEBYKAN_EINVAL;
    HostPipe& p = g_pipes[dev];
    if (!p.ready) {
        int rc;
        if ((rc = check_cuda(cudaStreamCreateWithFlags(&p.s_in, cudaStreamNonBlocking)))) return rc;
        if ((rc = check_cuda(cudaStreamCreateWithFlags(&p.s_out, cudaStreamNonBlocking)))) return rc;
        if ((rc = check_cuda(cudaEventCreateWithFlags(&p.e_start, cudaEventDisableTiming)))) return rc;
        for (int k = 0; k < HOST_SLOTS; ++k)
            for (cudaEvent_t* e : {&p.e_in[k], &p.e_cmp[k], &p.e_free_x[k], &p.e_free_y[k]})
                if ((rc = check_cuda(cudaEventCreateWithFlags(e, cudaEventDisableTiming)))) return rc;
        p.ready = true;
    }
    *out = &p;
    return CHEBYKAN_OK;
}
}  // namespace

int64_t chebykan_fwd_host_packed_scratch_bytes(int64_t chunk_rows, int64_t in, int64_t out) {
    if (chunk_rows <= 0 || in <= 0 || out <= 0) return CHEBYKAN_EINVAL;
    return HOST_SLOTS * (a256(chunk_rows * in * 4) + a256(chunk_rows * out * 4)) + 256;
}

int chebykan_fwd_host_packed(const float* x_host, const void* packed, float* y_host, void* device_scratch,
                             int64_t scratch_bytes, int64_t B, int64_t in, int64_t out, int64_t deg, int mode,
                             int64_t chunk_rows, void* stream) {
    if (!shape_ok(B, in, out, deg) || !mode_ok(mode) || !packed || !device_scratch || chunk_rows <= 0)
        return CHEBYKAN_EINVAL;
    if (B == 0) return CHEBYKAN_OK;
    if (!x_host || !y_host) return CHEBYKAN_EINVAL;
    if (!aligned16(device_scratch) || !aligned16(packed)) return CHEBYKAN_EALIGN;
    if (chunk_rows > B) chunk_rows = B;
    if (scratch_bytes < chebykan_fwd_host_packed_scratch_bytes(chunk_rows, in, out)) return CHEBYKAN_EWORKSPACE;
    int rc = check_device();
    if (rc) return rc;
    int dev = 0;
    if ((rc = check_cuda(cudaGetDevice(&dev)))) return rc;
    std::lock_guard<std::mutex> lock(g_pipe_mutex);
    HostPipe* p = nullptr;
    if ((rc = pipe_for_device(dev, &p))) return rc;

    cudaStream_t cur = (cudaStream_t)stream;
    char* base = reinterpret_cast<char*>(device_scratch);
    float* xd[HOST_SLOTS]; float* yd[HOST_SLOTS];
    for (int k = 0; k < HOST_SLOTS; ++k) { xd[k] = reinterpret_cast<float*>(base); base += a256(chunk_rows * in * 4); }
    for (int k = 0; k < HOST_SLOTS; ++k) { yd[k] = reinterpret_cast<float*>(base); base += a256(chunk_rows * out * 4); }
    int32_t* st = reinterpret_cast<int32_t*>(base);

#define CK(call) do { if ((rc = check_cuda(call))) return rc; } while (0)
    CK(cudaMemsetAsync(st, 0, 4, cur));
    // the copy streams start after whatever the caller has queued on its stream (the packed coefficients, say)
    CK(cudaEventRecord(p->e_start, cur));
    CK(cudaStreamWaitEvent(p->s_in, p->e_start, 0));
    CK(cudaStreamWaitEvent(p->s_out, p->e_start, 0));
    // Block schedule: full blocks of chunk_rows rows, but the first and the last blocks ramp (1/8, 1/4, 1/2 of a
    // block): nothing overlaps the first block's copy in and the last block's copy out, so they are kept short.
    // CHEBYKAN_HOST_RAMP=0 in the environment switches the ramp off (uniform blocks).
    static const bool ramp_on = [] { const char* e = getenv("CHEBYKAN_HOST_RAMP"); return !(e && e[0] == '0'); }();
    const bool ramp = ramp_on && B >= 4 * chunk_rows && chunk_rows >= 1024;
    const int64_t ramp_rows = ramp ? chunk_rows / 8 + chunk_rows / 4 + chunk_rows / 2 : 0;
    auto block_rows = [&](int64_t b) -> int64_t {       // rows of the block that starts at row b
        if (ramp && b < ramp_rows) return b == 0 ? chunk_rows / 8 : (b == chunk_rows / 8 ? chunk_rows / 4 : chunk_rows / 2);
        const int64_t body_end = B - ramp_rows;
        if (b < body_end) return (body_end - b < chunk_rows) ? body_end - b : chunk_rows;
        const int64_t t = b - body_end;                 // inside the tail: 1/2, 1/4, 1/8 of a block
        return t == 0 ? chunk_rows / 2 : (t == chunk_rows / 2 ? chunk_rows / 4 : B - b);
    };
    int64_t n_chunks = 0;
    for (int64_t b = 0; b < B; ++n_chunks) {
        const int64_t k = n_chunks;
        const int64_t rows = block_rows(b);
        const int slot = (int)(k % HOST_SLOTS);
        if (k >= HOST_SLOTS) CK(cudaStreamWaitEvent(p->s_in, p->e_free_x[slot], 0));    // the block that last used this buffer has been computed
        CK(cudaMemcpyAsync(xd[slot], x_host + b * in, rows * in * 4, cudaMemcpyHostToDevice, p->s_in));
        CK(cudaEventRecord(p->e_in[slot], p->s_in));
        CK(cudaStreamWaitEvent(cur, p->e_in[slot], 0));
        if (k >= HOST_SLOTS) CK(cudaStreamWaitEvent(cur, p->e_free_y[slot], 0));        // the block that last used this buffer has been copied back
        if ((rc = chebykan_fwd(xd[slot], packed, yd[slot], rows, in, out, deg, mode, st, stream))) return rc;
        CK(cudaEventRecord(p->e_cmp[slot], cur));
        CK(cudaEventRecord(p->e_free_x[slot], cur));
        CK(cudaStreamWaitEvent(p->s_out, p->e_cmp[slot], 0));
        CK(cudaMemcpyAsync(y_host + b * out, yd[slot], rows * out * 4, cudaMemcpyDeviceToHost, p->s_out));
        CK(cudaEventRecord(p->e_free_y[slot], p->s_out));
        b += rows;
    }
    // the caller's stream ends after the last copy back
    for (int64_t k = n_chunks - 1; k >= 0 && k > n_chunks - 1 - HOST_SLOTS; --k)
        CK(cudaStreamWaitEvent(cur, p->e_free_y[k % HOST_SLOTS], 0));
    int32_t st_host = 0;
    CK(cudaMemcpyAsync(&st_host, st, 4, cudaMemcpyDeviceToHost, cur));
    CK(cudaStreamSynchronize(cur));
#undef CK
    return st_host ? CHEBYKAN_ETIMEOUT : CHEBYKAN_OK;
}

}  // extern "C"
