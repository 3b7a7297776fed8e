/*
 * chebykan_b200 — C ABI of the B200 (sm_100a) ChebyKAN layer hot path.
 *
 * The layer computes  y[b,o] = sum_i sum_d C[i,o,d] * T_d(tanh(x[b,i]))
 * (T_d = Chebyshev polynomial of the first kind) and its gradients.  The
 * reference project (0xEodum/KAN) implements this path in Python on top of
 * PyTorch; it has no FFI of its own, so every entry point below cites the
 * reference lines whose work it replaces (paths inside that project).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless its name ends in _host;
 *   - x, y, dy, dx are row-major fp32: x[B][in], y[B][out];
 *   - coeffs / dcoeffs use the parameter's own layout [in][out][deg+1] fp32;
 *   - `stream` is a cudaStream_t passed as void* (NULL = default stream);
 *   - all launches are asynchronous on `stream`; nothing synchronises;
 *   - return value: 0 on success, a negative CHEBYKAN_E* code otherwise
 *     (no exception ever crosses this boundary);
 *   - the library allocates no device memory: callers own every buffer
 *     (sizes from chebykan_packed_bytes / chebykan_workspace_bytes).
 */
#ifndef CHEBYKAN_B200_H_
#define CHEBYKAN_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CHEBYKAN_ABI_VERSION 7

/* error codes */
#define CHEBYKAN_OK            0
#define CHEBYKAN_EINVAL       -1  /* bad shape / null pointer / bad enum            */
#define CHEBYKAN_EALIGN       -2  /* pointer not 16-byte aligned                    */
#define CHEBYKAN_EUNSUPPORTED -3  /* shape outside what this mode's kernel handles  */
#define CHEBYKAN_ECUDA        -4  /* CUDA runtime error (see chebykan_last_cuda_error) */
#define CHEBYKAN_ETIMEOUT     -5  /* a bounded device-side wait gave up             */
#define CHEBYKAN_EWORKSPACE   -6  /* workspace / packed buffer too small            */
#define CHEBYKAN_EDEVICE      -7  /* current device is not compute capability 10.x  */
#define CHEBYKAN_ESTATIC      -8  /* problem needs more than the built-in 16 MiB scratch */

/* arithmetic mode of the contraction */
#define CHEBYKAN_MODE_FP32 0  /* fp32 FFMA on CUDA cores, correctly rounded tanh   */
#define CHEBYKAN_MODE_TF32 1  /* tcgen05 kind::tf32 (narrow layers: fp16 operands,   */
                              /* the same 11 bits), fp32 accumulate in TMEM        */
#define CHEBYKAN_MODE_BF16 2  /* tcgen05 kind::f16 (bf16 x bf16), fp32 accumulate  */
/* fp32-grade forward on the tensor cores: basis values and coefficients are each
 * split into a tf32 head and a tf32 tail and three tcgen05 kind::tf32 products
 * (head*head, head*tail, tail*head) are accumulated in fp32, with the library's
 * single-precision tanh (2 ulp).  Same 1e-5 tolerance as CHEBYKAN_MODE_FP32.  The
 * backward entry points do the same for large products (the tf32 kernels run
 * three times on heads and tails, over short batch slices for dC; their
 * workspace then also holds the tails of dY and, for dC, one partial result per
 * 1536 batch rows) and run their fp32 kernels for small ones and for dx with
 * more than 2048 outputs. */
#define CHEBYKAN_MODE_FP32X3 3

/* operations that may need a caller-provided workspace */
#define CHEBYKAN_OP_FWD        0
#define CHEBYKAN_OP_BWD_DCOEFF 1
#define CHEBYKAN_OP_BWD_DX     2

int         chebykan_abi_version(void);
const char* chebykan_strerror(int code);
/* cudaError_t of the most recent CHEBYKAN_ECUDA on the calling thread */
int         chebykan_last_cuda_error(void);

/*
 * Packed coefficient matrix for one mode.
 * Replaces the permute + copy that torch.einsum performs on the coefficient
 * tensor before its bmm (kan/basis/chebyshev.py:101).  The packed layout is
 * private to the library; it is rebuilt after every optimizer step.
 */
int64_t chebykan_packed_bytes(int64_t in, int64_t out, int64_t deg, int mode);
int chebykan_pack_coeffs(const float* coeffs, void* packed,
                         int64_t in, int64_t out, int64_t deg, int mode,
                         void* stream);

/* bytes of caller-owned workspace an operation needs (0 = none, <0 = error) */
int64_t chebykan_workspace_bytes(int op, int64_t B, int64_t in, int64_t out,
                                 int64_t deg, int mode);

/*
 * Forward.  Replaces ChebyKANLayer.forward -> ChebyshevBasis.forward
 * (kan/layers/chebykan.py:53-67, kan/basis/chebyshev.py:80-145): tanh,
 * basis expansion and einsum('bid,iod->bo') in one fused kernel; the basis
 * tensor never exists in device memory.  `packed` comes from
 * chebykan_pack_coeffs with the same (in, out, deg, mode).
 * `status` is a device int32 the kernel sets non-zero if a bounded wait gave
 * up (tensor-core modes; may be NULL in FP32 mode).
 */
int chebykan_fwd(const float* x, const void* packed, float* y,
                 int64_t B, int64_t in, int64_t out, int64_t deg, int mode,
                 int32_t* status, void* stream);

/*
 * Forward with the LayerNorm that sits between two ChebyKAN layers of a stack
 * fused in (tensor-core modes only; FP32 mode returns CHEBYKAN_EUNSUPPORTED).
 * The reference chains layers through torch.nn.LayerNorm modules in a
 * Sequential (kan/layers/base.py:144-153); each LayerNorm costs a read and a
 * write of the whole activation.  Here
 *   - ln_stats_out (nullable, float[B][2], zeroed by the caller): the kernel adds
 *     each produced row's sum and sum of squares of y;
 *   - ln_stats_in / ln_gamma / ln_beta / ln_eps (stats nullable): the kernel
 *     normalises its input rows, x' = (x - mean) * rstd * gamma + beta with
 *     mean and rstd from the previous layer's sums over `in` features, before tanh.
 * So y of layer k is written once, un-normalised, and layer k+1 applies the
 * LayerNorm while it loads it.
 */
int chebykan_fwd_ln(const float* x, const void* packed, float* y,
                    int64_t B, int64_t in, int64_t out, int64_t deg, int mode,
                    const float* ln_stats_in, const float* ln_gamma,
                    const float* ln_beta, float ln_eps, float* ln_stats_out,
                    int32_t* status, void* stream);

/*
 * Coefficient gradient dC[i,o,d] = sum_b T_d(tanh x[b,i]) * dY[b,o].
 * Replaces the dW half of autograd's BmmBackward plus the permute back to
 * [in,out,deg+1] (backward of kan/basis/chebyshev.py:101,119-145).
 * accumulate != 0 adds into dcoeffs, otherwise dcoeffs is overwritten.
 * TF32 and BF16 modes both contract in tcgen05 kind::tf32 (bf16 operands would
 * miss the 2e-3 tolerance for this product); FP32 mode uses the FFMA pipe.
 */
int chebykan_bwd_dcoeff(const float* x, const float* dy, float* dcoeffs,
                        void* workspace, int64_t workspace_bytes,
                        int64_t B, int64_t in, int64_t out, int64_t deg,
                        int mode, int accumulate, int32_t* status, void* stream);

/*
 * chebykan_bwd_dcoeff without a workspace argument, for callers that cannot
 * allocate device memory: code that only receives raw pointers from a host
 * owning all of the GPU's memory (a server that gave the whole device to its
 * own pool, a plugin callback where CUDA allocation calls are off limits, a
 * real-time loop that must not hit cudaMalloc's implicit synchronisation).
 * It has no counterpart in the reference, which leaves all memory to PyTorch.
 *   - Scratch is a 16 MiB array built into the library; every GPU that loads
 *     the library keeps it reserved until the process exits.
 *   - Shapes whose batch-split partial sums need more than 16 MiB (what
 *     chebykan_workspace_bytes(CHEBYKAN_OP_BWD_DCOEFF, ...) reports) are
 *     refused with CHEBYKAN_ESTATIC; use chebykan_bwd_dcoeff for those.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current); make that first call
 *     outside any stream capture.  The lookup is guarded by a mutex, so first
 *     calls from several host threads are safe.  No call allocates or frees
 *     anything.  The current device must be compute capability 10.x
 *     (CHEBYKAN_EDEVICE otherwise), as for every other entry point.
 *   - All calls share the one array.  A call overwrites every byte it later
 *     reads, so leftovers of earlier calls are harmless, but two calls that
 *     may run on the GPU at the same time (different streams, different host
 *     threads) race on it: keep calls on one device in stream order.
 * This entry point always runs the fp32 FFMA kernels, whatever modes the
 * workspace variant offers; its result is bit-identical to
 * chebykan_bwd_dcoeff(..., CHEBYKAN_MODE_FP32, ...).
 */
int chebykan_bwd_dcoeff_static(const float* x, const float* dy, float* dcoeffs,
                               int64_t B, int64_t in, int64_t out, int64_t deg,
                               int accumulate, void* stream);

/*
 * Input gradient dx[b,i] = (1-t^2) * sum_d T_d'(t) * sum_o dY[b,o] C[i,o,d],
 * t = tanh x[b,i].  Replaces the dPhi half of BmmBackward and the
 * Cos/Mul/Acos/Clamp/Tanh backward chain (backward of
 * kan/basis/chebyshev.py:78,136-145).  Where tanh saturates to exactly +-1
 * the reference produces NaN (0 * inf); this library returns 0 there.
 * Reads the coefficients in their own [in][out][deg+1] layout.  The tensor-core
 * modes repack them into `workspace` on every call
 * (chebykan_workspace_bytes(CHEBYKAN_OP_BWD_DX, ...) bytes; 0 in FP32 mode).
 * TF32 mode contracts in tcgen05 kind::tf32.  BF16 mode does the same on layers
 * of fewer than 512 outputs and contracts fp16 operands (tf32's 11 significant
 * bits, half the MMAs) on wider ones: the workspace then also holds a copy of dY
 * as fp16, every row scaled by a power of two taken from its largest element,
 * and the coefficients are scaled likewise; both scales are exact and undone
 * before dx is written.
 */
int chebykan_bwd_dx(const float* x, const float* dy, const float* coeffs,
                    float* dx, void* workspace, int64_t workspace_bytes,
                    int64_t B, int64_t in, int64_t out, int64_t deg,
                    int mode, int32_t* status, void* stream);

/*
 * Jacobian jac[b][o][i] = d y[b,o] / d x[b,i] (fp32).  Stands where the
 * reference has KANLayer.jacobian / compute_derivatives
 * (kan/layers/base.py:102-141 over kan/basis/chebyshev.py:174-267); those do
 * not return this derivative (their coefficient rule is wrong), this entry
 * point returns what autograd gives.  The output has B*out*in elements.
 */
int chebykan_jacobian(const float* x, const float* coeffs, float* jac,
                      int64_t B, int64_t in, int64_t out, int64_t deg,
                      void* stream);

/*
 * The basis object's own methods, on flat fp32 arrays of n = B*in elements:
 *   chebykan_normalize_input   t = tanh(x), correctly rounded
 *                              (ChebyshevBasis.normalize_input, kan/basis/chebyshev.py:68-78);
 *   chebykan_basis_functions   phi[e][d] = T_d(clamp(t[e], -1, 1)), d = 0..deg, by the three-term
 *                              recurrence (ChebyshevBasis.basis_functions, kan/basis/chebyshev.py:103-172);
 *                              phi has n*(deg+1) elements.
 * The layer's forward never builds phi; these serve callers that want the basis tensor itself.
 */
int chebykan_normalize_input(const float* x, float* t, int64_t n, void* stream);
int chebykan_basis_functions(const float* t, float* phi, int64_t n, int64_t deg,
                             void* stream);

/*
 * The reference's other polynomial layers have the Chebyshev layer's structure - normalise the
 * input, evaluate a three-term recurrence, contract with coefficients[in][out][deg+1] through
 * einsum('bid,iod->bo') - and run on the same fp32 kernels with the recurrence swapped:
 *   CHEBYKAN_FAMILY_JACOBI       P_d^(alpha,beta)(tanh x), alpha, beta > -1
 *                                (JacobiKANLayer / JacobiBasis, kan/layers/jacobikan.py:20-68,
 *                                 kan/basis/jacobi.py:84-188);
 *   CHEBYKAN_FAMILY_HERMITE      physicist's H_d(u),  H_{d+1} = 2u H_d - 2d H_{d-1}
 *   CHEBYKAN_FAMILY_HERMITE_PROB probabilist's He_d(u), He_{d+1} = u He_d - d He_{d-1}
 *                                (HermiteKANLayer / HermiteBasis, kan/layers/hermitekan.py:22-83,
 *                                 kan/basis/hermite.py:85-233), u = 3 tanh x, or - for a finite
 *                                 domain [lo, hi] with domain normalisation on - the affine map
 *                                 u = 6/(hi-lo) * (x - lo) - 3;
 *   CHEBYKAN_FAMILY_CHEBYSHEV    T_d(tanh x) through the same table-driven kernels (a cross-check of
 *                                them against the Chebyshev entry points above).
 * A family is described on the HOST by a chebykan_family; the library turns it into the recurrence
 * table the kernels take as a launch parameter, so there is nothing to upload or keep alive.
 * `packed` is chebykan_pack_coeffs' layout for `mode` (the packing does not depend on the family);
 * the workspaces of the two bwd functions are sized by chebykan_family_workspace_bytes(op, ..., mode).
 * Modes: CHEBYKAN_MODE_FP32 (FFMA pipe, correctly rounded tanh; status may be NULL), CHEBYKAN_MODE_TF32
 * and CHEBYKAN_MODE_BF16 (the tcgen05 kernels of chebykan_fwd / chebykan_bwd_dcoeff / chebykan_bwd_dx
 * with the family's recurrence - and, for dx, its derivative - in their producer and epilogue warps;
 * the backward contracts in tf32 in both modes; status as for the Chebyshev functions);
 * CHEBYKAN_MODE_FP32X3 returns CHEBYKAN_EUNSUPPORTED.  The reference has no hand-written backward: the
 * two bwd functions return what autograd derives from the forward.  chebykan_family_normalize / chebykan_family_basis are the basis object's
 * normalize_input / basis_functions on flat arrays of n elements (phi has n*(deg+1) elements), and
 * chebykan_family_table copies the recurrence P_d = (a[d] u + b[d]) P_{d-1} - c[d] P_{d-2}
 * (d = 1..deg, P_0 = 1, P_{-1} = 0; deg+1 floats per HOST array; entry 0 is a = 0, b = 1, c = 0)
 * for inspection.
 */
#define CHEBYKAN_FAMILY_CHEBYSHEV    0
#define CHEBYKAN_FAMILY_JACOBI       1
#define CHEBYKAN_FAMILY_HERMITE      2
#define CHEBYKAN_FAMILY_HERMITE_PROB 3

typedef struct chebykan_family {
    int32_t kind;        /* CHEBYKAN_FAMILY_*                                                   */
    float   alpha, beta; /* Jacobi parameters; ignored by the other kinds                       */
    int32_t affine;      /* 0: u = scale * tanh(x);  1: u = scale * (x - shift) + offset        */
    float   scale;       /* 0 selects the kind's default (3 for the Hermite kinds, 1 otherwise) */
    float   shift, offset;
} chebykan_family;

int chebykan_family_table(const chebykan_family* family, int64_t deg, float* a_host, float* b_host,
                          float* c_host);
int chebykan_family_fwd(const chebykan_family* family, const float* x, const void* packed, float* y,
                        int64_t B, int64_t in, int64_t out, int64_t deg, int mode, int32_t* status,
                        void* stream);
int64_t chebykan_family_workspace_bytes(int op, int64_t B, int64_t in, int64_t out, int64_t deg,
                                        int mode);
int chebykan_family_bwd_dcoeff(const chebykan_family* family, const float* x, const float* dy,
                               float* dcoeffs, void* workspace, int64_t workspace_bytes, int64_t B,
                               int64_t in, int64_t out, int64_t deg, int mode, int accumulate,
                               int32_t* status, void* stream);
int chebykan_family_bwd_dx(const chebykan_family* family, const float* x, const float* dy,
                           const float* coeffs, float* dx, void* workspace, int64_t workspace_bytes,
                           int64_t B, int64_t in, int64_t out, int64_t deg, int mode, int32_t* status,
                           void* stream);
int chebykan_family_normalize(const chebykan_family* family, const float* x, float* u, int64_t n,
                              void* stream);
int chebykan_family_basis(const chebykan_family* family, const float* u, float* phi, int64_t n,
                          int64_t deg, void* stream);

/*
 * Mean-squared-error loss and its gradient in one pass: *loss = sum (y - target)^2 / n_mean and
 * dy[e] = 2 (y[e] - target[e]) / n_mean * grad_scale, over n elements.  Replaces the
 * nn.MSELoss() forward and backward of the reference's training loop (README.md:57-69), which
 * read y and the target three times and write a temporary.  n_mean is the element count the mean
 * runs over (n on one GPU; the global count when the batch is sharded, so that the summed
 * gradients of all ranks equal the single-GPU gradient).  `workspace` holds per-block partial
 * sums (chebykan_mse_workspace_bytes() bytes); they are added in a fixed order, so the loss is
 * repeatable bit for bit.
 */
int64_t chebykan_mse_workspace_bytes(void);
int chebykan_mse_loss_grad(const float* y, const float* target, float* dy, float* loss,
                           void* workspace, int64_t workspace_bytes, int64_t n,
                           int64_t n_mean, float grad_scale, void* stream);
/*
 * dy[e] *= *scalar (a device float) unless *scalar == 1, in which case nothing is written: the
 * chain-rule factor autograd hands to the loss's backward (torch's MseLossBackward multiplies
 * unconditionally).  No other counterpart in the reference.
 */
int chebykan_scale_by_device_scalar(float* dy, const float* scalar, int64_t n, void* stream);

/*
 * Optimizer updates on a flat fp32 parameter of n elements.  Replace
 * torch.optim.SGD(lr) / torch.optim.Adam(lr) as called by the reference's
 * training loop (README.md:59-66).  grad_scale multiplies the gradient first
 * (1/world_size after a sum all-reduce).  `step` is 1-based.
 */
int chebykan_sgd_step(float* param, const float* grad, int64_t n, float lr,
                      float grad_scale, void* stream);
int chebykan_adam_step(float* param, const float* grad, float* exp_avg,
                       float* exp_avg_sq, int64_t n, float lr, float beta1,
                       float beta2, float eps, int64_t step, float grad_scale,
                       void* stream);

/*
 * Adam update whose step count lives in device memory (*step_dev = number of
 * updates already applied; the call uses step_dev + 1 and then increments it),
 * so that a training step captured in a CUDA graph can be replayed.  Same
 * replaced reference line as chebykan_adam_step (torch.optim.Adam.step,
 * README.md:59-66).
 */
int chebykan_adam_step_graph(float* param, const float* grad, float* exp_avg,
                             float* exp_avg_sq, int64_t n, float lr, float beta1,
                             float beta2, float eps, int64_t* step_dev,
                             float grad_scale, void* stream);

/*
 * One-launch training step of a single SMALL layer: forward, mean-squared-error loss, backward and the
 * optimizer update as one kernel of one CTA.  Replaces one iteration of the reference's example loop
 * (README.md:57-69: optimizer.zero_grad(); loss = MSELoss()(layer(x), target); loss.backward();
 * optimizer.step()), whose dozen microsecond-scale kernels are bound by launch overhead when each stage
 * is its own launch.  coeffs [in][out][deg+1] is updated in place; optimizer 0 = SGD (lr), 1 = Adam
 * (lr, beta1, beta2, eps; exp_avg / exp_avg_sq like coeffs, *step_dev = steps taken so far, advanced
 * by the kernel: bias corrections as torch.optim.Adam computes them).  *loss = mean((y - target)^2) of
 * the step's forward (before the update); dcoeffs_out (may be NULL) receives the gradient that was
 * applied.  fp32, tanh correctly rounded; gradient sums run over the rows in order, so a step is
 * bitwise repeatable.  chebykan_small_train_step_supported: at most 2048 coefficients, 16 outputs and
 * B * (in + out) <= 49152; other shapes return CHEBYKAN_EUNSUPPORTED.
 */
int chebykan_small_train_step_supported(int64_t B, int64_t in, int64_t out, int64_t deg);
int chebykan_small_train_step(const float* x, const float* target, float* coeffs, float* exp_avg,
                              float* exp_avg_sq, int64_t* step_dev, float* loss, float* dcoeffs_out,
                              int64_t B, int64_t in, int64_t out, int64_t deg, int optimizer, float lr,
                              float beta1, float beta2, float eps, void* stream);

/*
 * Self-test of the bounded device-side wait the tensor-core kernels use: one
 * CTA waits (at most limit_ns, <= 1 s) on an mbarrier nothing arrives on,
 * gives up, and writes `code` to the device word *status.  The context stays
 * usable.  No counterpart in the reference (it has no device code).
 */
int chebykan_selftest_bounded_wait(int32_t* status, int64_t limit_ns, int code,
                                   void* stream);

/*
 * Forward with HOST buffers: copies x and the coefficients to the device,
 * packs, runs chebykan_fwd and copies y back; synchronous.  The caller lends
 * device scratch of at least chebykan_fwd_host_scratch_bytes(...) bytes.
 * Same replaced reference lines as chebykan_fwd.
 */
int64_t chebykan_fwd_host_scratch_bytes(int64_t B, int64_t in, int64_t out,
                                        int64_t deg, int mode);
int chebykan_fwd_host(const float* x_host, const float* coeffs_host,
                      float* y_host, void* device_scratch,
                      int64_t scratch_bytes, int64_t B, int64_t in,
                      int64_t out, int64_t deg, int mode, void* stream);

/*
 * Forward with HOST x and y and device-resident packed coefficients,
 * pipelined: the batch is cut into blocks of chunk_rows rows; block k+1 is
 * copied to the device while block k is computed and block k-1 is copied
 * back, on two copy streams the library creates per device at first use, so
 * both directions of the host link work at the same time.  x_host and y_host
 * should be page-locked (the copies are synchronous otherwise).  Synchronous:
 * returns once y_host is complete.  The caller lends device scratch of at
 * least chebykan_fwd_host_packed_scratch_bytes(chunk_rows, in, out) bytes
 * (two x blocks, two y blocks, a status word).  Calls that overlap on one
 * device serialise on the library's copy streams.  Same replaced reference
 * lines as chebykan_fwd.
 */
int64_t chebykan_fwd_host_packed_scratch_bytes(int64_t chunk_rows, int64_t in,
                                               int64_t out);
int chebykan_fwd_host_packed(const float* x_host, const void* packed,
                             float* y_host, void* device_scratch,
                             int64_t scratch_bytes, int64_t B, int64_t in,
                             int64_t out, int64_t deg, int mode,
                             int64_t chunk_rows, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CHEBYKAN_B200_H_ */
