// FP32 backward kernels on the FFMA pipe.
//
// The reference has no hand-written backward; these are the closed forms of
// what autograd derives from kan/basis/chebyshev.py:78-145:
//   dC[i,o,d] = sum_b T_d(t_bi) dY[b,o]
//   dx[b,i]   = (1 - t^2) sum_d d U_{d-1}(t) sum_o dY[b,o] C[i,o,d],  t = tanh x[b,i]
// Both kernels index the contraction "input-major" (kk = ii*(deg+1) + d for the
// TI inputs a CTA owns), which is the coefficient tensor's own memory order, so
// neither needs a packed copy of the coefficients.
#include <mutex>
#include "common.cuh"

namespace chebykan {

constexpr int BWD_KK = 128;  // flattened (input, degree) slots per CTA tile

// number of inputs whose (deg+1) slots fit one tile
static inline int tile_inputs(int64_t in, int dp1) {
    int ti = BWD_KK / dp1;
    if (ti > in) ti = (int)in;
    return ti;
}

// ---------------------------------------------------------------------------
// dC: tile = (TI inputs x all degrees) x BN outputs, contraction over a slice of
// the batch, 8 rows per stage.  Partial sums of the batch slices go to the
// workspace and are added up by dcoeff_reduce_kernel in a fixed order.
// ---------------------------------------------------------------------------
template <int G_N, class REC>
__global__ void __launch_bounds__(256)
dcoeff_ffma_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                   float* __restrict__ dst, int64_t B, int in, int out, int dp1, int TI,
                   int i_tiles, int n_tiles, int64_t rows_per_split, int64_t split_stride,
                   int add_to_dst, const __grid_constant__ REC rec) {
    constexpr int BN = 64 * G_N;
    constexpr int LDA = BWD_KK + 4;
    constexpr int MAXP = 4;  // (row, input) pairs per thread per stage: 8*TI <= 1024
    constexpr int DV = (8 * BN / 4 + 255) / 256;
    __shared__ __align__(16) float As[2][8][LDA];
    __shared__ __align__(16) float Bs[2][8][BN];

    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    int bid = blockIdx.x;
    const int n_t = bid % n_tiles; bid /= n_tiles;
    const int i_t = bid % i_tiles; bid /= i_tiles;
    const int split = bid;
    const int i0 = i_t * TI, n0 = n_t * BN;
    const int ti = min(TI, in - i0);
    const int64_t b_begin = (int64_t)split * rows_per_split;
    const int64_t b_end = min(B, b_begin + rows_per_split);
    const int S = (int)((b_end - b_begin + 7) / 8);
    const int npairs = 8 * ti;
    const bool vec = (out & 3) == 0;

    // slots past ti*dp1 are never written: clear both buffers once
    for (int e = tid; e < 2 * 8 * LDA; e += 256) (&As[0][0][0])[e] = 0.f;
    __syncthreads();

    float acc[8][4 * G_N];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4 * G_N; ++j) acc[i][j] = 0.f;

    float xreg[MAXP];
    float4 dreg[DV];

    auto load_stage = [&](int s) {
        const int64_t b0 = b_begin + (int64_t)s * 8;
#pragma unroll
        for (int j = 0; j < MAXP; ++j) {
            const int p = tid + j * 256;
            float v = 0.f;
            if (p < npairs && s < S) {
                const int bb = p / ti, ii = p % ti;
                if (b0 + bb < b_end) v = x[(b0 + bb) * in + i0 + ii];
            }
            xreg[j] = v;
        }
#pragma unroll
        for (int v = 0; v < DV; ++v) {
            const int idx = tid + v * 256;
            float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
            if (idx < 8 * BN / 4 && s < S) {
                const int bb = idx / (BN / 4), col = n0 + (idx % (BN / 4)) * 4;
                const int64_t row = b0 + bb;
                if (row < b_end) {
                    const float* src = dy + row * out + col;
                    if (vec && col + 3 < out) r = *reinterpret_cast<const float4*>(src);
                    else {
                        if (col < out) r.x = src[0];
                        if (col + 1 < out) r.y = src[1];
                        if (col + 2 < out) r.z = src[2];
                        if (col + 3 < out) r.w = src[3];
                    }
                }
            }
            dreg[v] = r;
        }
    };
    // rows beyond b_end carry x = 0 -> a non-zero basis value, but their dY row is zero
    auto generate = [&](int buf) {
#pragma unroll
        for (int j = 0; j < MAXP; ++j) {
            const int p = tid + j * 256;
            if (p < npairs) {
                const int bb = p / ti, ii = p % ti;
                const float u = rec.normalize(xreg[j]);
                const float c = rec.carry(u);
                float* dstA = &As[buf][bb][ii * dp1];
                float tm1 = 1.f, tm2 = rec.before_first(u);
                dstA[0] = 1.f;
                for (int d = 1; d < dp1; ++d) {
                    const float v = rec.next(d, c, tm1, tm2);
                    dstA[d] = v; tm2 = tm1; tm1 = v;
                }
            }
        }
#pragma unroll
        for (int v = 0; v < DV; ++v) {
            const int idx = tid + v * 256;
            if (idx < 8 * BN / 4)
                *reinterpret_cast<float4*>(&Bs[buf][idx / (BN / 4)][(idx % (BN / 4)) * 4]) = dreg[v];
        }
    };

    load_stage(0);
    generate(0);
    load_stage(1);
    __syncthreads();

    for (int s = 0; s < S; ++s) {
        const int buf = s & 1;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
            float a[8], b[4 * G_N];
#pragma unroll
            for (int g = 0; g < 2; ++g) {
                const float4 v = *reinterpret_cast<const float4*>(&As[buf][kk][g * 64 + ty * 4]);
                a[4 * g] = v.x; a[4 * g + 1] = v.y; a[4 * g + 2] = v.z; a[4 * g + 3] = v.w;
            }
#pragma unroll
            for (int g = 0; g < G_N; ++g) {
                const float4 v = *reinterpret_cast<const float4*>(&Bs[buf][kk][g * 64 + tx * 4]);
                b[4 * g] = v.x; b[4 * g + 1] = v.y; b[4 * g + 2] = v.z; b[4 * g + 3] = v.w;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 4 * G_N; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (s + 1 < S) { generate(buf ^ 1); load_stage(s + 2); }
        __syncthreads();
    }

    float* base = dst + (int64_t)split * split_stride;
#pragma unroll
    for (int g = 0; g < 2; ++g)
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int kk = g * 64 + ty * 4 + r;
            if (kk >= ti * dp1) continue;
            const int ii = kk / dp1, d = kk % dp1;
#pragma unroll
            for (int h = 0; h < G_N; ++h)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int col = n0 + h * 64 + tx * 4 + c;
                    if (col < out) {
                        float* q = base + ((int64_t)(i0 + ii) * out + col) * dp1 + d;
                        const float v = acc[4 * g + r][4 * h + c];
                        *q = add_to_dst ? (*q + v) : v;
                    }
                }
        }
}

__global__ void __launch_bounds__(256)
dcoeff_reduce_kernel(const float* __restrict__ ws, float* __restrict__ dc, int64_t n, int splits,
                     int accumulate) {
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < n;
         e += (int64_t)gridDim.x * blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < splits; ++k) s += ws[(int64_t)k * n + e];
        dc[e] = accumulate ? dc[e] + s : s;
    }
}

int launch_dcoeff_reduce(const float* ws, float* dc, int64_t n, int splits, int accumulate, cudaStream_t s) {
    int64_t blocks = ceil_div(n, 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    dcoeff_reduce_kernel<<<(unsigned)blocks, 256, 0, s>>>(ws, dc, n, splits, accumulate);
    return check_cuda(cudaGetLastError());
}

struct DcoeffPlan { int TI, i_tiles, n_tiles, g_n, splits; int64_t rows_per_split; };

static DcoeffPlan dcoeff_plan(int64_t B, int64_t in, int64_t out, int64_t deg) {
    DcoeffPlan p{};
    const int dp1 = (int)deg + 1;
    p.TI = tile_inputs(in, dp1);
    p.i_tiles = (int)ceil_div(in, p.TI);
    p.g_n = out > 64 ? 2 : 1;
    p.n_tiles = (int)ceil_div(out, 64 * p.g_n);
    const int64_t base = (int64_t)p.i_tiles * p.n_tiles;
    int64_t splits = ceil_div(2 * 148, base);
    const int64_t max_splits = ceil_div(B, 64);     // a slice as short as 64 rows still amortises the tile setup
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    p.rows_per_split = round_up(ceil_div(B, splits), 8);
    p.splits = (int)ceil_div(B, p.rows_per_split);
    if (p.splits < 1) p.splits = 1;
    return p;
}

int64_t dcoeff_workspace_bytes(int64_t B, int64_t in, int64_t out, int64_t deg, int mode) {
    if (mode == CHEBYKAN_MODE_FP32X3 && dcoeff_tc_supported(B, in, out, deg) &&
        x3_backward_on_tensor_cores(B, in, out, deg))
        return dcoeff_tc_workspace_bytes(B, in, out, deg, 1);
    if (mode != CHEBYKAN_MODE_FP32 && mode != CHEBYKAN_MODE_FP32X3 && dcoeff_tc_supported(B, in, out, deg))
        return dcoeff_tc_workspace_bytes(B, in, out, deg);
    const DcoeffPlan p = dcoeff_plan(B, in, out, deg);
    return p.splits > 1 ? (int64_t)p.splits * in * out * (deg + 1) * 4 : 0;
}

template <class REC>
static int launch_dcoeff_ffma_rec(const float* x, const float* dy, float* dc, void* ws, int64_t ws_bytes,
                                  int64_t B, int64_t in, int64_t out, int64_t deg, int accumulate,
                                  cudaStream_t s, const REC& rec) {
    const DcoeffPlan p = dcoeff_plan(B, in, out, deg);
    const int dp1 = (int)deg + 1;
    const int64_t n = in * out * dp1;
    const bool direct = p.splits == 1;
    if (!direct && (ws == nullptr || ws_bytes < (int64_t)p.splits * n * 4)) return CHEBYKAN_EWORKSPACE;
    float* dst = direct ? dc : reinterpret_cast<float*>(ws);
    const unsigned grid = (unsigned)((int64_t)p.i_tiles * p.n_tiles * p.splits);
    const int add = direct && accumulate;
    if (p.g_n == 2)
        dcoeff_ffma_kernel<2, REC><<<grid, 256, 0, s>>>(x, dy, dst, B, (int)in, (int)out, dp1, p.TI,
                                                       p.i_tiles, p.n_tiles, p.rows_per_split, n, add, rec);
    else
        dcoeff_ffma_kernel<1, REC><<<grid, 256, 0, s>>>(x, dy, dst, B, (int)in, (int)out, dp1, p.TI,
                                                       p.i_tiles, p.n_tiles, p.rows_per_split, n, add, rec);
    int rc = check_cuda(cudaGetLastError());
    if (rc) return rc;
    if (!direct) rc = launch_dcoeff_reduce(reinterpret_cast<const float*>(ws), dc, n, p.splits, accumulate, s);
    return rc;
}

int launch_dcoeff_ffma(const float* x, const float* dy, float* dc, void* ws, int64_t ws_bytes,
                       int64_t B, int64_t in, int64_t out, int64_t deg, int accumulate,
                       cudaStream_t s, const RecurrenceTable* rec) {
    if (rec == nullptr)
        return launch_dcoeff_ffma_rec(x, dy, dc, ws, ws_bytes, B, in, out, deg, accumulate, s, ChebyshevRec());
    TableRec t;
    t.t = *rec;
    return launch_dcoeff_ffma_rec(x, dy, dc, ws, ws_bytes, B, in, out, deg, accumulate, s, t);
}

// ---------------------------------------------------------------------------
// Workspace-free entry point.
//
// chebykan_bwd_dcoeff needs a caller-provided workspace whenever it splits the
// batch over several CTAs.  Some callers have no way to provide one: they are
// handed raw device pointers by a host that owns all device memory (a serving
// process that reserved the whole GPU for its own pool at start-up, a plugin
// callback in which CUDA allocation calls are forbidden, a latency-critical
// loop that cannot afford the device-wide synchronisation cudaMalloc implies).
// For them the same kernels run against a fixed scratch array that is part of
// the library image: it is reserved on every GPU that loads the library, for
// the life of the process, whether or not this entry point is ever called.
// ---------------------------------------------------------------------------
constexpr int64_t STATIC_SCRATCH_BYTES = (int64_t)16 << 20;   // 16 MiB
static __device__ __align__(256) unsigned char g_dcoeff_scratch[STATIC_SCRATCH_BYTES];

// Device address of g_dcoeff_scratch per device ordinal.  In host code the
// array's name is only a handle for the runtime, not a device address, so the
// address is looked up once per device with that device current.  The cache is
// guarded by a mutex: first calls may come from several host threads at once.
static void* g_dcoeff_scratch_addr[64] = {nullptr};
static std::mutex g_dcoeff_scratch_mutex;

static int static_scratch_address(void** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return check_cuda(e);
    if (dev < 0 || dev >= 64) return CHEBYKAN_EDEVICE;
    std::lock_guard<std::mutex> lock(g_dcoeff_scratch_mutex);
    if (g_dcoeff_scratch_addr[dev] == nullptr) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_dcoeff_scratch);
        if (e != cudaSuccess) return check_cuda(e);
        if (ptr == nullptr) return CHEBYKAN_ECUDA;
        g_dcoeff_scratch_addr[dev] = ptr;
    }
    *out = g_dcoeff_scratch_addr[dev];
    return CHEBYKAN_OK;
}

// ---------------------------------------------------------------------------
// dx: tile = 64 rows x (TI inputs x all degrees); G = dY * C^T accumulated over
// all outputs (8 per stage), then each (row, input) pair folds its deg+1 values
// of G with d*U_{d-1}(t) and the tanh derivative.
// ---------------------------------------------------------------------------
template <class REC>
__global__ void __launch_bounds__(256)
dx_ffma_kernel(const float* __restrict__ x, const float* __restrict__ dy,
               const float* __restrict__ coeffs, float* __restrict__ dx, int64_t B, int in,
               int out, int dp1, int TI, int i_tiles, const __grid_constant__ REC rec) {
    constexpr int BM = 64;
    constexpr int LDA = BM + 4;
    constexpr int LDG = BWD_KK + 1;
    __shared__ __align__(16) float As[2][8][LDA];     // dY^T: [o][row]
    __shared__ __align__(16) float Bs[2][8][BWD_KK];  // C:    [o][kk]
    __shared__ float Gs[BM][LDG];

    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int i_t = blockIdx.x % i_tiles;
    const int64_t m0 = (int64_t)(blockIdx.x / i_tiles) * BM;
    const int i0 = i_t * TI;
    const int ti = min(TI, in - i0);
    const int S = (out + 7) / 8;

    // loader roles, fixed for the whole kernel
    const int a_oo = tid & 7, a_r = tid >> 3;          // dY: rows a_r, a_r+32
    const int b_kk = tid & 127, b_o = tid >> 7;        // C:  outputs b_o + 2j
    const bool b_valid = b_kk < ti * dp1;
    const int64_t b_base = b_valid
        ? ((int64_t)(i0 + b_kk / dp1) * out) * dp1 + (b_kk % dp1) : 0;

    float acc[4][8];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

    float areg[2], breg[4];
    auto load_stage = [&](int s) {
        const int o0 = s * 8;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int64_t row = m0 + a_r + 32 * j;
            const int o = o0 + a_oo;
            areg[j] = (row < B && o < out && s < S) ? dy[row * out + o] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int o = o0 + b_o + 2 * j;
            breg[j] = (b_valid && o < out && s < S) ? coeffs[b_base + (int64_t)o * dp1] : 0.f;
        }
    };
    auto commit = [&](int buf) {
#pragma unroll
        for (int j = 0; j < 2; ++j) As[buf][a_oo][a_r + 32 * j] = areg[j];
#pragma unroll
        for (int j = 0; j < 4; ++j) Bs[buf][b_o + 2 * j][b_kk] = breg[j];
    };

    load_stage(0);
    commit(0);
    load_stage(1);
    __syncthreads();

    for (int s = 0; s < S; ++s) {
        const int buf = s & 1;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
            float a[4], b[8];
            {
                const float4 v = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 4]);
                a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w;
            }
#pragma unroll
            for (int g = 0; g < 2; ++g) {
                const float4 v = *reinterpret_cast<const float4*>(&Bs[buf][kk][g * 64 + tx * 4]);
                b[4 * g] = v.x; b[4 * g + 1] = v.y; b[4 * g + 2] = v.z; b[4 * g + 3] = v.w;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (s + 1 < S) { commit(buf ^ 1); load_stage(s + 2); }
        __syncthreads();
    }

#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int g = 0; g < 2; ++g)
#pragma unroll
            for (int c = 0; c < 4; ++c) Gs[ty * 4 + r][g * 64 + tx * 4 + c] = acc[r][4 * g + c];
    __syncthreads();

    for (int p = tid; p < BM * ti; p += 256) {
        const int bb = p / ti, ii = p % ti;
        const int64_t row = m0 + bb;
        if (row >= B) continue;
        const float* g = &Gs[bb][ii * dp1];
        if constexpr (REC::kChebyshev) {
            const float t = tanh_exact(x[row * in + i0 + ii]);
            const float t2 = 2.f * t;
            float um1 = 1.f, um2 = 0.f, sum = 0.f;  // U_0 = 1, U_{-1} = 0
            for (int d = 1; d < dp1; ++d) {
                sum = fmaf((float)d * um1, g[d], sum);   // T_d' = d U_{d-1}
                const float u = fmaf(t2, um1, -um2);
                um2 = um1; um1 = u;
            }
            dx[row * in + i0 + ii] = fmaf(-t, t, 1.f) * sum;
        } else {
            // P_d and dP_d/du side by side from the recurrence and its derivative
            const float u = rec.normalize(x[row * in + i0 + ii]);
            float pm1 = 1.f, pm2 = 0.f, dpm1 = 0.f, dpm2 = 0.f, sum = 0.f;
            for (int d = 1; d < dp1; ++d) {
                const float dp = rec.dnext(d, u, pm1, dpm1, dpm2);
                const float p = rec.next(d, u, pm1, pm2);
                sum = fmaf(dp, g[d], sum);
                pm2 = pm1; pm1 = p; dpm2 = dpm1; dpm1 = dp;
            }
            dx[row * in + i0 + ii] = rec.dnormalize(u) * sum;
        }
    }
}

int launch_dx_ffma(const float* x, const float* dy, const float* coeffs, float* dx, int64_t B,
                   int64_t in, int64_t out, int64_t deg, cudaStream_t s, const RecurrenceTable* rec) {
    const int dp1 = (int)deg + 1;
    const int TI = tile_inputs(in, dp1);
    const int i_tiles = (int)ceil_div(in, TI);
    const int64_t grid = ceil_div(B, 64) * i_tiles;
    if (grid > 0x7fffffffLL) return CHEBYKAN_EUNSUPPORTED;
    if (rec == nullptr) {
        dx_ffma_kernel<ChebyshevRec><<<(unsigned)grid, 256, 0, s>>>(x, dy, coeffs, dx, B, (int)in, (int)out, dp1, TI,
                                                                    i_tiles, ChebyshevRec());
    } else {
        TableRec t;
        t.t = *rec;
        dx_ffma_kernel<TableRec><<<(unsigned)grid, 256, 0, s>>>(x, dy, coeffs, dx, B, (int)in, (int)out, dp1, TI,
                                                                i_tiles, t);
    }
    return check_cuda(cudaGetLastError());
}

}  // namespace chebykan

// Declared in include/chebykan_b200.h.  Same result as chebykan_bwd_dcoeff (same
// kernels, same batch split, same summation order), no workspace argument.
extern "C" int chebykan_bwd_dcoeff_static(const float* x, const float* dy, float* dcoeffs, int64_t B,
                                          int64_t in, int64_t out, int64_t deg, int accumulate,
                                          void* stream) {
    using namespace chebykan;
    if (B < 0 || in < 1 || out < 1 || deg < 0 || deg > 127 || in > (1 << 20) || out > (1 << 20) ||
        B > ((int64_t)1 << 31) || in * (deg + 1) > ((int64_t)1 << 24) || !dcoeffs)
        return CHEBYKAN_EINVAL;
    if (!aligned16(dcoeffs)) return CHEBYKAN_EALIGN;
    cudaStream_t s = (cudaStream_t)stream;
    if (B == 0) {
        if (!accumulate) return check_cuda(cudaMemsetAsync(dcoeffs, 0, in * out * (deg + 1) * 4, s));
        return CHEBYKAN_OK;
    }
    if (!x || !dy) return CHEBYKAN_EINVAL;
    if (!aligned16(x) || !aligned16(dy)) return CHEBYKAN_EALIGN;
    int rc = check_device();        // same device rule as every other entry point: compute capability 10.x only
    if (rc) return rc;
    // the partial sums of every batch slice must fit the fixed array
    const int64_t need = dcoeff_workspace_bytes(B, in, out, deg, CHEBYKAN_MODE_FP32);
    if (need > STATIC_SCRATCH_BYTES) return CHEBYKAN_ESTATIC;
    void* scratch = nullptr;
    rc = static_scratch_address(&scratch);
    if (rc) return rc;
    // Every slice's tile overwrites its whole part of the scratch before the
    // reduction reads it, so nothing left by an earlier call needs clearing.
    return launch_dcoeff_ffma(x, dy, dcoeffs, scratch, STATIC_SCRATCH_BYTES, B, in, out, deg, accumulate, s);
}
