// FP32 forward: y[b,o] = sum_i sum_d C[i,o,d] T_d(tanh x[b,i]) on the FFMA pipe.
//
// Replaces reference kan/basis/chebyshev.py:92-101,119-145 (tanh, basis
// expansion, einsum) with one kernel.  A CTA owns a BM x BN tile of y.  The
// contraction index runs degree-major inside blocks of 8 inputs: one stage is
// one degree d of 8 inputs, so every thread carries the three-term recurrence
// T_d = 2t T_{d-1} - T_{d-2} for its few (row, input) pairs in registers and
// emits the next basis column straight into shared memory.  The basis tensor
// never exists in device memory.  W is the packed fp32 matrix Wf[K_pad][N_pad].
//
// Small batches leave most SMs without a tile while each tile runs through the whole contraction.
// The KSPLIT variant launches a thread-block cluster per tile: the CTAs of a cluster split the
// input blocks among themselves, park their partial tiles in shared memory and add them up through
// distributed shared memory in rank order (so the result does not depend on timing).
#include "common.cuh"

namespace chebykan {

// two CTAs per SM (<= 128 registers): the second CTA covers the first one's FFMA and LDS latency
__device__ __forceinline__ uint32_t ffma_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t ffma_cluster_size() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void ffma_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_peer_smem(const float* local, uint32_t rank) {
    uint32_t addr = (uint32_t)__cvta_generic_to_shared(local), peer;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer) : "r"(addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(peer) : "memory");
    return v;
}

template <int G_M, int G_N, bool KSPLIT, class REC>
__global__ void __launch_bounds__(256, 2)
fwd_ffma_kernel(const float* __restrict__ x, const float* __restrict__ wf, float* __restrict__ y,
                int64_t B, int in, int out, int dp1, int n_pad, int n_tiles, const __grid_constant__ REC rec) {
    constexpr int BM = 64 * G_M, BN = 64 * G_N;
    constexpr int LDA = BM + 4;         // +4 keeps the producer's stores bank-conflict free
    constexpr int EPT = BM / 32;        // (row, input) pairs per thread per stage
    constexpr int WV = (8 * BN / 4 + 255) / 256;  // float4 W loads per thread per stage
    __shared__ __align__(16) float As[2][8][LDA];
    __shared__ __align__(16) float Bs[2][8][BN];

    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const uint32_t crank = KSPLIT ? ffma_cluster_rank() : 0u;
    const uint32_t csize = KSPLIT ? ffma_cluster_size() : 1u;
    const unsigned tile = KSPLIT ? blockIdx.x / csize : blockIdx.x;
    const int64_t m0 = (int64_t)(tile / n_tiles) * BM;
    const int n0 = (int)(tile % n_tiles) * BN;

    const int p_ii = tid & 7;   // producer: input inside the block of 8
    const int p_r = tid >> 3;   // producer: first row (then +32 per pair)

    const int n_iblk = (in + 7) / 8;
    // stages [S0, S): this CTA's share of the input blocks (all of them without KSPLIT)
    const int S0 = KSPLIT ? (int)((int64_t)n_iblk * crank / csize) * dp1 : 0;
    const int S = KSPLIT ? (int)((int64_t)n_iblk * (crank + 1) / csize) * dp1 : n_iblk * dp1;

    float acc[4 * G_M][4 * G_N];
#pragma unroll
    for (int i = 0; i < 4 * G_M; ++i)
#pragma unroll
        for (int j = 0; j < 4 * G_N; ++j) acc[i][j] = 0.f;

    float tt[EPT], tm1[EPT], tm2[EPT], xpre[EPT], phi[EPT];
    float4 wreg[WV];

    auto load_x = [&](int iblk) {
        const int i = iblk * 8 + p_ii;
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            const int64_t row = m0 + p_r + 32 * j;
            xpre[j] = (row < B && i < in && iblk * dp1 < S) ? x[row * in + i] : 0.f;
        }
    };
    // next basis column of stage s into registers (phi) and its W rows into wreg
    auto produce = [&](int s) {
        const int d = s % dp1;
        if (d == 0) {
#pragma unroll
            for (int j = 0; j < EPT; ++j) {
                const float u = rec.normalize(xpre[j]);
                tt[j] = rec.carry(u); tm1[j] = 1.f; tm2[j] = rec.before_first(u);   // Chebyshev: T_0 = 1, T_{-1} = T_1 = t
                phi[j] = 1.f;
            }
            load_x(s / dp1 + 1);
        } else {
#pragma unroll
            for (int j = 0; j < EPT; ++j) {
                phi[j] = rec.next(d, tt[j], tm1[j], tm2[j]);
                tm2[j] = tm1[j]; tm1[j] = phi[j];
            }
        }
#pragma unroll
        for (int v = 0; v < WV; ++v) {
            const int idx = tid + v * 256;
            if (idx < 8 * BN / 4) {
                const int kk = idx / (BN / 4), c4 = idx % (BN / 4);
                wreg[v] = *reinterpret_cast<const float4*>(wf + ((int64_t)s * 8 + kk) * n_pad + n0 + c4 * 4);
            }
        }
    };
    auto commit = [&](int buf) {
#pragma unroll
        for (int j = 0; j < EPT; ++j) As[buf][p_ii][p_r + 32 * j] = phi[j];
#pragma unroll
        for (int v = 0; v < WV; ++v) {
            const int idx = tid + v * 256;
            if (idx < 8 * BN / 4) {
                const int kk = idx / (BN / 4), c4 = idx % (BN / 4);
                *reinterpret_cast<float4*>(&Bs[buf][kk][c4 * 4]) = wreg[v];
            }
        }
    };

    if (S0 < S) {
        load_x(S0 / dp1);
        produce(S0);
        commit(S0 & 1);
    }
    __syncthreads();

    for (int s = S0; s < S; ++s) {
        const int buf = s & 1;
        if (s + 1 < S) produce(s + 1);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
            float a[4 * G_M], b[4 * G_N];
#pragma unroll
            for (int g = 0; g < G_M; ++g) {
                const float4 v = *reinterpret_cast<const float4*>(&As[buf][kk][g * 64 + ty * 4]);
                a[4 * g] = v.x; a[4 * g + 1] = v.y; a[4 * g + 2] = v.z; a[4 * g + 3] = v.w;
            }
#pragma unroll
            for (int g = 0; g < G_N; ++g) {
                const float4 v = *reinterpret_cast<const float4*>(&Bs[buf][kk][g * 64 + tx * 4]);
                b[4 * g] = v.x; b[4 * g + 1] = v.y; b[4 * g + 2] = v.z; b[4 * g + 3] = v.w;
            }
#pragma unroll
            for (int i = 0; i < 4 * G_M; ++i)
#pragma unroll
                for (int j = 0; j < 4 * G_N; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (s + 1 < S) commit(buf ^ 1);
        __syncthreads();
    }

    if (KSPLIT) {
        // partial tile -> shared memory; every CTA then sums its rows' partials over all ranks in rank
        // order and writes them; nobody leaves while a peer may still read its shared memory
        __shared__ float red[BM][BN + 1];
#pragma unroll
        for (int r = 0; r < 4 * G_M; ++r)
#pragma unroll
            for (int c = 0; c < 4 * G_N; ++c)
                red[(r / 4) * 64 + ty * 4 + (r & 3)][(c / 4) * 64 + tx * 4 + (c & 3)] = acc[r][c];
        ffma_cluster_sync();
        const int rows_per = (BM + (int)csize - 1) / (int)csize;
        const int r_begin = (int)crank * rows_per, r_end = min(BM, r_begin + rows_per);
        for (int e = r_begin * BN + tid; e < r_end * BN; e += 256) {
            const int r = e / BN, c = e % BN;
            float v = 0.f;
            for (uint32_t q = 0; q < csize; ++q) v += ld_peer_smem(&red[r][c], q);
            const int64_t row = m0 + r;
            const int col = n0 + c;
            if (row < B && col < out) y[row * out + col] = v;
        }
        ffma_cluster_sync();
        return;
    }
    const bool vec = (out & 3) == 0;
#pragma unroll
    for (int g = 0; g < G_M; ++g)
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int64_t row = m0 + g * 64 + ty * 4 + r;
            if (row >= B) continue;
#pragma unroll
            for (int h = 0; h < G_N; ++h) {
                const int col = n0 + h * 64 + tx * 4;
                float* dst = y + row * out + col;
                const float* v = &acc[4 * g + r][4 * h];
                if (vec && col + 3 < out) {
                    *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
                } else {
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        if (col + c < out) dst[c] = v[c];
                }
            }
        }
}

template <class REC>
static int launch_fwd_ffma_rec(const float* x, const float* wf, float* y, int64_t B, int64_t in, int64_t out,
                               int64_t deg, cudaStream_t s, const REC& rec) {
    const PackedDims p = packed_dims(in, out, deg, CHEBYKAN_MODE_FP32);
    const int dp1 = (int)deg + 1;
    const bool wide = (p.n_pad % 128) == 0;
    // 128-row tiles once they still give every SM a few CTAs; 64-row tiles otherwise
    const int64_t tiles128 = ceil_div(B, 128) * (p.n_pad / (wide ? 128 : 64));
    if (tiles128 >= 2 * 148) {
        if (wide) {
            const int nt = (int)(p.n_pad / 128);
            fwd_ffma_kernel<2, 2, false, REC><<<(unsigned)(ceil_div(B, 128) * nt), 256, 0, s>>>(
                x, wf, y, B, (int)in, (int)out, dp1, (int)p.n_pad, nt, rec);
        } else {
            const int nt = (int)(p.n_pad / 64);
            fwd_ffma_kernel<2, 1, false, REC><<<(unsigned)(ceil_div(B, 128) * nt), 256, 0, s>>>(
                x, wf, y, B, (int)in, (int)out, dp1, (int)p.n_pad, nt, rec);
        }
    } else {
        const int nt = (int)(p.n_pad / 64);
        const int64_t tiles = ceil_div(B, 64) * nt;
        // few tiles and a long contraction: split the input blocks over a cluster per tile (2, 4 or 8 CTAs)
        const int64_t n_iblk = ceil_div(in, 8);
        int ks = 1;
        while (ks < 8 && tiles * ks * 2 <= 2 * 148 && n_iblk >= 4 * ks) ks *= 2;   // up to two CTAs per SM
        if (ks > 1) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((unsigned)(tiles * ks)); cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = 0; cfg.stream = s;
            cudaLaunchAttribute attrs[1];
            attrs[0].id = cudaLaunchAttributeClusterDimension;
            attrs[0].val.clusterDim.x = (unsigned)ks; attrs[0].val.clusterDim.y = 1; attrs[0].val.clusterDim.z = 1;
            cfg.attrs = attrs; cfg.numAttrs = 1;
            return check_cuda(cudaLaunchKernelEx(&cfg, fwd_ffma_kernel<1, 1, true, REC>, x, wf, y, B, (int)in, (int)out, dp1,
                                                 (int)p.n_pad, nt, rec));
        }
        fwd_ffma_kernel<1, 1, false, REC><<<(unsigned)tiles, 256, 0, s>>>(
            x, wf, y, B, (int)in, (int)out, dp1, (int)p.n_pad, nt, rec);
    }
    return check_cuda(cudaGetLastError());
}

int launch_fwd_ffma(const float* x, const float* wf, float* y, int64_t B, int64_t in, int64_t out,
                    int64_t deg, cudaStream_t s, const RecurrenceTable* rec) {
    if (rec == nullptr) return launch_fwd_ffma_rec(x, wf, y, B, in, out, deg, s, ChebyshevRec());
    TableRec t;
    t.t = *rec;
    return launch_fwd_ffma_rec(x, wf, y, B, in, out, deg, s, t);
}

}  // namespace chebykan
