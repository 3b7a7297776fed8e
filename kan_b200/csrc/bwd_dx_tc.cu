// Tensor-core input gradient for sm_100a (tcgen05 kind::tf32):
//   dx[b,i] = (1 - t^2) * sum_d U_{d-1}(t) * G[b,(i,d)],   G = dY * Wd^T,  Wd[(i,d)][o] = d C[i,o,d],
//   t = tanh x[b,i]   (T_d' = d U_{d-1}; the factor d rides in the packed coefficients)
// i.e. the dPhi half of autograd's BmmBackward followed by the Cos/Mul/Acos/Clamp/Tanh
// backward chain of reference kan/basis/chebyshev.py:78,136-145, in one kernel: G lives only
// in TMEM and is folded with the derivative recurrence (T_d' = d U_{d-1}) by the epilogue.
//
//   A (dY):  K-major tile [128 rows][32 outputs] fp32 read as tf32, TMA, 128B swizzle.
//   B (Wd):  packed coefficients Wd[(i,d)][out_pad], d = 1..deg (slot = i*deg + d-1: degree 0 has
//            no derivative and takes no slot; outputs contiguous, rounded to tf32), K-major tile
//            [256 slots][32 outputs], TMA, 128B swizzle.
//   D (G):   128 x 256 fp32 in TMEM, two buffers: the epilogue of one tile overlaps the
//            MMAs of the other.  A tile covers TI = 256/deg inputs with all their degrees.
//   warp 0 TMA, warp 1 MMA, warps 2-17 epilogue (two groups of eight, one per accumulator; in a
//   group two warps per TMEM lane quarter, each taking half of the tile's inputs, two inputs at a
//   time; a thread owns one batch row).
// With more than 128 rows the kernel runs as CTA pairs (cluster of 2, cta_group::2): the pair
// covers 256 rows, each CTA loads the dY tile of its own 128 rows and half of the Wd tile, and
// the even CTA issues M = 256 MMAs, so every coefficient byte is fetched once per 256 rows.
// Every mbarrier wait is bounded, as in the forward kernel.
//
// fp16-operand variant (template flag H; wide layers in the bf16 mode): the same kernel with kind::f16 MMAs on
// K blocks of 64 outputs, i.e. twice the contraction per 128-byte row and half the MMAs.  fp16 carries the 11
// significant bits of tf32, so the accuracy is that of the tf32 variant; what fp16 lacks is range, and exact
// power-of-two scales supply it: one pass over dY scales every batch row by the power of two that puts the row's
// largest element into [2^14, 2^15) and writes it as fp16 (dx is linear in a row of dY, and an epilogue thread owns one
// row), the coefficient repack writes d * C * s_W with max |C| * s_W in [2^14, 2^15) / 2^ceil(log2 deg), so that the
// degree factor cannot overflow, and the epilogue multiplies each dx by its row's 1/s_b and by 1/s_W.
#include <cuda_fp16.h>
#include "tc_common.cuh"

namespace chebykan {

namespace {
using namespace tc;

constexpr int DX_TMA_WARP = 0;
constexpr int DX_MMA_WARP = 1;
constexpr int DX_EPI_WARP0 = 2;
constexpr int DX_EPI_WARPS = 16;
// The epilogue warps form one group per accumulator; group g folds the tiles that land in accumulator g, so the
// groups work on different tiles at different points of their cycle: while one waits for its TMEM loads or its
// MMAs another issues its FMAs.  With all sixteen warps on the same tile they moved through the phases in lock
// step and every stall was exposed.  Inside a group, the warps of a TMEM lane quarter share the tile's inputs.
constexpr int DX_THREADS = (2 + DX_EPI_WARPS) * 32;
constexpr int DX_BM = 128, DX_BN = 256, DX_KB = 32;   // DX_BN: the widest tile (slots per accumulator)
constexpr int DX_A_STAGE = DX_BM * 128;
constexpr int DX_KB_HALF = 64;            // outputs per K block with fp16 operands (128 bytes all the same)
constexpr int DX_HEADER = 256;            // fp16 variant's workspace header: [0] max |C| as bits, [1] 1 / s_W (float)
// BN slots per accumulator, 512 / BN accumulators, one epilogue group each.  256 is what runs: four accumulators
// of 128 slots (four groups of four warps) measured slower on the narrow layers they were meant for (0.94 against
// 0.81 ms at 1048576 x 64 -> 64, degree 32: 22 tiles per row block instead of 10, each with its own set-up, and a
// wasted half round per tile of three inputs) and re-read dY twice as often on wide ones.
// a CTA of a pair stages half of every Wd tile (a ring deeper than 4 stages measured no faster)
template <int CG, int BN>
struct DxSmem {
    static constexpr int NS = 4;
    static constexpr int NACC = 512 / BN;
    static constexpr int NUM_BARS = 2 * NS + 2 * NACC + 1;     // full, empty, acc_full[NACC], acc_empty[NACC], drain
    static constexpr int B_STAGE = BN * 128 / CG;
    static constexpr int STAGE = DX_A_STAGE + B_STAGE;
    static constexpr int BAR_OFFSET = NS * STAGE;
    static constexpr int TOTAL = BAR_OFFSET + NUM_BARS * 8 + 16 + 1024;
};

enum { XST_TMA = 21, XST_MMA_FULL = 22, XST_MMA_ACC = 23, XST_EPILOGUE = 24 };

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr) : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, uint32_t (&r)[4]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld2(uint32_t taddr, uint32_t (&r)[2]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0, %1}, [%2];"
                 : "=r"(r[0]), "=r"(r[1]) : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld1(uint32_t taddr, uint32_t& r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr) : "memory");
}

// Wd[(i,d)][out_pad] <- tf32(d * C[i][o][d]); columns o >= out are zero.  The degree factor of
// T_d' = d U_{d-1} is folded in here so that the epilogue only needs U_{d-1} * G per value.
// PART 0: rounded to tf32 (the tf32 / bf16 modes).  PART 1: head = the value truncated to tf32, and the tail
// (value - head, fp32) in a second matrix right behind the first (the fp32-grade three-product mode).
// degree_factor = 0: plain C (other polynomial families: their P_d' comes whole from the differentiated recurrence).
template <int PART>
__global__ void __launch_bounds__(256)
pack_dx_kernel(const float* __restrict__ c, uint32_t* __restrict__ wd, int in, int out, int nd, int out_pad,
               int degree_factor) {
    const int64_t total = (int64_t)in * nd * out_pad;
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total;
         e += (int64_t)gridDim.x * blockDim.x) {
        const int o = (int)(e % out_pad);
        const int64_t slot = e / out_pad;
        const int64_t i = slot / nd;
        const int d = (int)(slot % nd) + 1;          // degree 0 has no slot: its derivative is zero
        float v = 0.f;
        if (o < out) v = (degree_factor ? (float)d : 1.f) * c[(i * out + o) * (nd + 1) + d];
        if (PART == 0) {
            uint32_t r;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
            wd[e] = r;
        } else {
            const uint32_t hi = __float_as_uint(v) & 0xFFFFE000u;
            wd[e] = hi;
            wd[total + e] = __float_as_uint(v - __uint_as_float(hi));
        }
    }
}

// tail of dY for the three-product mode: dY minus dY truncated to tf32 (what the tensor pipe reads of dY itself)
__global__ void __launch_bounds__(256)
dy_tail_kernel(const float* __restrict__ dy, float* __restrict__ lo, int64_t n) {
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x) {
        const float v = dy[e];
        lo[e] = v - __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
    }
}

// ---- pre-pass of the fp16-operand variant ----------------------------------------------------------------------
// max |v| as the bit pattern of a non-negative float (integer max then is float max; a NaN beats every finite value
// and turns the scaling off)
__global__ void __launch_bounds__(256)
dx_absmax_kernel(const float* __restrict__ v, int64_t n, uint32_t* __restrict__ out_bits) {
    uint32_t m = 0u;
    const int64_t n4 = n >> 2;
    const float4* v4 = reinterpret_cast<const float4*>(v);
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < n4; e += (int64_t)gridDim.x * blockDim.x) {
        const float4 a = v4[e];
        m = max(m, __float_as_uint(fabsf(a.x))); m = max(m, __float_as_uint(fabsf(a.y)));
        m = max(m, __float_as_uint(fabsf(a.z))); m = max(m, __float_as_uint(fabsf(a.w)));
    }
    if (blockIdx.x == 0 && threadIdx.x < (n & 3)) m = max(m, __float_as_uint(fabsf(v[(n4 << 2) + threadIdx.x])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0 && m != 0u) atomicMax(out_bits, m);
}

// s_W: max |C| * s_W lies in [2^14, 2^15) / 2^ceil(log2 max_factor), so max_factor * |C| * s_W stays below 2^15
__device__ __forceinline__ float dx_w_scale(uint32_t maxbits, int max_factor) {
    int sh = 0;
    while ((1 << sh) < max_factor) ++sh;
    return half_scale_for(maxbits) * __uint_as_float((uint32_t)(127 - sh) << 23);
}

// Wd[(i,d)][out_pad] <- fp16(d * C[i][o][d] * s_W); also writes the inverse scale the epilogue applies
__global__ void __launch_bounds__(256)
pack_dx_half_kernel(const float* __restrict__ c, uint32_t* __restrict__ header, __half* __restrict__ wd, int in, int out,
                    int nd, int out_pad, int degree_factor) {
    const float s_w = dx_w_scale(header[0], degree_factor ? nd : 1);
    if (blockIdx.x == 0 && threadIdx.x == 0) reinterpret_cast<float*>(header)[1] = 1.f / s_w;
    const int64_t total = (int64_t)in * nd * out_pad;
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total;
         e += (int64_t)gridDim.x * blockDim.x) {
        const int o = (int)(e % out_pad);
        const int64_t slot = e / out_pad;
        const int64_t i = slot / nd;
        const int d = (int)(slot % nd) + 1;
        float v = 0.f;
        if (o < out) v = (degree_factor ? (float)d : 1.f) * c[(i * out + o) * (nd + 1) + d] * s_w;
        wd[e] = __float2half_rn(v);
    }
}

// dYh[b][pitch] <- fp16(dY[b][o] * s_b) for o < out, s_b the power of two that puts the row's largest |element| into
// [2^14, 2^15) (1 for a row of zeros, and for a row with an inf or a NaN, which then reaches the tensor pipe as it
// is); row_inv[b] = 1 / s_b.  One warp per row, the row read twice (the second time from L1).  `out` is a multiple
// of 4; the pad columns are never read: the tensor map ends at `out`.
__global__ void __launch_bounds__(256)
dy_half_rows_kernel(const float* __restrict__ dy, __half* __restrict__ dyh, float* __restrict__ row_inv, int64_t B,
                    int out, int64_t pitch) {
    const int lane = threadIdx.x & 31;
    const int q = out >> 2;
    for (int64_t b = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5; b < B;
         b += ((int64_t)gridDim.x * blockDim.x) >> 5) {
        const float4* row = reinterpret_cast<const float4*>(dy + b * out);
        uint32_t m = 0u;
        for (int c4 = lane; c4 < q; c4 += 32) {
            const float4 v = row[c4];
            m = max(m, __float_as_uint(fabsf(v.x))); m = max(m, __float_as_uint(fabsf(v.y)));
            m = max(m, __float_as_uint(fabsf(v.z))); m = max(m, __float_as_uint(fabsf(v.w)));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
        const float s = half_scale_for(m);
        if (lane == 0) row_inv[b] = 1.f / s;
        __half* dst = dyh + b * pitch;
        for (int c4 = lane; c4 < q; c4 += 32) {
            const float4 v = row[c4];
            const __half2 h0 = __floats2half2_rn(v.x * s, v.y * s), h1 = __floats2half2_rn(v.z * s, v.w * s);
            uint2 w;
            w.x = *reinterpret_cast<const uint32_t*>(&h0); w.y = *reinterpret_cast<const uint32_t*>(&h1);
            *reinterpret_cast<uint2*>(dst + 4 * c4) = w;
        }
    }
}

// Running state of one input's fold: sum += U_{d-1}(t) G_d column by column, U advanced by its recurrence.
struct DxFold {
    float ua = 1.f, ub = 0.f, sum = 0.f, t2;       // (U_0, U_{-1}): the first column is degree 1, weight U_0 = 1
    __device__ __forceinline__ explicit DxFold(float two_t) : t2(two_t) {}
    // two columns: sum += U_{d-1} G_d, advance U, twice (ua / ub swap roles)
    __device__ __forceinline__ void two(uint32_t g0, uint32_t g1) {
        sum = fmaf(ua, __uint_as_float(g0), sum);
        ub = fmaf(t2, ua, -ub);
        sum = fmaf(ub, __uint_as_float(g1), sum);
        ua = fmaf(t2, ub, -ua);
    }
    __device__ __forceinline__ void one(uint32_t g) { sum = fmaf(ua, __uint_as_float(g), sum); }
};

// The same for a table-driven family: sum += P_d'(u) G_d with P and P' carried side by side through the recurrence
// and its derivative, from degree 1 on (start state P_0 = 1, P_{-1} = 0, P_0' = 0).
struct DxFoldTable {
    float p1 = 1.f, p2 = 0.f, d1 = 0.f, d2 = 0.f, sum = 0.f, u;
    __device__ __forceinline__ explicit DxFoldTable(float u_) : u(u_) {}
    __device__ __forceinline__ void one(const RecurrenceTable& t, int d, uint32_t g) {
        const float a = t.A[d], c = t.C[d];
        const float k = fmaf(a, u, t.B[d]);
        const float dp = fmaf(a, p1, fmaf(k, d1, -(c * d2)));
        const float p = fmaf(k, p1, -(c * p2));
        sum = fmaf(dp, __uint_as_float(g), sum);
        p2 = p1; p1 = p; d2 = d1; d1 = dp;
    }
};
struct DxNoTable {};
template <bool FAM> struct DxTable { using type = DxNoTable; };
template <> struct DxTable<true> { using type = RecurrenceTable; };

template <int CG, int BN, bool FAM, bool H = false>
__global__ void __launch_bounds__(DX_THREADS, 1)
dx_tc_kernel(const __grid_constant__ CUtensorMap tmap_dy, const __grid_constant__ CUtensorMap tmap_w,
             const float* __restrict__ x, float* __restrict__ dx, int64_t B, int in, int out, int nd, int TI,
             int i_tiles, int64_t num_tiles, int32_t* status, int accumulate, int exact_tanh,
             const __grid_constant__ typename DxTable<FAM>::type rec, const float* __restrict__ w_inv_scale,
             const float* __restrict__ row_inv_scale) {
    static_assert(!(H && FAM), "the fp16-operand variant exists for the Chebyshev fold only");
    constexpr int KB = H ? DX_KB_HALF : DX_KB;           // outputs per K block (one 128-byte row of either operand)
    constexpr int OPMODE = H ? CHEBYKAN_MODE_BF16 : CHEBYKAN_MODE_TF32;   // kind::f16 / kind::tf32
    using L = DxSmem<CG, BN>;
    constexpr int NS = L::NS, DX_NUM_BARS = L::NUM_BARS, NACC = L::NACC;
    constexpr int GROUP_WARPS = DX_EPI_WARPS / NACC;     // epilogue warps per accumulator
    constexpr int PARTS = GROUP_WARPS / 4;               // warps per TMEM lane quarter within a group
    constexpr int DX_STAGE = L::STAGE, DX_BAR_OFFSET = L::BAR_OFFSET;
    // fp32 accumulate; operand formats tf32 (2) or fp16 (0); both operands K-major
    constexpr uint32_t IDESC = (1u << 4) | (H ? 0u : ((2u << 7) | (2u << 10))) | ((uint32_t)(BN >> 3) << 17) |
                               ((uint32_t)((DX_BM * CG) >> 4) << 24);
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bars = smem_base + DX_BAR_OFFSET;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (NS + s); };
    auto acc_full_bar = [&](int a) { return bars + 8u * (2 * NS + a); };
    auto acc_empty_bar = [&](int a) { return bars + 8u * (2 * NS + NACC + a); };
    const uint32_t drain_bar = bars + 8u * (2 * NS + 2 * NACC);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + DX_BAR_OFFSET + DX_NUM_BARS * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + DX_BAR_OFFSET + DX_NUM_BARS * 8 + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nkb = (out + KB - 1) / KB;
    // CTA pair: a tile is 256 rows, this CTA owns rows [128 rank, 128 rank + 128) of it
    const uint32_t rank = (CG == 2) ? cluster_ctarank() : 0u;
    const int64_t unit = (CG == 2) ? (blockIdx.x >> 1) : blockIdx.x;
    const int64_t nunits = (CG == 2) ? (gridDim.x >> 1) : gridDim.x;
    // tile = row block * i_tiles + input tile.  The roles walk their tiles with (row block, input tile) counters:
    // a 64-bit division per tile and warp costs about as many instructions as folding one input.
    const int64_t rb_first = unit / i_tiles, rb_step = nunits / i_tiles;
    const int it_first = (int)(unit % i_tiles), it_step = (int)(nunits % i_tiles);

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < NACC; ++a) { mbar_init(acc_full_bar(a), 1); mbar_init(acc_empty_bar(a), GROUP_WARPS * CG); }
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == DX_MMA_WARP) {
        if (CG == 2) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                         ::"r"(smem_u32((const void*)tmem_slot)), "r"(512u) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                         ::"r"(smem_u32((const void*)tmem_slot)), "r"(512u) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if (CG == 2) cluster_sync_all();      // the peer's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == DX_TMA_WARP) {
        if (lane == 0) {
            int s = 0; uint32_t ph = 0;
            bool alive = true;
            int64_t rb = rb_first; int it = it_first;
            for (int64_t tile = unit; tile < num_tiles && alive; tile += nunits) {
                const int m0 = (int)(rb * (DX_BM * CG) + rank * DX_BM);
                const int slot0 = it * TI * nd;
                rb += rb_step; it += it_step;
                if (it >= i_tiles) { it -= i_tiles; ++rb; }
                for (int kb = 0; kb < nkb; ++kb) {
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, status, XST_TMA)) { alive = false; break; }
                    const uint32_t st = smem_base + s * DX_STAGE;
                    if (CG == 2) {
                        // both CTAs' bytes count on the even CTA's barrier
                        if (rank == 0) mbar_arrive_expect_tx(full_bar(s), 2 * DX_STAGE);
                        const uint32_t bar0 = mapa_cluster(full_bar(s), 0);
                        tma_load_2d_pair(st, &tmap_dy, kb * KB, m0, bar0);
                        tma_load_2d_pair(st + DX_A_STAGE, &tmap_w, kb * KB, slot0 + (int)rank * (BN / 2), bar0);
                    } else {
                        mbar_arrive_expect_tx(full_bar(s), DX_STAGE);
                        tma_load_2d(st, &tmap_dy, kb * KB, m0, full_bar(s));
                        tma_load_2d(st + DX_A_STAGE, &tmap_w, kb * KB, slot0, full_bar(s));
                    }
                    if (++s == NS) { s = 0; ph ^= 1u; }
                }
            }
            if (!alive) {
                const uint64_t t0 = globaltimer_ns();
                while (globaltimer_ns() - t0 < 200000ull) { }
            }
        }
    } else if (warp == DX_MMA_WARP) {
        // The warp runs the loop in lock step; one elected lane executes the MMAs and commits (see elect_one_sync).
        if (rank == 0) {
            const bool elected = elect_one_sync();
            int s = 0; uint32_t ph = 0;
            int acc = 0; uint32_t acc_ph = 0;
            bool alive = true;
            const uint64_t a_desc0 = make_smem_desc(smem_base);
            const uint64_t b_desc0 = make_smem_desc(smem_base + DX_A_STAGE);
            const uint32_t a_hi = (uint32_t)(a_desc0 >> 32), b_hi = (uint32_t)(b_desc0 >> 32);
            for (int64_t tile = unit; tile < num_tiles && alive; tile += nunits) {
                if (!__all_sync(0xffffffffu, mbar_wait(acc_empty_bar(acc), acc_ph ^ 1u, abort_flag, status, XST_MMA_ACC))) { alive = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < nkb; ++kb) {
                    if (!__all_sync(0xffffffffu, mbar_wait(full_bar(s), ph, abort_flag, status, XST_MMA_FULL))) { alive = false; break; }
                    tc_fence_after();
                    const uint32_t a_lo = (uint32_t)a_desc0 + (uint32_t)((s * DX_STAGE) >> 4);
                    const uint32_t b_lo = (uint32_t)b_desc0 + (uint32_t)((s * DX_STAGE) >> 4);
                    const uint32_t later = (uint32_t)(kb != 0);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint64_t ad = desc_from_words(a_lo + 2u * k, a_hi), bd = desc_from_words(b_lo + 2u * k, b_hi);
                        if (elected) {
                            if (CG == 2) {
                                if (k != 0) umma2<OPMODE>(d_tmem, ad, bd, IDESC, 1u);
                                else umma2<OPMODE>(d_tmem, ad, bd, IDESC, later);
                            } else {
                                if (k != 0) umma<OPMODE>(d_tmem, ad, bd, IDESC, 1u);
                                else umma<OPMODE>(d_tmem, ad, bd, IDESC, later);
                            }
                        }
                    }
                    if (elected) { if (CG == 2) umma2_commit_both(empty_bar(s)); else umma_commit(empty_bar(s)); }
                    __syncwarp();
                    if (++s == NS) { s = 0; ph ^= 1u; }
                }
                if (alive && elected) { if (CG == 2) umma2_commit_both(acc_full_bar(acc)); else umma_commit(acc_full_bar(acc)); }
                __syncwarp();
                if (++acc == NACC) { acc = 0; acc_ph ^= 1u; }
            }
            if (!alive && elected) {
                if (CG == 2) umma2_commit(drain_bar); else umma_commit(drain_bar);
                const uint64_t t0 = globaltimer_ns();
                while (!mbar_try_wait(drain_bar, 0) && globaltimer_ns() - t0 < 10000000ull) { }
            }
            __syncwarp();
        }
    } else {
        // ------------------------------ epilogue ------------------------------
        const int q = warp & 3;                          // TMEM lane quarter
        const int group = (warp - DX_EPI_WARP0) / GROUP_WARPS;          // which accumulator's tiles
        const int part = ((warp - DX_EPI_WARP0) % GROUP_WARPS) >> 2;     // which share of a tile's inputs
        const int acc = group; uint32_t acc_ph = 0;
        bool alive = true;
        const float osc_w = H ? __ldg(w_inv_scale) : 1.f;
        // this group's tiles: unit + group * nunits, then every NACC * nunits
        const int64_t first = unit + group * nunits;
        int64_t rb = first / i_tiles; int it = (int)(first % i_tiles);
        const int64_t rb_step2 = (NACC * nunits) / i_tiles; const int it_step2 = (int)((NACC * nunits) % i_tiles);
        for (int64_t tile = first; tile < num_tiles && alive; tile += NACC * nunits) {
            const int64_t row = rb * (DX_BM * CG) + rank * DX_BM + q * 32 + lane;
            const int i0 = it * TI;
            rb += rb_step2; it += it_step2;
            if (it >= i_tiles) { it -= i_tiles; ++rb; }
            const int ti = min(TI, in - i0);
            const int per = (ti + PARTS - 1) / PARTS;
            const int ii_begin = min(ti, part * per), ii_end = min(ti, ii_begin + per);
            const bool row_ok = row < B;
            const float osc_dy = (H && row_ok) ? __ldg(row_inv_scale + row) : 1.f;
            const float* xrow = x + (row_ok ? row : 0) * in + i0;
            float* dxrow = dx + (row_ok ? row : 0) * in + i0;
            // The warp folds its inputs two at a time (A and B): both inputs' TMEM loads are in flight together and
            // their recurrences are four independent FMA chains instead of two.  One input at a time, a warp spent
            // most of a tile waiting (a TMEM load, then 64 dependent FMAs, then the next load), and sixteen such
            // warps, not the MMAs, set the kernel's time.
            // x of the first pair in flight before the accumulator is awaited
            float xa = (row_ok && ii_begin < ii_end) ? __ldg(xrow + ii_begin) : 0.f;
            float xb = (row_ok && ii_begin + 1 < ii_end) ? __ldg(xrow + ii_begin + 1) : 0.f;
            const bool ok = mbar_wait(acc_full_bar(acc), acc_ph, abort_flag, status, XST_EPILOGUE);
            if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
            if constexpr (FAM) {
                // table-driven family: same pairing of inputs, one column per step (P and P' both advance)
                for (int ii = ii_begin; ii < ii_end; ii += 2) {
                    const bool has_b = ii + 1 < ii_end;
                    const float tha = tanh_fast(xa), thb = tanh_fast(xb);
                    const float ua = rec.affine ? fmaf(rec.scale, xa - rec.shift, rec.offset) : rec.scale * tha;
                    const float ub = rec.affine ? fmaf(rec.scale, xb - rec.shift, rec.offset) : rec.scale * thb;
                    const float dua = rec.affine ? rec.scale : rec.scale * fmaf(-tha, tha, 1.f);     // du/dx
                    const float dub = rec.affine ? rec.scale : rec.scale * fmaf(-thb, thb, 1.f);
                    if (row_ok && ii + 2 < ii_end) xa = __ldg(xrow + ii + 2);
                    if (row_ok && ii + 3 < ii_end) xb = __ldg(xrow + ii + 3);
                    float old_a = 0.f, old_b = 0.f;
                    if (accumulate && row_ok) { old_a = dxrow[ii]; if (has_b) old_b = dxrow[ii + 1]; }
                    DxFoldTable fa(ua), fb(ub);
                    const uint32_t col_a = taddr + (uint32_t)(ii * nd);
                    const uint32_t col_b = has_b ? col_a + (uint32_t)nd : col_a;
                    int c = 0;
                    for (; c + 16 <= nd; c += 16) {
                        uint32_t ra[16], rb[16];
                        tmem_ld16(col_a + c, ra); tmem_ld16(col_b + c, rb); tmem_ld_wait();
#pragma unroll
                        for (int e = 0; e < 16; ++e) { fa.one(rec, c + e + 1, ra[e]); fb.one(rec, c + e + 1, rb[e]); }
                    }
                    if ((nd - c) & 8) {
                        uint32_t ra[8], rb[8];
                        tmem_ld8(col_a + c, ra); tmem_ld8(col_b + c, rb); tmem_ld_wait();
#pragma unroll
                        for (int e = 0; e < 8; ++e) { fa.one(rec, c + e + 1, ra[e]); fb.one(rec, c + e + 1, rb[e]); }
                        c += 8;
                    }
                    if ((nd - c) & 4) {
                        uint32_t ra[4], rb[4];
                        tmem_ld4(col_a + c, ra); tmem_ld4(col_b + c, rb); tmem_ld_wait();
#pragma unroll
                        for (int e = 0; e < 4; ++e) { fa.one(rec, c + e + 1, ra[e]); fb.one(rec, c + e + 1, rb[e]); }
                        c += 4;
                    }
                    if ((nd - c) & 2) {
                        uint32_t ra[2], rb[2];
                        tmem_ld2(col_a + c, ra); tmem_ld2(col_b + c, rb); tmem_ld_wait();
                        fa.one(rec, c + 1, ra[0]); fb.one(rec, c + 1, rb[0]); fa.one(rec, c + 2, ra[1]); fb.one(rec, c + 2, rb[1]);
                        c += 2;
                    }
                    if ((nd - c) & 1) {
                        uint32_t ra = 0u, rb = 0u;
                        tmem_ld1(col_a + c, ra); tmem_ld1(col_b + c, rb); tmem_ld_wait();
                        fa.one(rec, c + 1, ra); fb.one(rec, c + 1, rb);
                    }
                    if (row_ok) {
                        const float va = dua * fa.sum;
                        dxrow[ii] = accumulate ? old_a + va : va;
                        if (has_b) {
                            const float vb = dub * fb.sum;
                            dxrow[ii + 1] = accumulate ? old_b + vb : vb;
                        }
                    }
                }
            } else {
            for (int ii = ii_begin; ii < ii_end; ii += 2) {
                const bool has_b = ii + 1 < ii_end;          // warp-uniform; without B the second lane of work repeats A
                const float ta = exact_tanh ? tanhf(xa) : tanh_fast(xa);
                const float tb = exact_tanh ? tanhf(xb) : tanh_fast(xb);
                if (row_ok && ii + 2 < ii_end) xa = __ldg(xrow + ii + 2);
                if (row_ok && ii + 3 < ii_end) xb = __ldg(xrow + ii + 3);
                // accumulating launches: what is in dx already, in flight while the columns are folded (one lane
                // per row: each of these loads is its own sector, and its latency would end the round otherwise)
                float old_a = 0.f, old_b = 0.f;
                if (accumulate && row_ok) { old_a = dxrow[ii]; if (has_b) old_b = dxrow[ii + 1]; }
                // ua / ub alternate as (U_{d-1}, U_{d-2}), starting at degree 1
                DxFold fa(2.f * ta), fb(2.f * tb);
                const uint32_t col_a = taddr + (uint32_t)(ii * nd);
                const uint32_t col_b = has_b ? col_a + (uint32_t)nd : col_a;
                int c = 0;
                for (; c + 32 <= nd; c += 32) {
                    uint32_t ra[32], rb[32];
                    tmem_ld32(col_a + c, ra);
                    tmem_ld32(col_b + c, rb);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 32; e += 2) { fa.two(ra[e], ra[e + 1]); fb.two(rb[e], rb[e + 1]); }
                }
                // the last 1-31 columns: loads of 16, 8, 4, 2 and 1 columns as the count's bits say, so that no lane
                // touches a column past its input's last one; each size is loaded, awaited and folded in turn (few
                // registers live at once; configurations whose time the epilogue sets have one or two bits set)
                const int rem = nd - c;
                int cc = c;
                if (rem & 16) {
                    uint32_t a[16], b[16];
                    tmem_ld16(col_a + cc, a); tmem_ld16(col_b + cc, b); tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 16; e += 2) { fa.two(a[e], a[e + 1]); fb.two(b[e], b[e + 1]); }
                    cc += 16;
                }
                if (rem & 8) {
                    uint32_t a[8], b[8];
                    tmem_ld8(col_a + cc, a); tmem_ld8(col_b + cc, b); tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 8; e += 2) { fa.two(a[e], a[e + 1]); fb.two(b[e], b[e + 1]); }
                    cc += 8;
                }
                if (rem & 4) {
                    uint32_t a[4], b[4];
                    tmem_ld4(col_a + cc, a); tmem_ld4(col_b + cc, b); tmem_ld_wait();
                    fa.two(a[0], a[1]); fb.two(b[0], b[1]); fa.two(a[2], a[3]); fb.two(b[2], b[3]);
                    cc += 4;
                }
                if (rem & 2) {
                    uint32_t a[2], b[2];
                    tmem_ld2(col_a + cc, a); tmem_ld2(col_b + cc, b); tmem_ld_wait();
                    fa.two(a[0], a[1]); fb.two(b[0], b[1]);
                    cc += 2;
                }
                if (rem & 1) {
                    uint32_t a = 0u, b = 0u;
                    tmem_ld1(col_a + cc, a); tmem_ld1(col_b + cc, b); tmem_ld_wait();
                    fa.one(a); fb.one(b);
                }
                if (row_ok) {
                    float va = fmaf(-ta, ta, 1.f) * fa.sum;
                    if (H) va = va * osc_dy * osc_w;       // undo the operands' power-of-two scales (one after the other:
                    dxrow[ii] = accumulate ? old_a + va : va;       // their product may leave the float range)
                    if (has_b) {
                        float vb = fmaf(-tb, tb, 1.f) * fb.sum;
                        if (H) vb = vb * osc_dy * osc_w;
                        dxrow[ii + 1] = accumulate ? old_b + vb : vb;
                    }
                }
            }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (CG == 2 && rank != 0) mbar_arrive_cluster(mapa_cluster(acc_empty_bar(acc), 0));
                else mbar_arrive(acc_empty_bar(acc));
            }
            acc_ph ^= 1u;
        }
    }

    tc_fence_before();
    __syncthreads();
    // neither CTA of a pair leaves (or frees TMEM) while the other may still arrive on its barriers
    if (CG == 2) cluster_sync_all();
    if (warp == DX_MMA_WARP) {
        tc_fence_after();
        if (CG == 2)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

}  // namespace

int launch_dy_tail(const float* dy, float* lo, int64_t n, cudaStream_t s) {
    int64_t blocks = ceil_div(n, 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (blocks < 1) blocks = 1;
    dy_tail_kernel<<<(unsigned)blocks, 256, 0, s>>>(dy, lo, n);
    return check_cuda(cudaGetLastError());
}

// dY and Wd rows must be TMA-addressable (16-byte pitch) and one input's degrees must fit a tile
bool dx_tc_supported(int64_t B, int64_t in, int64_t out, int64_t deg) {
    return B > 0 && (out % 4) == 0 && deg + 1 <= DX_BN && in * (deg + 1) < ((int64_t)1 << 31);
}

// tf32 / bf16 modes: the repacked coefficients.  Three-product (fp32-grade) mode: their heads and tails, and the
// tails of dY.
// fp16-operand variant (x3 == 2): a header, the fp16 coefficients and the scaled fp16 copy of dY.
int64_t dx_tc_workspace_bytes(int64_t B, int64_t in, int64_t out, int64_t deg, int x3) {
    if (x3 == 2) {
        const int64_t out_pad = round_up(out, DX_KB_HALF);
        return DX_HEADER + round_up(in * (deg > 0 ? deg : 1) * out_pad * 2, 256) + round_up(B * out_pad * 2, 256) +
               round_up(B * 4, 256);
    }
    const int64_t wd = round_up(in * (deg + 1) * round_up(out, 32) * 4, 256);
    return x3 ? 2 * wd + round_up(B * out * 4, 256) : wd;
}

namespace {
template <int CG, int BN, bool FAM, bool H = false>
int launch_dx_kernel(const CUtensorMap& tmap_dy, const CUtensorMap& tmap_w, const float* x, float* dx, int64_t B,
                     int in, int out, int nd, int32_t* status, cudaStream_t s, int accumulate, int exact_tanh,
                     const typename DxTable<FAM>::type& rec, const float* w_inv_scale = nullptr,
                     const float* row_inv_scale = nullptr) {
    using L = DxSmem<CG, BN>;
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kernel = dx_tc_kernel<CG, BN, FAM, H>;
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        int rc = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
        if (rc) return rc;
        attr_set[dev] = true;
    }
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int TI = BN / nd;
    if (TI > in) TI = in;
    const int i_tiles = (int)ceil_div(in, TI);
    const int64_t num_tiles = ceil_div(B, DX_BM * CG) * i_tiles;
    const int64_t max_units = sms / CG;
    const unsigned units = (unsigned)(num_tiles < max_units ? num_tiles : max_units);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(units * CG); cfg.blockDim = dim3(DX_THREADS); cfg.dynamicSmemBytes = L::TOTAL; cfg.stream = s;
    cudaLaunchAttribute attrs[1];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = CG; attrs[0].val.clusterDim.y = 1; attrs[0].val.clusterDim.z = 1;
    cfg.attrs = attrs; cfg.numAttrs = 1;
    return check_cuda(cudaLaunchKernelEx(&cfg, kernel, tmap_dy, tmap_w, x, dx, B, in, out, nd, TI, i_tiles, num_tiles,
                                         status, accumulate, exact_tanh, rec, w_inv_scale, row_inv_scale));
}

// The fp16-operand variant: row-scaled fp16 copy of dY, absmax and scaled fp16 repack of the coefficients, the kernel.
int launch_dx_half(const float* x, const float* dy, const float* coeffs, float* dx, void* ws, int64_t B, int64_t in,
                   int64_t out, int nd, int32_t* status, cudaStream_t s) {
    EncodeTiledFn encode = get_encode_fn();
    if (!encode) return CHEBYKAN_ECUDA;
    const int64_t out_pad = round_up(out, DX_KB_HALF);
    const int64_t slots = in * nd;
    uint32_t* header = reinterpret_cast<uint32_t*>(ws);
    __half* wd = reinterpret_cast<__half*>(reinterpret_cast<char*>(ws) + DX_HEADER);
    __half* dyh = reinterpret_cast<__half*>(reinterpret_cast<char*>(ws) + DX_HEADER + round_up(slots * out_pad * 2, 256));
    float* row_inv = reinterpret_cast<float*>(reinterpret_cast<char*>(dyh) + round_up(B * out_pad * 2, 256));
    int rc;
    if ((rc = check_cuda(cudaMemsetAsync(header, 0, 16, s)))) return rc;
    auto grid_for = [](int64_t work) {
        int64_t blocks = ceil_div(work, 256);
        if (blocks > 148 * 8) blocks = 148 * 8;
        return (unsigned)(blocks < 1 ? 1 : blocks);
    };
    dx_absmax_kernel<<<grid_for(ceil_div(in * out * (nd + 1), 4)), 256, 0, s>>>(coeffs, in * out * (nd + 1), header);
    pack_dx_half_kernel<<<grid_for(slots * out_pad), 256, 0, s>>>(coeffs, header, wd, (int)in, (int)out, nd, (int)out_pad, 1);
    dy_half_rows_kernel<<<grid_for(B * 32), 256, 0, s>>>(dy, dyh, row_inv, B, (int)out, out_pad);
    if ((rc = check_cuda(cudaGetLastError()))) return rc;
    const int cg = B > DX_BM ? 2 : 1;
    const cuuint32_t estr[2] = {1, 1};
    CUtensorMap m_dy, m_w;
    {
        // dYh[B][out_pad] fp16, valid columns [0, out): boxes of 64 outputs (128 bytes) x 128 rows
        const cuuint64_t dims[2] = {(cuuint64_t)out, (cuuint64_t)B};
        const cuuint64_t strides[1] = {(cuuint64_t)(out_pad * 2)};
        const cuuint32_t box[2] = {DX_KB_HALF, DX_BM};
        const CUresult r = encode(&m_dy, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, dyh, dims, strides, box, estr,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { set_last_cuda_error((int)r); return CHEBYKAN_ECUDA; }
    }
    {
        const cuuint64_t dims[2] = {(cuuint64_t)out_pad, (cuuint64_t)slots};
        const cuuint64_t strides[1] = {(cuuint64_t)(out_pad * 2)};
        const cuuint32_t box[2] = {DX_KB_HALF, (cuuint32_t)(DX_BN / cg)};
        const CUresult r = encode(&m_w, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, wd, dims, strides, box, estr,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { set_last_cuda_error((int)r); return CHEBYKAN_ECUDA; }
    }
    const float* w_inv = reinterpret_cast<const float*>(header) + 1;
    if (cg == 2) return launch_dx_kernel<2, DX_BN, false, true>(m_dy, m_w, x, dx, B, (int)in, (int)out, nd, status, s, 0, 0, DxNoTable(), w_inv, row_inv);
    return launch_dx_kernel<1, DX_BN, false, true>(m_dy, m_w, x, dx, B, (int)in, (int)out, nd, status, s, 0, 0, DxNoTable(), w_inv, row_inv);
}
}  // namespace

int launch_dx_tc(const float* x, const float* dy, const float* coeffs, float* dx, void* ws, int64_t ws_bytes,
                 int64_t B, int64_t in, int64_t out, int64_t deg, int32_t* status, cudaStream_t s, int x3,
                 const RecurrenceTable* rec) {
    // x3: 0 = tf32 operands, 1 = three tf32 products of heads and tails (the fp32 tolerance), 2 = fp16 operands
    if (rec != nullptr && x3) return CHEBYKAN_EUNSUPPORTED;
    const int degree_factor = rec == nullptr;
    // T_0' = 0 (P_0' = 0): degree 0 takes no slot of G.  A tile's 256 slots then hold 256 / deg inputs: 8 instead of
    // 7 at degree 32 (one 32-column TMEM load per input, no remainder), 32 instead of 28 at degree 8.
    const int nd = (int)deg;
    if (nd == 0) return check_cuda(cudaMemsetAsync(dx, 0, B * in * 4, s));
    const int64_t out_pad = round_up(out, 32);
    const int64_t slots = in * nd;
    if (ws == nullptr || ws_bytes < dx_tc_workspace_bytes(B, in, out, deg, x3)) return CHEBYKAN_EWORKSPACE;
    if (x3 == 2) return launch_dx_half(x, dy, coeffs, dx, ws, B, in, out, nd, status, s);
    EncodeTiledFn encode = get_encode_fn();
    if (!encode) return CHEBYKAN_ECUDA;
    const int64_t wd_bytes = round_up(slots * out_pad * 4, 256);
    uint32_t* wd_hi = reinterpret_cast<uint32_t*>(ws);
    uint32_t* wd_lo = wd_hi + slots * out_pad;                       // written right behind the heads by the pack kernel
    float* dy_lo = reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + 2 * wd_bytes);
    {
        int64_t blocks = ceil_div(slots * out_pad, 256);
        if (blocks > 148 * 16) blocks = 148 * 16;
        if (x3) pack_dx_kernel<1><<<(unsigned)blocks, 256, 0, s>>>(coeffs, wd_hi, (int)in, (int)out, nd, (int)out_pad, degree_factor);
        else pack_dx_kernel<0><<<(unsigned)blocks, 256, 0, s>>>(coeffs, wd_hi, (int)in, (int)out, nd, (int)out_pad, degree_factor);
        int rc = check_cuda(cudaGetLastError());
        if (rc) return rc;
        if (x3) {
            int64_t b2 = ceil_div(B * out, 256);
            if (b2 > 148 * 16) b2 = 148 * 16;
            dy_tail_kernel<<<(unsigned)b2, 256, 0, s>>>(dy, dy_lo, B * out);
            if ((rc = check_cuda(cudaGetLastError()))) return rc;
        }
    }
    const int cg = B > DX_BM ? 2 : 1;
    const int bn = DX_BN;
    const cuuint32_t estr[2] = {1, 1};
    auto map_dy = [&](CUtensorMap* m, const float* p) -> int {
        const cuuint64_t dims[2] = {(cuuint64_t)out, (cuuint64_t)B};
        const cuuint64_t strides[1] = {(cuuint64_t)(out * 4)};
        const cuuint32_t box[2] = {DX_KB, DX_BM};
        const CUresult r = encode(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(p), dims, strides,
                                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { set_last_cuda_error((int)r); return CHEBYKAN_ECUDA; }
        return CHEBYKAN_OK;
    };
    auto map_w = [&](CUtensorMap* m, void* p) -> int {
        const cuuint64_t dims[2] = {(cuuint64_t)out_pad, (cuuint64_t)slots};
        const cuuint64_t strides[1] = {(cuuint64_t)(out_pad * 4)};
        const cuuint32_t box[2] = {DX_KB, (cuuint32_t)(bn / cg)};
        const CUresult r = encode(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, p, dims, strides, box, estr,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { set_last_cuda_error((int)r); return CHEBYKAN_ECUDA; }
        return CHEBYKAN_OK;
    };
    auto run = [&](const CUtensorMap& mdy, const CUtensorMap& mw, int accumulate) -> int {
        if (rec != nullptr) {
            if (cg == 2) return launch_dx_kernel<2, DX_BN, true>(mdy, mw, x, dx, B, (int)in, (int)out, nd, status, s, accumulate, 0, *rec);
            return launch_dx_kernel<1, DX_BN, true>(mdy, mw, x, dx, B, (int)in, (int)out, nd, status, s, accumulate, 0, *rec);
        }
        if (cg == 2) return launch_dx_kernel<2, DX_BN, false>(mdy, mw, x, dx, B, (int)in, (int)out, nd, status, s, accumulate, x3, DxNoTable());
        return launch_dx_kernel<1, DX_BN, false>(mdy, mw, x, dx, B, (int)in, (int)out, nd, status, s, accumulate, x3, DxNoTable());
    };
    CUtensorMap m_dy, m_w;
    int rc;
    if ((rc = map_dy(&m_dy, dy)) || (rc = map_w(&m_w, wd_hi))) return rc;
    if ((rc = run(m_dy, m_w, 0))) return rc;
    if (!x3) return CHEBYKAN_OK;
    // dx = fold(dY_head Wd_head) + fold(dY_head Wd_tail) + fold(dY_tail Wd_head): the fold is linear in G, so the
    // three products are three launches that add into dx (tail x tail is below fp32 rounding)
    CUtensorMap m_wlo, m_dylo;
    if ((rc = map_w(&m_wlo, wd_lo)) || (rc = map_dy(&m_dylo, dy_lo))) return rc;
    if ((rc = run(m_dy, m_wlo, 1))) return rc;
    return run(m_dylo, m_w, 1);
}

}  // namespace chebykan
