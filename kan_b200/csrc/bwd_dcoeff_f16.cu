// Coefficient gradient of NARROW layers (at most 128 outputs) on the tensor cores with 16-bit operands:
//   dC[(i,d), o] = sum_b T_d(tanh x[b,i]) * dY[b,o]          (tcgen05 kind::f16, fp32 accumulate)
// the dW half of what autograd derives from reference kan/basis/chebyshev.py:101,119-145, with Phi regenerated on
// chip.  Same tiling as bwd_dcoeff_tc.cu (a CTA owns TI inputs with all their degrees, up to 512 slots, all outputs
// and a slice of the batch), different operands:
//
//   * Why.  On a narrow layer the kind::tf32 kernel is bound by shared-memory traffic: every basis value is stored
//     once (4 bytes) and read once by the tensor pipe, and an N = 64 MMA is too short to hide it.  fp16 carries the
//     same 11 significant bits as tf32, so fp16 operands give the same accuracy with half the bytes and half the
//     MMAs (K = 16 per instruction).  Basis values lie in [-1, 1], well inside fp16's range.  dY does not: a
//     pre-pass finds max |dY| and scales dY by the power of two that puts the maximum in [2^14, 2^15) (exact; what
//     then falls below fp16's normal range is 2^-28 of the maximum and cannot matter at 11 bits), and the epilogue
//     multiplies the accumulators by the inverse.
//   * A (Phi^T, generated): K-major [128 slots][64 batch rows] fp16, 128B swizzle; a producer lane owns one input and
//     eight consecutive batch rows and writes one 16-byte chunk per degree.
//   * B (dY, scaled, fp16): the same pre-pass transposes dY to [out][B] so that the operand is K-major like every
//     forward operand (one TMA box of 64 rows x BN outputs, 128B swizzle).
//
// Pre-pass cost: dY is read twice and written once at half size (about a tenth of the kernel's time on a
// 1048576 x 64 layer).  Every mbarrier wait is bounded, as in the other kernels.
#include <cuda_fp16.h>
#include <stdlib.h>
#include <string.h>
#include "tc_common.cuh"

namespace chebykan {

namespace {
using namespace tc;

constexpr int F_PRODUCER_WARPS = 8;
constexpr int F_TMA_WARP = 8, F_MMA_WARP = 9, F_X_WARP = 10;
constexpr int F_THREADS = 11 * 32;
constexpr int F_KB = 64;                  // batch rows per K block (128 bytes of fp16)
constexpr int F_A_TILE = 128 * 128;       // one M tile of A: 128 slots x 64 fp16
constexpr int F_NS = 2;                   // stages; the 8 producer warps split into two groups of four
constexpr int F_G = F_PRODUCER_WARPS / F_NS;
constexpr int F_MAX_ROUNDS = 2;           // (input, 8-row chunk) pairs per lane per K block
constexpr int F_MAX_TI = 28;              // TI + 3 columns of x fit a 32-float row of the x tile
constexpr int F_XSLOTS = 4;               // ring of x tiles, 64 rows x 32 floats each
constexpr int F_XSLOT_BYTES = F_KB * 32 * 4;
constexpr int F_HEADER = 256;             // workspace header: [0] max |dY| as bits, [1] inverse scale

enum { FST_PRODUCER = 31, FST_TMA = 32, FST_MMA = 33, FST_EPILOGUE = 34, FST_X = 35 };

template <int BN>
struct FSmem {
    static constexpr int MT = (BN == 64) ? 4 : 2;            // M tiles per CTA: MT * BN = 256 accumulator columns
    static constexpr int A_STAGE = MT * F_A_TILE;
    static constexpr int B_STAGE = BN * 128;                 // BN outputs x 64 fp16
    static constexpr int STAGE = A_STAGE + B_STAGE;
    static constexpr int X_OFFSET = F_NS * STAGE;
    static constexpr int BAR_OFFSET = X_OFFSET + F_XSLOTS * F_XSLOT_BYTES;
    static constexpr int NUM_BARS = 2 * F_NS + 2 * F_XSLOTS + 2;   // full, empty, xfull, xempty, acc_full, drain
    static constexpr int TOTAL = BAR_OFFSET + NUM_BARS * 8 + 16 + 1024;
    static constexpr uint32_t TMEM_COLS = 256;
};

// ---------------------------------------------------------------------------------------------------------------
// pre-pass 1: max |dY| (as the bit pattern of a non-negative float: integer max then is float max)
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
absmax_kernel(const float* __restrict__ v, int64_t n, uint32_t* __restrict__ out_bits) {
    uint32_t m = 0u;
    const int64_t n4 = n >> 2;
    const float4* v4 = reinterpret_cast<const float4*>(v);
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < n4; e += (int64_t)gridDim.x * blockDim.x) {
        const float4 a = v4[e];
        // a NaN has a larger bit pattern than any finite value: it wins the max and turns scaling off
        m = max(m, __float_as_uint(fabsf(a.x))); m = max(m, __float_as_uint(fabsf(a.y)));
        m = max(m, __float_as_uint(fabsf(a.z))); m = max(m, __float_as_uint(fabsf(a.w)));
    }
    if (blockIdx.x == 0 && threadIdx.x < (n & 3)) m = max(m, __float_as_uint(fabsf(v[(n4 << 2) + threadIdx.x])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0 && m != 0u) atomicMax(out_bits, m);
}

// power of two that puts `maxbits` (a non-negative float's bit pattern) into [2^14, 2^15); 1 for zero, inf and NaN
__device__ __forceinline__ float scale_for(uint32_t maxbits) {
    const int e = (int)(maxbits >> 23);            // biased exponent; 0 = zero / subnormal, 255 = inf / NaN
    if (e == 0 || e == 255) return 1.f;
    int k = 14 - (e - 127);
    if (k > 126) k = 126;                           // keep the scale a normal float
    if (k < -126) k = -126;
    return __uint_as_float((uint32_t)(k + 127) << 23);
}

// ---------------------------------------------------------------------------------------------------------------
// pre-pass 2: dYt[o][b] = fp16(dY[b][o] * scale), rows b >= B of the padded pitch written as zeros
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
transpose_scale_kernel(const float* __restrict__ dy, __half* __restrict__ dyt, int64_t B, int out, int64_t b_pitch,
                       uint32_t* __restrict__ header) {
    __shared__ float tile[64][65];
    const float scale = scale_for(header[0]);
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) reinterpret_cast<float*>(header)[1] = 1.f / scale;
    const int64_t b0 = (int64_t)blockIdx.x * 64;
    const int o0 = blockIdx.y * 64;
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;      // 64 x 4
#pragma unroll
    for (int r = 0; r < 16; ++r) {
        const int64_t b = b0 + ty + 4 * r;
        const int o = o0 + tx;
        tile[ty + 4 * r][tx] = (b < B && o < out) ? dy[b * out + o] * scale : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 16; ++r) {
        const int o = o0 + ty + 4 * r;
        const int64_t b = b0 + tx;
        if (o < out && b < b_pitch) dyt[(int64_t)o * b_pitch + b] = __float2half_rn(tile[tx][ty + 4 * r]);
    }
}

// ---------------------------------------------------------------------------------------------------------------
// the GEMM
// ---------------------------------------------------------------------------------------------------------------
template <int BN>
__global__ void __launch_bounds__(F_THREADS, 1)
dcoeff_f16_kernel(const __grid_constant__ CUtensorMap tmap_dyt, const __grid_constant__ CUtensorMap tmap_x,
                  float* __restrict__ dst, int64_t B, int in, int out, int dp1, int TI, int i_tiles,
                  int64_t rows_per_split, int64_t split_stride, int add_to_dst, const uint32_t* __restrict__ header,
                  int32_t* status) {
    using L = FSmem<BN>;
    // f16 x f16 -> f32, both operands K-major, M = 128, N = BN
    constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bars = smem_base + L::BAR_OFFSET;
    auto full = [&](int s) { return bars + 8u * s; };             // producers of the stage + the dY tile's bytes
    auto empty = [&](int s) { return bars + 8u * (F_NS + s); };
    auto xfull = [&](int xs) { return bars + 8u * (2 * F_NS + xs); };
    auto xempty = [&](int xs) { return bars + 8u * (2 * F_NS + F_XSLOTS + xs); };
    const uint32_t acc_full_bar = bars + 8u * (2 * F_NS + 2 * F_XSLOTS);
    const uint32_t drain_bar = bars + 8u * (2 * F_NS + 2 * F_XSLOTS + 1);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L::BAR_OFFSET + L::NUM_BARS * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + L::BAR_OFFSET + L::NUM_BARS * 8 + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int i_t = (int)blockIdx.x % i_tiles;
    const int split = (int)blockIdx.x / i_tiles;
    const int i0 = i_t * TI;
    const int ti = max(0, min(TI, in - i0));
    const int64_t b_begin = (int64_t)split * rows_per_split;      // a multiple of 64
    const int64_t b_end = min(B, b_begin + rows_per_split);
    const int nkb = (int)((b_end - b_begin + F_KB - 1) / F_KB);

    if (threadIdx.x == 0) {
        for (int s = 0; s < F_NS; ++s) { mbar_init(full(s), F_G + 1); mbar_init(empty(s), 1); }
        for (int xs = 0; xs < F_XSLOTS; ++xs) { mbar_init(xfull(xs), 1); mbar_init(xempty(xs), F_G); }
        mbar_init(acc_full_bar, 1);
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == F_MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32((const void*)tmem_slot)), "r"(L::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < F_PRODUCER_WARPS) {
        // ------------------------------ producers ------------------------------
        // warps w and w + 2 ... share stage w % 2; a lane's pairs are (input ii, chunk c of eight batch rows)
        const int my_stage = warp % F_NS, sub = warp / F_NS;
        const int npairs = ti * 8;
        const int x_col0 = i0 & 3;                 // the x tile starts at the 16-byte boundary below input i0
        bool alive = true;
        for (int kb = my_stage; kb < nkb && alive; kb += F_NS) {
            const int s = my_stage;
            const uint32_t ph = (uint32_t)((kb / F_NS) & 1);
            const int xslot = kb % F_XSLOTS;
            const uint32_t xph = (uint32_t)((kb / F_XSLOTS) & 1);
            if (!mbar_wait(xfull(xslot), xph, abort_flag, status, FST_PRODUCER)) { alive = false; break; }
            const uint32_t xs = smem_base + L::X_OFFSET + xslot * F_XSLOT_BYTES;
            float xc[F_MAX_ROUNDS][8];
#pragma unroll
            for (int r = 0; r < F_MAX_ROUNDS; ++r) {
                const int pair = lane + 32 * (F_G * r + sub);
#pragma unroll
                for (int e = 0; e < 8; ++e) xc[r][e] = 0.f;
                if (pair < npairs) {
                    const int ii = pair >> 3, c = pair & 7;
#pragma unroll
                    for (int e = 0; e < 8; ++e)
                        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(xc[r][e])
                                     : "r"(xs + (uint32_t)(((8 * c + e) * 32 + x_col0 + ii) * 4)));
                }
            }
            if (!mbar_wait(empty(s), ph ^ 1u, abort_flag, status, FST_PRODUCER)) { alive = false; break; }
            const uint32_t a_stage = smem_base + s * L::STAGE;
#pragma unroll
            for (int r = 0; r < F_MAX_ROUNDS; ++r) {
                const int pair = lane + 32 * (F_G * r + sub);
                if (pair < npairs) {
                    const int ii = pair >> 3, c = pair & 7;
                    float t2[8], ta[8], tb[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const float t = tanh_fast(xc[r][e]);
                        t2[e] = 2.f * t; ta[e] = 1.f; tb[e] = t;     // T_0 = 1, T_{-1} = T_1 = t
                    }
                    // slot row = ii*(deg+1) + d lives at a_stage + row * 128 (M tiles are 128 rows = 16 KB apart, so
                    // the address is linear in the row); its chunk c sits at chunk position c ^ (row % 8), and
                    // since a_stage is 1024-byte aligned, row % 8 is bits 7-9 of the linear address
                    uint32_t lin = a_stage + (uint32_t)(ii * dp1) * 128u + ((uint32_t)c << 4);
                    auto store8 = [&](const float (&v)[8]) {
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const __half2 h = __floats2half2_rn(v[2 * e], v[2 * e + 1]);
                            w[e] = *reinterpret_cast<const uint32_t*>(&h);
                        }
                        const uint32_t dsta = lin ^ ((lin >> 3) & 0x70u);
                        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};"
                                     ::"r"(dsta), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
                        lin += 128u;
                    };
                    store8(ta);                                        // degree 0
                    int d = 1;
                    for (; d + 7 < dp1; d += 8) {                      // eight degrees per trip
#pragma unroll
                        for (int h = 0; h < 4; ++h) {
#pragma unroll
                            for (int e = 0; e < 8; ++e) tb[e] = fmaf(t2[e], ta[e], -tb[e]);
                            store8(tb);
#pragma unroll
                            for (int e = 0; e < 8; ++e) ta[e] = fmaf(t2[e], tb[e], -ta[e]);
                            store8(ta);
                        }
                    }
                    for (; d < dp1; d += 2) {
#pragma unroll
                        for (int e = 0; e < 8; ++e) tb[e] = fmaf(t2[e], ta[e], -tb[e]);
                        store8(tb);
                        if (d + 1 < dp1) {
#pragma unroll
                            for (int e = 0; e < 8; ++e) ta[e] = fmaf(t2[e], tb[e], -ta[e]);
                            store8(ta);
                        }
                    }
                }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(full(s));
                // the x values were consumed above (their loads fed the stores), so the slot can be refilled
                mbar_arrive(xempty(xslot));
            }
        }
    } else if (warp == F_TMA_WARP) {
        // ------------------------------ dY tiles ------------------------------
        if (lane == 0) {
            bool alive = true;
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % F_NS;
                const uint32_t ph = (uint32_t)((kb / F_NS) & 1);
                if (!mbar_wait(empty(s), ph ^ 1u, abort_flag, status, FST_TMA)) { alive = false; break; }
                mbar_arrive_expect_tx(full(s), (uint32_t)L::B_STAGE);
                tma_load_2d(smem_base + s * L::STAGE + L::A_STAGE, &tmap_dyt, (int)(b_begin + (int64_t)kb * F_KB), 0, full(s));
            }
            if (!alive) {
                const uint64_t t0 = globaltimer_ns();
                while (globaltimer_ns() - t0 < 200000ull) { }
            }
        }
    } else if (warp == F_X_WARP) {
        // ------------------------------ x tiles ------------------------------
        if (lane == 0) {
            bool alive = true;
            for (int kb = 0; kb < nkb; ++kb) {
                const int xslot = kb % F_XSLOTS;
                const uint32_t xph = (uint32_t)((kb / F_XSLOTS) & 1);
                if (!mbar_wait(xempty(xslot), xph ^ 1u, abort_flag, status, FST_X)) { alive = false; break; }
                mbar_arrive_expect_tx(xfull(xslot), (uint32_t)F_XSLOT_BYTES);
                tma_load_2d(smem_base + L::X_OFFSET + xslot * F_XSLOT_BYTES, &tmap_x, i0 & ~3,
                            (int)(b_begin + (int64_t)kb * F_KB), xfull(xslot));
            }
            if (!alive) {
                const uint64_t t0 = globaltimer_ns();
                while (globaltimer_ns() - t0 < 200000ull) { }
            }
        }
    } else if (warp == F_MMA_WARP) {
        // ------------------------------ MMA issue (warp-uniform loop, one elected lane issues) ------------------------------
        const bool elected = elect_one_sync();
        bool alive = true;
        const uint64_t a_desc0 = make_smem_desc(smem_base);
        const uint64_t b_desc0 = make_smem_desc(smem_base + L::A_STAGE);
        const uint32_t a_hi = (uint32_t)(a_desc0 >> 32), b_hi = (uint32_t)(b_desc0 >> 32);
        const int mt_used = (ti * dp1 + 127) / 128;
        int s = 0; uint32_t ph = 0;
        for (int kb = 0; kb < nkb; ++kb) {
            if (!__all_sync(0xffffffffu, mbar_wait(full(s), ph, abort_flag, status, FST_MMA))) { alive = false; break; }
            tc_fence_after();
            const uint32_t a_lo = (uint32_t)a_desc0 + (uint32_t)((s * L::STAGE) >> 4);
            const uint32_t b_lo = (uint32_t)b_desc0 + (uint32_t)((s * L::STAGE) >> 4);
            const uint32_t later = (uint32_t)(kb != 0);
#pragma unroll
            for (int mt = 0; mt < L::MT; ++mt) {
                if (mt < mt_used) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) {            // 16 batch rows per MMA: +32 bytes in both operands' rows
                        const uint64_t ad = desc_from_words(a_lo + (uint32_t)((mt * F_A_TILE) >> 4) + 2u * k, a_hi);
                        const uint64_t bd = desc_from_words(b_lo + 2u * k, b_hi);
                        if (elected) {
                            if (k != 0) umma<CHEBYKAN_MODE_BF16>(tmem_base + (uint32_t)(mt * BN), ad, bd, IDESC, 1u);
                            else umma<CHEBYKAN_MODE_BF16>(tmem_base + (uint32_t)(mt * BN), ad, bd, IDESC, later);
                        }
                    }
                }
            }
            if (elected) umma_commit(empty(s));
            __syncwarp();
            if (++s == F_NS) { s = 0; ph ^= 1u; }
        }
        if (elected) {
            if (alive) umma_commit(acc_full_bar);
            else {
                umma_commit(drain_bar);
                const uint64_t t0 = globaltimer_ns();
                while (!mbar_try_wait(drain_bar, 0) && globaltimer_ns() - t0 < 10000000ull) { }
            }
        }
        __syncwarp();
    }

    // ------------------------------ epilogue: warps 0-3 own TMEM lanes 32w..32w+31 ------------------------------
    if (warp < 4) {
        const bool ok = nkb == 0 ? true : mbar_wait(acc_full_bar, 0, abort_flag, status, FST_EPILOGUE);
        if (__all_sync(0xffffffffu, ok)) {
            tc_fence_after();
            const float inv_scale = __ldg(reinterpret_cast<const float*>(header) + 1);
#pragma unroll 1
            for (int mt = 0; mt < L::MT; ++mt) {
                if (mt * 128 >= ti * dp1) break;
                const int kk = mt * 128 + warp * 32 + lane;      // slot: M tile mt, TMEM lane warp*32+lane
                const bool valid = kk < ti * dp1;
                const int ii = kk / dp1, d = kk % dp1;
                float* base = dst + (int64_t)split * split_stride + ((int64_t)(i0 + ii) * out) * dp1 + d;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    if (c0 >= out) break;
                    uint32_t r[32];
                    if (nkb > 0) {
                        tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(mt * BN + c0), r);
                        tmem_ld_wait();
                    } else {
#pragma unroll
                        for (int e = 0; e < 32; ++e) r[e] = 0u;
                    }
                    if (valid) {
#pragma unroll
                        for (int e = 0; e < 32; ++e) {
                            const int col = c0 + e;
                            if (col < out) {
                                float* q = base + (int64_t)col * dp1;
                                const float v = __uint_as_float(r[e]) * inv_scale;
                                *q = add_to_dst ? (*q + v) : v;
                            }
                        }
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == F_MMA_WARP) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(L::TMEM_COLS) : "memory");
    }
}

struct FPlan { int TI, i_tiles, bn, splits; int64_t rows_per_split, b_pitch; };

FPlan f16_plan(int64_t B, int64_t in, int64_t out, int64_t deg) {
    FPlan p{};
    const int dp1 = (int)deg + 1;
    p.bn = out <= 64 ? 64 : 128;
    const int mt = p.bn == 64 ? 4 : 2;
    p.TI = mt * 128 / dp1;
    if (p.TI > F_MAX_TI) p.TI = F_MAX_TI;
    if (p.TI > in) p.TI = (int)in;
    p.i_tiles = (int)ceil_div(in, p.TI);
    // split the batch so that the CTAs fill whole waves of the 148 SMs (least waves x rows per CTA)
    int64_t max_splits = ceil_div(B, 2048);
    if (max_splits < 1) max_splits = 1;
    int64_t cand_hi = ceil_div(4 * 148, p.i_tiles);
    if (cand_hi > max_splits) cand_hi = max_splits;
    int64_t best_s = 1, best_cost = -1;
    for (int64_t sp = 1; sp <= cand_hi; ++sp) {
        const int64_t rows = round_up(ceil_div(B, sp), F_KB);
        const int64_t ctas = p.i_tiles * ceil_div(B, rows);
        const int64_t cost = ceil_div(ctas, 148) * (rows + 4096);     // + fixed cost of a CTA (setup, epilogue)
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_s = sp; }
    }
    p.rows_per_split = round_up(ceil_div(B, best_s), F_KB);
    p.splits = (int)ceil_div(B, p.rows_per_split);
    if (p.splits < 1) p.splits = 1;
    p.b_pitch = round_up(B, 64);          // fp16 row pitch of dYt: a multiple of 16 bytes, zero-filled past B
    return p;
}

template <int BN>
int launch_f16(const CUtensorMap& tm_dyt, const CUtensorMap& tm_x, float* dst, int64_t B, int in, int out, int dp1,
               const FPlan& p, int64_t split_stride, int add, const uint32_t* header, int32_t* status, cudaStream_t s) {
    using L = FSmem<BN>;
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kernel = dcoeff_f16_kernel<BN>;
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        int rc = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
        if (rc) return rc;
        attr_set[dev] = true;
    }
    const unsigned grid = (unsigned)((int64_t)p.i_tiles * p.splits);
    kernel<<<grid, F_THREADS, L::TOTAL, s>>>(tm_dyt, tm_x, dst, B, in, out, dp1, p.TI, p.i_tiles, p.rows_per_split,
                                             split_stride, add, header, status);
    return check_cuda(cudaGetLastError());
}

}  // namespace

// CHEBYKAN_DCOEFF_NARROW=tf32 in the environment keeps narrow layers on the kind::tf32 kernel (A/B timing; read once)
static bool narrow_dcoeff_in_tf32() {
    static const bool v = [] {
        const char* e = getenv("CHEBYKAN_DCOEFF_NARROW");
        return e != nullptr && strcmp(e, "tf32") == 0;
    }();
    return v;
}

bool dcoeff_f16_supported(int64_t B, int64_t in, int64_t out, int64_t deg) {
    return B > 0 && B < ((int64_t)1 << 31) - 128 && out <= 128 && (in % 4) == 0 && deg + 1 <= 128 && !narrow_dcoeff_in_tf32();
}

int64_t dcoeff_f16_workspace_bytes(int64_t B, int64_t in, int64_t out, int64_t deg) {
    const FPlan p = f16_plan(B, in, out, deg);
    const int64_t partials = p.splits > 1 ? (int64_t)p.splits * in * out * (deg + 1) * 4 : 0;
    return F_HEADER + round_up(out * p.b_pitch * 2, 256) + partials;
}

int launch_dcoeff_f16(const float* x, const float* dy, float* dc, void* ws, int64_t ws_bytes, int64_t B, int64_t in,
                      int64_t out, int64_t deg, int accumulate, int32_t* status, cudaStream_t s) {
    const FPlan p = f16_plan(B, in, out, deg);
    const int dp1 = (int)deg + 1;
    const int64_t n = in * out * dp1;
    if (ws == nullptr || ws_bytes < dcoeff_f16_workspace_bytes(B, in, out, deg)) return CHEBYKAN_EWORKSPACE;
    EncodeTiledFn encode = get_encode_fn();
    if (!encode) return CHEBYKAN_ECUDA;
    uint32_t* header = reinterpret_cast<uint32_t*>(ws);
    __half* dyt = reinterpret_cast<__half*>(reinterpret_cast<char*>(ws) + F_HEADER);
    float* partials = reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + F_HEADER + round_up(out * p.b_pitch * 2, 256));
    int rc;
    // pre-pass: max |dY|, then the scaled fp16 transpose (and the inverse scale for the epilogue)
    if ((rc = check_cuda(cudaMemsetAsync(header, 0, 8, s)))) return rc;
    {
        int64_t blocks = ceil_div(ceil_div(B * out, 4), 256);
        if (blocks > 148 * 8) blocks = 148 * 8;
        if (blocks < 1) blocks = 1;
        absmax_kernel<<<(unsigned)blocks, 256, 0, s>>>(dy, B * out, header);
        if ((rc = check_cuda(cudaGetLastError()))) return rc;
        const dim3 grid((unsigned)ceil_div(p.b_pitch, 64), (unsigned)ceil_div(out, 64));
        transpose_scale_kernel<<<grid, 256, 0, s>>>(dy, dyt, B, (int)out, p.b_pitch, header);
        if ((rc = check_cuda(cudaGetLastError()))) return rc;
    }
    const cuuint32_t estr[2] = {1, 1};
    CUtensorMap tm_dyt, tm_x;
    {
        // dYt[out][b_pitch] fp16: boxes of 64 batch rows (128 bytes) x BN outputs, outputs past `out` read as zeros
        const cuuint64_t dims[2] = {(cuuint64_t)p.b_pitch, (cuuint64_t)out};
        const cuuint64_t strides[1] = {(cuuint64_t)(p.b_pitch * 2)};
        const cuuint32_t box[2] = {(cuuint32_t)F_KB, (cuuint32_t)p.bn};
        const CUresult r = encode(&tm_dyt, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, dyt, dims, strides, box, estr,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { set_last_cuda_error((int)r); return CHEBYKAN_ECUDA; }
    }
    {
        // x[B][in] fp32: a K block's tile is 64 rows by 32 floats starting at the 16-byte boundary below the
        // CTA's first input (rows and columns outside x read as zeros)
        const cuuint64_t dims[2] = {(cuuint64_t)in, (cuuint64_t)B};
        const cuuint64_t strides[1] = {(cuuint64_t)(in * 4)};
        const cuuint32_t box[2] = {32, (cuuint32_t)F_KB};
        const CUresult r = encode(&tm_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(x), dims, strides, box,
                                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { set_last_cuda_error((int)r); return CHEBYKAN_ECUDA; }
    }
    const bool direct = p.splits == 1;
    float* dst = direct ? dc : partials;
    const int add = direct && accumulate;
    if (p.bn == 64) rc = launch_f16<64>(tm_dyt, tm_x, dst, B, (int)in, (int)out, dp1, p, n, add, header, status, s);
    else rc = launch_f16<128>(tm_dyt, tm_x, dst, B, (int)in, (int)out, dp1, p, n, add, header, status, s);
    if (rc) return rc;
    if (!direct) rc = launch_dcoeff_reduce(partials, dc, n, p.splits, accumulate, s);
    return rc;
}

}  // namespace chebykan
