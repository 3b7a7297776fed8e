// Tensor-core forward for NARROW layers (at most 128 outputs) on sm_100a, with the generated basis tile held in
// TENSOR MEMORY instead of shared memory.
//
// Same math as fwd_tc.cu (reference kan/basis/chebyshev.py:92-101,119-145: tanh, basis expansion, einsum):
// Y[B, out] = Phi[B, K] * W[K, out], K = in*(deg+1), Phi generated on chip by the three-term recurrence.
//
// Why a second kernel.  With one tile of 64 or 128 outputs an MMA (M=128, N=64) is so small that the shared-memory
// traffic of its A operand bounds it: every basis value is written once by a producer (4 bytes in tf32) and read once
// by the tensor pipe, 8 KB per MMA against 128 bytes per clock of shared-memory bandwidth, more than the MMA's own
// 32 cycles.  tcgen05.mma can take A from tensor memory: the producers store their values with tcgen05.st, one TMEM
// lane per batch row, and the MMA reads them there, so shared memory only carries the coefficient tiles (TMA) and
// the x tiles.
//
//   producer warps   one thread per (row, 16 tf32 / 32 bf16 inputs): x from the shared-memory tile (TMA, 128B
//                    swizzle) -> tanh -> recurrence in registers -> tcgen05.st of 16 columns per degree
//   warp MMA         one lane issues tcgen05.mma [D], [A in TMEM], B descriptor (K-major W tile, 128B swizzle)
//   warp W           TMA loads of the packed coefficient tiles, KP K blocks per stage
//   warp X           TMA loads of the x tiles (two slots per row sub-tile)
//   4 epilogue warps tcgen05.ld of the accumulator -> y
//
// A K block is 32 TMEM columns (one degree of 32 tf32 or 64 bf16 inputs = four MMAs); a stage is KP K blocks of A in
// TMEM plus the matching W panels in shared memory, handed over with one full and one empty barrier; the ring takes
// whatever TMEM columns the accumulators leave.  A CTA may work on two row sub-tiles of 128 rows at once (two sets of
// eight producer warps, two accumulators): every W stage then feeds 256 rows, which halves the coefficient bytes the
// SM pulls from L2 per row (the whole packed matrix is re-read for every row tile).
//
// Every mbarrier wait is bounded; on expiry the kernel records a role code in *status, drains and frees its TMEM.
#include <cuda_fp16.h>
#include <stdlib.h>
#include <string.h>
#include "tc_common.cuh"

namespace chebykan {

namespace {
using namespace tc;

enum { TS_PRODUCER = 21, TS_TMA_W = 22, TS_MMA_A = 23, TS_MMA_B = 24, TS_MMA_ACC = 25, TS_EPILOGUE = 26, TS_X_LOAD = 27,
       TS_X_WAIT = 28 };

// NSUBM: row sub-tiles (of 128 rows) a CTA works on at once; KP: K blocks per stage; NACC: accumulator buffers.
// The A ring takes the tensor-memory columns the accumulators leave: NSTG = (512 - NACC*NSUBM*BN) / (NSUBM*KP*32).
#define TOTAL_CHECK(v) ((v) <= 232448)
// Internal mode of this file: fp16 operands (basis values and a power-of-two scaled fp16 copy of the coefficients)
// with the bf16 kernel's layouts.  fp16 carries tf32's 11 significant bits at half the tensor-memory columns, stores
// and MMAs, and the basis values lie in [-1, 1]: this is what the TF32 math mode runs on narrow layers.
constexpr int TS_MODE_F16 = 16;
template <int MODE, int BN, int NSUBM_, int KP_, int NACC_>
struct TsCfg {
    static constexpr bool BF16 = MODE == CHEBYKAN_MODE_BF16 || MODE == TS_MODE_F16;   // 16-bit operands
    static constexpr int NSUBM = NSUBM_;
    static constexpr int KP = KP_;
    static constexpr int NACC = NACC_;
    static constexpr int IB = BF16 ? 64 : 32;           // inputs per K block
    static constexpr int EPT = IB / 2;                  // inputs per producer thread (two threads share a row's block)
    static constexpr int XBOXES = IB / 32;              // x boxes of 32 fp32 per input block
    static constexpr int NPW = 8 * NSUBM;               // producer warps
    static constexpr int EPI_WARP0 = NPW, MMA_WARP = NPW + 4, W_WARP = NPW + 5, X_WARP = NPW + 6;
    static constexpr int NUM_THREADS = (NPW + 8) * 32;  // + 4 epilogue, MMA, W, X, one idle (whole warpgroups)
    // register split (setmaxnreg): 65536 = producers + others
    static constexpr int PRODUCER_REGS = NSUBM == 1 ? 168 : 96;
    static constexpr int OTHER_REGS = NSUBM == 1 ? 88 : 48;
    static constexpr int D_COLS = NACC * NSUBM * BN;
    static constexpr int NSTG = (512 - D_COLS) / (NSUBM * KP * 32);      // A stages (TMEM)
    static constexpr int A_COLS = NSUBM * NSTG * KP * 32;
    static constexpr int B_PANEL_BYTES = BN * 128;
    static constexpr int B_STAGE_BYTES = KP * B_PANEL_BYTES;
    static constexpr int NSB = NSTG;                    // one ring: stage s holds the W panels and the A columns of the same K blocks
    static constexpr int X_SLOT_BYTES = XBOXES * 128 * 128;       // 128 rows x 128 bytes per box
    static constexpr int NXS = 2;                                 // x slots per sub-tile
    static constexpr int B_OFFSET = 0;
    static constexpr int X_OFFSET = NSB * B_STAGE_BYTES;
    static constexpr int BAR_OFFSET = X_OFFSET + NSUBM * NXS * X_SLOT_BYTES;
    // full[NSTG] empty[NSTG] acc_full[2] acc_empty[2] x_full[NSUBM*NXS] x_empty[NSUBM*NXS] drain
    static constexpr int NUM_BARS = 2 * NSTG + 4 + 2 * NSUBM * NXS + 1;
    static_assert(TOTAL_CHECK(BAR_OFFSET + NUM_BARS * 8 + 16 + 1024), "shared memory");
    static constexpr int TOTAL = BAR_OFFSET + NUM_BARS * 8 + 16 + 1024;
    static_assert(NSTG >= 2 && D_COLS + A_COLS <= 512, "tensor memory holds 512 columns");
};

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem descriptor]
template <int MODE>
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    if (MODE == CHEBYKAN_MODE_BF16 || MODE == TS_MODE_F16) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
            ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
            ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
    }
}

template <int MODE, int BN, int NSUBM_, int KP_, int NACC_>
__global__ void __launch_bounds__(TsCfg<MODE, BN, NSUBM_, KP_, NACC_>::NUM_THREADS, 1)
fwd_ts_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
              float* __restrict__ y, int64_t B, int in, int out, int dp1, int64_t num_tiles, int32_t* status,
              const float* __restrict__ out_scale, const float* __restrict__ bias) {
    // `dp1` counts the degrees that take K slots: degrees 1..deg (K slot d holds T_{d+1}).  Degree 0, the constant 1,
    // is the bias vector the epilogue adds.
    using C = TsCfg<MODE, BN, NSUBM_, KP_, NACC_>;
    constexpr int NSUBM = C::NSUBM, KP = C::KP, NSTG = C::NSTG, NSB = C::NSB, NACC = C::NACC, NXS = C::NXS;
    constexpr int IB = C::IB, EPT = C::EPT;
    constexpr uint32_t FMT = MODE == TS_MODE_F16 ? 0u : (C::BF16 ? 1u : 2u);      // f16, bf16, tf32
    constexpr uint32_t IDESC = (1u << 4) | (FMT << 7) | (FMT << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    constexpr uint32_t D_COL0 = 0, A_COL0 = C::D_COLS;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bars = smem_base + C::BAR_OFFSET;
    // full(s): all producer warps have stored the stage's A columns and the stage's W panels have landed;
    // empty(s): the MMAs that read the stage have retired
    auto full = [&](int s) { return bars + 8u * s; };
    auto empty = [&](int s) { return bars + 8u * (NSTG + s); };
    auto acc_full_bar = [&](int a) { return bars + 8u * (2 * NSTG + a); };
    auto acc_empty_bar = [&](int a) { return bars + 8u * (2 * NSTG + 2 + a); };
    auto x_full = [&](int sub, int slot) { return bars + 8u * (2 * NSTG + 4 + sub * NXS + slot); };
    auto x_empty = [&](int sub, int slot) { return bars + 8u * (2 * NSTG + 4 + NSUBM * NXS + sub * NXS + slot); };
    const uint32_t drain_bar = bars + 8u * (2 * NSTG + 4 + 2 * NSUBM * NXS);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + C::BAR_OFFSET + C::NUM_BARS * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + C::BAR_OFFSET + C::NUM_BARS * 8 + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_iblk = (in + IB - 1) / IB;
    const int nkb = n_iblk * dp1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTG; ++s) { mbar_init(full(s), C::NPW + 1); mbar_init(empty(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(acc_full_bar(a), 1); mbar_init(acc_empty_bar(a), 4); }
        for (int sub = 0; sub < NSUBM; ++sub)
            for (int slot = 0; slot < NXS; ++slot) { mbar_init(x_full(sub, slot), 1); mbar_init(x_empty(sub, slot), 8); }
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == C::MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32((const void*)tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < C::NPW) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(C::PRODUCER_REGS));
    else               asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(C::OTHER_REGS));

    if (warp < C::NPW) {
        // ------------------------------ producers ------------------------------
        const int sub = warp >> 3;               // row sub-tile of this warp set
        const int q = warp & 3;                  // TMEM lane quarter (a warp may only touch lanes 32*(warp%4)..+31)
        const int h = (warp >> 2) & 1;           // which half of the K block's 32 columns this thread writes
        const int r = q * 32 + lane;             // row inside the sub-tile = TMEM lane
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        float tt[EPT], ta[EPT], tb[EPT];
        uint32_t inc = TF32_HALF_ULP;
        int s = 0; uint32_t ph = 0;
        int xs = 0; uint32_t xph = 0;
        bool alive = true;

        // one K block's values of this thread -> 16 columns of the stage, straight-line code
        auto emit = [&](uint32_t taddr, const float (&v)[EPT]) {
            uint32_t w[16];
            if (C::BF16) {
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    if (MODE == TS_MODE_F16) {
                        const __half2 p2 = __floats2half2_rn(v[(2 * c) % EPT], v[(2 * c + 1) % EPT]);
                        w[c] = *reinterpret_cast<const uint32_t*>(&p2);
                    } else {
                        const __nv_bfloat162 p2 = __floats2bfloat162_rn(v[(2 * c) % EPT], v[(2 * c + 1) % EPT]);
                        w[c] = *reinterpret_cast<const uint32_t*>(&p2);
                    }
                }
            } else {
#pragma unroll
                for (int c = 0; c < 16; ++c) w[c] = tf32_rna(v[c % EPT], inc);
            }
            tmem_st16(taddr, w);
        };

        // A stage never spans two input blocks: the K blocks of an input block are cut into stages of KP degrees (the
        // last one shorter), so that inside a stage the degree parity, the column offsets and the trip count are
        // compile-time and the recurrence runs as straight-line code.  KP is even: a stage starts on an even degree
        // with ta = T_{d0-2}, tb = T_{d0-1}.
        static_assert(KP % 2 == 0, "stages start on even degrees");
        for (int64_t tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
            for (int ib = 0; ib < n_iblk && alive; ++ib) {
                {
                    const bool ok = mbar_wait(x_full(sub, xs), xph, abort_flag, status, TS_X_WAIT);
                    if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
                }
                // this thread's EPT inputs of row r: box (h for bf16, 0 for tf32), 16-byte chunks c0..; the tile is
                // 128B-swizzled: chunk c of row r sits at chunk position c ^ (r & 7)
                const uint32_t xbase = smem_base + C::X_OFFSET + (uint32_t)((sub * NXS + xs) * C::X_SLOT_BYTES) +
                                       (C::BF16 ? (uint32_t)(h * 16384) : 0u) + (uint32_t)(r * 128);
                const int c0 = C::BF16 ? 0 : h * 4;
                bool finite = true;
#pragma unroll
                for (int c = 0; c < EPT / 4; ++c) {
                    float v0, v1, v2, v3;
                    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                                 : "=f"(v0), "=f"(v1), "=f"(v2), "=f"(v3)
                                 : "r"(xbase + (uint32_t)((((c0 + c) ^ (r & 7))) << 4)));
                    const float vv[4] = {v0, v1, v2, v3};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float t = tanh_fast(vv[e]);
                        finite = finite && (t == t);
                        tt[4 * c + e] = 2.f * t; ta[4 * c + e] = t; tb[4 * c + e] = fmaf(2.f * t, t, -1.f);   // T_1, T_2
                    }
                }
                inc = finite ? TF32_HALF_ULP : 0u;
                for (int d0 = 0; d0 < dp1 && alive; d0 += KP) {
                    const int np = (dp1 - d0 < KP) ? dp1 - d0 : KP;
                    {
                        const bool ok = mbar_wait(empty(s), ph ^ 1u, abort_flag, status, TS_PRODUCER);
                        if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
                        tc_fence_after();
                    }
                    const uint32_t st0 = lane_addr + A_COL0 + (uint32_t)((sub * NSTG + s) * KP * 32 + h * 16);
                    if (d0 == 0) {
                        emit(st0, ta);                                     // the block's first degree (T_1)
                        // the x slot goes back after a store whose data derives from it has been issued (an mbarrier
                        // arrive does not wait for this thread's outstanding ld.shared, the store does)
                        __syncwarp();
                        if (lane == 0) mbar_arrive(x_empty(sub, xs));
                        if (1 < np) emit(st0 + 32, tb);                    // T_2
                    } else {
#pragma unroll
                        for (int e = 0; e < EPT; ++e) ta[e] = fmaf(tt[e], tb[e], -ta[e]);
                        emit(st0, ta);
                        if (1 < np) {
#pragma unroll
                            for (int e = 0; e < EPT; ++e) tb[e] = fmaf(tt[e], ta[e], -tb[e]);
                            emit(st0 + 32, tb);
                        }
                    }
#pragma unroll
                    for (int p = 2; p < KP; p += 2) {
                        if (p < np) {
#pragma unroll
                            for (int e = 0; e < EPT; ++e) ta[e] = fmaf(tt[e], tb[e], -ta[e]);
                            emit(st0 + (uint32_t)(p * 32), ta);
                        }
                        if (p + 1 < np) {
#pragma unroll
                            for (int e = 0; e < EPT; ++e) tb[e] = fmaf(tt[e], ta[e], -tb[e]);
                            emit(st0 + (uint32_t)((p + 1) * 32), tb);
                        }
                    }
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(full(s));
                    if (++s == NSTG) { s = 0; ph ^= 1u; }
                }
                if (++xs == NXS) { xs = 0; xph ^= 1u; }
            }
        }
    } else if (warp == C::W_WARP) {
        // ------------------------------ coefficient tiles ------------------------------
        if (lane == 0) {
            int s = 0; uint32_t ph = 0;
            bool alive = true;
            for (int64_t tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
                for (int ib = 0; ib < n_iblk && alive; ++ib) {
                    for (int d0 = 0; d0 < dp1 && alive; d0 += KP) {      // the producers' stages: KP degrees of one input block
                        const int np = (dp1 - d0 < KP) ? dp1 - d0 : KP;
                        const int kb = ib * dp1 + d0;
                        if (!mbar_wait(empty(s), ph ^ 1u, abort_flag, status, TS_TMA_W)) { alive = false; break; }
                        const uint32_t dst = smem_base + C::B_OFFSET + s * C::B_STAGE_BYTES;
                        mbar_arrive_expect_tx(full(s), (uint32_t)(np * C::B_PANEL_BYTES));
                        for (int p = 0; p < np; ++p)
                            tma_load_2d(dst + p * C::B_PANEL_BYTES, &tmap_w, (kb + p) * IB, 0, full(s));
                        if (++s == NSTG) { s = 0; ph ^= 1u; }
                    }
                }
            }
            if (!alive) {
                const uint64_t t0 = globaltimer_ns();
                while (globaltimer_ns() - t0 < 200000ull) { }      // let the copies in flight land
            }
        }
    } else if (warp == C::X_WARP) {
        // ------------------------------ x tiles ------------------------------
        if (lane == 0) {
            int xs = 0; uint32_t xph = 0;
            bool alive = true;
            for (int64_t tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
                for (int ib = 0; ib < n_iblk && alive; ++ib) {
                    for (int sub = 0; sub < NSUBM; ++sub) {
                        if (!mbar_wait(x_empty(sub, xs), xph ^ 1u, abort_flag, status, TS_X_LOAD)) { alive = false; break; }
                        const int m0 = (int)(tile * (128 * NSUBM) + sub * 128);
                        const uint32_t dst = smem_base + C::X_OFFSET + (uint32_t)((sub * NXS + xs) * C::X_SLOT_BYTES);
                        mbar_arrive_expect_tx(x_full(sub, xs), (uint32_t)C::X_SLOT_BYTES);
                        for (int bx = 0; bx < C::XBOXES; ++bx)      // rows past B and inputs past `in` read as zeros
                            tma_load_2d(dst + bx * 16384, &tmap_x, ib * IB + bx * 32, m0, x_full(sub, xs));
                    }
                    if (++xs == NXS) { xs = 0; xph ^= 1u; }
                }
            }
            if (!alive) {
                const uint64_t t0 = globaltimer_ns();
                while (globaltimer_ns() - t0 < 200000ull) { }
            }
        }
    } else if (warp == C::MMA_WARP) {
        // ------------------------------ MMA issue ------------------------------
        // The whole warp runs this loop in lock step and only the MMA / commit instructions themselves are executed by
        // one elected lane.  The operands of tcgen05.mma live in uniform registers: inside a divergent region (a loop
        // under `if (lane == 0)`) the compiler has to move every address from a vector register first, which costs
        // more than the 32 cycles an N = 64 MMA occupies the tensor pipe.  Operand addresses are per-stage bases plus
        // compile-time offsets (the descriptor's high word never changes; its low word is a 32-bit add), the accumulate
        // predicate is a constant except for a tile's very first MMA, and a stage takes one wait and one commit.
        {
            const bool elected = elect_one_sync();
            int sa = 0; uint32_t pha = 0;
            int acc = 0; uint32_t acc_ph = 0;
            bool alive = true;
            const uint64_t desc0 = make_smem_desc(smem_base + C::B_OFFSET);
            const uint32_t desc_hi = (uint32_t)(desc0 >> 32), desc_lo0 = (uint32_t)desc0;
            auto issue = [&](uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, bool acc_const_one, uint32_t acc_dyn) {
                const uint64_t b_desc = desc_from_words(b_lo, desc_hi);
                if (elected) {
                    if (acc_const_one) umma_ts<MODE>(d_tmem, a_tmem, b_desc, IDESC, 1u);
                    else umma_ts<MODE>(d_tmem, a_tmem, b_desc, IDESC, acc_dyn);
                }
            };
            for (int64_t tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
                if (!__all_sync(0xffffffffu, mbar_wait(acc_empty_bar(acc), acc_ph ^ 1u, abort_flag, status, TS_MMA_ACC))) { alive = false; break; }
                tc_fence_after();
                const uint32_t dacc = tmem_base + D_COL0 + (uint32_t)(acc * NSUBM * BN);
                for (int ib = 0; ib < n_iblk && alive; ++ib) {
                  for (int d0 = 0; d0 < dp1 && alive; d0 += KP) {        // the producers' stages
                    const int np = (dp1 - d0 < KP) ? dp1 - d0 : KP;
                    const uint32_t a0 = tmem_base + A_COL0 + (uint32_t)(sa * KP * 32);
                    const uint32_t b0 = desc_lo0 + (uint32_t)((sa * C::B_STAGE_BYTES) >> 4);
                    if (!__all_sync(0xffffffffu, mbar_wait(full(sa), pha, abort_flag, status, TS_MMA_A))) { alive = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int p = 0; p < KP; ++p) {
                        if (p < np) {
#pragma unroll
                            for (int k = 0; k < 4; ++k) {          // 4 x 8 columns of A, 4 x 32 bytes of each W row
#pragma unroll
                                for (int sub = 0; sub < NSUBM; ++sub)
                                    issue(dacc + (uint32_t)(sub * BN), a0 + (uint32_t)(sub * NSTG * KP * 32 + p * 32 + k * 8),
                                          b0 + (uint32_t)((p * C::B_PANEL_BYTES) >> 4) + 2u * k, (p | k) != 0, (uint32_t)((ib | d0) != 0));
                            }
                        }
                    }
                    if (elected) umma_commit(empty(sa));
                    __syncwarp();
                    if (++sa == NSTG) { sa = 0; pha ^= 1u; }
                  }
                }
                if (alive && elected) umma_commit(acc_full_bar(acc));
                __syncwarp();
                if (++acc == NACC) { acc = 0; acc_ph ^= 1u; }
            }
            if (!alive && elected) {
                umma_commit(drain_bar);
                const uint64_t t0 = globaltimer_ns();
                while (!mbar_try_wait(drain_bar, 0) && globaltimer_ns() - t0 < 10000000ull) { }
            }
            __syncwarp();
        }
    } else if (warp >= C::EPI_WARP0 && warp < C::EPI_WARP0 + 4) {
        // ------------------------------ epilogue ------------------------------
        const int q = warp & 3;
        int acc = 0; uint32_t acc_ph = 0;
        bool alive = true;
        const bool vec4 = (out & 3) == 0;
        // fp16 operands: the coefficients were scaled by a power of two when they were packed; its inverse is exact
        const float osc = (MODE == TS_MODE_F16) ? __ldg(out_scale) : 1.f;
        for (int64_t tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
            const bool ok = mbar_wait(acc_full_bar(acc), acc_ph, abort_flag, status, TS_EPILOGUE);
            if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
            tc_fence_after();
            const int nchunks = (out + 15) >> 4;
#pragma unroll
            for (int sub = 0; sub < NSUBM; ++sub) {
                const int64_t row = tile * (128 * NSUBM) + sub * 128 + q * 32 + lane;
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + D_COL0 + (uint32_t)((acc * NSUBM + sub) * BN);
#pragma unroll 1
                for (int ch = 0; ch < nchunks; ++ch) {
                    uint32_t rg[16];
                    tmem_ld16(taddr + ch * 16, rg);
                    tmem_ld_wait();
                    {
                        // degree 0's part of y: lane l fetches bias[16 ch + (l & 15)] (the vector is padded to 128
                        // outputs) and the warp passes the values round
                        const float bl = __ldg(bias + ch * 16 + (lane & 15));
#pragma unroll
                        for (int e = 0; e < 16; ++e) {
                            const float v = __uint_as_float(rg[e]);
                            rg[e] = __float_as_uint(fmaf(v, osc, __shfl_sync(0xffffffffu, bl, e)));
                        }
                    }
                    if (row < B) {
                        float* dst = y + row * out + ch * 16;
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            const int col = ch * 16 + 4 * g;
                            if (vec4 && col + 3 < out) {
                                *reinterpret_cast<float4*>(dst + 4 * g) =
                                    make_float4(__uint_as_float(rg[4 * g]), __uint_as_float(rg[4 * g + 1]),
                                                __uint_as_float(rg[4 * g + 2]), __uint_as_float(rg[4 * g + 3]));
                            } else {
#pragma unroll
                                for (int e = 0; e < 4; ++e)
                                    if (col + e < out) dst[4 * g + e] = __uint_as_float(rg[4 * g + e]);
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty_bar(acc));
            if (++acc == NACC) { acc = 0; acc_ph ^= 1u; }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == C::MMA_WARP) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

template <int MODE, int BN, int NSUBM_, int KP_, int NACC_>
int launch_ts(const CUtensorMap& tmap_w, const CUtensorMap& tmap_x, float* y, int64_t B, int in, int out, int dp1,
              int32_t* status, cudaStream_t s, const float* bias, const float* out_scale = nullptr) {
    using C = TsCfg<MODE, BN, NSUBM_, KP_, NACC_>;
    static bool attr_set[64] = {false};
    static int sms[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return CHEBYKAN_EINVAL;
    auto kernel = fwd_ts_kernel<MODE, BN, NSUBM_, KP_, NACC_>;
    if (!attr_set[dev]) {
        int rc = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::TOTAL));
        if (rc) return rc;
        int n = 148;
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        sms[dev] = n;
        attr_set[dev] = true;
    }
    const int64_t num_tiles = ceil_div(B, 128 * C::NSUBM);
    const unsigned grid = (unsigned)(num_tiles < sms[dev] ? num_tiles : sms[dev]);
    kernel<<<grid, C::NUM_THREADS, C::TOTAL, s>>>(tmap_w, tmap_x, y, B, in, out, dp1, num_tiles, status, out_scale, bias);
    return check_cuda(cudaGetLastError());
}

}  // namespace

static bool narrow_forward_tf32_operands() {
    static const bool v = [] {
        const char* e = getenv("CHEBYKAN_NARROW_FWD");
        return e != nullptr && strcmp(e, "tf32") == 0;
    }();
    return v;
}

// narrow layers in the plain tf32 / bf16 modes whose x rows are TMA-addressable
bool fwd_ts_supported(int64_t B, int64_t in, int64_t out, int64_t deg, int mode) {
    return (mode == CHEBYKAN_MODE_TF32 || mode == CHEBYKAN_MODE_BF16) && out <= 128 && (in % 4) == 0 && B >= 1 && deg >= 1 &&
           B <= (int64_t)0x7fffffff - 512;
}

int launch_fwd_ts(const float* x, const void* wt, float* y, int64_t B, int64_t in, int64_t out, int64_t deg, int mode,
                  int32_t* status, cudaStream_t s) {
    // TF32 mode: the fp16 plane behind the tf32 matrix (same layout as the bf16 matrix), unless the environment
    // asks for tf32 operands (CHEBYKAN_NARROW_FWD=tf32, for A/B runs)
    const bool half_plane = mode == CHEBYKAN_MODE_TF32 && tf32_has_half_plane(in, out) && !narrow_forward_tf32_operands();
    const PackedDims p = packed_dims(in, out, deg, half_plane ? CHEBYKAN_MODE_BF16 : mode);
    const char* plane = reinterpret_cast<const char*>(wt) + (half_plane ? tf32_half_plane_offset(in, out, deg) : 0);
    const float* out_scale = half_plane ? reinterpret_cast<const float*>(plane) + 1 : nullptr;   // header: {max bits, 1/scale}
    if (half_plane) plane += HALF_PLANE_HEADER;
    EncodeTiledFn encode = get_encode_fn();
    if (!encode) return CHEBYKAN_ECUDA;
    const int bn = out <= 64 ? 64 : 128;
    const cuuint32_t estr[2] = {1, 1};
    CUtensorMap tmap_w, tmap_x;
    {
        const cuuint64_t dims[2] = {(cuuint64_t)p.k_pad, (cuuint64_t)p.n_pad};
        const cuuint64_t strides[1] = {(cuuint64_t)(p.k_pad * p.elem)};
        const cuuint32_t box[2] = {(cuuint32_t)p.ib, (cuuint32_t)bn};
        const CUtensorMapDataType dt = half_plane ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                       : (mode == CHEBYKAN_MODE_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                                      : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
        const CUresult r = encode(&tmap_w, dt, 2, const_cast<char*>(plane), dims, strides, box, estr,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { set_last_cuda_error((int)r); return CHEBYKAN_ECUDA; }
    }
    {
        // x[B][in] fp32 in boxes of 32 inputs x 128 rows, 128B-swizzled so that a thread reading its own row's
        // chunks meets no bank conflicts; rows / inputs outside the tensor read as zeros
        const cuuint64_t dims[2] = {(cuuint64_t)in, (cuuint64_t)B};
        const cuuint64_t strides[1] = {(cuuint64_t)(in * 4)};
        const cuuint32_t box[2] = {32, 128};
        const CUresult r = encode(&tmap_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(x), dims, strides, box,
                                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { set_last_cuda_error((int)r); return CHEBYKAN_ECUDA; }
    }
    const int dp1 = (int)p.nd;        // degrees 1..deg take K slots; degree 0 is the bias vector behind the matrices
    const float* bias = reinterpret_cast<const float*>(reinterpret_cast<const char*>(wt) + packed_bias_offset(in, out, deg, mode));
#ifdef TS_PROBE_VARIANTS
    TS_PROBE_VARIANTS
#endif
    if (half_plane) {
        if (bn == 64) return launch_ts<TS_MODE_F16, 64, 1, 4, 2>(tmap_w, tmap_x, y, B, (int)in, (int)out, dp1, status, s, bias, out_scale);
        return launch_ts<TS_MODE_F16, 128, 1, 4, 2>(tmap_w, tmap_x, y, B, (int)in, (int)out, dp1, status, s, bias, out_scale);
    }
    if (mode == CHEBYKAN_MODE_BF16) {
        if (bn == 64) return launch_ts<CHEBYKAN_MODE_BF16, 64, 1, 4, 2>(tmap_w, tmap_x, y, B, (int)in, (int)out, dp1, status, s, bias);
        return launch_ts<CHEBYKAN_MODE_BF16, 128, 1, 4, 2>(tmap_w, tmap_x, y, B, (int)in, (int)out, dp1, status, s, bias);
    }
    if (bn == 64) return launch_ts<CHEBYKAN_MODE_TF32, 64, 1, 4, 2>(tmap_w, tmap_x, y, B, (int)in, (int)out, dp1, status, s, bias);
    return launch_ts<CHEBYKAN_MODE_TF32, 128, 1, 4, 1>(tmap_w, tmap_x, y, B, (int)in, (int)out, dp1, status, s, bias);
}

}  // namespace chebykan
