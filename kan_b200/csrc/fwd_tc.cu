// Tensor-core forward for sm_100a:  Y[B, out] = Phi[B, K] * W[K, out],
// K = in*(deg+1), with the basis tile Phi generated on chip.
//
// Replaces reference kan/basis/chebyshev.py:92-101,119-145 (tanh, basis
// expansion, einsum) with one persistent, warp-specialised kernel:
//
//   warps 0-7   producers: coalesced x loads -> tanh -> three-term recurrence
//               T_d = 2t T_{d-1} - T_{d-2} held in registers -> bf16 (or tf32)
//               -> 128-byte-swizzled K-major A tile in shared memory.  One K
//               block is one degree d of IB consecutive inputs, so a thread
//               advances its recurrence by one step per K block.
//   warp  8     TMA: cp.async.bulk.tensor loads of the packed coefficient tile
//               Wt[N][K] (B operand, K-major, 128B swizzle), no multicast.
//   warp  9     MMA: one elected lane issues tcgen05.mma (cta_group::1,
//               M=128, N=BN) and tcgen05.commit releases shared-memory stages
//               / publishes the accumulator.
//   warps 10-13 epilogue: tcgen05.ld TMEM -> registers -> y.
//   warp  14    TMA: prefetches the next [128 rows x IB inputs] fp32 tile of x into
//               shared memory while the producers work on the current one, so no
//               producer ever waits on a global load (when in % 4 != 0 the tile is
//               not TMA-addressable and the producers load x themselves).
//
// With 512 or more (padded) outputs and more than 128 rows the kernel runs as CTA pairs (cluster of 2,
// tcgen05 cta_group::2): each CTA generates the basis tile of its own 128 rows and stages half of
// every W tile; one thread of the even CTA issues M=256 MMAs that read both CTAs' shared memory and
// write both CTAs' TMEM.  The odd CTA's producers and epilogue arrive on the even CTA's barriers
// (mapa + mbarrier.arrive.shared::cluster), both W halves count on the even CTA's full barrier
// (cp.async.bulk.tensor with .cta_group::2, no multicast), and tcgen05.commit multicasts the
// "stage free" / "accumulator ready" arrivals to both CTAs.  Halving the W bytes per CTA frees
// shared memory for an 8-deep A ring.
//
// A CTA tile is 128 rows x (NSUB*BN) outputs.  Each generated A stage feeds
// NSUB MMAs groups (one per BN-wide sub-accumulator), so with BN=256, NSUB=2
// all 512 TMEM columns hold one tile's accumulators and every basis value is
// generated out/512 times instead of out/256 times: basis generation, not the
// tensor pipe, is what limits this kernel.  A and B stages live in separate
// rings (A: 16 KB per stage, B: BN x 128 bytes per stage) with their own
// full/empty mbarriers.  With NSUB*BN <= 256 two accumulator buffers
// alternate, so the epilogue overlaps the next tile's main loop.
//
// Phi never reaches device memory.  Every mbarrier wait is bounded: when one
// gives up the kernel raises an abort flag, records a code in *status, drains
// what it has in flight, frees its TMEM and returns.
#include "tc_common.cuh"

namespace chebykan {

namespace {
using namespace tc;

constexpr int BM = 128;
constexpr int NUM_PRODUCER_WARPS = 8;
constexpr int TMA_WARP = 8;
constexpr int MMA_WARP = 9;
constexpr int X_WARP = 14;
// 16 warps = four warpgroups (warp 15 idles): the two producer warpgroups take registers from the
// other two with setmaxnreg, 8*32*168 + 8*32*88 = 65536
constexpr int NUM_THREADS = 16 * 32;
constexpr int PRODUCER_REGS = 168;
constexpr int OTHER_REGS = 88;
constexpr int A_PANEL_BYTES = BM * 128;     // one K block of A: 128 rows x 128 bytes

// status codes recorded by a wait that gave up
enum { ST_PRODUCER = 1, ST_TMA = 2, ST_MMA_A = 3, ST_MMA_B = 4, ST_MMA_ACC = 5, ST_EPILOGUE = 6, ST_X_LOAD = 7,
       ST_X_WAIT = 8 };

// PP = 2: every K block is staged twice, as a tf32 head and a tf32 tail (the fp32-grade FP32X3 mode)
template <int BN, int NSUB, int CG = 1, int PP = 1>
struct Smem {
    // A ring depth / B ring depth (a CTA of a pair stages half of each W tile, which frees room for more A stages)
    // K blocks per stage.  On narrow layers (one tile of 128 or 64 outputs) an MMA is so small that the
    // hand-over of a stage (barrier waits, proxy fence, arrive, commit) costs more than its math: three
    // or four K blocks share one hand-over there, in rings of two stages.
    static constexpr int KP = (PP == 2) ? 1 : ((BN == 128 && NSUB == 1) ? 3 : (BN == 64 ? 4 : 1));
    static constexpr int NSA = (PP == 2) ? ((BN == 256) ? (CG == 2 ? 3 : 2) : (BN == 128 ? 3 : 4))
                                         : ((KP > 1) ? 2 : ((CG == 2) ? 8 : 4));
    static constexpr int NSB = (PP == 2) ? ((BN == 256) ? (CG == 2 ? 3 : 2) : (BN == 128 ? 3 : 4))
                                         : ((KP > 1) ? 2 : ((CG == 2 || BN == 256) ? 4 : 8));
    static constexpr int NACC = (NSUB * BN <= 256) ? 2 : 1;
    static constexpr int B_PANEL_BYTES = BN * 128 / CG;   // a CTA of a pair holds half of the tile's W rows
    static constexpr int A_STAGE_BYTES = KP * PP * A_PANEL_BYTES;
    static constexpr int B_STAGE_BYTES = KP * PP * B_PANEL_BYTES;
    static constexpr int A_OFFSET = 0;
    static constexpr int B_OFFSET = NSA * A_STAGE_BYTES;
    static constexpr int X_OFFSET = B_OFFSET + NSB * B_STAGE_BYTES;   // x tile: 128 rows x 128 bytes... x 2
    static constexpr int X_BYTES = BM * 256;                          // up to 64 fp32 inputs per row
    static constexpr int GB_OFFSET = X_OFFSET + X_BYTES;               // LayerNorm gamma | beta of the input block
    static constexpr int GB_BYTES = 512;                              // 2 x 64 fp32
    static constexpr int BAR_OFFSET = GB_OFFSET + GB_BYTES;
    // barriers: fullA[NSA] emptyA[NSA] fullB[NSB] emptyB[NSB] acc_full[2] acc_empty[2] drain x_full x_empty
    static constexpr int NUM_BARS = 2 * NSA + 2 * NSB + 7;
    static constexpr int TOTAL = BAR_OFFSET + NUM_BARS * 8 + 16 + 1024;  // +1024 alignment slack
    static constexpr uint32_t TMEM_COLS = NACC * NSUB * BN;
};

// Kernel variants: 0 = the plain Chebyshev layer, 1 = with LayerNorm fused on either side, 2 = another polynomial
// family, whose recurrence table arrives as one more by-value parameter (the other variants pass an empty struct).
constexpr int VAR_PLAIN = 0, VAR_LN = 1, VAR_FAMILY = 2;
struct NoTable {};
template <int VAR> struct VariantTable { using type = NoTable; };
template <> struct VariantTable<VAR_FAMILY> { using type = RecurrenceTable; };

template <int MODE, int BN, int NSUB, int VAR, int CG>
__global__ void __launch_bounds__(NUM_THREADS, 1)
fwd_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
              int use_x_tma, const float* __restrict__ x,
              float* __restrict__ y, int64_t B, int in, int out, int dp1, int n_tiles,
              int64_t num_tiles, int32_t* status, LnFusion ln, int n_pad, const float* __restrict__ bias,
              const __grid_constant__ typename VariantTable<VAR>::type rec) {
    // `dp1` counts the degrees that take K slots per input block: degrees 1..deg.  Degree 0, the constant 1, is one
    // last K block of ones per tile, against the bias row of the packed matrix (a layer of degree 0 never gets
    // here: its output is the bias alone).
    constexpr bool LN = VAR == VAR_LN;
    constexpr bool FAM = VAR == VAR_FAMILY;
    constexpr bool X3 = MODE == CHEBYKAN_MODE_FP32X3;
    constexpr int PP = X3 ? 2 : 1;
    using L = Smem<BN, NSUB, CG, PP>;
    constexpr int NSA = L::NSA, NSB = L::NSB, NACC = L::NACC, KP = L::KP;
    constexpr int A_STAGE_BYTES = L::A_STAGE_BYTES;
    constexpr int BNT = BN * NSUB;                              // outputs per CTA tile
    constexpr int IB = (MODE == CHEBYKAN_MODE_BF16) ? 64 : 32;  // inputs per K block
    constexpr int CH = (MODE == CHEBYKAN_MODE_BF16) ? 8 : 4;    // elements per 16-byte chunk
    constexpr uint32_t FMT = (MODE == CHEBYKAN_MODE_BF16) ? 1u : 2u;
    constexpr uint32_t IDESC = (1u << 4) | (FMT << 7) | (FMT << 10) | ((uint32_t)(BN >> 3) << 17) |
                               ((uint32_t)((BM * CG) >> 4) << 24);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bars = smem_base + L::BAR_OFFSET;
    auto fullA = [&](int s) { return bars + 8u * s; };
    auto emptyA = [&](int s) { return bars + 8u * (NSA + s); };
    auto fullB = [&](int s) { return bars + 8u * (2 * NSA + s); };
    auto emptyB = [&](int s) { return bars + 8u * (2 * NSA + NSB + s); };
    auto acc_full_bar = [&](int a) { return bars + 8u * (2 * NSA + 2 * NSB + a); };
    auto acc_empty_bar = [&](int a) { return bars + 8u * (2 * NSA + 2 * NSB + 2 + a); };
    const uint32_t drain_bar = bars + 8u * (2 * NSA + 2 * NSB + 4);
    const uint32_t x_full_bar = bars + 8u * (2 * NSA + 2 * NSB + 5);
    const uint32_t x_empty_bar = bars + 8u * (2 * NSA + 2 * NSB + 6);
    constexpr uint32_t X_TILE_BYTES = BM * IB * 4;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L::BAR_OFFSET + L::NUM_BARS * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + L::BAR_OFFSET + L::NUM_BARS * 8 + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // CTA pair: the even CTA (rank 0) issues every MMA; each CTA owns 128 of the pair's 256 rows
    const uint32_t rank = (CG == 2) ? cluster_ctarank() : 0u;
    const int64_t unit = (CG == 2) ? (blockIdx.x >> 1) : blockIdx.x;
    const int64_t nunits = (CG == 2) ? (gridDim.x >> 1) : gridDim.x;
    const int n_iblk = (in + IB - 1) / IB;
    const int nkb = n_iblk * dp1 + 1;      // + the bias block: a K block of ones against the packed bias row
    // FP32X3: the tensor pipe's fp32 accumulation truncates, a bias that grows with the number of MMAs added
    // into one accumulator (6e-5 after 3456 of them).  So an accumulator takes only X3_CHUNK K blocks (192 MMAs);
    // the epilogue adds the chunks' partial sums into y with ordinary fp32 additions.
    constexpr int X3_CHUNK = 16;
    const int kb_chunk = X3 ? X3_CHUNK : nkb;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NSA; ++s) { mbar_init(fullA(s), NUM_PRODUCER_WARPS * CG); mbar_init(emptyA(s), 1); }
        for (int s = 0; s < NSB; ++s) { mbar_init(fullB(s), 1); mbar_init(emptyB(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(acc_full_bar(a), 1); mbar_init(acc_empty_bar(a), 4 * 32 * CG); }
        mbar_init(drain_bar, 1);
        mbar_init(x_full_bar, 1);
        mbar_init(x_empty_bar, NUM_PRODUCER_WARPS);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) {
        if (CG == 2) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                         ::"r"(smem_u32((const void*)tmem_slot)), "r"(L::TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                         ::"r"(smem_u32((const void*)tmem_slot)), "r"(L::TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if (CG == 2) cluster_sync_all();      // the peer's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < NUM_PRODUCER_WARPS) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(PRODUCER_REGS));
    else                           asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(OTHER_REGS));

    if (warp < NUM_PRODUCER_WARPS) {
        // ------------------------------ producers ------------------------------
        // thread -> 16-byte chunk c of rows r0, r0+32, r0+64, r0+96: 8 lanes cover one
        // 128-byte row, so x loads are coalesced and the swizzled stores conflict-free
        const int p = threadIdx.x;
        const int c = p & 7;
        const int r0 = p >> 3;
        const bool vec = (in & 3) == 0;
        const uint32_t st_off = (uint32_t)(r0 * 128 + ((c ^ (r0 & 7)) << 4));  // (r0+32j)&7 == r0&7
        // recurrence state: ta/tb alternate as (T_{d-1}, T_{d-2}); tt = 2t
        float tt[4][CH], ta[4][CH], tb[4][CH];
        uint32_t inc[4];        // tf32 rounding increment per row: 0 where the row's inputs of this block hold a NaN
        int s = 0; uint32_t ph = 0;
        int kpos = 0;           // K block inside the current stage
        int kb_left = 0;        // K blocks of the current tile not yet emitted
        uint32_t xph = 0;
        bool alive = true;

        // pack one K block's values, wait for the stage (at its first K block), store, publish (at its last)
        auto emit = [&](const float (&v)[4][CH]) -> bool {
            uint32_t w[4][4];
            uint32_t wl[X3 ? 4 : 1][4];       // tails (FP32X3)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (X3) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        // head = value truncated to tf32; tail = the rest, exact in fp32
                        const uint32_t hi = __float_as_uint(v[j][q % CH]) & 0xFFFFE000u;
                        w[j][q] = hi;
                        wl[X3 ? j : 0][q] = __float_as_uint(v[j][q % CH] - __uint_as_float(hi));
                    }
                } else if (MODE == CHEBYKAN_MODE_BF16) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const __nv_bfloat162 h = __floats2bfloat162_rn(v[j][(2 * q) % CH], v[j][(2 * q + 1) % CH]);
                        w[j][q] = *reinterpret_cast<const uint32_t*>(&h);
                    }
                } else {
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        w[j][q] = tf32_rna(v[j][q % CH], inc[j]);
                }
            }
            if (kpos == 0 && !mbar_wait(emptyA(s), ph ^ 1u, abort_flag, status, ST_PRODUCER)) return false;
            const uint32_t dst = smem_base + L::A_OFFSET + s * A_STAGE_BYTES + kpos * (PP * A_PANEL_BYTES) + st_off;
#pragma unroll
            for (int j = 0; j < 4; ++j)
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};"
                             ::"r"(dst + j * 4096), "r"(w[j][0]), "r"(w[j][1]), "r"(w[j][2]), "r"(w[j][3]) : "memory");
            if (X3) {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};"
                                 ::"r"(dst + A_PANEL_BYTES + j * 4096), "r"(wl[X3 ? j : 0][0]), "r"(wl[X3 ? j : 0][1]),
                                   "r"(wl[X3 ? j : 0][2]), "r"(wl[X3 ? j : 0][3]) : "memory");
            }
            --kb_left;
            if (KP > 1 && kpos + 1 < KP && kb_left > 0) { ++kpos; return true; }   // the stage takes another K block
            kpos = 0;
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                if (CG == 2 && rank != 0) mbar_arrive_cluster(mapa_cluster(fullA(s), 0));
                else mbar_arrive(fullA(s));
            }
            if (++s == NSA) { s = 0; ph ^= 1u; }
            return true;
        };

        for (int64_t tile = unit; tile < num_tiles && alive; tile += nunits) {
            const int64_t m0 = (tile / n_tiles) * (BM * CG) + rank * BM;
            kb_left = nkb;
            // fused LayerNorm of the input rows: per-row mean and 1/std from the previous layer's sums
            float ln_mean[4], ln_rstd[4];
            if (LN && ln.stats_in != nullptr) {
                const float inv_n = 1.f / (float)in;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int64_t row = m0 + r0 + 32 * j;
                    float s1 = 0.f, s2 = 0.f;
                    if (row < B) { s1 = __ldg(ln.stats_in + 2 * row); s2 = __ldg(ln.stats_in + 2 * row + 1); }
                    const float mean = s1 * inv_n;
                    const float var = fmaxf(fmaf(-mean, mean, s2 * inv_n), 0.f);
                    ln_rstd[j] = rsqrtf(var + ln.eps);
                    ln_mean[j] = -mean * ln_rstd[j];       // (x - mean) * rstd as one fma
                }
            }
            for (int ib = 0; ib < n_iblk && alive; ++ib) {
                const int i_base = ib * IB + c * CH;
                float ln_g[CH], ln_b[CH];
                if (LN && ln.stats_in != nullptr && !use_x_tma) {
#pragma unroll
                    for (int e = 0; e < CH; ++e) {
                        const bool ok = i_base + e < in;       // padded inputs stay exactly 0
                        ln_g[e] = ok ? __ldg(ln.gamma + i_base + e) : 0.f;
                        ln_b[e] = ok ? __ldg(ln.beta + i_base + e) : 0.f;
                    }
                }
                if (use_x_tma) {
                    if (!mbar_wait(x_full_bar, xph, abort_flag, status, ST_X_WAIT)) { alive = false; break; }
                    xph ^= 1u;
                    if (LN && ln.stats_in != nullptr) {
                        // gamma and beta of this input block arrived next to the x tile
                        const uint32_t gsrc = smem_base + L::GB_OFFSET + (uint32_t)(c * (CH * 4));
#pragma unroll
                        for (int q = 0; q < CH / 4; ++q) {
                            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                                         : "=f"(ln_g[4 * q]), "=f"(ln_g[4 * q + 1]), "=f"(ln_g[4 * q + 2]), "=f"(ln_g[4 * q + 3])
                                         : "r"(gsrc + 16 * q));
                            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                                         : "=f"(ln_b[4 * q]), "=f"(ln_b[4 * q + 1]), "=f"(ln_b[4 * q + 2]), "=f"(ln_b[4 * q + 3])
                                         : "r"(gsrc + 256 + 16 * q));
                        }
#pragma unroll
                        for (int e = 0; e < CH; ++e)
                            if (i_base + e >= in) { ln_g[e] = 0.f; ln_b[e] = 0.f; }   // padded inputs stay exactly 0
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int64_t row = m0 + r0 + 32 * j;
                    float v[CH];
#pragma unroll
                    for (int e = 0; e < CH; ++e) v[e] = 0.f;
                    if (use_x_tma) {
                        // x tile in shared memory: [128 rows][IB fp32]; rows and inputs past the ends read as 0
                        const uint32_t src = smem_base + L::X_OFFSET + (uint32_t)((r0 + 32 * j) * (IB * 4) + c * (CH * 4));
#pragma unroll
                        for (int q = 0; q < CH / 4; ++q)
                            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                                         : "=f"(v[4 * q]), "=f"(v[4 * q + 1]), "=f"(v[4 * q + 2]), "=f"(v[4 * q + 3])
                                         : "r"(src + 16 * q));
                    } else if (row < B) {
                        const float* src = x + row * in + i_base;
                        if (vec) {
#pragma unroll
                            for (int q = 0; q < CH / 4; ++q)
                                if (i_base + 4 * q < in) {
                                    const float4 f = __ldg(reinterpret_cast<const float4*>(src) + q);
                                    v[4 * q] = f.x; v[4 * q + 1] = f.y; v[4 * q + 2] = f.z; v[4 * q + 3] = f.w;
                                }
                        } else {
#pragma unroll
                            for (int e = 0; e < CH; ++e)
                                if (i_base + e < in) v[e] = __ldg(src + e);
                        }
                    }
                    if (LN && ln.stats_in != nullptr) {
#pragma unroll
                        for (int e = 0; e < CH; ++e)
                            v[e] = fmaf(fmaf(v[e], ln_rstd[j], ln_mean[j]), ln_g[e], ln_b[e]);
                    }
                    bool finite = true;
#pragma unroll
                    for (int e = 0; e < CH; ++e) {
                        float t = X3 ? tanhf(v[e]) : tanh_fast(v[e]);
                        if constexpr (FAM) {
                            // the family's normalised input u; first emitted degree in ta, the one before it in tb: (P_1, P_0)
                            t = rec.affine ? fmaf(rec.scale, v[e] - rec.shift, rec.offset) : rec.scale * t;
                            tt[j][e] = t;
                            ta[j][e] = fmaf(rec.A[1], t, rec.B[1]);
                            tb[j][e] = 1.f;
                        } else {
                            tt[j][e] = 2.f * t; ta[j][e] = t; tb[j][e] = 1.f;      // (T_1, T_0)
                        }
                        finite = finite && (t == t);
                    }
                    inc[j] = finite ? TF32_HALF_ULP : 0u;
                }
                // Hand the x buffer back for the next prefetch only after a shared-memory store whose
                // data derives from the tile has been issued: an mbarrier arrive does not wait for this
                // thread's outstanding ld.shared, the store (and everything after it) does.
                bool x_held = use_x_tma != 0;
                auto release_x = [&]() {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(x_empty_bar);
                    x_held = false;
                };
                // degree 1 (ta); then degrees alternate between tb and ta.  K slot d holds degree d + 1.
                constexpr int sh = 1;
                if (!emit(ta)) { alive = false; break; }
                if (x_held && dp1 == 1) release_x();      // a single degree: nothing else reads the tile
                for (int d = 1; d < dp1; d += 2) {
                    if constexpr (FAM) {
                        const float ra = rec.A[d + sh], rb = rec.B[d + sh], rc = rec.C[d + sh];   // P_d = (A u + B) P_{d-1} - C P_{d-2}
#pragma unroll
                        for (int j = 0; j < 4; ++j)
#pragma unroll
                            for (int e = 0; e < CH; ++e)
                                tb[j][e] = fmaf(fmaf(ra, tt[j][e], rb), ta[j][e], -(rc * tb[j][e]));
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j)
#pragma unroll
                            for (int e = 0; e < CH; ++e) tb[j][e] = fmaf(tt[j][e], ta[j][e], -tb[j][e]);
                    }
                    if (!emit(tb)) { alive = false; break; }
                    if (x_held) release_x();
                    if (d + 1 < dp1) {
                        if constexpr (FAM) {
                            const float ra = rec.A[d + 1 + sh], rb = rec.B[d + 1 + sh], rc = rec.C[d + 1 + sh];
#pragma unroll
                            for (int j = 0; j < 4; ++j)
#pragma unroll
                                for (int e = 0; e < CH; ++e)
                                    ta[j][e] = fmaf(fmaf(ra, tt[j][e], rb), tb[j][e], -(rc * ta[j][e]));
                        } else {
#pragma unroll
                            for (int j = 0; j < 4; ++j)
#pragma unroll
                                for (int e = 0; e < CH; ++e) ta[j][e] = fmaf(tt[j][e], tb[j][e], -ta[j][e]);
                        }
                        if (!emit(ta)) { alive = false; break; }
                    }
                }
            }
            // the tile's last K block: ones (degree 0 of every input at once) against the packed bias row
            if (alive) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    inc[j] = 0u;                       // 1.0 is exact in tf32: no rounding increment
#pragma unroll
                    for (int e = 0; e < CH; ++e) ta[j][e] = 1.f;
                }
                if (!emit(ta)) alive = false;
            }
        }
    } else if (warp == TMA_WARP) {
        // ------------------------------ coefficient loads ------------------------------
        if (lane == 0) {
            int s = 0; uint32_t ph = 0;
            bool alive = true;
            for (int64_t tile = unit; tile < num_tiles && alive; tile += nunits) {
                const int n0 = (int)(tile % n_tiles) * BNT;
                for (int kb = 0; kb < nkb && alive; kb += KP) {
                    const int np = (nkb - kb < KP) ? nkb - kb : KP;     // K blocks in this stage
#pragma unroll
                    for (int sub = 0; sub < NSUB; ++sub) {
                        if (!mbar_wait(emptyB(s), ph ^ 1u, abort_flag, status, ST_TMA)) { alive = false; break; }
                        const uint32_t dst = smem_base + L::B_OFFSET + s * L::B_STAGE_BYTES;
                        if (CG == 2) {
                            // both halves count on the even CTA's barrier, which expects the whole tile
                            if (rank == 0) mbar_arrive_expect_tx(fullB(s), (uint32_t)(np * PP * L::B_PANEL_BYTES * 2));
                            const uint32_t bar0 = mapa_cluster(fullB(s), 0);
                            for (int p = 0; p < np * PP; ++p)      // FP32X3: the tails' rows start at row n_pad
                                tma_load_2d_pair(dst + p * L::B_PANEL_BYTES, &tmap_w, (kb + p / PP) * IB,
                                                 n0 + sub * BN + (int)rank * (BN / 2) + (p % PP) * n_pad, bar0);
                        } else {
                            mbar_arrive_expect_tx(fullB(s), (uint32_t)(np * PP * L::B_PANEL_BYTES));
                            for (int p = 0; p < np * PP; ++p)
                                tma_load_2d(dst + p * L::B_PANEL_BYTES, &tmap_w, (kb + p / PP) * IB,
                                            n0 + sub * BN + (p % PP) * n_pad, fullB(s));
                        }
                        if (++s == NSB) { s = 0; ph ^= 1u; }
                    }
                }
            }
            if (!alive) {
                // let the copies already issued land before the CTA gives up its shared memory
                const uint64_t t0 = globaltimer_ns();
                while (globaltimer_ns() - t0 < 200000ull) { }
            }
        }
    } else if (warp == X_WARP) {
        // ------------------------------ x tile prefetch ------------------------------
        if (lane == 0 && use_x_tma) {
            uint32_t xph = 0;
            bool alive = true;
            for (int64_t tile = unit; tile < num_tiles && alive; tile += nunits) {
                const int m0 = (int)((tile / n_tiles) * (BM * CG) + rank * BM);
                for (int ib = 0; ib < n_iblk; ++ib) {
                    if (!mbar_wait(x_empty_bar, xph ^ 1u, abort_flag, status, ST_X_LOAD)) { alive = false; break; }
                    if (LN && ln.stats_in != nullptr) {
                        // gamma | beta of this block of inputs ride on the same barrier (plain bulk copies)
                        const int i0 = ib * IB;
                        const uint32_t gb_bytes = (uint32_t)(min(IB, in - i0) * 4);     // in % 4 == 0 here
                        mbar_arrive_expect_tx(x_full_bar, X_TILE_BYTES + 2 * gb_bytes);
                        bulk_load_1d(smem_base + L::GB_OFFSET, ln.gamma + i0, gb_bytes, x_full_bar);
                        bulk_load_1d(smem_base + L::GB_OFFSET + 256, ln.beta + i0, gb_bytes, x_full_bar);
                    } else {
                        mbar_arrive_expect_tx(x_full_bar, X_TILE_BYTES);
                    }
                    tma_load_2d(smem_base + L::X_OFFSET, &tmap_x, ib * IB, m0, x_full_bar);
                    xph ^= 1u;
                }
            }
            if (!alive) {
                const uint64_t t0 = globaltimer_ns();
                while (globaltimer_ns() - t0 < 200000ull) { }
            }
        }
    } else if (warp == MMA_WARP) {
        // ------------------------------ MMA issue ------------------------------
        // The warp runs the loop in lock step; one elected lane executes the MMAs and commits (see elect_one_sync).
        // Operand descriptors are per-stage low words plus compile-time offsets.
        if (rank == 0) {
            const bool elected = elect_one_sync();
            int sa = 0; uint32_t pha = 0;
            int sb = 0; uint32_t phb = 0;
            int acc = 0; uint32_t acc_ph = 0;
            bool alive = true;
            const uint64_t a_desc0 = make_smem_desc(smem_base + L::A_OFFSET);
            const uint64_t b_desc0 = make_smem_desc(smem_base + L::B_OFFSET);
            const uint32_t a_hi = (uint32_t)(a_desc0 >> 32), b_hi = (uint32_t)(b_desc0 >> 32);
            for (int64_t tile = unit; tile < num_tiles && alive; tile += nunits) {
              for (int kb0 = 0; kb0 < nkb && alive; kb0 += kb_chunk) {     // one accumulator per chunk of K blocks
                const int kb_end = (nkb - kb0 < kb_chunk) ? nkb : kb0 + kb_chunk;
                if (!__all_sync(0xffffffffu, mbar_wait(acc_empty_bar(acc), acc_ph ^ 1u, abort_flag, status, ST_MMA_ACC))) { alive = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BNT);
                for (int kb = kb0; kb < kb_end && alive; kb += KP) {
                    const int np = (kb_end - kb < KP) ? kb_end - kb : KP;     // K blocks in this stage
                    if (!__all_sync(0xffffffffu, mbar_wait(fullA(sa), pha, abort_flag, status, ST_MMA_A))) { alive = false; break; }
                    const uint32_t a_lo = (uint32_t)a_desc0 + (uint32_t)((sa * A_STAGE_BYTES) >> 4);
                    const uint32_t later = (uint32_t)(kb != kb0);       // 0 only for the first stage of an accumulator
#pragma unroll
                    for (int sub = 0; sub < NSUB; ++sub) {
                        if (!__all_sync(0xffffffffu, mbar_wait(fullB(sb), phb, abort_flag, status, ST_MMA_B))) { alive = false; break; }
                        tc_fence_after();
                        const uint32_t b_lo = (uint32_t)b_desc0 + (uint32_t)((sb * L::B_STAGE_BYTES) >> 4);
#pragma unroll
                        for (int p = 0; p < KP; ++p) {
                            if (p < np) {
                                auto mma = [&](uint32_t a_off, uint32_t b_off, bool acc_is_one) {
                                    const uint64_t ad = desc_from_words(a_lo + a_off, a_hi), bd = desc_from_words(b_lo + b_off, b_hi);
                                    if (elected) {
                                        if (CG == 2) {
                                            if (acc_is_one) umma2<MODE>(d_tmem + sub * BN, ad, bd, IDESC, 1u);
                                            else umma2<MODE>(d_tmem + sub * BN, ad, bd, IDESC, later);
                                        } else {
                                            if (acc_is_one) umma<MODE>(d_tmem + sub * BN, ad, bd, IDESC, 1u);
                                            else umma<MODE>(d_tmem + sub * BN, ad, bd, IDESC, later);
                                        }
                                    }
                                };
                                constexpr uint32_t A_P = (uint32_t)((PP * A_PANEL_BYTES) >> 4), B_P = (uint32_t)((PP * L::B_PANEL_BYTES) >> 4);
#pragma unroll
                                for (int k = 0; k < 4; ++k) {  // 4 x 32 bytes of K per 128-byte row
                                    mma(p * A_P + 2u * k, p * B_P + 2u * k, (p | k) != 0);
                                    if (X3) {
                                        // head x tail and tail x head (tail x tail is below fp32 rounding); descriptors
                                        // address 16-byte units
                                        mma(p * A_P + 2u * k, p * B_P + (uint32_t)(L::B_PANEL_BYTES >> 4) + 2u * k, true);
                                        mma(p * A_P + (uint32_t)(A_PANEL_BYTES >> 4) + 2u * k, p * B_P + 2u * k, true);
                                    }
                                }
                            }
                        }
                        if (elected) { if (CG == 2) umma2_commit_both(emptyB(sb)); else umma_commit(emptyB(sb)); }
                        __syncwarp();
                        if (++sb == NSB) { sb = 0; phb ^= 1u; }
                    }
                    if (elected) { if (CG == 2) umma2_commit_both(emptyA(sa)); else umma_commit(emptyA(sa)); }
                    __syncwarp();
                    if (++sa == NSA) { sa = 0; pha ^= 1u; }
                }
                if (alive && elected) { if (CG == 2) umma2_commit_both(acc_full_bar(acc)); else umma_commit(acc_full_bar(acc)); }
                __syncwarp();
                if (++acc == NACC) { acc = 0; acc_ph ^= 1u; }
              }
            }
            if (!alive && elected) {
                // wait (bounded) until the MMAs already issued have retired
                if (CG == 2) umma2_commit(drain_bar); else umma_commit(drain_bar);
                const uint64_t t0 = globaltimer_ns();
                while (!mbar_try_wait(drain_bar, 0) && globaltimer_ns() - t0 < 10000000ull) { }
            }
            __syncwarp();
        }
    } else if (warp < X_WARP) {
        // ------------------------------ epilogue ------------------------------
        const int q = warp & 3;  // TMEM lane quarter this warp may read
        int acc = 0; uint32_t acc_ph = 0;
        bool alive = true;
        const bool vec4 = (out & 3) == 0;
        const bool vec8 = (out & 7) == 0 && (reinterpret_cast<uintptr_t>(y) & 31u) == 0;
        // one row's 32 consecutive outputs from registers to y
        float ln_s1 = 0.f, ln_s2 = 0.f;    // this row's sum and sum of squares over the tile (fused LayerNorm)
        auto store32 = [&](uint32_t (&r)[32], int64_t row, int col0, bool add) {
            if (row >= B) return;
            if (X3 && add) {
                // later chunk of the K range: y already holds the earlier chunks' sum
                const float* src = y + row * out + col0;
                if (vec4 && col0 + 32 <= out) {
                    float4 p[8];
#pragma unroll
                    for (int g = 0; g < 8; ++g) p[g] = *reinterpret_cast<const float4*>(src + 4 * g);
#pragma unroll
                    for (int g = 0; g < 8; ++g) {
                        r[4 * g] = __float_as_uint(__uint_as_float(r[4 * g]) + p[g].x);
                        r[4 * g + 1] = __float_as_uint(__uint_as_float(r[4 * g + 1]) + p[g].y);
                        r[4 * g + 2] = __float_as_uint(__uint_as_float(r[4 * g + 2]) + p[g].z);
                        r[4 * g + 3] = __float_as_uint(__uint_as_float(r[4 * g + 3]) + p[g].w);
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 32; ++e)
                        if (col0 + e < out) r[e] = __float_as_uint(__uint_as_float(r[e]) + src[e]);
                }
            }
            if (LN && ln.stats_out != nullptr) {
#pragma unroll
                for (int e = 0; e < 32; ++e)
                    if (col0 + e < out) {
                        const float v = __uint_as_float(r[e]);
                        ln_s1 += v; ln_s2 = fmaf(v, v, ln_s2);
                    }
            }
            float* dst = y + row * out + col0;
            if (vec8 && col0 + 32 <= out) {
#pragma unroll
                for (int g = 0; g < 4; ++g)
                    asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                                 ::"l"(dst + 8 * g), "r"(r[8 * g]), "r"(r[8 * g + 1]), "r"(r[8 * g + 2]),
                                   "r"(r[8 * g + 3]), "r"(r[8 * g + 4]), "r"(r[8 * g + 5]), "r"(r[8 * g + 6]),
                                   "r"(r[8 * g + 7]) : "memory");
            } else {
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    const int col = col0 + 4 * g;
                    if (vec4 && col + 3 < out) {
                        *reinterpret_cast<float4*>(dst + 4 * g) =
                            make_float4(__uint_as_float(r[4 * g]), __uint_as_float(r[4 * g + 1]),
                                        __uint_as_float(r[4 * g + 2]), __uint_as_float(r[4 * g + 3]));
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            if (col + e < out) dst[4 * g + e] = __uint_as_float(r[4 * g + e]);
                    }
                }
            }
        };
        auto arrive_acc_empty = [&](int a) {
            if (CG == 2 && rank != 0) mbar_arrive_cluster(mapa_cluster(acc_empty_bar(a), 0));
            else mbar_arrive(acc_empty_bar(a));
        };
        for (int64_t tile = unit; tile < num_tiles && alive; tile += nunits) {
          for (int kb0 = 0; kb0 < nkb && alive; kb0 += kb_chunk) {
            const bool add = kb0 > 0;
            const int64_t row = (tile / n_tiles) * (BM * CG) + rank * BM + q * 32 + lane;
            const int n0 = (int)(tile % n_tiles) * BNT;
            // tcgen05.ld is warp-collective: leave the loop only as a whole warp
            const bool ok = mbar_wait(acc_full_bar(acc), acc_ph, abort_flag, status, ST_EPILOGUE);
            if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BNT);
            // columns that hold real outputs (a ragged last tile ends early), in chunks of 32
            int ncols = out - n0;
            if (ncols > BNT) ncols = BNT;
            const int nchunks = (ncols + 31) >> 5;
            // two register buffers: the TMEM load of chunk i+1 is in flight while chunk i is stored
            uint32_t ra[32], rb[32];
            tmem_ld32(taddr, ra);
#pragma unroll 1
            for (int ch = 0; ch < nchunks; ch += 2) {
                tmem_ld_wait();
                if (ch + 1 < nchunks) tmem_ld32(taddr + (ch + 1) * 32, rb);
                else { tc_fence_before(); arrive_acc_empty(acc); }   // accumulator fully read
                store32(ra, row, n0 + ch * 32, add);
                if (ch + 1 < nchunks) {
                    tmem_ld_wait();
                    if (ch + 2 < nchunks) tmem_ld32(taddr + (ch + 2) * 32, ra);
                    else { tc_fence_before(); arrive_acc_empty(acc); }
                    store32(rb, row, n0 + (ch + 1) * 32, add);
                }
            }
            if (LN && ln.stats_out != nullptr) {
                if (row < B) {
                    atomicAdd(ln.stats_out + 2 * row, ln_s1);
                    atomicAdd(ln.stats_out + 2 * row + 1, ln_s2);
                }
                ln_s1 = 0.f; ln_s2 = 0.f;
            }
            if (++acc == NACC) { acc = 0; acc_ph ^= 1u; }
          }
        }
    }

    tc_fence_before();
    __syncthreads();
    // neither CTA of a pair leaves (or frees TMEM) while the other may still arrive on its barriers
    if (CG == 2) cluster_sync_all();
    if (warp == MMA_WARP) {
        tc_fence_after();
        if (CG == 2)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(L::TMEM_COLS) : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(L::TMEM_COLS) : "memory");
    }
}

template <int MODE, int BN, int NSUB, int VAR, int CG>
int launch_one_ln(const CUtensorMap& tmap, const CUtensorMap& tmap_x, int use_x_tma, const float* x, float* y,
               int64_t B, int in, int out, int dp1, int n_pad, int32_t* status, cudaStream_t s, const LnFusion& ln,
               const float* bias, const typename VariantTable<VAR>::type& rec) {
    using L = Smem<BN, NSUB, CG, (MODE == CHEBYKAN_MODE_FP32X3) ? 2 : 1>;
    static bool attr_set[64] = {false};
    static int max_units[64] = {0};       // CTAs (or CTA pairs) that can be resident at once
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return CHEBYKAN_EINVAL;
    auto kernel = fwd_tc_kernel<MODE, BN, NSUB, VAR, CG>;
    if (!attr_set[dev]) {
        int rc = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
        if (rc) return rc;
        int sms = 148;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        max_units[dev] = sms / CG;
        if (CG == 2) {
            cudaLaunchConfig_t q = {};
            q.gridDim = dim3((unsigned)(sms & ~1)); q.blockDim = dim3(NUM_THREADS); q.dynamicSmemBytes = L::TOTAL;
            cudaLaunchAttribute qa[1];
            qa[0].id = cudaLaunchAttributeClusterDimension;
            qa[0].val.clusterDim.x = 2; qa[0].val.clusterDim.y = 1; qa[0].val.clusterDim.z = 1;
            q.attrs = qa; q.numAttrs = 1;
            int nclusters = 0;
            rc = check_cuda(cudaOccupancyMaxActiveClusters(&nclusters, kernel, &q));
            if (rc) return rc;
            if (nclusters < 1) return CHEBYKAN_ECUDA;
            if (nclusters < max_units[dev]) max_units[dev] = nclusters;
        }
        attr_set[dev] = true;
    }
    const int n_tiles = (int)ceil_div(out, BN * NSUB);      // n_pad is out rounded up to a divisor of the tile
    const int64_t num_tiles = ceil_div(B, BM * CG) * n_tiles;
    const unsigned units = (unsigned)(num_tiles < max_units[dev] ? num_tiles : max_units[dev]);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(units * CG); cfg.blockDim = dim3(NUM_THREADS); cfg.dynamicSmemBytes = L::TOTAL; cfg.stream = s;
    cudaLaunchAttribute attrs[1];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = CG; attrs[0].val.clusterDim.y = 1; attrs[0].val.clusterDim.z = 1;
    cfg.attrs = attrs; cfg.numAttrs = 1;
    return check_cuda(cudaLaunchKernelEx(&cfg, kernel, tmap, tmap_x, use_x_tma, x, y, B, in, out, dp1, n_tiles,
                                         num_tiles, status, ln, n_pad, bias, rec));
}

// the LayerNorm-fused and the family variants are separate instantiations, so the plain kernel carries none of
// their registers
template <int MODE, int BN, int NSUB, int CG = 1>
int launch_one(const CUtensorMap& tmap, const CUtensorMap& tmap_x, int use_x_tma, const float* x, float* y,
               int64_t B, int in, int out, int dp1, int n_pad, int32_t* status, cudaStream_t s, const LnFusion& ln,
               const float* bias, const RecurrenceTable* rec) {
    if constexpr (MODE != CHEBYKAN_MODE_FP32X3) {   // neither LayerNorm fusion nor families in the FP32X3 mode (the entry points refuse)
        if (rec != nullptr)
            return launch_one_ln<MODE, BN, NSUB, VAR_FAMILY, CG>(tmap, tmap_x, use_x_tma, x, y, B, in, out, dp1, n_pad, status, s, ln, bias, *rec);
        if (ln.stats_in != nullptr || ln.stats_out != nullptr)
            return launch_one_ln<MODE, BN, NSUB, VAR_LN, CG>(tmap, tmap_x, use_x_tma, x, y, B, in, out, dp1, n_pad, status, s, ln, bias, NoTable());
    }
    return launch_one_ln<MODE, BN, NSUB, VAR_PLAIN, CG>(tmap, tmap_x, use_x_tma, x, y, B, in, out, dp1, n_pad, status, s, ln, bias, NoTable());
}

template <int MODE>
int launch_mode(const CUtensorMap& tmap, const CUtensorMap& tmx, int xt, int bn, int nsub, int cg, const float* x, float* y,
                int64_t B, int in, int out, int dp1, int n_pad, int32_t* status, cudaStream_t s, const LnFusion& ln,
                const float* bias, const RecurrenceTable* rec) {
    if (bn == 64) return launch_one<MODE, 64, 1>(tmap, tmx, xt, x, y, B, in, out, dp1, n_pad, status, s, ln, bias, rec);
    if (bn == 256 && nsub == 2 && cg == 2) return launch_one<MODE, 256, 2, 2>(tmap, tmx, xt, x, y, B, in, out, dp1, n_pad, status, s, ln, bias, rec);
    if (bn == 256 && nsub == 2) return launch_one<MODE, 256, 2>(tmap, tmx, xt, x, y, B, in, out, dp1, n_pad, status, s, ln, bias, rec);
    if (bn == 256) return launch_one<MODE, 256, 1>(tmap, tmx, xt, x, y, B, in, out, dp1, n_pad, status, s, ln, bias, rec);
    return launch_one<MODE, 128, 1>(tmap, tmx, xt, x, y, B, in, out, dp1, n_pad, status, s, ln, bias, rec);
}

}  // namespace

int launch_fwd_tc(const float* x, const void* wt, float* y, int64_t B, int64_t in, int64_t out,
                  int64_t deg, int mode, int32_t* status, cudaStream_t s, const LnFusion& ln, const RecurrenceTable* rec) {
    if (rec != nullptr && (mode == CHEBYKAN_MODE_FP32X3 || ln.stats_in != nullptr || ln.stats_out != nullptr))
        return CHEBYKAN_EUNSUPPORTED;
    const PackedDims p = packed_dims(in, out, deg, mode);
    EncodeTiledFn encode = get_encode_fn();
    if (!encode) return CHEBYKAN_ECUDA;
    // tile width: 2 x 256 outputs (all of TMEM) when there are that many, else 256 or 128
    int bn = 128, nsub = 1;
    int cg = 1;
    if (p.n_pad >= 384 && mode == CHEBYKAN_MODE_FP32X3) { bn = 256; }   // two accumulators: a chunk drains while the next one runs
    else if (p.n_pad >= 384) { bn = 256; nsub = 2; cg = (B > BM) ? 2 : 1; }
    else if (out <= 64) { bn = 64; }     // smallest tile that holds the outputs: smaller W panels, more K blocks per stage
    else if (p.n_pad == 256) { bn = 256; }
    CUtensorMap tmap;
    const cuuint64_t dims[2] = {(cuuint64_t)p.k_pad, (cuuint64_t)(p.n_pad * p.planes)};
    const cuuint64_t strides[1] = {(cuuint64_t)(p.k_pad * p.elem)};
    const cuuint32_t box[2] = {(cuuint32_t)p.ib, (cuuint32_t)(bn / cg)};
    const cuuint32_t estr[2] = {1, 1};
    const CUtensorMapDataType dt = (mode == CHEBYKAN_MODE_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                                : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    // rows of the box past n_pad (ragged last tile) are filled with zeros
    const CUresult r = encode(&tmap, dt, 2, const_cast<void*>(wt), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_last_cuda_error((int)r); return CHEBYKAN_ECUDA; }
    // x[B][in] fp32 as a TMA tensor: needs a 16-byte row pitch; rows/inputs outside read as zeros
    CUtensorMap tmap_x = tmap;
    const int use_x_tma = (in % 4 == 0) ? 1 : 0;
    if (use_x_tma) {
        const cuuint64_t xdims[2] = {(cuuint64_t)in, (cuuint64_t)B};
        const cuuint64_t xstrides[1] = {(cuuint64_t)(in * 4)};
        const cuuint32_t xbox[2] = {(cuuint32_t)p.ib, (cuuint32_t)BM};
        const CUresult rx = encode(&tmap_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(x), xdims, xstrides,
                                   xbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (rx != CUDA_SUCCESS) { set_last_cuda_error((int)rx); return CHEBYKAN_ECUDA; }
    }
    // degrees that take K slots, and degree 0 as the bias vector behind the matrices (see packed_degrees)
    const int dp1 = (int)p.nd;
    const float* bias = reinterpret_cast<const float*>(reinterpret_cast<const char*>(wt) + packed_bias_offset(in, out, deg, mode));
    if (deg == 0) return CHEBYKAN_EUNSUPPORTED;      // the bias alone: the entry points broadcast it (launch_bias_rows)
    if (mode == CHEBYKAN_MODE_FP32X3)
        return launch_mode<CHEBYKAN_MODE_FP32X3>(tmap, tmap_x, use_x_tma, bn, nsub, cg, x, y, B, (int)in, (int)out, dp1,
                                                 (int)p.n_pad, status, s, ln, bias, rec);
    if (mode == CHEBYKAN_MODE_BF16)
        return launch_mode<CHEBYKAN_MODE_BF16>(tmap, tmap_x, use_x_tma, bn, nsub, cg, x, y, B, (int)in, (int)out, dp1,
                                               (int)p.n_pad, status, s, ln, bias, rec);
    return launch_mode<CHEBYKAN_MODE_TF32>(tmap, tmap_x, use_x_tma, bn, nsub, cg, x, y, B, (int)in, (int)out, dp1,
                                           (int)p.n_pad, status, s, ln, bias, rec);
}

}  // namespace chebykan
