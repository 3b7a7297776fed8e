// Tensor-core coefficient gradient for sm_100a (tcgen05 kind::tf32):
//   dC[(i,d), o] = sum_b T_d(tanh x[b,i]) * dY[b,o]
// i.e. D[M, N] = A[M, K] * B[K, N] with M = (input, degree) slots, N = outputs and the
// BATCH as the contraction dimension K.  It is the dW half of what autograd derives
// from reference kan/basis/chebyshev.py:101,119-145, with Phi regenerated on chip.
//
//   A (Phi^T, generated): K-major tile [128 slots][32 batch rows] tf32, 128B swizzle.  A CTA owns
//       TI = 128/(deg+1) inputs with all their degrees (slot = ii*(deg+1) + d, the
//       coefficient tensor's own order).  A producer lane owns one input and four
//       consecutive batch rows: it runs four recurrences side by side and writes one
//       16-byte chunk per degree.  A producer warp is bound to one stage of the ring
//       (alone, or as one of two warps that split the stage's pairs) and prefetches the
//       x values of its next K block before it generates the current one.
//   B (dY, via TMA): MN-major tile [32 batch rows][BN outputs] fp32 straight from the
//       row-major dY, as BN/32 boxes of 32 rows x 128 bytes in the 32-byte-atom 128B
//       swizzle (the only layout the tensor pipe takes for MN-major 32-bit operands).
//       The tensor pipe reads fp32 as tf32.
//   D: 128 x BN fp32 in TMEM for the CTA's whole slice of the batch; the batch is split
//      over CTAs and the slices' partial sums are added by dcoeff_reduce (fixed order).
//
// Precision: tf32 operands, fp32 accumulate (plain bf16 operands would miss the 2e-3
// tolerance for this product).  Every mbarrier wait is bounded, as in the forward kernel.
#include "tc_common.cuh"

namespace chebykan {

namespace {
using namespace tc;

constexpr int DC_PRODUCER_WARPS = 8;
constexpr int DC_TMA_WARP = 8;
constexpr int DC_MMA_WARP = 9;
constexpr int DC_X_WARP = 10;             // prefetches x tiles by TMA
constexpr int DC_THREADS = 11 * 32;
constexpr int DC_A_TILE = 128 * 128;      // one M tile of A: 128 slots x 32 tf32
constexpr int DC_KB = 32;                 // batch rows per K block
constexpr int DC_MAX_ROUNDS = 8;          // (input, 4-row chunk) pairs per lane per K block: TI*8/32
constexpr int DC_MAX_TI = 28;             // inputs per tile: TI + 3 columns of x fit the 32-float x buffer
constexpr int DC_X_REGION = 32 * 1024;    // shared memory for the ring of x tiles
constexpr int DC_MAX_XSLOTS = 16;         // ring depth: twice the stage count where the tiles are small enough

enum { DST_PRODUCER = 11, DST_TMA = 12, DST_MMA_A = 13, DST_EPILOGUE = 15 };

// A CTA owns MT M tiles (MT*128 slots): every dY tile loaded feeds MT groups of MMAs, and the cost
// of a stage hand-over is spread over MT times more work.  Narrow outputs (tiny MMAs) take MT = 4.
// BN = 512 is two 256-wide accumulators (all of TMEM) fed by the same generated A tile, which halves
// the basis generation per MMA on wide layers.
template <int BN, int CG = 1>
struct DcSmem {
    static constexpr int MT = (BN == 64) ? 4 : (BN == 128 ? 2 : 1);
    static constexpr int BNI = BN > 256 ? 256 : BN;          // N of one MMA
    static constexpr int NSUB = BN / BNI;
    static constexpr int A_STAGE = MT * DC_A_TILE;
    static constexpr int B_STAGE = BN * 128 / CG;            // 32 rows x BN fp32; a CTA of a pair stages half
    static constexpr int STAGE = A_STAGE + B_STAGE;
    // NS divides the 8 producer warps: 8/NS warps share one stage and split its pairs, and a
    // warp only ever fills its own stage, so it is never more than one mbarrier phase ahead
    static constexpr int NS = (BN == 64 || (BN == 512 && CG == 1)) ? 2 : 4;
    static constexpr int X_OFFSET = NS * STAGE;
    static constexpr int BAR_OFFSET = X_OFFSET + DC_X_REGION;
    static constexpr int NUM_BARS = 2 * NS + 2 * DC_MAX_XSLOTS + 2;   // full, empty, xfull, xempty, acc_full, drain
    static constexpr int TOTAL = BAR_OFFSET + NUM_BARS * 8 + 16 + 1024;
    static constexpr uint32_t TMEM_COLS = MT * BN < 32 ? 32 : MT * BN;
};

// MN-major tf32 operand.  32-bit MN-major operands exist only in the "128B swizzle with 32-byte
// atoms" layout: rows of 128 bytes (32 outputs), groups of 4 K rows (512 B) inside which the
// 32-byte chunk index is XORed with the row index; TMA writes it with SWIZZLE_128B_ATOM_32B.
// Column blocks of 32 outputs are 32 rows = 4096 B apart.
__device__ __forceinline__ uint64_t make_smem_desc_mn(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(4096 >> 4) << 16;   // leading byte offset: next 128-byte block along N
    d |= (uint64_t)(512 >> 4) << 32;    // stride byte offset: next group of 4 K rows
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)1 << 61;             // SWIZZLE_128B_BASE32B
    return d;
}

// FAM: another polynomial family; its recurrence table arrives as one more by-value parameter (an empty struct
// otherwise) and the producer warps run the table recurrence instead of the Chebyshev one.
struct DcNoTable {};
template <bool FAM> struct DcTable { using type = DcNoTable; };
template <> struct DcTable<true> { using type = RecurrenceTable; };

template <int BN, int CG, bool FAM>
__global__ void __launch_bounds__(DC_THREADS, 1)
dcoeff_tc_kernel(const __grid_constant__ CUtensorMap tmap_dy, const __grid_constant__ CUtensorMap tmap_x,
                 int use_x_tma, int x_box_w, int nxs, int x_slot_bytes, const float* __restrict__ x,
                 float* __restrict__ dst, int64_t B, int in, int out, int dp1, int nd, int TI, int i_tiles,
                 int n_tiles, int64_t rows_per_split, int64_t split_stride, int add_to_dst,
                 int32_t* status, int part, int exact_tanh,
                 const __grid_constant__ typename DcTable<FAM>::type rec) {
    using L = DcSmem<BN, CG>;
    constexpr int NS = L::NS;
    // tf32 x tf32 -> f32, A K-major, B MN-major, M = 128 per CTA, N = BNI
    constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 16) | ((uint32_t)(L::BNI >> 3) << 17) |
                               ((uint32_t)((128 * CG) >> 4) << 24);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bars = smem_base + L::BAR_OFFSET;
    // one "full" barrier per stage: the producer warps of the stage and the TMA's byte count
    auto full = [&](int s) { return bars + 8u * s; };
    auto empty = [&](int s) { return bars + 8u * (NS + s); };
    // x tiles live in their own ring of nxs slots (K block kb uses slot kb % nxs), deeper than the
    // stage ring so that the prefetch runs well ahead of the producers
    auto xfull = [&](int xs) { return bars + 8u * (2 * NS + xs); };                     // tile has landed
    auto xempty = [&](int xs) { return bars + 8u * (2 * NS + DC_MAX_XSLOTS + xs); };    // tile has been consumed
    const uint32_t acc_full_bar = bars + 8u * (2 * NS + 2 * DC_MAX_XSLOTS);
    const uint32_t drain_bar = bars + 8u * (2 * NS + 2 * DC_MAX_XSLOTS + 1);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L::BAR_OFFSET + L::NUM_BARS * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + L::BAR_OFFSET + L::NUM_BARS * 8 + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // CTA pair (CG == 2): two neighbouring input tiles share every dY tile; the even CTA issues the
    // pair's M = 256 MMAs.  i_tiles is even then, and a tile past the last input has ti = 0.
    const uint32_t rank = (CG == 2) ? cluster_ctarank() : 0u;
    int bid = (CG == 2) ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int n_t = bid % n_tiles; bid /= n_tiles;
    const int i_t = (CG == 2) ? (bid % (i_tiles / 2)) * 2 + (int)rank : bid % i_tiles;
    bid /= (CG == 2) ? (i_tiles / 2) : i_tiles;
    const int split = bid;
    const int i0 = i_t * TI, n0 = n_t * BN;
    const int ti = max(0, min(TI, in - i0));
    const int64_t b_begin = (int64_t)split * rows_per_split;      // a multiple of 32
    const int64_t b_end = min(B, b_begin + rows_per_split);
    const int nkb = (int)((b_end - b_begin + DC_KB - 1) / DC_KB);

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(full(s), CG * DC_PRODUCER_WARPS / NS + 1); mbar_init(empty(s), 1);
        }
        for (int xs = 0; xs < DC_MAX_XSLOTS; ++xs) {
            mbar_init(xfull(xs), 1); mbar_init(xempty(xs), DC_PRODUCER_WARPS / NS);
        }
        mbar_init(acc_full_bar, 1);
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == DC_MMA_WARP) {
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

    if (warp < DC_PRODUCER_WARPS) {
        // ------------------------------ producers ------------------------------
        constexpr int G = DC_PRODUCER_WARPS / NS;   // warps sharing a stage
        const int my_stage = warp % NS, sub = warp / NS;
        const int npairs = ti * 8;                  // (input, chunk of 4 batch rows)
        const int rounds = (npairs + 32 * G - 1) / (32 * G);      // <= DC_MAX_ROUNDS
        float xn[DC_MAX_ROUNDS][4];
        auto load_x = [&](int kb) {
            const int64_t b0 = b_begin + (int64_t)kb * DC_KB;
#pragma unroll
            for (int r = 0; r < DC_MAX_ROUNDS; ++r) {
                const int pair = lane + 32 * (G * r + sub);
#pragma unroll
                for (int e = 0; e < 4; ++e) xn[r][e] = 0.f;
                if (r < rounds && pair < npairs && kb < nkb) {
                    const int ii = pair >> 3, c = pair & 7;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int64_t row = b0 + 4 * c + e;
                        if (row < b_end) xn[r][e] = __ldg(x + row * in + i0 + ii);
                    }
                }
            }
        };
        bool alive = true;
        // x tile in shared memory: [32 rows][x_box_w floats], first column = input (i0 & ~3)
        const int x_col0 = i0 & 3;
        if (!use_x_tma) load_x(my_stage);
        for (int kb = my_stage; kb < nkb && alive; kb += NS) {
            const int s = my_stage;
            const uint32_t ph = (uint32_t)((kb / NS) & 1);
            float xc[DC_MAX_ROUNDS][4];
            if (use_x_tma) {
                // the x warp loaded this tile as soon as the previous one in this slot had been read
                const int xslot = kb % nxs;
                const uint32_t xph = (uint32_t)((kb / nxs) & 1);
                if (!mbar_wait(xfull(xslot), xph, abort_flag, status, DST_PRODUCER)) { alive = false; break; }
                const uint32_t xs = smem_base + L::X_OFFSET + xslot * x_slot_bytes;
#pragma unroll
                for (int r = 0; r < DC_MAX_ROUNDS; ++r) {
                    const int pair = lane + 32 * (G * r + sub);
#pragma unroll
                    for (int e = 0; e < 4; ++e) xc[r][e] = 0.f;
                    if (r < rounds && pair < npairs) {
                        const int ii = pair >> 3, c = pair & 7;
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            asm volatile("ld.shared.f32 %0, [%1];" : "=f"(xc[r][e])
                                         : "r"(xs + (uint32_t)(((4 * c + e) * x_box_w + x_col0 + ii) * 4)));
                    }
                }
                if (!mbar_wait(empty(s), ph ^ 1u, abort_flag, status, DST_PRODUCER)) { alive = false; break; }
            } else {
#pragma unroll
                for (int r = 0; r < DC_MAX_ROUNDS; ++r)
#pragma unroll
                    for (int e = 0; e < 4; ++e) xc[r][e] = xn[r][e];
                load_x(kb + NS);            // in flight while this block is generated
                if (!mbar_wait(empty(s), ph ^ 1u, abort_flag, status, DST_PRODUCER)) { alive = false; break; }
            }
            const uint32_t a_stage = smem_base + s * L::STAGE;
#pragma unroll
            for (int r = 0; r < DC_MAX_ROUNDS; ++r) {
                const int pair = lane + 32 * (G * r + sub);
                if (r < rounds && pair < npairs) {
                    const int ii = pair >> 3, c = pair & 7;
                    float t2[4], ta[4], tb[4];
                    bool finite = true;           // a NaN input makes every degree NaN: no rounding add then
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float t = exact_tanh ? tanhf(xc[r][e]) : tanh_fast(xc[r][e]);
                        if constexpr (FAM) {
                            // the family's normalised input u
                            t = rec.affine ? fmaf(rec.scale, xc[r][e] - rec.shift, rec.offset) : rec.scale * t;
                            t2[e] = t; ta[e] = fmaf(rec.A[1], t, rec.B[1]); tb[e] = 1.f;       // (P_1, P_0)
                        } else {
                            t2[e] = 2.f * t; ta[e] = t; tb[e] = 1.f;     // (T_1, T_0): slots start at degree 1
                        }
                        finite = finite && (t == t);
                    }
                    // slot d (degree d + 1) from the two before it: into tb from (ta, tb), or into ta from (tb, ta)
                    auto next_b = [&](int d) {
                        if constexpr (FAM) {
                            const float ra = rec.A[d + 1], rb = rec.B[d + 1], rc = rec.C[d + 1];
#pragma unroll
                            for (int e = 0; e < 4; ++e) tb[e] = fmaf(fmaf(ra, t2[e], rb), ta[e], -(rc * tb[e]));
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e) tb[e] = fmaf(t2[e], ta[e], -tb[e]);
                        }
                    };
                    auto next_a = [&](int d) {
                        if constexpr (FAM) {
                            const float ra = rec.A[d + 1], rb = rec.B[d + 1], rc = rec.C[d + 1];
#pragma unroll
                            for (int e = 0; e < 4; ++e) ta[e] = fmaf(fmaf(ra, t2[e], rb), tb[e], -(rc * ta[e]));
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e) ta[e] = fmaf(t2[e], tb[e], -ta[e]);
                        }
                    };
                    const uint32_t inc = finite ? TF32_HALF_ULP : 0u;
                    // one 16-byte chunk (4 batch rows) per degree; ta / tb alternate as the newest value
                    // Slot `row` lives in M tile row / 128 at row % 128 (tiles are 16 KB apart): its chunk c sits
                    // at lin = a_stage + row * 128 + c * 16 with the 16-byte chunk index XORed by row % 8, and
                    // since a_stage is 1024-byte aligned, row % 8 is bits 7-9 of lin itself.
                    uint32_t lin = a_stage + (uint32_t)(ii * nd) * 128u + ((uint32_t)c << 4);
                    auto store4 = [&](const float (&v)[4]) {
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            // part 0: rounded to tf32.  Three-product mode: part 1 = head (the tensor pipe drops
                            // the low 13 bits itself), part 2 = tail, the value minus its head
                            if (part == 0) w[e] = tf32_rna(v[e], inc);
                            else if (part == 1) w[e] = __float_as_uint(v[e]);
                            else w[e] = __float_as_uint(v[e] - __uint_as_float(__float_as_uint(v[e]) & 0xFFFFE000u));
                        }
                        const uint32_t dsta = lin ^ ((lin >> 3) & 0x70u);
                        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};"
                                     ::"r"(dsta), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
                        lin += 128u;
                    };
                    store4(ta);                                        // degree 1
                    int d = 1;
                    // eight degrees per trip: the loop's branches, not its arithmetic, were what the
                    // producers waited on
                    for (; d + 7 < nd; d += 8) {
#pragma unroll
                        for (int h = 0; h < 4; ++h) {
                            next_b(d + 2 * h);
                            store4(tb);
                            next_a(d + 2 * h + 1);
                            store4(ta);
                        }
                    }
                    for (; d < nd; d += 2) {
                        next_b(d);
                        store4(tb);
                        if (d + 1 < nd) {
                            next_a(d + 1);
                            store4(ta);
                        }
                    }
                }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                if (CG == 2 && rank != 0) mbar_arrive_cluster(mapa_cluster(full(s), 0));
                else mbar_arrive(full(s));
                // every x value of this stage has been consumed by now (the loads' results were used
                // above), so the slot can take the tile of K block kb + NS
                if (use_x_tma) mbar_arrive(xempty(kb % nxs));
            }
        }
    } else if (warp == DC_TMA_WARP) {
        // ------------------------------ dY loads ------------------------------
        if (lane == 0) {
            bool alive = true;
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % NS;
                const uint32_t ph = (uint32_t)((kb / NS) & 1);
                if (!mbar_wait(empty(s), ph ^ 1u, abort_flag, status, DST_TMA)) { alive = false; break; }
                const int row0 = (int)(b_begin + (int64_t)kb * DC_KB);
                const uint32_t b_stage = smem_base + s * L::STAGE + L::A_STAGE;
                if (CG == 2) {
                    // this CTA stages outputs [128 rank, 128 rank + 128) of each 256-wide half; every byte
                    // counts on the even CTA's barrier, which expects the whole dY tile
                    if (rank == 0) mbar_arrive_expect_tx(full(s), L::B_STAGE * 2);
                    const uint32_t bar0 = mapa_cluster(full(s), 0);
#pragma unroll
                    for (int m = 0; m < BN / 64; ++m)
                        tma_load_2d_pair(b_stage + m * 4096, &tmap_dy,
                                         n0 + (m / 4) * L::BNI + (int)rank * (L::BNI / 2) + 32 * (m % 4), row0, bar0);
                } else {
                    mbar_arrive_expect_tx(full(s), L::B_STAGE);
#pragma unroll
                    for (int m = 0; m < BN / 32; ++m)
                        tma_load_2d(b_stage + m * 4096, &tmap_dy, n0 + 32 * m, row0, full(s));
                }
            }
            if (!alive) {
                const uint64_t t0 = globaltimer_ns();
                while (globaltimer_ns() - t0 < 200000ull) { }
            }
        }
    } else if (warp == DC_X_WARP) {
        // ------------------------------ x tile prefetch ------------------------------
        if (lane == 0 && use_x_tma) {
            bool alive = true;
            for (int kb = 0; kb < nkb; ++kb) {
                const int xslot = kb % nxs;
                const uint32_t xph = (uint32_t)((kb / nxs) & 1);
                if (!mbar_wait(xempty(xslot), xph ^ 1u, abort_flag, status, DST_TMA)) { alive = false; break; }
                mbar_arrive_expect_tx(xfull(xslot), (uint32_t)(DC_KB * x_box_w * 4));
                tma_load_2d(smem_base + L::X_OFFSET + xslot * x_slot_bytes, &tmap_x, i0 & ~3,
                            (int)(b_begin + (int64_t)kb * DC_KB), xfull(xslot));
            }
            if (!alive) {
                const uint64_t t0 = globaltimer_ns();
                while (globaltimer_ns() - t0 < 200000ull) { }
            }
        }
    } else if (warp == DC_MMA_WARP) {
        // ------------------------------ MMA issue ------------------------------
        // The warp runs the loop in lock step; one elected lane executes the MMAs and commits (see elect_one_sync).
        // Operand descriptors are per-stage low words plus compile-time offsets.
        if (rank == 0) {
            const bool elected = elect_one_sync();
            bool alive = true;
            const uint64_t a_desc0 = make_smem_desc(smem_base);
            const uint64_t b_desc0 = make_smem_desc_mn(smem_base + L::A_STAGE);
            const uint32_t a_hi = (uint32_t)(a_desc0 >> 32), b_hi = (uint32_t)(b_desc0 >> 32);
            // slots of the pair: the odd CTA's tile may hold fewer (or no) inputs, its MMAs run all the same
            const int mt_used = (ti * nd + 127) / 128;       // M tiles past the CTA's last slot stay unused
            int nsub_used = 1;                                // 256-wide halves that hold real outputs
            for (int sub = 1; sub < L::NSUB; ++sub)
                if (n0 + sub * L::BNI < out) nsub_used = sub + 1;
            int s = 0; uint32_t ph = 0;
            for (int kb = 0; kb < nkb; ++kb) {
                if (!__all_sync(0xffffffffu, mbar_wait(full(s), ph, abort_flag, status, DST_MMA_A))) { alive = false; break; }
                tc_fence_after();
                const uint32_t a_lo = (uint32_t)a_desc0 + (uint32_t)((s * L::STAGE) >> 4);
                const uint32_t b_lo = (uint32_t)b_desc0 + (uint32_t)((s * L::STAGE) >> 4);
                const uint32_t first = (uint32_t)(kb != 0);
#pragma unroll
                for (int mt = 0; mt < L::MT; ++mt) {
                    if (mt < mt_used) {
#pragma unroll
                        for (int sub = 0; sub < L::NSUB; ++sub) {
                            if (sub < nsub_used) {
#pragma unroll
                                for (int k = 0; k < 4; ++k) { // 8 batch rows per MMA: +32 B in A's rows, +1024 B in B
                                    // A: M tiles are DC_A_TILE apart; B: column blocks of 32 outputs are 4096 B apart
                                    const uint64_t ad = desc_from_words(a_lo + (uint32_t)((mt * DC_A_TILE) >> 4) + 2u * k, a_hi);
                                    const uint64_t bd = desc_from_words(
                                        b_lo + (uint32_t)((sub * (L::BNI / 32 / CG) * 4096) >> 4) + 64u * k, b_hi);
                                    const uint32_t d_tmem = tmem_base + (uint32_t)(mt * BN + sub * L::BNI);
                                    if (elected) {
                                        if (CG == 2) {
                                            if (k != 0) umma2<CHEBYKAN_MODE_TF32>(d_tmem, ad, bd, IDESC, 1u);
                                            else umma2<CHEBYKAN_MODE_TF32>(d_tmem, ad, bd, IDESC, first);
                                        } else {
                                            if (k != 0) umma<CHEBYKAN_MODE_TF32>(d_tmem, ad, bd, IDESC, 1u);
                                            else umma<CHEBYKAN_MODE_TF32>(d_tmem, ad, bd, IDESC, first);
                                        }
                                    }
                                }
                            }
                        }
                    }
                }
                if (elected) { if (CG == 2) umma2_commit_both(empty(s)); else umma_commit(empty(s)); }
                __syncwarp();
                if (++s == NS) { s = 0; ph ^= 1u; }
            }
            if (elected) {
                if (alive) { if (CG == 2) umma2_commit_both(acc_full_bar); else umma_commit(acc_full_bar); }
                else {
                    if (CG == 2) umma2_commit(drain_bar); else umma_commit(drain_bar);
                    const uint64_t t0 = globaltimer_ns();
                    while (!mbar_try_wait(drain_bar, 0) && globaltimer_ns() - t0 < 10000000ull) { }
                }
            }
            __syncwarp();
        }
    }

    // ------------------------------ epilogue: warps 0-3 own TMEM lanes 32w..32w+31 ------------------------------
    if (warp < 4) {
        const bool ok = nkb == 0 ? true : mbar_wait(acc_full_bar, 0, abort_flag, status, DST_EPILOGUE);
        if (__all_sync(0xffffffffu, ok)) {
            tc_fence_after();
#pragma unroll 1
            for (int mt = 0; mt < L::MT; ++mt) {
                if (mt * 128 >= ti * nd) break;
                const int kk = mt * 128 + warp * 32 + lane;      // slot: M tile mt, TMEM lane warp*32+lane
                const bool valid = kk < ti * nd;
                const int ii = kk / nd, d = kk % nd + 1;         // slots are degrees 1..deg; degree 0 is dY's column sums
                float* base = dst + (int64_t)split * split_stride + ((int64_t)(i0 + ii) * out) * dp1 + d;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    if (n0 + c0 >= out) break;
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
                            const int col = n0 + c0 + e;
                            if (col < out) {
                                float* q = base + (int64_t)col * dp1;
                                const float v = __uint_as_float(r[e]);
                                *q = add_to_dst ? (*q + v) : v;
                                // the degree-0 entry next to degree 1: cleared unless the destination accumulates,
                                // filled from the column sums of dY after the reduction
                                if (d == 1 && !add_to_dst) q[-1] = 0.f;
                            }
                        }
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    // neither CTA of a pair leaves (or frees TMEM) while the other may still arrive on its barriers
    if (CG == 2) cluster_sync_all();
    if (warp == DC_MMA_WARP) {
        tc_fence_after();
        if (CG == 2)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(L::TMEM_COLS) : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(L::TMEM_COLS) : "memory");
    }
}

// ---- degree 0 ---------------------------------------------------------------------------------------------
// T_0 = 1 (P_0 = 1), so dC[i][o][0] = sum_b dY[b][o] for every input i: no part of the GEMM.  Two small kernels:
// partial column sums per block of DC_CS_ROWS rows (a thread per column group walks its rows in order), then one
// warp per output adds the blocks' partials in a fixed order and writes the value to all inputs.
constexpr int DC_CS_ROWS = 2048;
__global__ void __launch_bounds__(256)
dy_colsum_kernel(const float* __restrict__ dy, float* __restrict__ part, int64_t B, int out) {
    // 32 columns x 8 row lanes per block; grid (column groups, row blocks)
    __shared__ float red[8][33];
    const int col = blockIdx.x * 32 + (threadIdx.x & 31), rl = threadIdx.x >> 5;
    const int64_t b0 = (int64_t)blockIdx.y * DC_CS_ROWS;
    const int64_t b1 = min(B, b0 + DC_CS_ROWS);
    float s = 0.f;
    if (col < out)
        for (int64_t b = b0 + rl; b < b1; b += 8) s += dy[b * out + col];
    red[rl][threadIdx.x & 31] = s;
    __syncthreads();
    if (rl == 0 && col < out) {
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) t += red[k][threadIdx.x & 31];
        part[(int64_t)blockIdx.y * out + col] = t;
    }
}
__global__ void __launch_bounds__(256)
degree0_fill_kernel(const float* __restrict__ part, int64_t nblocks, float* __restrict__ dc, int in, int out, int dp1,
                    int accumulate) {
    const int o = (int)((blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5);
    const int lane = threadIdx.x & 31;
    if (o >= out) return;
    float sum = 0.f;
    for (int64_t k = lane; k < nblocks; k += 32) sum += part[k * out + o];
#pragma unroll
    for (int w = 16; w > 0; w >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, w);
    for (int i = lane; i < in; i += 32) {
        float* q = dc + ((int64_t)i * out + o) * dp1;
        *q = accumulate ? *q + sum : sum;
    }
}
static int64_t dc_colsum_bytes(int64_t B, int64_t out) { return round_up(ceil_div(B, DC_CS_ROWS) * out * 4, 256); }

// inputs per CTA: as many as fit the CTA's MT*128 slots, the x tile buffer and the producers' registers
int dc_tile_inputs(int64_t in, int nd, int bn) {
    const int mt = bn == 64 ? 4 : (bn == 128 ? 2 : 1);
    const int g = (bn == 64 || bn == 512) ? 4 : 2;         // producer warps per stage (8 / NS)
    int ti = mt * 128 / nd;               // slots: degrees 1..deg of TI inputs
    if (ti > DC_MAX_TI) ti = DC_MAX_TI;
    if (ti * 8 > 32 * g * DC_MAX_ROUNDS) ti = 4 * g * DC_MAX_ROUNDS;
    if (ti > in) ti = (int)in;
    return ti;
}

struct DcTcPlan { int TI, i_tiles, bn, cg, n_tiles, splits; int64_t rows_per_split; };

// x3: at most DC_X3_ROWS batch rows (192 MMAs) go into one accumulator, because the tensor pipe's fp32
// accumulation truncates; the slices' partial sums are added by the reduction kernel in ordinary fp32
constexpr int64_t DC_X3_ROWS = 1536;

DcTcPlan dc_tc_plan(int64_t B, int64_t in, int64_t out, int64_t deg, int x3 = 0) {
    DcTcPlan p{};
    const int dp1 = (int)deg + 1;
    p.bn = out <= 64 ? 64 : (out <= 128 ? 128 : (out <= 256 ? 256 : 512));
    p.TI = dc_tile_inputs(in, (int)deg, p.bn);
    p.i_tiles = (int)ceil_div(in, p.TI);
    // wide layers run as CTA pairs over neighbouring input tiles (an odd count gets one empty tile)
    p.cg = (p.bn == 512 && p.i_tiles >= 2) ? 2 : 1;
    if (p.cg == 2) p.i_tiles = (int)round_up(p.i_tiles, 2);
    p.n_tiles = (int)ceil_div(out, p.bn);
    const int64_t base = (int64_t)p.i_tiles * p.n_tiles;
    // Split the batch so that the CTAs fill whole waves of the 148 SMs: among the candidate split
    // counts take the one with the least (waves x rows per CTA), i.e. the shortest critical path.
    int64_t max_splits = ceil_div(B, 1024);
    if (max_splits < 1) max_splits = 1;
    int64_t cand_hi = ceil_div(4 * 148, base);
    if (cand_hi > max_splits) cand_hi = max_splits;
    int64_t best_s = 1, best_cost = -1;
    for (int64_t sp = 1; sp <= cand_hi; ++sp) {
        const int64_t rows = round_up(ceil_div(B, sp), DC_KB);
        const int64_t ctas = base * ceil_div(B, rows);
        const int64_t cost = ceil_div(ctas, 148) * (rows + 2048);   // + fixed cost of a CTA (setup, epilogue)
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_s = sp; }
    }
    if (x3 && best_s < ceil_div(B, DC_X3_ROWS)) best_s = ceil_div(B, DC_X3_ROWS);
    p.rows_per_split = round_up(ceil_div(B, best_s), DC_KB);
    p.splits = (int)ceil_div(B, p.rows_per_split);
    if (p.splits < 1) p.splits = 1;
    return p;
}

template <int BN, int CG, bool FAM>
int launch_dc_fam(const CUtensorMap& tmap, const CUtensorMap& tmap_x, int use_x_tma, int x_box_w, const float* x, float* dst, int64_t B, int in, int out, int dp1,
                  const DcTcPlan& p, int64_t split_stride, int add, int32_t* status, cudaStream_t s, int part, int exact,
                  const typename DcTable<FAM>::type& rec) {
    using L = DcSmem<BN, CG>;
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kernel = dcoeff_tc_kernel<BN, CG, FAM>;
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        int rc = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
        if (rc) return rc;
        attr_set[dev] = true;
    }
    const unsigned grid = (unsigned)((int64_t)p.i_tiles * p.n_tiles * p.splits);
    // x ring: slots of one tile each (128-byte aligned), twice as many as stages when they fit
    const int x_slot_bytes = (int)round_up((int64_t)DC_KB * x_box_w * 4, 128);
    int nxs = 2 * L::NS;
    if (nxs > DC_MAX_XSLOTS) nxs = DC_MAX_XSLOTS;
    if (nxs * x_slot_bytes > DC_X_REGION) nxs = L::NS;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(DC_THREADS); cfg.dynamicSmemBytes = L::TOTAL; cfg.stream = s;
    cudaLaunchAttribute attrs[1];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = CG; attrs[0].val.clusterDim.y = 1; attrs[0].val.clusterDim.z = 1;
    cfg.attrs = attrs; cfg.numAttrs = 1;
    return check_cuda(cudaLaunchKernelEx(&cfg, kernel, tmap, tmap_x, use_x_tma, x_box_w, nxs, x_slot_bytes, x, dst, B, in,
                                         out, dp1, dp1 - 1, p.TI, p.i_tiles, p.n_tiles, p.rows_per_split, split_stride, add,
                                         status, part, exact, rec));
}

template <int BN, int CG = 1>
int launch_dc(const CUtensorMap& tmap, const CUtensorMap& tmap_x, int use_x_tma, int x_box_w, const float* x, float* dst, int64_t B, int in, int out, int dp1,
              const DcTcPlan& p, int64_t split_stride, int add, int32_t* status, cudaStream_t s, int part, int exact,
              const RecurrenceTable* rec) {
    if (rec != nullptr)
        return launch_dc_fam<BN, CG, true>(tmap, tmap_x, use_x_tma, x_box_w, x, dst, B, in, out, dp1, p, split_stride, add, status, s, part, exact, *rec);
    return launch_dc_fam<BN, CG, false>(tmap, tmap_x, use_x_tma, x_box_w, x, dst, B, in, out, dp1, p, split_stride, add, status, s, part, exact, DcNoTable());
}

}  // namespace

// shapes the tensor-core kernel handles: dY rows must be TMA-addressable (16-byte pitch) and a
// lane must hold its (input, chunk) pairs in registers (TI*8 <= 32*DC_MAX_ROUNDS)
bool dcoeff_tc_supported(int64_t B, int64_t in, int64_t out, int64_t deg) {
    const int dp1 = (int)deg + 1;
    return B > 0 && (out % 4) == 0 && deg >= 1 && dp1 <= 128;
}

// FP32X3 keeps one partial result per DC_X3_ROWS batch rows.  So that the workspace does not grow with the batch
// (43 partial copies of a 37.7 MB gradient on a 65536 x 1024 -> 1024 degree-8 layer), the batch is worked off in
// groups of slices whose partial results fit about 512 MB; each group's reduction adds into dC.
static int64_t x3_group_rows(int64_t in, int64_t out, int64_t deg) {
    const int64_t n_bytes = in * out * (deg + 1) * 4;
    int64_t slices = ((int64_t)512 << 20) / n_bytes;
    if (slices < 2) slices = 2;
    return slices * DC_X3_ROWS;
}

int64_t dcoeff_tc_workspace_bytes(int64_t B, int64_t in, int64_t out, int64_t deg, int x3, int family) {
    // (the fp16-operand kernel of narrow layers is for the Chebyshev basis only: its values stay in [-1, 1])
    if (!x3 && !family && dcoeff_f16_supported(B, in, out, deg)) return dcoeff_f16_workspace_bytes(B, in, out, deg);
    if (x3 && B > x3_group_rows(in, out, deg)) B = x3_group_rows(in, out, deg);
    const DcTcPlan p = dc_tc_plan(B, in, out, deg, x3);
    const int64_t partials = round_up(p.splits > 1 ? (int64_t)p.splits * in * out * (deg + 1) * 4 : 0, 256);
    // x3: the tails of dY come first; last, the partial column sums of dY (degree 0)
    return (x3 ? round_up(B * out * 4, 256) : 0) + partials + dc_colsum_bytes(B, out);
}

// dY minus dY truncated to tf32 (defined next to the dx kernel, which needs the same split)
int launch_dy_tail(const float* dy, float* lo, int64_t n, cudaStream_t s);

int launch_dcoeff_tc(const float* x, const float* dy, float* dc, void* ws, int64_t ws_bytes, int64_t B,
                     int64_t in, int64_t out, int64_t deg, int accumulate, int32_t* status, cudaStream_t s, int x3,
                     const RecurrenceTable* rec) {
    if (rec != nullptr && x3) return CHEBYKAN_EUNSUPPORTED;
    if (!x3 && rec == nullptr && dcoeff_f16_supported(B, in, out, deg))
        return launch_dcoeff_f16(x, dy, dc, ws, ws_bytes, B, in, out, deg, accumulate, status, s);
    if (x3 && B > x3_group_rows(in, out, deg)) {
        // group after group of batch slices through the same workspace (stream order keeps them apart)
        const int64_t rows = x3_group_rows(in, out, deg);
        for (int64_t b0 = 0; b0 < B; b0 += rows) {
            const int64_t bg = (B - b0 < rows) ? B - b0 : rows;
            const int rc = launch_dcoeff_tc(x + b0 * in, dy + b0 * out, dc, ws, ws_bytes, bg, in, out, deg,
                                            (b0 > 0) ? 1 : accumulate, status, s, x3);
            if (rc) return rc;
        }
        return CHEBYKAN_OK;
    }
    const DcTcPlan p = dc_tc_plan(B, in, out, deg, x3);
    const int dp1 = (int)deg + 1;
    const int64_t n = in * out * dp1;
    const bool direct = p.splits == 1;
    if (dcoeff_tc_workspace_bytes(B, in, out, deg, x3, rec != nullptr) > 0 &&
        (ws == nullptr || ws_bytes < dcoeff_tc_workspace_bytes(B, in, out, deg, x3, rec != nullptr)))
        return CHEBYKAN_EWORKSPACE;
    EncodeTiledFn encode = get_encode_fn();
    if (!encode) return CHEBYKAN_ECUDA;
    float* dy_lo = reinterpret_cast<float*>(ws);
    float* partials = x3 ? reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + round_up(B * out * 4, 256))
                         : reinterpret_cast<float*>(ws);
    float* colsum_part = reinterpret_cast<float*>(reinterpret_cast<char*>(partials) +
                                                  round_up(p.splits > 1 ? (int64_t)p.splits * n * 4 : 0, 256));
    const cuuint32_t estr[2] = {1, 1};
    auto map_dy = [&](CUtensorMap* m, const float* ptr) -> int {
        const cuuint64_t dims[2] = {(cuuint64_t)out, (cuuint64_t)B};
        const cuuint64_t strides[1] = {(cuuint64_t)(out * 4)};
        const cuuint32_t box[2] = {32, (cuuint32_t)DC_KB};
        const CUresult r = encode(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(ptr), dims, strides, box,
                                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { set_last_cuda_error((int)r); return CHEBYKAN_ECUDA; }
        return CHEBYKAN_OK;
    };
    CUtensorMap tmap, tmap_lo;
    int rc;
    if ((rc = map_dy(&tmap, dy))) return rc;
    if (x3) {
        if ((rc = launch_dy_tail(dy, dy_lo, B * out, s))) return rc;
        if ((rc = map_dy(&tmap_lo, dy_lo))) return rc;
    }
    // x[B][in] as a TMA tensor when its row pitch allows (in % 4 == 0): a K block's x tile is 32 rows by
    // TI inputs; the box starts at the 16-byte boundary below the tile's first input and is wide enough
    // to cover the tile from there (rows and columns outside x read as zeros)
    CUtensorMap tmap_x = tmap;
    const int use_x_tma = (in % 4 == 0) ? 1 : 0;
    const int x_box_w = (int)round_up(p.TI + 3, 4);
    if (use_x_tma) {
        const cuuint64_t xdims[2] = {(cuuint64_t)in, (cuuint64_t)B};
        const cuuint64_t xstrides[1] = {(cuuint64_t)(in * 4)};
        const cuuint32_t xbox[2] = {(cuuint32_t)x_box_w, (cuuint32_t)DC_KB};
        const CUresult rx = encode(&tmap_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(x), xdims, xstrides,
                                   xbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (rx != CUDA_SUCCESS) { set_last_cuda_error((int)rx); return CHEBYKAN_ECUDA; }
    }
    float* dst = direct ? dc : partials;
    // one pass in the tf32 / bf16 modes; three in the fp32-grade mode: basis heads x dY, basis heads x dY tails,
    // basis tails x dY (the tensor pipe reads the head of whatever fp32 value it is given), each added into dC
    const int passes = x3 ? 3 : 1;
    for (int pass = 0; pass < passes; ++pass) {
        const CUtensorMap& m = (pass == 1) ? tmap_lo : tmap;
        const int part = x3 ? (pass == 2 ? 2 : 1) : 0;
        const int acc = (pass == 0) ? accumulate : 1;
        const int add = direct && acc;
        if (p.bn == 64) rc = launch_dc<64>(m, tmap_x, use_x_tma, x_box_w, x, dst, B, (int)in, (int)out, dp1, p, n, add, status, s, part, x3, rec);
        else if (p.bn == 128) rc = launch_dc<128>(m, tmap_x, use_x_tma, x_box_w, x, dst, B, (int)in, (int)out, dp1, p, n, add, status, s, part, x3, rec);
        else if (p.bn == 256) rc = launch_dc<256>(m, tmap_x, use_x_tma, x_box_w, x, dst, B, (int)in, (int)out, dp1, p, n, add, status, s, part, x3, rec);
        else if (p.cg == 2) rc = launch_dc<512, 2>(m, tmap_x, use_x_tma, x_box_w, x, dst, B, (int)in, (int)out, dp1, p, n, add, status, s, part, x3, rec);
        else rc = launch_dc<512>(m, tmap_x, use_x_tma, x_box_w, x, dst, B, (int)in, (int)out, dp1, p, n, add, status, s, part, x3, rec);
        if (rc) return rc;
        if (!direct && (rc = launch_dcoeff_reduce(partials, dc, n, p.splits, acc, s))) return rc;
    }
    // degree 0: the column sums of dY (exact fp32 sums in every mode), the same for every input
    const int64_t nblk = ceil_div(B, DC_CS_ROWS);
    dy_colsum_kernel<<<dim3((unsigned)ceil_div(out, 32), (unsigned)nblk), 256, 0, s>>>(dy, colsum_part, B, (int)out);
    if ((rc = check_cuda(cudaGetLastError()))) return rc;
    degree0_fill_kernel<<<(unsigned)ceil_div(out * 32, 256), 256, 0, s>>>(colsum_part, nblk, dc, (int)in, (int)out, dp1, accumulate);
    return check_cuda(cudaGetLastError());
}

}  // namespace chebykan
