// Fused unpack + dequantise + split-KV attention over the packed cache
// (kernel b).  One launch covers every (batch, KV head) pair of a layer.
//
// Work distribution.  The live tokens of every pair are cut into n_splits
// "items" of whole 32-token warp units; items are numbered head-major and each
// CTA (one per SM, 16 warps) takes a contiguous range of them, computed on the
// device from the live token count.  Consecutive items of one pair inside a
// CTA form a "run": one stream of tiles, one softmax state, ONE partial (O, LSE)
// written to the slot of the run's first item; the other slots of the run, and
// the slots past the live items, get LSE = -inf, which the combine skips.  So
// every SM works on the same number of tiles (to within one) whatever the
// batch, head count or length, and per-CTA set-up happens once per SM.
//
// Per CTA:
//   * the head's lookup tables arrive as a prebuilt, lane-replicated image
//     (bgtq_plan.h) copied into shared memory with bulk (TMA) copies, before
//     the programmatic dependency wait, and again only when the range crosses
//     into another head;
//   * tiles of 16 warps x 32 tokens of the four cache arrays (packed K, K
//     norms, packed V, V norms) are streamed with 1-D bulk copies completed on
//     mbarriers, two stages deep.  There is no producer warp: the last warp to
//     finish with a stage refills it (a counter in shared memory tells a warp
//     that it is the last);
//   * each warp owns 32 tokens of a tile.  Codes are expanded straight into
//     tensor-core operand registers through the tables:
//        S^T(16 tok x 8 q)  = sum_seg norm_seg[tok] * ( Khat_seg(16 x k) . Qrot_seg^T )
//        O^T(128 dim x 8 q) += Vhat^T(dim x 16 tok) . P^T(16 tok x 8 q)
//     so the GQA group (<= 8 query heads) is the N dimension of m16n8k16 and no
//     tile row is padding.  The K loop is specialised at compile time per stored
//     width (immediate rotates and masks, one body per width with a run-time
//     trip count); the segment list of the head drives which bodies run;
//   * softmax state is fp32 and per warp; warps are merged at the end of a run
//     through the (then idle) stage buffers.
//   * rounding points follow the reference kernel
//     (blockgtq/kernels/fused_packed_attention.py:770-873): fp32 logits,
//     p rounded to fp16 for the PV product while the denominator uses fp32 p,
//     vhat = fp16(fp16 centroid * fp16 norm), fp32 accumulation.
//
// This text is compiled twice.  Ahead of time (nvcc) it yields the general kernel, whose K loop reads the
// head's segment list from the plan at run time.  At run time (NVRTC, bgtq_decode_jit.cu, with BGTQ_JIT
// defined and the same text passed as a string after a generated prelude) it yields a kernel specialised
// for the heads of ONE layer: the prelude spells every head's segment list as compile-time constants, so
// the K loop unrolls into straight-line code with immediate offsets, rotates and masks -- the reference
// specialises its Triton kernel per head with constexprs in the same way
// (blockgtq/production_cache.py:19-22).  Everything but the K side is shared.
#pragma once
#ifndef BGTQ_JIT
#include "bgtq_common.cuh"
#include "bgtq_plan.h"
#endif

namespace bgtq {

constexpr int kDecWarps = 16;
constexpr int kDecThreads = 32 * kDecWarps;
constexpr int kDecStages = 2;
constexpr int kMergeSlot = 9 * 32;   // float4 per warp in the end-of-run merge buffer: 8 of O and (m, l), per lane
// shared-memory layout (byte offsets from the start of dynamic shared memory)
// [barriers | query fragments | pad | lookup tables | stages (merge buffer at run end)]
// The lookup tables start at the first address past kOffMisc whose ABSOLUTE shared-window address is a
// multiple of kLutAlign (table bases are OR-ed into addresses); the stages follow at a fixed offset that
// leaves room for the worst-case pad.
constexpr uint32_t kOffQf = 1024, kOffMisc = kOffQf + kMaxSteps * 32 * 8;
constexpr uint32_t kOffStagesMin = kOffMisc + kLutAlign;     // + lut_bytes = P.stage_off
static_assert(kOffMisc % 128 == 0, "layout");
// two regions the tree merge alternates between: 8 slots (first level) and 4 (second); later levels fit in them
constexpr uint32_t kMergeBytes = (kDecWarps / 2 + kDecWarps / 4) * kMergeSlot * 16;
#define BGTQ_INF __int_as_float(0x7f800000)

struct DecParams {
    const uint16_t* q_rot;  // fp16 bit patterns
    const uint8_t* kp;
    const uint8_t* kn;  // byte pointers; strides below are in bytes
    const uint8_t* vp;
    const uint8_t* vn;
    int64_t kp_sb, kp_sh, kn_sb, kn_sh, vp_sb, vp_sh, vn_sb, vn_sh;
    int32_t kp_st, kn_st, vp_st, vn_st;  // bytes per token
    int32_t n_batch, n_q, n_kv, gqa;
    int32_t t_begin, t_end, n_splits;
    const int32_t* pos_dev;
    int32_t pos_add;
    float scale_log2;
    float* part_o;
    float* part_lse;
    int32_t* status;
    uint32_t stage_off, stage_bytes, off_kn, off_v, off_vn;  // shared-memory layout
    DecPlanDev plan;
};

// V unpack parameters per stored width: mask of the even-indexed codes of one
// 32-bit group, groups per 16 codes, lane replication of the table.
template <int VB> struct VCfg;
template <> struct VCfg<1> { static constexpr uint32_t M = 0x5555u, GROUPS = 1, REP_SHIFT = 5; };
template <> struct VCfg<2> { static constexpr uint32_t M = 0x33333333u, GROUPS = 1, REP_SHIFT = 5; };
template <> struct VCfg<3> { static constexpr uint32_t M = 0x001C71C7u, GROUPS = 2, REP_SHIFT = 5; };
template <> struct VCfg<4> { static constexpr uint32_t M = 0x0F0F0F0Fu, GROUPS = 2, REP_SHIFT = 3; };

// Shared-memory loads of the hot loop take ABSOLUTE 32-bit shared-window addresses: every base the loop uses
// (stage rows, table bases with the lane's replica column, query fragments) has the window address of the
// dynamic shared memory folded in once, so a table lookup is rotate/shift + one and-or + the load, with no
// add in between.  (`sm` is unused; it keeps the call sites readable.)
__device__ __forceinline__ uint32_t ld32(const uint8_t* sm, uint32_t addr) {
    (void)sm;
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 ld64(const uint8_t* sm, uint32_t addr) {
    (void)sm;
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t ld16(const uint8_t* sm, uint32_t addr) {
    (void)sm;
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
// 2^x for the softmax: the hardware approximation (relative error 2^-22; the IEEE-style wrapper of exp2f
// costs two more multiplies and a compare per value for denormal results that the fp16 rounding of p and the
// fp32 denominator cannot see).  ex2(-inf) = 0.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t rotl32(uint32_t x, uint32_t n) { return __funnelshift_l(x, x, n); }
// a / b (b > 0) for the start-up arithmetic every CTA waits on: dividends below 2^22 through the fp32 reciprocal
// (quotient within one of the truth, then corrected), a third of the latency of the integer sequence.
__device__ __forceinline__ uint32_t udiv_fast(uint32_t a, uint32_t b) {
    if (a >= (1u << 22)) return a / b;
    uint32_t q = (uint32_t)__fdividef(__uint2float_rn(a), __uint2float_rn(b));
    const uint32_t p = q * b;
    if (p > a) --q;
    else if (a - p >= b) ++q;
    return q;
}

// 16 codes of one token (bits [bit, bit + 16*VB) past word-aligned offset `row_al`) as one or two
// 32-bit groups of 8 codes.
// WORD_ROWS: the token's row starts on a 32-bit boundary, so the 16-code group (16 VB bits at a multiple of
// 16 VB) never reaches into a third word.
template <int VB, bool WORD_ROWS>
__device__ __forceinline__ void load_v16(const uint8_t* sm, uint32_t row_al, uint32_t bit, uint32_t (&g)[2]) {
    const uint32_t wa = row_al + ((bit >> 5) << 2);
    const uint32_t w0 = ld32(sm, wa), w1 = ld32(sm, wa + 4);
    const uint32_t sh = bit & 31u;
    if constexpr (VB <= 2) {
        g[0] = __funnelshift_r(w0, w1, sh);
        g[1] = 0;
    } else {
        const uint32_t w2 = (!WORD_ROWS && sh + 16u * VB > 64u) ? ld32(sm, wa + 8) : 0u;
        const uint32_t lo = __funnelshift_r(w0, w1, sh), hi = __funnelshift_r(w1, w2, sh);
        if constexpr (VB == 3) {
            g[0] = lo & 0xFFFFFFu;
            g[1] = __funnelshift_r(lo, hi, 24) & 0xFFFFFFu;
        } else {
            g[0] = lo;
            g[1] = hi;
        }
    }
}

#ifndef BGTQ_JIT
// ---------------------------------------------------------------------------------------------
// One K segment of a warp's token tile: acc[u] += Khat_seg(16 tokens x codes) . Qrot_seg^T.
// KIND = stored bits per code.  Lane (r, j): token rows r + 8 i (i < 2 NU), the run of `q` codes at bit
// `lbit` of each row; `tb` = table base with this lane's replica column; `qf` = this lane's query
// fragments, one uint2 per k-tile, 32 apart.  Returns the number of k-tiles consumed.
// ---------------------------------------------------------------------------------------------
template <int KIND, int NU>
__device__ __forceinline__ int k_segment(float (&acc)[NU][4], const uint8_t* sm, const uint32_t rowK,
                                         const uint32_t k_row8, const uint32_t lbit, const int q, const uint32_t tb,
                                         const uint32_t esh8, const uint32_t mask8, const uint32_t qf, const bool f16n,
                                         const uint32_t (&n2)[2 * NU]) {
    constexpr int SB = KIND;                                   // stored bits
    constexpr int CAP = KIND == 3 ? 8 : 32 / SB;               // codes per 32-bit unit
    constexpr int TILES = CAP / 4;                             // k-tiles per unit
    int step = 0;
    for (int c = 0; c < q; c += CAP) {
        const uint32_t pbit = lbit + (uint32_t)(c * SB);
        const uint32_t wa = rowK + ((pbit >> 5) << 2);
        uint32_t cur[2 * NU];
#pragma unroll
        for (int i = 0; i < 2 * NU; ++i)
            cur[i] = __funnelshift_r(ld32(sm, wa + i * k_row8), ld32(sm, wa + i * k_row8 + 4), pbit);
        const int n = q - c;                                   // codes left in the run (even)
#pragma unroll
        for (int t = 0; t < TILES; ++t) {
            if (4 * t >= n) break;
            const uint2 bq = ld64(sm, qf + step * 256);
            ++step;
            uint32_t lo[2 * NU], hi[2 * NU];                   // fp16x2 of codes (0,1) and (2,3) of this k-tile, per row
            if constexpr (KIND == 1) {                         // quad table: one 64-bit lookup per row
                constexpr uint32_t FW = 4 * SB;
                const uint32_t MASK = ((1u << FW) - 1u) << esh8, R = (32u + esh8 - FW * t) & 31u;
#pragma unroll
                for (int i = 0; i < 2 * NU; ++i) {
                    const uint2 v = ld64(sm, (rotl32(cur[i], R) & MASK) | tb);
                    lo[i] = v.x;
                    hi[i] = v.y;
                }
            } else if constexpr (KIND <= 4) {                  // pair tables
                constexpr uint32_t FW = 2 * SB;
                const uint32_t MASK = ((1u << FW) - 1u) << esh8;
                const uint32_t R0 = (64u + esh8 - 2 * FW * t) & 31u, R1 = (64u + esh8 - 2 * FW * t - FW) & 31u;
                const bool full = n - 4 * t >= 4;              // else codes 2, 3 meet a zero query fragment
#pragma unroll
                for (int i = 0; i < 2 * NU; ++i) {
                    lo[i] = ld32(sm, (rotl32(cur[i], R0) & MASK) | tb);
                    hi[i] = full ? ld32(sm, (rotl32(cur[i], R1) & MASK) | tb) : 0u;
                }
            } else {                                           // raw bytes, one code per lookup (fp16 in both halves)
                const bool full = n - 4 * t >= 4;
#pragma unroll
                for (int i = 0; i < 2 * NU; ++i) {
                    const uint32_t c0 = ld32(sm, (rotl32(cur[i], esh8) & mask8) | tb);
                    const uint32_t c1 = ld32(sm, (rotl32(cur[i], esh8 + 24u) & mask8) | tb);
                    lo[i] = __byte_perm(c0, c1, 0x5410);
                    if (full) {
                        const uint32_t c2 = ld32(sm, (rotl32(cur[i], esh8 + 16u) & mask8) | tb);
                        const uint32_t c3 = ld32(sm, (rotl32(cur[i], esh8 + 8u) & mask8) | tb);
                        hi[i] = __byte_perm(c2, c3, 0x5410);
                    } else {
                        hi[i] = 0u;
                    }
                }
            }
            if (f16n) {
#pragma unroll
                for (int i = 0; i < 2 * NU; ++i) {
                    lo[i] = hmul2_u32(lo[i], n2[i]);
                    hi[i] = hmul2_u32(hi[i], n2[i]);
                }
            }
            const uint32_t b[2] = {bq.x, bq.y};
#pragma unroll
            for (int u = 0; u < NU; ++u) {
                const uint32_t a[4] = {lo[2 * u], lo[2 * u + 1], hi[2 * u], hi[2 * u + 1]};
                mma_16816(acc[u], a, b);
            }
        }
    }
    return step;
}
#endif

// Lane-constant inputs of the K side of a warp's token tile.
struct KLane {
    uint32_t lut;              // absolute shared address of the lookup tables
    uint32_t qf;               // absolute shared address of this lane's first query fragment
    uint32_t rowK, rowN;       // absolute shared addresses of the lane's first packed row (word aligned) / norm row
    uint32_t k_row8, kn_row8;  // byte distance between rows r and r + 8
    uint32_t k_p0;             // bit phase of the packed rows inside their first aligned word
    uint32_t j, lane;
    bool kn_words;             // norm rows start on 4-byte boundaries
};

#ifndef BGTQ_JIT
// S^T = Khat . Qrot^T of a warp's NU 16-token row tiles, segment list read from the plan.
template <int NU>
__device__ __forceinline__ void k_side(float (&S)[NU][4], const uint8_t* sm, const KLane& kl, const DecHeadPlan& hp) {
    const int n_seg = hp.n_seg;
    uint32_t qf = kl.qf;
    for (int sg = 0; sg < n_seg; ++sg) {
        const DecSeg sd = hp.seg[sg];
        // Norm handling: the bit-packed layout scales the fp32 dot product of a segment by its fp16 norm; the
        // nibble layout rounds centroid * norm to fp16 per element before the product
        // (fused_packed_attention.py:1449-1452), so there the norm is folded into the operand.
        const bool f16n = sd.f16_norm != 0;
        float nrm[2 * NU];
        uint32_t n2[2 * NU];
#pragma unroll
        for (int i = 0; i < 2 * NU; ++i) {
            const uint32_t nh = ld16(sm, kl.rowN + 2u * sd.norm_idx + i * kl.kn_row8);
            n2[i] = nh | (nh << 16);
            nrm[i] = f16n ? 1.0f : f16_bits_to_float(nh);
        }
        float acc[NU][4];
#pragma unroll
        for (int u = 0; u < NU; ++u) acc[u][0] = acc[u][1] = acc[u][2] = acc[u][3] = 0.f;
        const uint32_t lbit = kl.k_p0 + sd.bit0 + kl.j * sd.lane_bits;
        const uint32_t tb = kl.lut + sd.tbl + ((kl.lane & ((1u << sd.rep_log2) - 1u)) << sd.ent_log2);
        const int q = sd.q;
        int used;
        switch (sd.kind) {
            case 1: used = k_segment<1, NU>(acc, sm, kl.rowK, kl.k_row8, lbit, q, tb, (uint32_t)sd.esh, 0u, qf, f16n, n2); break;
            case 2: used = k_segment<2, NU>(acc, sm, kl.rowK, kl.k_row8, lbit, q, tb, (uint32_t)sd.esh, 0u, qf, f16n, n2); break;
            case 3: used = k_segment<3, NU>(acc, sm, kl.rowK, kl.k_row8, lbit, q, tb, (uint32_t)sd.esh, 0u, qf, f16n, n2); break;
            case 4: used = k_segment<4, NU>(acc, sm, kl.rowK, kl.k_row8, lbit, q, tb, (uint32_t)sd.esh, 0u, qf, f16n, n2); break;
            default:
                used = k_segment<8, NU>(acc, sm, kl.rowK, kl.k_row8, lbit, q, tb, (uint32_t)sd.esh,
                                        ((1u << sd.bw) - 1u) << sd.esh, qf, f16n, n2);
                break;
        }
        qf += used * 256;
#pragma unroll
        for (int u = 0; u < NU; ++u) {
            S[u][0] = fmaf(nrm[2 * u], acc[u][0], S[u][0]);
            S[u][1] = fmaf(nrm[2 * u], acc[u][1], S[u][1]);
            S[u][2] = fmaf(nrm[2 * u + 1], acc[u][2], S[u][2]);
            S[u][3] = fmaf(nrm[2 * u + 1], acc[u][3], S[u][3]);
        }
    }
}
#else
// ---------------------------------------------------------------------------------------------
// Specialised K side: the generated prelude declares, per KV head H of the layer,
//     template <> struct jit::Head<H> { static constexpr int n_seg; static constexpr jit::SegC seg[8]; };
// and every loop below has a compile-time trip count.
// ---------------------------------------------------------------------------------------------
// Bring the bit field that starts at bit POS of x to bit TO (a plain shift: which pipe executes it is the
// compiler's choice, unlike a funnel shift).
// Both positions are constants once the loops around the call are unrolled.
__device__ __forceinline__ uint32_t field_to(uint32_t x, uint32_t to, uint32_t pos) {
    return pos < to ? x << (to - pos) : x >> (pos - to);
}
// PW = index of the 32-bit word of the token's norm row that `nw` holds (norms 2 PW and 2 PW + 1), -1: none yet.
template <class HeadT, int SG, int NU, int PW>
__device__ __forceinline__ void k_segment_c(float (&S)[NU][4], const uint8_t* sm, const KLane& kl, uint32_t (&nw)[2 * NU]) {
    constexpr jit::SegC c = HeadT::seg[SG];
    constexpr int SB = c.kind, Q = c.q;
    constexpr int CAP = c.kind == 3 ? 8 : 32 / SB, TILES = CAP / 4;
    constexpr bool f16n = c.f16_norm != 0;
    constexpr int W = c.norm_idx >> 1;
    if constexpr (W != PW) {
        // the token's norms two at a time when its norm row sits on a 4-byte boundary (the four lanes of a quad
        // read one address, so a row costs one wavefront either way, but half as many loads)
        if (kl.kn_words) {
#pragma unroll
            for (int i = 0; i < 2 * NU; ++i) nw[i] = ld32(sm, kl.rowN + 4u * W + i * kl.kn_row8);
        } else {
#pragma unroll
            for (int i = 0; i < 2 * NU; ++i)
                nw[i] = ld16(sm, kl.rowN + 4u * W + i * kl.kn_row8) | (ld16(sm, kl.rowN + 4u * W + 2u + i * kl.kn_row8) << 16);
        }
    }
    float nrm[2 * NU];
    uint32_t n2[2 * NU];
#pragma unroll
    for (int i = 0; i < 2 * NU; ++i) {
        n2[i] = __byte_perm(nw[i], 0u, (c.norm_idx & 1) ? 0x3232 : 0x1010);
        nrm[i] = f16n ? 1.0f : f16_bits_to_float((c.norm_idx & 1) ? nw[i] >> 16 : nw[i]);
    }
    float acc[NU][4];     // the segment's first k-tile starts it from zero
    // Lanes of a quad past the segment's last code (short segments: c.jv < 4 lanes hold codes) meet zero query
    // fragments.  They read what the quad's last live lane reads, and the lookup-table replica is chosen per
    // (token row, live lane), so that the 8 c.jv distinct addresses of a lookup fall into different banks
    // whenever the table has that many replicas.
    const uint32_t jj = c.jv < 4 ? min(kl.j, (uint32_t)(c.jv - 1)) : kl.j;
    const uint32_t rep = c.jv < 4 ? (kl.lane >> 2) * (uint32_t)c.jv + jj : kl.lane;
    const uint32_t lbit = kl.k_p0 + (uint32_t)c.bit0 + jj * (uint32_t)c.lane_bits;
    const uint32_t tb = kl.lut + (uint32_t)c.tbl + ((rep & ((1u << c.rep_log2) - 1u)) << c.ent_log2);
#pragma unroll
    for (int cc = 0; cc < Q; cc += CAP) {
        const uint32_t pbit = lbit + (uint32_t)(cc * SB);
        const uint32_t wa = kl.rowK + ((pbit >> 5) << 2);
        uint32_t cur[2 * NU];
#pragma unroll
        for (int i = 0; i < 2 * NU; ++i)
            cur[i] = __funnelshift_r(ld32(sm, wa + i * kl.k_row8), ld32(sm, wa + i * kl.k_row8 + 4), pbit);
#pragma unroll
        for (int t = 0; t < TILES; ++t) {
            if (cc + 4 * t < Q) {
                const bool full = Q - cc - 4 * t >= 4;         // else codes 2, 3 meet a zero query fragment
                const uint2 bq = ld64(sm, kl.qf + (c.step0 + (cc + 4 * t) / 4) * 256);
                uint32_t lo[2 * NU], hi[2 * NU];
                if constexpr (c.kind == 1) {                   // quad table: one 64-bit lookup per row
                    constexpr uint32_t ESH = c.esh, FW = 4 * SB;
                    constexpr uint32_t MASK = ((1u << FW) - 1u) << ESH;
#pragma unroll
                    for (int i = 0; i < 2 * NU; ++i) {
                        const uint2 v = ld64(sm, (field_to(cur[i], ESH, FW * t) & MASK) | tb);
                        lo[i] = v.x;
                        hi[i] = v.y;
                    }
                } else if constexpr (c.kind <= 4) {            // pair tables
                    constexpr uint32_t ESH = c.esh, FW = 2 * SB;
                    constexpr uint32_t MASK = ((1u << FW) - 1u) << ESH;
#pragma unroll
                    for (int i = 0; i < 2 * NU; ++i) {
                        lo[i] = ld32(sm, (field_to(cur[i], ESH, 2 * FW * t) & MASK) | tb);
                        hi[i] = full ? ld32(sm, (field_to(cur[i], ESH, 2 * FW * t + FW) & MASK) | tb) : 0u;
                    }
                } else {                                       // raw bytes, one code per lookup
                    constexpr uint32_t ESH = c.esh, MASK = ((1u << c.bw) - 1u) << ESH;
#pragma unroll
                    for (int i = 0; i < 2 * NU; ++i) {
                        const uint32_t c0 = ld32(sm, (field_to(cur[i], ESH, 0) & MASK) | tb);
                        const uint32_t c1 = ld32(sm, (field_to(cur[i], ESH, 8) & MASK) | tb);
                        lo[i] = __byte_perm(c0, c1, 0x5410);
                        if (full) {
                            const uint32_t c2 = ld32(sm, (field_to(cur[i], ESH, 16) & MASK) | tb);
                            const uint32_t c3 = ld32(sm, (field_to(cur[i], ESH, 24) & MASK) | tb);
                            hi[i] = __byte_perm(c2, c3, 0x5410);
                        } else {
                            hi[i] = 0u;
                        }
                    }
                }
                if (f16n) {
#pragma unroll
                    for (int i = 0; i < 2 * NU; ++i) {
                        lo[i] = hmul2_u32(lo[i], n2[i]);
                        hi[i] = hmul2_u32(hi[i], n2[i]);
                    }
                }
                const uint32_t b[2] = {bq.x, bq.y};
#pragma unroll
                for (int u = 0; u < NU; ++u) {
                    const uint32_t a[4] = {lo[2 * u], lo[2 * u + 1], hi[2 * u], hi[2 * u + 1]};
                    if (cc + 4 * t == 0) mma_16816_z(acc[u], a, b);
                    else mma_16816(acc[u], a, b);
                }
            }
        }
    }
#pragma unroll
    for (int u = 0; u < NU; ++u) {
        S[u][0] = fmaf(nrm[2 * u], acc[u][0], S[u][0]);
        S[u][1] = fmaf(nrm[2 * u], acc[u][1], S[u][1]);
        S[u][2] = fmaf(nrm[2 * u + 1], acc[u][2], S[u][2]);
        S[u][3] = fmaf(nrm[2 * u + 1], acc[u][3], S[u][3]);
    }
}
template <class HeadT, int SG, int NU, int PW>
__device__ __forceinline__ void k_side_from(float (&S)[NU][4], const uint8_t* sm, const KLane& kl, uint32_t (&nw)[2 * NU]) {
    if constexpr (SG < HeadT::n_seg) {
        k_segment_c<HeadT, SG, NU, PW>(S, sm, kl, nw);
        k_side_from<HeadT, SG + 1, NU, (HeadT::seg[SG].norm_idx >> 1)>(S, sm, kl, nw);
    }
}
template <int NU>
__device__ __forceinline__ void k_side(float (&S)[NU][4], const uint8_t* sm, const KLane& kl, const int h) {
    uint32_t nw[2 * NU];
#define BGTQ_JIT_CASE(H) case H: k_side_from<jit::Head<H>, 0, NU, -1>(S, sm, kl, nw); break;
    switch (h) { BGTQ_JIT_CASES }       // one case per head of the layer, spelled by the prelude
#undef BGTQ_JIT_CASE
}
#endif

#ifndef BGTQ_JIT
template <int VB, int NU>
__global__ void __launch_bounds__(kDecThreads, 1) decode_kernel(const __grid_constant__ DecParams P) {
#else
constexpr int VB = BGTQ_JIT_VB, NU = BGTQ_JIT_NU;
extern "C" __global__ void __launch_bounds__(kDecThreads, 1) bgtq_decode_jit(const __grid_constant__ DecParams P) {
#endif
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int kWarpTok = 16 * NU;              // tokens per warp and tile
    constexpr int kTileTok = kDecWarps * kWarpTok; // tokens per CTA tile
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r = lane >> 2, j = lane & 3;
    // Row strides and the stage layout: compile-time constants when the kernel was specialised for them (the
    // launch wrapper then also guarantees 16-byte aligned array slices, so every phase below is zero and row
    // offsets fold into the load instructions), launch parameters otherwise.
#ifdef BGTQ_JIT_STRIDES
    constexpr uint32_t kp_st = BGTQ_JIT_KP_ST, kn_st = BGTQ_JIT_KN_ST, vp_st = BGTQ_JIT_VP_ST, vn_st = BGTQ_JIT_VN_ST;
    constexpr StageLayout kSL = stage_layout(kTileTok, kp_st, kn_st, vp_st, vn_st);
    constexpr uint32_t off_kn = kSL.off_kn, off_v = kSL.off_v, off_vn = kSL.off_vn, stage_bytes = kSL.stage_bytes;
    constexpr uint32_t stage_off = BGTQ_JIT_STAGE_OFF;
    constexpr bool kAligned = true;
    constexpr bool kWordRowsV = vp_st % 4u == 0u && (off_v % 4u) == 0u;
#else
    const uint32_t kp_st = (uint32_t)P.kp_st, kn_st = (uint32_t)P.kn_st, vp_st = (uint32_t)P.vp_st, vn_st = (uint32_t)P.vn_st;
    const uint32_t off_kn = P.off_kn, off_v = P.off_v, off_vn = P.off_vn, stage_bytes = P.stage_bytes;
    const uint32_t stage_off = P.stage_off;
    constexpr bool kAligned = false;
    constexpr bool kWordRowsV = false;
#endif

    // Everything up to grid_dependency_wait() touches only static tables, so under a programmatic
    // launch it overlaps the tail of the preceding kernel (the step's append / query rotation).
    grid_launch_dependents();

    uint64_t* full = reinterpret_cast<uint64_t*>(smem);                      // [kDecStages]
    uint64_t* lutbar = full + kDecStages;
    unsigned int* done = reinterpret_cast<unsigned int*>(lutbar + 1);        // warps finished with a stage, ever
    uint2* qfrag = reinterpret_cast<uint2*>(smem + kOffQf);                  // [step][lane]
    const uint8_t* sm = smem;
    const uint32_t sbase = smem_u32(smem);
    const uint32_t lut_abs = (sbase + kOffMisc + kLutAlign - 1u) & ~(kLutAlign - 1u);   // see the layout comment
    const uint32_t lut_rel = lut_abs - sbase;

    if (tid == 0) {
        for (int i = 0; i < kDecStages; ++i) {
            mbar_init(&full[i], 1);
            done[i] = 0u;
        }
        mbar_init(lutbar, 1);
        mbar_fence_init();
    }
    __syncthreads();

    // ---- lookup tables of one head: bulk copies of the prebuilt image --------------------------------
    int h_loaded = -1;
    uint32_t lut_uses = 0;
    bool ok = true;
    auto load_tables = [&](int h) {       // called by all threads; the previous tables are no longer read
        if (tid == 0) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            const uint32_t bytes = (P.plan.head[h].image_bytes + 15u) & ~15u;
            const uint8_t* src = P.plan.image + (size_t)h * P.plan.lut_bytes;
            mbar_arrive_expect_tx(lutbar, bytes);
            for (uint32_t o = 0; o < bytes; o += 32768u)
                bulk_g2s(smem + lut_rel + o, src + o, min(32768u, bytes - o), lutbar);
        }
        h_loaded = h;
    };
    auto wait_tables = [&]() {
        if (!mbar_wait_bounded(lutbar, lut_uses & 1u)) ok = false;
        ++lut_uses;
    };
    const int n_cta = (int)gridDim.x, cta = (int)blockIdx.x;
    load_tables(min(P.n_kv - 1, (int)(((int64_t)cta * P.n_kv) / n_cta)));   // the head this CTA most likely starts in
    bool tables_pending = true;
    // The item-range table, if the plan carries one, is requested here, ahead of the dependency wait, so that its
    // latency passes behind the start-up work (it is written by a copy ordered before the launch that precedes
    // this one, never by that launch itself).
    const int32_t* part = P.plan.partition;
    uint32_t pk0 = 0, pk1 = 0, pk2 = 0, pk3 = 0, p_lo = 0, p_hi = 0;
    if (part) {
        pk0 = (uint32_t)__ldg(part);
        pk1 = (uint32_t)__ldg(part + 1);
        pk2 = (uint32_t)__ldg(part + 2);
        pk3 = (uint32_t)__ldg(part + 3);
        p_lo = (uint32_t)__ldg(part + kPartHeader + cta);
        p_hi = (uint32_t)__ldg(part + kPartHeader + cta + 1);
    }

    // With early fetch (see bgtq_decode_plan_set_early_fetch) the wait moves behind the first tile requests.
    const int early_fresh = P.plan.early_fresh;
    bool dep_waited = early_fresh <= 0;
    if (dep_waited) grid_dependency_wait();
    // ---- this CTA's range of items ---------------------------------------------------------------------
    // (32-bit unsigned arithmetic: a 64-bit division costs a few hundred cycles of every CTA's start-up, and
    // item counts that need one do not occur: the launch wrapper rejects them)
    const int t_live = P.pos_dev ? min(P.t_end, *P.pos_dev + P.pos_add) : P.t_end;
    const uint32_t n_tok = (uint32_t)max(0, t_live - P.t_begin);
    const uint32_t units = (n_tok + 31u) >> 5;                          // 32-token warp units per pair
    const uint32_t c_units = max(1u, udiv_fast(units + (uint32_t)P.n_splits - 1u, (uint32_t)P.n_splits));  // units per item
    const uint32_t n_live = udiv_fast(units + c_units - 1u, c_units);   // non-empty items per pair (<= n_splits)
    const uint32_t n_items = (uint32_t)(P.n_batch * P.n_kv) * n_live;
    if (n_items == 0) {     // no tokens at all: every slot of every row is an empty split
        if (!dep_waited) grid_dependency_wait();
        for (int64_t i = (int64_t)cta * kDecThreads + tid; i < (int64_t)P.n_batch * P.n_q * P.n_splits;
             i += (int64_t)n_cta * kDecThreads)
            P.part_lse[i] = -BGTQ_INF;
        if (tables_pending) wait_tables();
        return;
    }
    // Equal item counts, unless the caller's table was made for exactly this launch (the same items per pair,
    // pairs, CTAs and units per item: every CTA sees the same four words, so all take the same branch)
    uint32_t item_lo, item_hi;
    if (part && pk0 == n_live && pk1 == (uint32_t)(P.n_batch * P.n_kv) && pk2 == (uint32_t)n_cta && pk3 == c_units) {
        item_lo = min(p_lo, n_items);
        item_hi = min(max(p_hi, item_lo), n_items);
    } else {
        item_lo = udiv_fast((uint32_t)cta * n_items, (uint32_t)n_cta);
        item_hi = udiv_fast(((uint32_t)cta + 1u) * n_items, (uint32_t)n_cta);
    }

    const uint64_t pol = l2_evict_first_policy();
    uint32_t g_it = 0;                      // tiles streamed so far by this CTA (stage = g_it % stages)
    const uint32_t lane4 = (uint32_t)lane << 2;
    constexpr uint32_t kVSh = VCfg<VB>::REP_SHIFT + 2;

    // The run that starts at item `item`: consecutive items of one (head, batch) pair, up to the CTA's last.
    struct Run { int h, b, s0, cnt, t0, t1; };
    auto run_at = [&](uint32_t item) {
        Run R;
        const uint32_t pair = udiv_fast(item, n_live);
        R.s0 = (int)(item - pair * n_live);
        R.cnt = (int)min(n_live - (uint32_t)R.s0, item_hi - item);
        R.h = (int)udiv_fast(item, n_live * (uint32_t)P.n_batch);   // = pair / n_batch, without waiting for `pair`
        R.b = (int)pair - R.h * P.n_batch;
        R.t0 = P.t_begin + 32 * R.s0 * (int)c_units;
        R.t1 = min(t_live, P.t_begin + 32 * (R.s0 + R.cnt) * (int)c_units);
        return R;
    };
    // Stream tile `it` of a run into the stage of running tile number `git`.  Called by a whole warp: lanes
    // 0..3 each request one of the four arrays (packed K, K norms, packed V, V norms), so the address
    // arithmetic of a tile takes one lane's worth of time instead of four.
    auto issue_tile = [&](const Run& R, int it, uint32_t git) {
        const int st = git % kDecStages;
        const int t = R.t0 + it * kTileTok;
        const int nt = min(kTileTok, R.t1 - t);
        const int a = lane & 3;
        const uint8_t* base = a == 0 ? P.kp : a == 1 ? P.kn : a == 2 ? P.vp : P.vn;
        const int64_t sb_ = a == 0 ? P.kp_sb : a == 1 ? P.kn_sb : a == 2 ? P.vp_sb : P.vn_sb;
        const int64_t sh_ = a == 0 ? P.kp_sh : a == 1 ? P.kn_sh : a == 2 ? P.vp_sh : P.vn_sh;
        const uint32_t st_ = a == 0 ? kp_st : a == 1 ? kn_st : a == 2 ? vp_st : vn_st;
        const uint32_t off = a == 0 ? 0u : a == 1 ? off_kn : a == 2 ? off_v : off_vn;
        const uint8_t* src = base + (size_t)R.b * sb_ + (size_t)R.h * sh_ + (size_t)t * st_;
        const uint32_t ph = kAligned ? 0u : (uint32_t)(reinterpret_cast<uintptr_t>(src) & 15u);
        const uint32_t z = (ph + (uint32_t)nt * st_ + 15u) & ~15u;
        uint32_t tot = z + __shfl_xor_sync(0xffffffffu, z, 1);
        tot += __shfl_xor_sync(0xffffffffu, tot, 2);
        if (lane < 4) {
            // the stage was last touched through the generic proxy (its previous tile's readers, or the merge)
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            if (lane == 0) mbar_arrive_expect_tx(&full[st], tot);
            bulk_g2s_hint(smem + stage_off + (size_t)st * stage_bytes + off, src - ph, z, &full[st], pol);
        }
    };
    // A run's first tile may already be on its way: the previous run's end requests it before merging its warps.
    bool first_tile_issued = false;

    for (uint32_t item = item_lo; item < item_hi;) {
        const Run R = run_at(item);
        item += (uint32_t)R.cnt;
        const int h = R.h, b = R.b, s0 = R.s0, cnt = R.cnt, t0 = R.t0, t1 = R.t1;
        const DecHeadPlan& hp = P.plan.head[h];
        const int n_tiles = (t1 - t0 + kTileTok - 1) / kTileTok;

        const size_t bh_kp = (size_t)b * P.kp_sb + (size_t)h * P.kp_sh;
        const size_t bh_kn = (size_t)b * P.kn_sb + (size_t)h * P.kn_sh;
        const size_t bh_vp = (size_t)b * P.vp_sb + (size_t)h * P.vp_sh;
        const size_t bh_vn = (size_t)b * P.vn_sb + (size_t)h * P.vn_sh;
        if (h != h_loaded) {                 // the range crossed into another head (all warps are past the
            if (tables_pending) {            // previous run's closing barrier, nobody reads the old tables)
                wait_tables();               // a copy still in flight (wrong first guess) lands before the next
                __syncthreads();             // one is armed on the same barrier
            }
            load_tables(h);
            tables_pending = true;
        }
        // first tiles of the run; their stages are idle (see the run's end).  Before the dependency wait only
        // tiles that end below the rows the preceding launch may still be writing are requested.
        {
            const int first = first_tile_issued ? 1 : 0, last = min(n_tiles, kDecStages);
            int held = last;                 // first tile held back until the wait
            if (!dep_waited) {
                held = first;
                while (held < last && t0 + (held + 1) * kTileTok <= t_live - early_fresh) ++held;
            }
            if (warp == 0)
                for (int it = first; it < held; ++it) issue_tile(R, it, g_it + it);
            if (!dep_waited) {
                grid_dependency_wait();
                dep_waited = true;
                if (warp == 0)
                    for (int it = held; it < last; ++it) issue_tile(R, it, g_it + it);
            }
        }
        // query fragments of this pair: step s, lane (g, jj)
        for (int s = kDecWarps - 1 - warp; s < hp.n_steps; s += kDecWarps) {     // (warp 0 is busy with the tiles)
            const DecStepQ st = hp.steps[s];
            const int g = lane >> 2, jj = lane & 3;
            const int pos = (int)st.pos + jj * (int)st.q;
            const bool q_ok = g < P.gqa;
            const uint16_t* qrow = P.q_rot + ((size_t)b * P.n_q + (size_t)h * P.gqa + (q_ok ? g : 0)) * kHD;
            uint2 v;
            v.x = (q_ok && pos < (int)st.end) ? __ldg(reinterpret_cast<const uint32_t*>(qrow + pos)) : 0u;
            v.y = (q_ok && (int)st.c4 + 2 < (int)st.q && pos + 2 < (int)st.end)
                      ? __ldg(reinterpret_cast<const uint32_t*>(qrow + pos + 2)) : 0u;
            qfrag[s * 32 + lane] = v;
        }
        if (tables_pending) {
            wait_tables();
            tables_pending = false;
        }
        __syncthreads();

        // -------------------------------- the run's tiles --------------------------------
        float O[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) O[i][0] = O[i][1] = O[i][2] = O[i][3] = 0.f;
        float m0 = -BGTQ_INF, m1 = -BGTQ_INF, l0 = 0.f, l1 = 0.f;

        // Byte phases of the four arrays inside a stage (tiles advance every array by a multiple of 16
        // bytes), and this lane's row offsets.  K side: tokens tok0 + 8 i; V side, row tile u: tokens
        // tkv + 16u + {0, 1, 8, 9}.
        const uint32_t k_pre = kAligned ? 0u : (uint32_t)((reinterpret_cast<uintptr_t>(P.kp) + bh_kp + (size_t)t0 * kp_st) & 15u);
        const uint32_t kn_pre = kAligned ? 0u : (uint32_t)((reinterpret_cast<uintptr_t>(P.kn) + bh_kn + (size_t)t0 * kn_st) & 15u);
        const uint32_t v_pre = kAligned ? 0u : (uint32_t)((reinterpret_cast<uintptr_t>(P.vp) + bh_vp + (size_t)t0 * vp_st) & 15u);
        const uint32_t vn_pre = kAligned ? 0u : (uint32_t)((reinterpret_cast<uintptr_t>(P.vn) + bh_vn + (size_t)t0 * vn_st) & 15u);
        const int tok0 = warp * kWarpTok + r, tkv = warp * kWarpTok + 2 * j;
        const uint32_t k_off = k_pre + tok0 * kp_st;
        const uint32_t k_row_al = k_off & ~3u, k_p0 = (k_off & 3u) << 3;
        const uint32_t kn_row = off_kn + kn_pre + tok0 * kn_st;
        const uint32_t v_off = off_v + v_pre + tkv * vp_st;
        const uint32_t vn_rowS = off_vn + vn_pre + tok0 * vn_st;   // V norms of the lane's score rows
        const uint32_t k_row8 = 8u * kp_st, kn_row8 = 8u * kn_st;
        const bool kn_words = ((kn_st | (off_kn + kn_pre)) & 3u) == 0u;
        const uint32_t vtbl = lut_abs + hp.v_tbl + (lane4 & ((1u << kVSh) - 1u));

        for (int it = 0; it < n_tiles; ++it, ++g_it) {
            const int st = g_it % kDecStages;
            const uint32_t use = g_it / kDecStages;
            if (!mbar_wait_bounded(&full[st], use & 1u)) ok = false;
            const int nt = min(kTileTok, t1 - (t0 + it * kTileTok));
            const uint32_t sb = sbase + stage_off + st * stage_bytes;
            if (warp * kWarpTok < nt) {
                // ---------------- S^T = Khat . Qrot^T for NU 16-token row tiles ----------------
                float S[NU][4];
#pragma unroll
                for (int u = 0; u < NU; ++u) S[u][0] = S[u][1] = S[u][2] = S[u][3] = 0.f;
                KLane kl;
                kl.lut = lut_abs;
                kl.qf = sbase + kOffQf + (uint32_t)lane * 8u;
                kl.rowK = sb + k_row_al;
                kl.rowN = sb + kn_row;
                kl.k_row8 = k_row8;
                kl.kn_row8 = kn_row8;
                kl.k_p0 = k_p0;
                kl.j = (uint32_t)j;
                kl.lane = (uint32_t)lane;
                kl.kn_words = kn_words;
#ifndef BGTQ_JIT
                k_side<NU>(S, sm, kl, hp);
#else
                k_side<NU>(S, sm, kl, h);
#endif
                // ---------------- online softmax (log2 domain) over the warp's tokens ----------------
                // Scores stay unscaled until the exponent: 2^(S * scale - max) is one fused multiply-add per value.
                float x0 = -BGTQ_INF, x1 = -BGTQ_INF;
                const bool partial = nt < kTileTok;     // only a run's last tile can hold rows past its end
                if (partial) {
#pragma unroll
                    for (int u = 0; u < NU; ++u) {
                        const bool okA = tok0 + 16 * u < nt, okB = tok0 + 16 * u + 8 < nt;
                        S[u][0] = okA ? S[u][0] : -BGTQ_INF;
                        S[u][1] = okA ? S[u][1] : -BGTQ_INF;
                        S[u][2] = okB ? S[u][2] : -BGTQ_INF;
                        S[u][3] = okB ? S[u][3] : -BGTQ_INF;
                    }
                }
#pragma unroll
                for (int u = 0; u < NU; ++u) {
                    x0 = fmaxf(x0, fmaxf(S[u][0], S[u][2]));
                    x1 = fmaxf(x1, fmaxf(S[u][1], S[u][3]));
                }
#pragma unroll
                for (int o = 4; o < 32; o <<= 1) {
                    x0 = fmaxf(x0, __shfl_xor_sync(0xffffffffu, x0, o));
                    x1 = fmaxf(x1, __shfl_xor_sync(0xffffffffu, x1, o));
                }
                const float n0 = fmaxf(m0, x0 * P.scale_log2), n1 = fmaxf(m1, x1 * P.scale_log2);
                const float z0 = n0 == -BGTQ_INF ? 0.f : n0, z1 = n1 == -BGTQ_INF ? 0.f : n1;
                const float al0 = fast_exp2(m0 - z0), al1 = fast_exp2(m1 - z1);
                m0 = n0;
                m1 = n1;
                // P^T fragments carry the V norm of their token (one fp16 per token), so the V side multiplies
                // nothing: sum_t p_t * (n_t * c_t) = sum_t (p_t * n_t) * c_t.  Rows past the run's end hold
                // stale bytes: their norm reads as zero, like their p.
                uint32_t pf[NU][2];
                float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
                for (int u = 0; u < NU; ++u) {
                    const float p0 = fast_exp2(fmaf(S[u][0], P.scale_log2, -z0)), p1 = fast_exp2(fmaf(S[u][1], P.scale_log2, -z1));
                    const float p2 = fast_exp2(fmaf(S[u][2], P.scale_log2, -z0)), p3 = fast_exp2(fmaf(S[u][3], P.scale_log2, -z1));
                    ps0 += p0 + p2;
                    ps1 += p1 + p3;
                    const uint32_t rn = sb + vn_rowS + 16u * u * vn_st;
                    float nA = f16_bits_to_float(ld16(sm, rn)), nB = f16_bits_to_float(ld16(sm, rn + 8u * vn_st));
                    if (partial) {
                        nA = tok0 + 16 * u < nt ? nA : 0.f;
                        nB = tok0 + 16 * u + 8 < nt ? nB : 0.f;
                    }
                    pf[u][0] = movmatrix_trans(pack_half2(p0 * nA, p1 * nA));
                    pf[u][1] = movmatrix_trans(pack_half2(p2 * nB, p3 * nB));
                }
                l0 = fmaf(l0, al0, ps0);
                l1 = fmaf(l1, al1, ps1);
                if (__any_sync(0xffffffffu, al0 != 1.f || al1 != 1.f)) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        O[i][0] *= al0;
                        O[i][1] *= al1;
                        O[i][2] *= al0;
                        O[i][3] *= al1;
                    }
                }

                // ---------------- O^T += Vhat^T . P^T ----------------
                // Row tile u, this lane: tokens tkv+16u+{0,1} (pair AB) and +{8,9} (pair CD); dims 16r .. 16r+15.
                constexpr uint32_t M = VCfg<VB>::M, G = VCfg<VB>::GROUPS, FW = 2 * VB;
                constexpr uint32_t IMS = ((1u << FW) - 1u) << kVSh;
                constexpr int PER = 8 / G;   // k-tiles (dim pairs) per 32-bit group
#pragma unroll
                for (int u = 0; u < NU; ++u) {
                    uint32_t gA[2], gB[2], gC[2], gD[2];
                    const uint32_t rv = sb + v_off + 16u * u * vp_st;
                    const uint32_t base = rv & ~3u, bit = ((rv & 3u) << 3) + 16u * VB * r;
                    load_v16<VB, kWordRowsV>(sm, base, bit, gA);
                    load_v16<VB, kWordRowsV>(sm, base, bit + 8u * vp_st, gB);
                    load_v16<VB, kWordRowsV>(sm, base, bit + 64u * vp_st, gC);
                    load_v16<VB, kWordRowsV>(sm, base, bit + 72u * vp_st, gD);
#pragma unroll
                    for (int g = 0; g < (int)G; ++g) {
                        const uint32_t xab = (gA[g] & M) | ((gB[g] & M) << VB), yab = ((gA[g] >> VB) & M) | (gB[g] & (M << VB));
                        const uint32_t xcd = (gC[g] & M) | ((gD[g] & M) << VB), ycd = ((gC[g] >> VB) & M) | (gD[g] & (M << VB));
#pragma unroll
                        for (int k = 0; k < PER; ++k) {
                            // index pre-scaled by the entry stride: rotate so the field sits at bit kVSh
                            const uint32_t rt = (32u + kVSh - FW * k) & 31u;
                            uint32_t a[4];
                            a[0] = ld32(sm, (rotl32(xab, rt) & IMS) | vtbl);
                            a[1] = ld32(sm, (rotl32(yab, rt) & IMS) | vtbl);
                            a[2] = ld32(sm, (rotl32(xcd, rt) & IMS) | vtbl);
                            a[3] = ld32(sm, (rotl32(ycd, rt) & IMS) | vtbl);
                            mma_16816(O[g * PER + k], a, pf[u]);
                        }
                    }
                }
            }
            __syncwarp();
            // Release the stage; the last warp to do so streams the tile that reuses it.  The counter only ever
            // grows: after `use + 1` rounds of this stage all warps have added to it that many times.
            uint32_t refill = 0u;
            if (lane == 0) {
                __threadfence_block();
                refill = atomicAdd(&done[st], 1u) == (use + 1u) * kDecWarps - 1u && it + kDecStages < n_tiles;
                __threadfence_block();
            }
            __syncwarp();
            if (__shfl_sync(0xffffffffu, refill, 0)) issue_tile(R, it + kDecStages, g_it + kDecStages);
        }

        // ---------------- merge the warps, write the run's partial ----------------
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            l0 += __shfl_xor_sync(0xffffffffu, l0, o);
            l1 += __shfl_xor_sync(0xffffffffu, l1, o);
        }
        // Every tile of the run has been consumed once all warps are here: both stages are idle.
        __syncthreads();
        // If this CTA has another run, that run's first tile is requested NOW, into the stage it will use (the
        // one the last tile did not), so its DRAM latency passes behind the merge, which then stays inside the
        // other stage.  Otherwise the merge may spread over both.
        const bool ahead = item < item_hi && kDecStages == 2 && stage_bytes >= kMergeBytes;
        if (ahead && warp == 0) issue_tile(run_at(item), 0, g_it);
        first_tile_issued = ahead;
        // Merge of the sixteen warps' (O, m, l).  Two tree levels (16 -> 8 -> 4): the upper half of the live warps
        // hands its state to the lower half through shared memory, fragment for fragment (thread t of warp w + n
        // stores what thread t of warp w reads, 16 bytes per access), and the lower half folds it into its
        // registers.  Then the four remaining warps split the eight dim tiles between them: each sends the other
        // three the tiles they own, sums what it receives for its own two, normalises and writes them, so the
        // run's partial leaves through four warps' stores.  The levels alternate between two regions of the
        // buffer; one barrier per level.
        float4* const mb = reinterpret_cast<float4*>(smem + stage_off + (ahead ? ((g_it + 1u) % kDecStages) * stage_bytes : 0u));
#pragma unroll
        for (int n = kDecWarps / 2, lvl = 0; n >= 4; n >>= 1, ++lvl) {
            float4* const reg = mb + ((lvl & 1) ? (kDecWarps / 2) * kMergeSlot : 0);
            if (warp >= n && warp < 2 * n) {
                float4* dst = reg + (warp - n) * kMergeSlot + lane;
#pragma unroll
                for (int i = 0; i < 8; ++i) dst[i * 32] = make_float4(O[i][0], O[i][1], O[i][2], O[i][3]);
                dst[8 * 32] = make_float4(m0, m1, l0, l1);
            }
            __syncthreads();
            if (warp < n) {
                const float4* src = reg + warp * kMergeSlot + lane;
                const float4 ms = src[8 * 32];
                const float M0 = fmaxf(m0, ms.x), M1 = fmaxf(m1, ms.y);
                const float Z0 = M0 == -BGTQ_INF ? 0.f : M0, Z1 = M1 == -BGTQ_INF ? 0.f : M1;
                const float a0 = fast_exp2(m0 - Z0), a1 = fast_exp2(m1 - Z1);
                const float b0 = fast_exp2(ms.x - Z0), b1 = fast_exp2(ms.y - Z1);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float4 v = src[i * 32];
                    O[i][0] = fmaf(O[i][0], a0, v.x * b0);
                    O[i][1] = fmaf(O[i][1], a1, v.y * b1);
                    O[i][2] = fmaf(O[i][2], a0, v.z * b0);
                    O[i][3] = fmaf(O[i][3], a1, v.w * b1);
                }
                l0 = fmaf(l0, a0, ms.z * b0);
                l1 = fmaf(l1, a1, ms.w * b1);
                m0 = M0;
                m1 = M1;
            }
        }
        // Warp w < 4 owns dim tiles 2 w and 2 w + 1.  Region 0 again (its first-level readers are past the
        // second level's barrier): piece (owner o, sender w, k) at ((o * 4 + w) * 2 + k) * 32 + lane, the
        // senders' (m, l) behind the 32 pieces.
        if (warp < 4) {
#pragma unroll
            for (int o = 0; o < 4; ++o)
                if (o != warp) {
#pragma unroll
                    for (int k = 0; k < 2; ++k)
                        mb[((o * 4 + warp) * 2 + k) * 32 + lane] =
                            make_float4(O[2 * o + k][0], O[2 * o + k][1], O[2 * o + k][2], O[2 * o + k][3]);
                }
            mb[(32 + warp) * 32 + lane] = make_float4(m0, m1, l0, l1);
        }
        __syncthreads();
        if (warp < 4) {
            float4 ms[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) ms[w] = w == warp ? make_float4(m0, m1, l0, l1) : mb[(32 + w) * 32 + lane];
            const float M0 = fmaxf(fmaxf(ms[0].x, ms[1].x), fmaxf(ms[2].x, ms[3].x));
            const float M1 = fmaxf(fmaxf(ms[0].y, ms[1].y), fmaxf(ms[2].y, ms[3].y));
            const float Z0 = M0 == -BGTQ_INF ? 0.f : M0, Z1 = M1 == -BGTQ_INF ? 0.f : M1;
            float w0[4], w1[4], L0 = 0.f, L1 = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                w0[w] = fast_exp2(ms[w].x - Z0);
                w1[w] = fast_exp2(ms[w].y - Z1);
                L0 = fmaf(ms[w].z, w0[w], L0);
                L1 = fmaf(ms[w].w, w1[w], L1);
            }
            float4 acc[2];
#pragma unroll
            for (int o = 0; o < 4; ++o)
                if (o == warp) {
#pragma unroll
                    for (int k = 0; k < 2; ++k)
                        acc[k] = make_float4(O[2 * o + k][0] * w0[o], O[2 * o + k][1] * w1[o], O[2 * o + k][2] * w0[o],
                                             O[2 * o + k][3] * w1[o]);
                }
#pragma unroll
            for (int w = 0; w < 4; ++w)
                if (w != warp) {
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const float4 v = mb[((warp * 4 + w) * 2 + k) * 32 + lane];
                        acc[k].x = fmaf(v.x, w0[w], acc[k].x);
                        acc[k].y = fmaf(v.y, w1[w], acc[k].y);
                        acc[k].z = fmaf(v.z, w0[w], acc[k].z);
                        acc[k].w = fmaf(v.w, w1[w], acc[k].w);
                    }
                }
            // lane (r, j): query heads 2 j, 2 j + 1; dims 16 r + 2 mt, + 1 for mt = 2 warp + k
            const float i0 = L0 > 0.f ? 1.f / L0 : 0.f, i1 = L1 > 0.f ? 1.f / L1 : 0.f;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int qi = 2 * j + e;
                if (qi < P.gqa) {
                    const size_t row = ((size_t)b * P.n_q + (size_t)h * P.gqa + qi) * P.n_splits + s0;
                    const float inv = e ? i1 : i0;
#pragma unroll
                    for (int k = 0; k < 2; ++k)
                        *reinterpret_cast<float2*>(P.part_o + row * kHD + 16 * r + 2 * (2 * warp + k)) =
                            e ? make_float2(acc[k].y * inv, acc[k].w * inv) : make_float2(acc[k].x * inv, acc[k].z * inv);
                    const float le = e ? L1 : L0, me = e ? M1 : M0;
                    if (warp == 0 && r == 0)
                        P.part_lse[row] = le > 0.f ? (me + log2f(le)) * 0.6931471805599453f : -BGTQ_INF;
                }
            }
        }
        {
            // slots merged into this partial, and (after the pair's last live item) the slots past them
            const int qi = tid >> 6;
            if (qi < P.gqa) {
                const size_t row = ((size_t)b * P.n_q + (size_t)h * P.gqa + qi) * P.n_splits;
                const int s_end = s0 + cnt == (int)n_live ? P.n_splits : s0 + cnt;
                for (int s = s0 + 1 + (tid & 63); s < s_end; s += 64) P.part_lse[row + s] = -BGTQ_INF;
            }
        }
        __syncthreads();      // the merge buffer is free again before the next run's tiles land in it
    }
    if (tables_pending) wait_tables();
    if (!dep_waited) grid_dependency_wait();     // (a CTA without items: the launch still completes behind its predecessor)
    if (!ok && P.status && lane == 0) atomicExch(P.status, kStatusWaitTimeout);
}

#ifndef BGTQ_JIT
// Launch one instantiation; defined once per stored V width in its own translation unit.
template <int VB>
cudaError_t launch_decode(const DecParams& P, int nu, dim3 grid, size_t smem, cudaStream_t stream, bool programmatic) {
    auto go = [&](void (*kern)(DecParams)) -> cudaError_t {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        return launch_kernel(kern, grid, dim3(kDecThreads), smem, stream, programmatic, P);
    };
    return nu == 2 ? go(decode_kernel<VB, 2>) : go(decode_kernel<VB, 1>);
}

cudaError_t launch_decode_vb1(const DecParams&, int, dim3, size_t, cudaStream_t, bool);
cudaError_t launch_decode_vb2(const DecParams&, int, dim3, size_t, cudaStream_t, bool);
cudaError_t launch_decode_vb3(const DecParams&, int, dim3, size_t, cudaStream_t, bool);
cudaError_t launch_decode_vb4(const DecParams&, int, dim3, size_t, cudaStream_t, bool);
cudaError_t launch_decode_jit(const DecParams&, dim3, size_t, cudaStream_t, bool);
#endif

}  // namespace bgtq
