// Fused unpack + dequantise + split-KV attention over the packed cache
// (kernel b).  One launch covers every (batch, KV head, token split) of a layer.
//
// Mapping (per CTA = one split of one (batch, KV head)):
//   * 256-token tiles of the four cache arrays (packed K, K norms, packed V, V
//     norms) are streamed into shared memory with 1-D bulk (TMA) copies
//     completed on mbarriers, kStages deep.  There is no producer warp: the
//     last of the eight warps to finish with a stage refills it (a counter in
//     shared memory tells a warp that it is the last).  A ninth warp would
//     cost more than its issue slots: 288 threads round up to 320 for register
//     allocation, which holds a two-CTA kernel to 96 registers (with spills in
//     the inner loop) where 256 threads get 128;
//   * each warp owns 32 tokens of a tile.  Codes are expanded
//     straight into tensor-core operand registers through small fp16x2 lookup
//     tables in shared memory (one per K width segment, one for V), replicated
//     per lane so lookups are bank-conflict free:
//        S^T(16 tok x 8 q)  = sum_seg norm_seg[tok] * ( Khat_seg(16 x k) . Qrot_seg^T )
//        O^T(128 dim x 8 q) += Vhat^T(dim x 16 tok) . P^T(16 tok x 8 q)
//     so the GQA group (<= 8 query heads) is the N dimension of m16n8k16 and no
//     tile row is padding.  Softmax state is fp32 and per warp; warps are
//     merged once at the end of the CTA.
//   * the four lanes of a quad share a token; each owns a contiguous run of
//     every K segment's codes, so one unaligned 32-bit shared load feeds several
//     k-tiles (see bgtq_plan.h).  Because 64-token tiles advance every array by
//     a multiple of 16 bytes, all byte phases are per-CTA constants.
//   * rounding points follow the reference kernel
//     (blockgtq/kernels/fused_packed_attention.py:770-873): fp32 logits,
//     p rounded to fp16 for the PV product while the denominator uses fp32 p,
//     vhat = fp16(fp16 centroid * fp16 norm), fp32 accumulation.
#include "bgtq_common.cuh"
#include "bgtq_plan.h"

#include <type_traits>

namespace bgtq {
namespace {

constexpr int kTileTok = 256;      // tokens per CTA tile
constexpr int kWarpTok = 32;       // tokens per consumer warp and tile (two 16-token MMA row tiles)
constexpr int kConsumerWarps = 8;
constexpr int kThreads = 32 * kConsumerWarps;
constexpr int kStages = 2;
constexpr int kMergeStride = 132;  // floats per query row in the end-of-CTA merge buffer
// shared-memory layout (byte offsets from the start of dynamic shared memory)
// [barriers | codebook staging | per-step uniform params | per-step per-lane params | tables | stages]
constexpr uint32_t kOffCbk = 128, kOffStepU = 1280, kOffStepL = kOffStepU + kMaxSteps * 16;   // StepU: per segment
constexpr uint32_t kOffLut = 12288;  // multiple of kLutTableBytes: table bases can be OR-ed into offsets
static_assert(kOffStepL + kMaxSteps * 32 * 16 <= kOffLut && kOffLut % kLutTableBytes == 0, "layout");

struct DecParams {
    const BgtqHeadDesc* desc;
    const __half* q_rot;
    const uint8_t* kp;
    const uint8_t* kn;  // byte pointers; strides below are in bytes
    const uint8_t* vp;
    const uint8_t* vn;
    int64_t kp_sb, kp_sh, kn_sb, kn_sh, vp_sb, vp_sh, vn_sb, vn_sh;
    int32_t kp_st, kn_st, vp_st, vn_st;  // bytes per token
    int32_t n_q, n_kv, gqa;
    int32_t t_begin, t_end, n_splits, chunk;
    const int32_t* pos_dev;
    int32_t pos_add;
    float scale_log2;
    float* part_o;
    float* part_lse;
    int32_t* status;
    // fused merge (optional): the last CTA of each (batch, KV head) to finish merges that pair's partials,
    // applies V's rotation and writes the fp16 result, so no combine launch follows
    int32_t* tickets;
    const float* v_rot;
    __half* out;
    int64_t o_sb, o_sh;
    uint32_t stage_off, stage_bytes, off_kn, off_v, off_vn;  // shared-memory layout
    DecPlanDev plan;
};

// V unpack parameters per stored width: mask of the even-indexed codes of one
// 32-bit group, groups per 16 codes, lane replication of the table.
template <int VB> struct VCfg;
template <> struct VCfg<1> { static constexpr uint32_t M = 0x5555u, GROUPS = 1, REP_SHIFT = 5; };
template <> struct VCfg<2> { static constexpr uint32_t M = 0x33333333u, GROUPS = 1, REP_SHIFT = 5; };
template <> struct VCfg<3> { static constexpr uint32_t M = 0x001C71C7u, GROUPS = 2, REP_SHIFT = 4; };
template <> struct VCfg<4> { static constexpr uint32_t M = 0x0F0F0F0Fu, GROUPS = 2, REP_SHIFT = 2; };

__device__ __forceinline__ uint32_t ld32(const uint8_t* sm, uint32_t off) {
    return *reinterpret_cast<const uint32_t*>(sm + off);
}
__device__ __forceinline__ uint32_t ld16(const uint8_t* sm, uint32_t off) {
    return *reinterpret_cast<const uint16_t*>(sm + off);
}
__device__ __forceinline__ uint32_t rotl32(uint32_t x, uint32_t n) { return __funnelshift_l(x, x, n); }

// 16 codes of one token (bits [bit, bit + 16*VB) past word-aligned offset `row_al`) as one or two
// 32-bit groups of 8 codes.
template <int VB>
__device__ __forceinline__ void load_v16(const uint8_t* sm, uint32_t row_al, uint32_t bit, uint32_t (&g)[2]) {
    const uint32_t wa = row_al + ((bit >> 5) << 2);
    const uint32_t w0 = ld32(sm, wa), w1 = ld32(sm, wa + 4);
    const uint32_t sh = bit & 31u;
    if constexpr (VB <= 2) {
        g[0] = __funnelshift_r(w0, w1, sh);
        g[1] = 0;
    } else {
        const uint32_t w2 = (sh + 16u * VB > 64u) ? ld32(sm, wa + 8) : 0u;
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

template <int VB>
__global__ void __launch_bounds__(kThreads, 2) decode_kernel(const __grid_constant__ DecParams P) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const DecHeadPlan& hp = P.plan.head[h];

    // Everything up to grid_dependency_wait() touches only static tables, so under a programmatic
    // launch it overlaps the tail of the preceding kernel (the step's append / query rotation).
    grid_launch_dependents();
    const int t0 = P.t_begin + split * P.chunk;

    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    unsigned int* done = reinterpret_cast<unsigned int*>(full + kStages);   // warps finished with a stage, ever
    uint16_t* cbk = reinterpret_cast<uint16_t*>(smem + kOffCbk);  // 512 K entries + 16 V entries
    // Per k-tile parameters, expanded once so the inner loop does no decoding:
    //   stepu[seg]     = per-segment constants (same for all lanes), see below
    //   stepl[s][lane] = {Qrot fragment lo, hi, table offset incl. lane column, unit bit offset of this lane}
    uint4* stepu = reinterpret_cast<uint4*>(smem + kOffStepU);
    uint4* stepl = reinterpret_cast<uint4*>(smem + kOffStepL);
    constexpr uint32_t lut_rel = kOffLut;
    uint32_t* lut = reinterpret_cast<uint32_t*>(smem + lut_rel);
    const uint8_t* sm = smem;

    if (tid == 0) {
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&full[i], 1);
            done[i] = 0u;
        }
        mbar_fence_init();
    }
    __syncthreads();
    const size_t bh_kp = (size_t)b * P.kp_sb + (size_t)h * P.kp_sh;
    const size_t bh_kn = (size_t)b * P.kn_sb + (size_t)h * P.kn_sh;
    const size_t bh_vp = (size_t)b * P.vp_sb + (size_t)h * P.vp_sh;
    const size_t bh_vn = (size_t)b * P.vn_sb + (size_t)h * P.vn_sh;
    // One lane streams tile `it` of the range [t0, t1) into its stage.
    auto issue_tile = [&](int it, int t1, uint64_t pol) {
        const int st = it % kStages;
        const int t = t0 + it * kTileTok;
        const int nt = min(kTileTok, t1 - t);
        uint8_t* sb = smem + P.stage_off + (size_t)st * P.stage_bytes;
        const uint8_t* s0 = P.kp + bh_kp + (size_t)t * P.kp_st;
        const uint8_t* s1 = P.kn + bh_kn + (size_t)t * P.kn_st;
        const uint8_t* s2 = P.vp + bh_vp + (size_t)t * P.vp_st;
        const uint8_t* s3 = P.vn + bh_vn + (size_t)t * P.vn_st;
        const uint32_t p0 = (uint32_t)(reinterpret_cast<uintptr_t>(s0) & 15u), p1 = (uint32_t)(reinterpret_cast<uintptr_t>(s1) & 15u);
        const uint32_t p2 = (uint32_t)(reinterpret_cast<uintptr_t>(s2) & 15u), p3 = (uint32_t)(reinterpret_cast<uintptr_t>(s3) & 15u);
        const uint32_t z0 = (p0 + (uint32_t)nt * P.kp_st + 15u) & ~15u, z1 = (p1 + (uint32_t)nt * P.kn_st + 15u) & ~15u;
        const uint32_t z2 = (p2 + (uint32_t)nt * P.vp_st + 15u) & ~15u, z3 = (p3 + (uint32_t)nt * P.vn_st + 15u) & ~15u;
        mbar_arrive_expect_tx(&full[st], z0 + z1 + z2 + z3);
        bulk_g2s_hint(sb, s0 - p0, z0, &full[st], pol);
        bulk_g2s_hint(sb + P.off_kn, s1 - p1, z1, &full[st], pol);
        bulk_g2s_hint(sb + P.off_v, s2 - p2, z2, &full[st], pol);
        bulk_g2s_hint(sb + P.off_vn, s3 - p3, z3, &full[st], pol);
    };
    const uint64_t pol = l2_evict_first_policy();
    constexpr int kBuildThreads = kThreads - 32;
    if (warp == kConsumerWarps - 1) {
        // First tiles: one lane of the last warp starts streaming as soon as the preceding kernel's rows
        // are visible, while the other warps build the tables.
        if (lane == 0) {
            grid_dependency_wait();
            const int t_end = P.pos_dev ? min(P.t_end, *P.pos_dev + P.pos_add) : P.t_end;
            const int t1 = min(t_end, t0 + P.chunk);
            const int n_tiles = (max(0, t1 - t0) + kTileTok - 1) / kTileTok;
            for (int it = 0; it < min(n_tiles, kStages); ++it) issue_tile(it, t1, pol);
        }
        __syncwarp();
    } else {
        // ------------------- tables (named barrier 2 = the building warps only) -------------------
        {
            const BgtqHeadDesc& d = P.desc[h];
            for (int i = tid; i < 528; i += kBuildThreads) cbk[i] = i < 512 ? d.codebook[i] : d.v_lut[i - 512];
        }
        if (warp == 1 && lane < hp.n_seg) {   // per segment: {n_kt | kt/unit << 8 | pair << 16 | norm offset << 20,
                                              //  first rotate, rotate step | pair stride << 8, scaled index mask}
            const DecSegTbl tb = hp.seg[lane];
            const uint32_t esh = tb.rep_shift + 2u;
            const uint32_t mask = (tb.pair ? (1u << (2 * tb.sbits)) - 1u : (1u << tb.bw) - 1u) << esh;
            stepu[lane] = make_uint4(tb.n_kt | ((uint32_t)tb.kt_per_unit << 8) | ((uint32_t)tb.pair << 16) |
                                         ((uint32_t)tb.f16_norm << 17) | ((2u * lane) << 20),
                                     esh, (4u * tb.sbits) | ((2u * tb.sbits) << 8), mask);
        }
        asm volatile("bar.sync 2, %0;" ::"n"(kBuildThreads) : "memory");
        // Expand codebooks into lane-replicated fp16x2 tables.
        for (int s = 0; s < hp.n_seg; ++s) {
            const DecSegTbl tb = hp.seg[s];
            const uint32_t cm = (1u << tb.bw) - 1u, smk = (1u << tb.sbits) - 1u;
            for (uint32_t i = tid; i < tb.n_words; i += kBuildThreads) {
                const uint32_t e = i >> tb.rep_shift;
                uint32_t v;
                if (tb.pair) v = cbk[tb.cb_off + ((e & smk) & cm)] | (uint32_t(cbk[tb.cb_off + ((e >> tb.sbits) & cm)]) << 16);
                else v = cbk[tb.cb_off + (e & cm)];
                lut[tb.word_off + i] = v;
            }
        }
        {
            const uint32_t vm = (1u << P.plan.v_bits) - 1u, smk = (1u << VB) - 1u;
            for (uint32_t i = tid; i < (uint32_t)P.plan.v_n_words; i += kBuildThreads) {
                const uint32_t e = i >> VCfg<VB>::REP_SHIFT;
                lut[hp.v_word_off + i] = cbk[512 + ((e & smk) & vm)] | (uint32_t(cbk[512 + ((e >> VB) & vm)]) << 16);
            }
        }
    }
    grid_dependency_wait();
    const int t_end = P.pos_dev ? min(P.t_end, *P.pos_dev + P.pos_add) : P.t_end;
    const int t1 = min(t_end, t0 + P.chunk);
    const int n_tiles = (max(0, t1 - t0) + kTileTok - 1) / kTileTok;
    if (warp == 0) {   // lane (r, j): query r, this lane's 4 codes of every k-tile
        const int r = lane >> 2, j = lane & 3;
        const bool q_ok = r < P.gqa;
        const __half* qrow = P.q_rot + ((size_t)b * P.n_q + (size_t)h * P.gqa + (q_ok ? r : 0)) * kHD;
        for (int s = 0; s < hp.n_steps; ++s) {
            const DecStep stp = hp.steps[s];
            const int d0 = (int)(stp.q & 0xFFu) + j * (int)((stp.q >> 8) & 0x3Fu);
            const int end = (int)((stp.q >> 14) & 0xFFu);
            const uint32_t* src = reinterpret_cast<const uint32_t*>(qrow + d0);
            const uint32_t esh = (stp.b >> 10) & 31u;
            uint4 v;
            v.x = (q_ok && d0 < end) ? __ldg(src) : 0u;
            v.y = (q_ok && d0 + 2 < end) ? __ldg(src + 1) : 0u;
            v.z = lut_rel + (stp.c >> 16) + (((uint32_t)lane << 2) & ((1u << esh) - 1u));
            v.w = (stp.a & 0xFFFu) + j * ((stp.a >> 12) & 0x3FFu);
            stepl[s * 32 + lane] = v;
        }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory");

    // -------------------------------- consumers --------------------------------
    const int r = lane >> 2, j = lane & 3;
    float O[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) O[i][0] = O[i][1] = O[i][2] = O[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    // Per-CTA byte phases of the four arrays inside a stage (tiles advance every array by a multiple
    // of 16 bytes), and this lane's row offsets for a warp whose first token in the tile is `base`.
    // K side: tokens tok0 + 8 i; V side, row tile u: tokens tkv + 16u + {0, 1, 8, 9}.
    const uint32_t k_pre = (uint32_t)((reinterpret_cast<uintptr_t>(P.kp) + bh_kp + (size_t)t0 * P.kp_st) & 15u);
    const uint32_t kn_pre = (uint32_t)((reinterpret_cast<uintptr_t>(P.kn) + bh_kn + (size_t)t0 * P.kn_st) & 15u);
    const uint32_t v_pre = (uint32_t)((reinterpret_cast<uintptr_t>(P.vp) + bh_vp + (size_t)t0 * P.vp_st) & 15u);
    const uint32_t vn_pre = (uint32_t)((reinterpret_cast<uintptr_t>(P.vn) + bh_vn + (size_t)t0 * P.vn_st) & 15u);
    struct Rows {
        int tok0, tkv;
        uint32_t k_row_al, k_p0, kn_row, v_off, vn_row;
    };
    auto rows_for = [&](int base) {
        Rows ra;
        ra.tok0 = base + r;
        const uint32_t k_off = k_pre + ra.tok0 * P.kp_st;
        ra.k_row_al = k_off & ~3u;
        ra.k_p0 = (k_off & 3u) << 3;
        ra.kn_row = P.off_kn + kn_pre + ra.tok0 * P.kn_st;
        ra.tkv = base + 2 * j;
        ra.v_off = P.off_v + v_pre + ra.tkv * P.vp_st;
        ra.vn_row = P.off_vn + vn_pre + ra.tkv * P.vn_st;
        return ra;
    };
    const Rows rows_full = rows_for(warp * kWarpTok);
    const uint32_t k_row8 = 8u * P.kp_st, kn_row8 = 8u * P.kn_st;

    const uint32_t lane4 = (uint32_t)lane << 2;
    constexpr uint32_t kVSh = VCfg<VB>::REP_SHIFT + 2;
    const uint32_t vtbl = lut_rel + (hp.v_word_off << 2) + (lane4 & ((1u << kVSh) - 1u));
    const int n_seg = hp.n_seg;

    // One warp's share of a tile: NU row tiles of 16 tokens starting at the warp's base token.  (Spreading a
    // short last tile over the warps as single row tiles, NU = 1, measured no faster: the kernel is bound by
    // the SM's instruction throughput, not by the slowest warp of a CTA.)
    auto tile_body = [&](auto nu_tag, const Rows& ra, const uint32_t sb, const int nt) {
        constexpr int NU = decltype(nu_tag)::value;
        const int tok0 = ra.tok0, tkv = ra.tkv;
        // ---------------- S^T = Khat . Qrot^T for NU 16-token row tiles ----------------
        float S[NU][4];
#pragma unroll
        for (int u = 0; u < NU; ++u) S[u][0] = S[u][1] = S[u][2] = S[u][3] = 0.f;
        const uint32_t rowK = sb + ra.k_row_al, rowN = sb + ra.kn_row, k_p0 = ra.k_p0;
        int s = 0;
        for (int sg = 0; sg < n_seg; ++sg) {
            const uint4 su = stepu[sg];
            const int n_kt = su.x & 0xFF, kpu = (su.x >> 8) & 0xFF;
            const uint32_t mask = su.w, dr = su.z & 0xFFu, dp = su.z >> 8;
            // Norm handling: bit-packed layout scales the fp32 dot product of a segment by its fp16
            // norm; the nibble layout rounds centroid * norm to fp16 per element before the product
            // (fused_packed_attention.py:1449-1452), so there the norm is folded into the operand.
            const bool f16n = su.x & 0x20000u;
            float nrm[2 * NU];
            uint32_t n2[2 * NU];
#pragma unroll
            for (int i = 0; i < 2 * NU; ++i) {
                const uint32_t nh = ld16(sm, rowN + (su.x >> 20) + i * kn_row8);
                n2[i] = nh | (nh << 16);
                nrm[i] = f16n ? 1.0f : __half2float(__ushort_as_half((unsigned short)nh));
            }
            float acc[NU][4];
#pragma unroll
            for (int u = 0; u < NU; ++u) acc[u][0] = acc[u][1] = acc[u][2] = acc[u][3] = 0.f;
            uint32_t cur[2 * NU];
#pragma unroll
            for (int i = 0; i < 2 * NU; ++i) cur[i] = 0u;
            uint32_t r0 = su.y;
            int left = 0;
            for (int kt = 0; kt < n_kt; ++kt, ++s) {
                const uint4 sl = stepl[s * 32 + lane];
                if (left == 0) {        // next unit: 32 bits of this lane's run, one word per token
                    const uint32_t pbit = k_p0 + sl.w;
                    const uint32_t wa = rowK + ((pbit >> 5) << 2);
#pragma unroll
                    for (int i = 0; i < 2 * NU; ++i)
                        cur[i] = __funnelshift_r(ld32(sm, wa + i * k_row8), ld32(sm, wa + i * k_row8 + 4), pbit);
                    left = kpu;
                    r0 = su.y;
                }
                --left;
                const uint32_t tb = sl.z;
                uint32_t lo[2 * NU], hi[2 * NU];   // fp16x2 of codes (0,1) and (2,3) of this k-tile, per token
                if (su.x & 0x10000u) {
                    const uint32_t r1 = r0 - dp;
#pragma unroll
                    for (int i = 0; i < 2 * NU; ++i) {
                        lo[i] = ld32(sm, (rotl32(cur[i], r0) & mask) | tb);
                        hi[i] = ld32(sm, (rotl32(cur[i], r1) & mask) | tb);
                    }
                } else {                   // raw bytes, one code per lookup
#pragma unroll
                    for (int i = 0; i < 2 * NU; ++i) {
                        const uint32_t c0 = ld32(sm, (rotl32(cur[i], r0) & mask) | tb);
                        const uint32_t c1 = ld32(sm, (rotl32(cur[i], r0 + 24u) & mask) | tb);
                        const uint32_t c2 = ld32(sm, (rotl32(cur[i], r0 + 16u) & mask) | tb);
                        const uint32_t c3 = ld32(sm, (rotl32(cur[i], r0 + 8u) & mask) | tb);
                        lo[i] = c0 | (c1 << 16);
                        hi[i] = c2 | (c3 << 16);
                    }
                }
                r0 -= dr;
                if (f16n) {
#pragma unroll
                    for (int i = 0; i < 2 * NU; ++i) {
                        lo[i] = hmul2_u32(lo[i], n2[i]);
                        hi[i] = hmul2_u32(hi[i], n2[i]);
                    }
                }
                const uint32_t bq[2] = {sl.x, sl.y};
#pragma unroll
                for (int u = 0; u < NU; ++u) {
                    const uint32_t a[4] = {lo[2 * u], lo[2 * u + 1], hi[2 * u], hi[2 * u + 1]};
                    mma_16816(acc[u], a, bq);
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
        // ---------------- online softmax (log2 domain) over the warp's tokens ----------------
        float sv[NU][4];
        float x0 = -INFINITY, x1 = -INFINITY;
#pragma unroll
        for (int u = 0; u < NU; ++u) {
            const bool okA = tok0 + 16 * u < nt, okB = tok0 + 16 * u + 8 < nt;
            sv[u][0] = okA ? S[u][0] * P.scale_log2 : -INFINITY;
            sv[u][1] = okA ? S[u][1] * P.scale_log2 : -INFINITY;
            sv[u][2] = okB ? S[u][2] * P.scale_log2 : -INFINITY;
            sv[u][3] = okB ? S[u][3] * P.scale_log2 : -INFINITY;
            x0 = fmaxf(x0, fmaxf(sv[u][0], sv[u][2]));
            x1 = fmaxf(x1, fmaxf(sv[u][1], sv[u][3]));
        }
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            x0 = fmaxf(x0, __shfl_xor_sync(0xffffffffu, x0, o));
            x1 = fmaxf(x1, __shfl_xor_sync(0xffffffffu, x1, o));
        }
        const float n0 = fmaxf(m0, x0), n1 = fmaxf(m1, x1);
        const float z0 = n0 == -INFINITY ? 0.f : n0, z1 = n1 == -INFINITY ? 0.f : n1;
        const float al0 = exp2f(m0 - z0), al1 = exp2f(m1 - z1);
        m0 = n0;
        m1 = n1;
        uint32_t pf[NU][2];
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int u = 0; u < NU; ++u) {
            const float p0 = exp2f(sv[u][0] - z0), p1 = exp2f(sv[u][1] - z1);
            const float p2 = exp2f(sv[u][2] - z0), p3 = exp2f(sv[u][3] - z1);
            ps0 += p0 + p2;
            ps1 += p1 + p3;
            pf[u][0] = movmatrix_trans(pack_half2(p0, p1));
            pf[u][1] = movmatrix_trans(pack_half2(p2, p3));
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
            const uint32_t rv = sb + ra.v_off + 16u * u * P.vp_st;
            const uint32_t base = rv & ~3u, bit = ((rv & 3u) << 3) + 16u * VB * r;
            load_v16<VB>(sm, base, bit, gA);
            load_v16<VB>(sm, base, bit + 8u * P.vp_st, gB);
            load_v16<VB>(sm, base, bit + 64u * P.vp_st, gC);
            load_v16<VB>(sm, base, bit + 72u * P.vp_st, gD);
            const int tq = tkv + 16 * u;
            const uint32_t rn = sb + ra.vn_row + 16u * u * P.vn_st;
            const uint32_t hA = tq + 0 < nt ? ld16(sm, rn) : 0u;
            const uint32_t hB = tq + 1 < nt ? ld16(sm, rn + P.vn_st) : 0u;
            const uint32_t hC = tq + 8 < nt ? ld16(sm, rn + 8 * P.vn_st) : 0u;
            const uint32_t hD = tq + 9 < nt ? ld16(sm, rn + 9 * P.vn_st) : 0u;
            const uint32_t nab = hA | (hB << 16), ncd = hC | (hD << 16);
#pragma unroll
            for (int g = 0; g < (int)G; ++g) {
                const uint32_t xab = (gA[g] & M) | ((gB[g] & M) << VB), yab = ((gA[g] >> VB) & M) | (gB[g] & (M << VB));
                const uint32_t xcd = (gC[g] & M) | ((gD[g] & M) << VB), ycd = ((gC[g] >> VB) & M) | (gD[g] & (M << VB));
#pragma unroll
                for (int k = 0; k < PER; ++k) {
                    // index pre-scaled by the entry stride: rotate so the field sits at bit kVSh
                    const uint32_t rt = (32u + kVSh - FW * k) & 31u;
                    uint32_t a[4];
                    a[0] = hmul2_u32(ld32(sm, (rotl32(xab, rt) & IMS) | vtbl), nab);
                    a[1] = hmul2_u32(ld32(sm, (rotl32(yab, rt) & IMS) | vtbl), nab);
                    a[2] = hmul2_u32(ld32(sm, (rotl32(xcd, rt) & IMS) | vtbl), ncd);
                    a[3] = hmul2_u32(ld32(sm, (rotl32(ycd, rt) & IMS) | vtbl), ncd);
                    mma_16816(O[g * PER + k], a, pf[u]);
                }
            }
        }
    };

    for (int it = 0; it < n_tiles; ++it) {
        const int st = it % kStages, use = it / kStages;
        if (!mbar_wait_bounded(&full[st], use & 1)) {
            if (P.status && lane == 0) atomicExch(P.status, kStatusWaitTimeout);
            break;
        }
        const int nt = min(kTileTok, t1 - (t0 + it * kTileTok));
        const uint32_t sb = P.stage_off + st * P.stage_bytes;
        if (warp * kWarpTok < nt) tile_body(std::integral_constant<int, 2>{}, rows_full, sb, nt);
        __syncwarp();
        // Release the stage; the last warp to do so streams the tile that reuses it.  The counter only ever
        // grows: after `use + 1` rounds of this stage all warps have added to it that many times.
        if (lane == 0 && it + kStages < n_tiles) {
            __threadfence_block();
            if (atomicAdd(&done[st], 1u) == (unsigned)(use + 1) * kConsumerWarps - 1u) {
                __threadfence_block();
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                issue_tile(it + kStages, t1, pol);
            }
        }
    }

    // ---------------- merge the warps, write the split's partial ----------------
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, o);
        l1 += __shfl_xor_sync(0xffffffffu, l1, o);
    }
    // All LUT reads are done once every consumer warp is here.
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32));
    float* mo = reinterpret_cast<float*>(lut);                           // [warp][8][kMergeStride]
    float* mm = mo + kConsumerWarps * 8 * kMergeStride;                   // [warp][8] running max
    float* ml = mm + kConsumerWarps * 8;                                  // [warp][8] denominators
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) {
        float* base = mo + (warp * 8 + 2 * j) * kMergeStride + 16 * r + 2 * mt;
        base[0] = O[mt][0];
        base[kMergeStride] = O[mt][1];
        base[1] = O[mt][2];
        base[kMergeStride + 1] = O[mt][3];
    }
    if (r == 0) {
        mm[warp * 8 + 2 * j] = m0;
        mm[warp * 8 + 2 * j + 1] = m1;
        ml[warp * 8 + 2 * j] = l0;
        ml[warp * 8 + 2 * j + 1] = l1;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32));
    {
        const int q = tid >> 5, d0 = (tid & 31) * 4;
        if (q < P.gqa) {
            float mx = -INFINITY;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) mx = fmaxf(mx, mm[w * 8 + q]);
            float wgt[kConsumerWarps], den = 0.f;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) {
                wgt[w] = mx == -INFINITY ? 0.f : exp2f(mm[w * 8 + q] - mx);
                den = fmaf(ml[w * 8 + q], wgt[w], den);
            }
            const float inv = den > 0.f ? 1.f / den : 0.f;
            float o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < kConsumerWarps; ++w) v = fmaf(mo[(w * 8 + q) * kMergeStride + d0 + i], wgt[w], v);
                o[i] = v * inv;
            }
            const size_t row = ((size_t)b * P.n_q + (size_t)h * P.gqa + q) * P.n_splits + split;
            *reinterpret_cast<float4*>(P.part_o + row * kHD + d0) = make_float4(o[0], o[1], o[2], o[3]);
            if ((tid & 31) == 0)
                P.part_lse[row] = den > 0.f ? (mx + log2f(den)) * 0.6931471805599453f : -INFINITY;
        }
    }
    if (P.tickets == nullptr) return;

    // ---------------- fused merge: the pair's last CTA combines all splits ----------------
    // Every CTA publishes its partial (fence), then takes a ticket; the one that draws the last ticket
    // knows all other partials are visible in L2 and reads them with cache-global loads.
    __threadfence();
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory");
    int* flag = reinterpret_cast<int*>(mm);           // the merge scratch is free again
    if (tid == 0) {
        const int t = atomicAdd(P.tickets + b * P.n_kv + h, 1);
        *flag = (t == (int)gridDim.x - 1) ? 1 : 0;
        if (t == (int)gridDim.x - 1) P.tickets[b * P.n_kv + h] = 0;      // ready for the next launch
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory");
    if (*flag == 0) return;
    __threadfence();
    {
        const int q = tid >> 5, d0 = (tid & 31) * 4;        // one warp per query head, four dims per lane
        float* merged = mo;                                   // [8][kHD] merged partial, V's rotated basis
        const int n_sp = (int)gridDim.x;
        if (q < P.gqa) {
            const size_t row = (size_t)b * P.n_q + (size_t)h * P.gqa + q;
            const float* lse = P.part_lse + row * n_sp;
            float mx = -INFINITY;
#pragma unroll 8
            for (int s = 0; s < n_sp; ++s) mx = fmaxf(mx, __ldcg(lse + s));
            float den = 0.f, o[4] = {0.f, 0.f, 0.f, 0.f};
            if (mx > -INFINITY) {
#pragma unroll 8
                for (int s = 0; s < n_sp; ++s) {
                    const float l = __ldcg(lse + s);
                    if (l == -INFINITY) continue;
                    const float a = expf(l - mx);
                    den += a;
                    const float4 v = __ldcg(reinterpret_cast<const float4*>(P.part_o + (row * n_sp + s) * kHD + d0));
                    o[0] = fmaf(a, v.x, o[0]); o[1] = fmaf(a, v.y, o[1]);
                    o[2] = fmaf(a, v.z, o[2]); o[3] = fmaf(a, v.w, o[3]);
                }
            }
            const float inv = den > 0.f ? 1.f / den : 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) merged[q * kHD + d0 + i] = o[i] * inv;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory");
        if (q < P.gqa) {
            float o[4] = {0.f, 0.f, 0.f, 0.f};
            if (P.v_rot) {
                const float* R = P.v_rot + (size_t)h * kHD * kHD + d0;
#pragma unroll 32
                for (int i = 0; i < kHD; ++i) {
                    const float4 rr = __ldg(reinterpret_cast<const float4*>(R + (size_t)i * kHD));
                    const float m = merged[q * kHD + i];
                    o[0] = fmaf(m, rr.x, o[0]); o[1] = fmaf(m, rr.y, o[1]);
                    o[2] = fmaf(m, rr.z, o[2]); o[3] = fmaf(m, rr.w, o[3]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) o[i] = merged[q * kHD + d0 + i];
            }
            __half* dst = P.out + b * P.o_sb + ((int64_t)h * P.gqa + q) * P.o_sh + d0;
            *reinterpret_cast<uint2*>(dst) = make_uint2(pack_half2(o[0], o[1]), pack_half2(o[2], o[3]));
        }
    }
}

constexpr uint32_t v_rep_shift_for(int vb) { return vb <= 2 ? 5 : (vb == 3 ? 4 : 2); }
constexpr uint32_t kMergeBytes = (kConsumerWarps * 8 * kMergeStride + 2 * kConsumerWarps * 8) * 4;

}  // namespace
}  // namespace bgtq

using namespace bgtq;

extern "C" __attribute__((visibility("default"))) int bgtq_decode_plan(const BgtqHeadDesc* desc_host, int32_t n_kv,
                                                                       int32_t flags, BgtqDecodePlan* out) {
    if (!desc_host || !out || n_kv < 1) return BGTQ_E_BADARG;
    if (n_kv > kMaxPlanHeads) return BGTQ_E_TOOBIG;
    static_assert(sizeof(DecPlanDev) <= sizeof(BgtqDecodePlan), "plan does not fit its public container");
    DecPlanDev pl;
    memset(&pl, 0, sizeof(pl));
    pl.n_heads = n_kv;
    pl.flags = flags;
    pl.v_bits = desc_host[0].v_bits;
    if (pl.v_bits < 1 || pl.v_bits > 4) return BGTQ_E_UNSUPPORTED;
    pl.v_sbits = (flags & BGTQ_DEC_V_NIBBLE) ? 4 : pl.v_bits;
    pl.v_rep_shift = v_rep_shift_for(pl.v_sbits);
    pl.v_n_words = (1u << (2 * pl.v_sbits)) << pl.v_rep_shift;
    uint32_t lut_words = 0;
    for (int h = 0; h < n_kv; ++h) {
        const BgtqHeadDesc& d = desc_host[h];
        if (d.v_bits != pl.v_bits) return BGTQ_E_UNSUPPORTED;
        if (d.n_seg < 1 || d.n_seg > BGTQ_MAX_SEGMENTS) return BGTQ_E_BADARG;
        DecHeadPlan& hp = pl.head[h];
        hp.n_seg = d.n_seg;
        int sbits_of[BGTQ_MAX_SEGMENTS];
        uint32_t bitbase_of[BGTQ_MAX_SEGMENTS];
        for (int s = 0; s < d.n_seg; ++s) {
            const int bw = d.seg_bw[s], len = d.seg_len[s], start = d.seg_start[s];
            if (bw < 1 || bw > 8 || len < 2 || (len & 1) || start < 0 || start + len > kHD) return BGTQ_E_BADARG;
            if (flags & BGTQ_DEC_K_MIXED) {
                sbits_of[s] = bw <= 4 ? 4 : 8;
                bitbase_of[s] = bw <= 4 ? start * 4u : 8u * (d.nopack_start / 2 + (start - d.nopack_start));
            } else {
                sbits_of[s] = bw <= 4 ? bw : 8;
                bitbase_of[s] = 8u * d.seg_pack_off[s];
            }
            const bool pair = sbits_of[s] <= 4;
            const uint32_t entries = pair ? 1u << (2 * sbits_of[s]) : 1u << bw;
            // Replication per table: as many per-lane copies as fit in kLutTableBytes.  (8 KB tables, which make
            // the 3-bit pair tables conflict-free, measured under 1 % faster and push some layers past the
            // shared-memory budget of two resident CTAs.)
            const uint32_t cap_bytes = kLutTableBytes;
            uint32_t rep = cap_bytes / 4 / entries;
            rep = rep < 1 ? 1 : (rep > 32 ? 32 : rep);
            DecSegTbl& tb = hp.seg[s];
            tb.cb_off = d.seg_lut_off[s];
            tb.sbits = sbits_of[s];
            tb.bw = bw;
            tb.rep_shift = 31 - __builtin_clz(rep);
            tb.pair = pair;
            tb.n_words = entries << tb.rep_shift;
            if (tb.n_words * 4 > kLutTableBytes) return BGTQ_E_UNSUPPORTED;
            const int n_kt_s = (len + 15) / 16;
            const int cap_s = tb.sbits == 1 ? 32 : tb.sbits == 2 ? 16 : tb.sbits == 8 ? 4 : 8;
            tb.n_kt = (uint8_t)n_kt_s;
            tb.kt_per_unit = (uint8_t)(cap_s / 4);
            tb.f16_norm = ((flags & BGTQ_DEC_K_MIXED) && len >= 16 && s < 5) ? 1 : 0;   // reference: segments 5-7 stay scalar
        }
        // Place tables largest first: every size is a power of two, so each lands on a multiple of its size.
        // (the V table takes part: index d.n_seg)
        uint32_t word = 0;
        bool placed[BGTQ_MAX_SEGMENTS + 1] = {false};
        auto words_of = [&](int s) { return s < d.n_seg ? hp.seg[s].n_words : pl.v_n_words; };
        for (int n = 0; n <= d.n_seg; ++n) {
            int best = -1;
            for (int s = 0; s <= d.n_seg; ++s)
                if (!placed[s] && (best < 0 || words_of(s) > words_of(best))) best = s;
            placed[best] = true;
            if (best < d.n_seg) hp.seg[best].word_off = (uint16_t)word;
            else hp.v_word_off = word;
            word += words_of(best);
        }
        if (word * 4 > 0xFFFFu) return BGTQ_E_TOOBIG;
        lut_words = word > lut_words ? word : lut_words;

        int step = 0;
        for (int s = 0; s < d.n_seg; ++s) {
            const DecSegTbl& tb = hp.seg[s];
            const int sbits = tb.sbits, len = d.seg_len[s], start = d.seg_start[s];
            const int n_kt = (len + 15) / 16;
            const int q = 4 * n_kt;                                  // codes per lane in this segment
            const int cap = sbits == 1 ? 32 : sbits == 2 ? 16 : sbits == 8 ? 4 : 8;   // codes per 32-bit unit
            const uint32_t esh = tb.rep_shift + 2u;
            const uint32_t mask = (tb.pair ? (1u << (2 * sbits)) - 1u : (1u << tb.bw) - 1u) << esh;
            for (int kt = 0; kt < n_kt; ++kt) {
                if (step >= kMaxSteps) return BGTQ_E_UNSUPPORTED;
                DecStep& stp = hp.steps[step++];
                const int code0 = 4 * kt;                            // first code of this k-tile in the lane's run
                const int unit = code0 / cap, in_unit = code0 % cap;
                const uint32_t ubit = bitbase_of[s] + (uint32_t)(unit * cap * sbits);
                const uint32_t jstride = (uint32_t)(q * sbits);
                if (ubit + 3 * jstride + 32 > 0x1000u || jstride > 0x3FFu) return BGTQ_E_UNSUPPORTED;
                const uint32_t ush = (uint32_t)(in_unit * sbits);
                stp.a = ubit | (jstride << 12) | (in_unit == 0 ? 1u << 22 : 0u) | (tb.pair ? 1u << 23 : 0u) |
                        (kt == 0 ? 1u << 24 : 0u);
                const uint32_t r0 = (esh + 64u - ush) & 31u, r1 = (esh + 64u - ush - 2u * sbits) & 31u;
                stp.b = r0 | (r1 << 5) | (esh << 10) | ((uint32_t)s << 15);
                stp.c = mask | (((uint32_t)tb.word_off * 4u) << 16);
                stp.q = (uint32_t)(start + code0) | ((uint32_t)q << 8) | ((uint32_t)(start + len) << 14);
            }
        }
        hp.n_steps = step;
    }
    pl.lut_bytes = ((lut_words * 4u > kMergeBytes ? lut_words * 4u : kMergeBytes) + 127u) / 128u * 128u;
    memcpy(out, &pl, sizeof(pl));
    return BGTQ_OK;
}

extern "C" __attribute__((visibility("default"))) int bgtq_decode_default_splits(int32_t n_batch, int32_t n_kv,
                                                                                 int32_t n_tokens) {
    // Pick the split count with the shortest makespan, counted in CTA tiles: a CTA works through
    // ceil(tiles / splits) tiles, two CTAs are resident per SM, and CTAs beyond the resident slots
    // queue behind the first wave; every CTA also pays a fixed set-up (tables, first tile latency, final
    // merge) worth about one and a half tiles.  Ties go to fewer splits (fewer partials to merge).
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long pairs = (long)n_batch * n_kv > 0 ? (long)n_batch * n_kv : 1;
    if (n_tokens <= kTileTok) return 1;
    const long slots = 2L * sms;
    if (2 * pairs > slots) {
        // More (batch, head) pairs than half the resident slots: the launch runs several waves whatever the
        // split count.  Measured (256 pairs x 16384 tokens): 4 splits of 16 tiles beat 2 splits of 32 tiles by
        // 10 % (2: 343 us, 3: 334, 4: 308, 6: 320, 8: 315), because CTAs that start together also set up
        // together, and many shorter CTAs drift apart and leave a shorter tail.  Aim at 16 tiles per CTA.
        const long tiles = (n_tokens + kTileTok - 1) / kTileTok;
        const long ns = (tiles + 8) / 16;
        return (int)(ns < 1 ? 1 : ns);
    }
    const long max_ns = (n_tokens + kWarpTok - 1) / kWarpTok;
    long best = 1;
    double best_span = -1.0;
    for (long ns = 1; ns <= max_ns && ns <= 512; ++ns) {
        long per = (n_tokens + ns - 1) / ns;                     // tokens per CTA, in warp units
        per = ((per + kWarpTok - 1) / kWarpTok) * kWarpTok;
        const long used = (n_tokens + per - 1) / per;            // non-empty splits
        const long ctas = pairs * used;
        const long waves = (ctas + slots - 1) / slots;
        // full tiles cost 16 units; a partial last tile costs in proportion to its busy warps but not
        // less than a third of a tile; fixed set-up / first-load / merge cost per CTA: 24 units
        const long full = per / kTileTok, rem = per % kTileTok;
        const double tail = rem ? (16.0 * rem / kTileTok > 5.5 ? 16.0 * rem / kTileTok : 5.5) : 0.0;
        double span = waves * (full * 16.0 + tail + 24.0);
        // single-CTA SMs run their CTA faster; charge a half-occupied machine a little more per tile
        if (ctas < slots) span += (double)(slots - ctas) * (full * 16.0 + tail) / 4.0 / slots;
        if (best_span < 0 || span < best_span - 1e-9) { best_span = span; best = used; }
    }
    return (int)best;
}

static int decode_impl(
    const BgtqDecodePlan* plan_host, const BgtqHeadDesc* desc, const void* q_rot, const uint8_t* k_packed,
    int64_t kp_sb, int64_t kp_sh, int64_t kp_st, const void* k_norms, int64_t kn_sb, int64_t kn_sh, int64_t kn_st,
    const uint8_t* v_packed, int64_t vp_sb, int64_t vp_sh, int64_t vp_st, const void* v_norms, int64_t vn_sb,
    int64_t vn_sh, int64_t vn_st, int32_t n_batch, int32_t n_q, int32_t n_kv, int32_t t_begin, int32_t t_end,
    int32_t n_splits, float scale, float* part_o, float* part_lse, int32_t* status, const int32_t* pos_dev,
    int32_t pos_add, void* stream, int32_t* tickets, const float* v_rot, void* out, int64_t o_sb, int64_t o_sh) {
    if (!plan_host || !desc || !q_rot || !k_packed || !k_norms || !v_packed || !v_norms || !part_o || !part_lse)
        return BGTQ_E_BADARG;
    if (n_batch < 1 || n_kv < 1 || n_q < n_kv || n_q % n_kv || n_splits < 1 || t_end < t_begin || t_begin < 0)
        return BGTQ_E_BADARG;
    DecParams P;
    memcpy(&P.plan, plan_host, sizeof(DecPlanDev));
    if (P.plan.n_heads != n_kv) return BGTQ_E_BADARG;
    const int gqa = n_q / n_kv;
    if (gqa > 8) return BGTQ_E_UNSUPPORTED;
    if (kp_st < 1 || kp_st > 160 || vp_st < 1 || vp_st > 128 || kn_st < 1 || kn_st > 16 || vn_st < 1 || vn_st > 8)
        return BGTQ_E_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(part_o) & 15u) || (reinterpret_cast<uintptr_t>(q_rot) & 3u)) return BGTQ_E_ALIGN;
    if (n_batch > 65535 || n_splits > 65535) return BGTQ_E_TOOBIG;

    P.desc = desc;
    P.q_rot = static_cast<const __half*>(q_rot);
    P.kp = k_packed;
    P.kn = static_cast<const uint8_t*>(k_norms);
    P.vp = v_packed;
    P.vn = static_cast<const uint8_t*>(v_norms);
    P.kp_sb = kp_sb; P.kp_sh = kp_sh; P.kp_st = (int32_t)kp_st;
    P.kn_sb = 2 * kn_sb; P.kn_sh = 2 * kn_sh; P.kn_st = (int32_t)(2 * kn_st);
    P.vp_sb = vp_sb; P.vp_sh = vp_sh; P.vp_st = (int32_t)vp_st;
    P.vn_sb = 2 * vn_sb; P.vn_sh = 2 * vn_sh; P.vn_st = (int32_t)(2 * vn_st);
    P.n_q = n_q; P.n_kv = n_kv; P.gqa = gqa;
    P.t_begin = t_begin; P.t_end = t_end; P.n_splits = n_splits;
    const int n_tok = t_end - t_begin;
    // Splits are equal runs of tokens rounded up to a warp's 32 tokens, not to the 256-token tile: the
    // last tile of a CTA may be partial (warps without tokens skip it), which lets the split count fill
    // the resident CTA slots exactly instead of jumping between whole-tile multiples.
    int chunk = (n_tok + n_splits - 1) / n_splits;
    chunk = ((chunk + kWarpTok - 1) / kWarpTok) * kWarpTok;
    P.chunk = chunk < kWarpTok ? kWarpTok : chunk;
    P.scale_log2 = scale * 1.4426950408889634f;
    P.part_o = part_o; P.part_lse = part_lse; P.status = status;
    P.pos_dev = pos_dev; P.pos_add = pos_add;
    P.tickets = tickets; P.v_rot = v_rot; P.out = static_cast<__half*>(out); P.o_sb = o_sb; P.o_sh = o_sh;

    auto r16 = [](uint32_t x) { return (x + 15u) & ~15u; };
    // each array: one tile of rows + 15 bytes of leading phase + rounding + slack for the bit-field over-read
    const uint32_t sz_k = r16(kTileTok * P.kp_st + 48), sz_kn = r16(kTileTok * P.kn_st + 48);
    const uint32_t sz_v = r16(kTileTok * P.vp_st + 48), sz_vn = r16(kTileTok * P.vn_st + 48);
    P.off_kn = sz_k; P.off_v = sz_k + sz_kn; P.off_vn = sz_k + sz_kn + sz_v;
    P.stage_bytes = sz_k + sz_kn + sz_v + sz_vn;
    P.stage_off = kOffLut + P.plan.lut_bytes;
    const size_t smem = (size_t)P.stage_off + (size_t)kStages * P.stage_bytes;
    if (smem > 227 * 1024) return BGTQ_E_TOOBIG;

    void (*kern)(DecParams) = nullptr;
    switch (P.plan.v_sbits) {
        case 1: kern = decode_kernel<1>; break;
        case 2: kern = decode_kernel<2>; break;
        case 3: kern = decode_kernel<3>; break;
        case 4: kern = decode_kernel<4>; break;
        default: return BGTQ_E_UNSUPPORTED;
    }
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return BGTQ_E_LAUNCH;
    }
    dim3 grid(n_splits, n_kv, n_batch);
    return launch_kernel(kern, grid, dim3(kThreads), smem, static_cast<cudaStream_t>(stream),
                         (P.plan.flags & BGTQ_DEC_PROGRAMMATIC) != 0, P) == cudaSuccess ? BGTQ_OK : BGTQ_E_LAUNCH;
}

extern "C" __attribute__((visibility("default"))) int bgtq_decode(
    const BgtqDecodePlan* plan_host, const BgtqHeadDesc* desc, const void* q_rot, const uint8_t* k_packed,
    int64_t kp_sb, int64_t kp_sh, int64_t kp_st, const void* k_norms, int64_t kn_sb, int64_t kn_sh, int64_t kn_st,
    const uint8_t* v_packed, int64_t vp_sb, int64_t vp_sh, int64_t vp_st, const void* v_norms, int64_t vn_sb,
    int64_t vn_sh, int64_t vn_st, int32_t n_batch, int32_t n_q, int32_t n_kv, int32_t t_begin, int32_t t_end,
    int32_t n_splits, float scale, float* part_o, float* part_lse, int32_t* status, const int32_t* pos_dev,
    int32_t pos_add, void* stream) {
    return decode_impl(plan_host, desc, q_rot, k_packed, kp_sb, kp_sh, kp_st, k_norms, kn_sb, kn_sh, kn_st, v_packed,
                       vp_sb, vp_sh, vp_st, v_norms, vn_sb, vn_sh, vn_st, n_batch, n_q, n_kv, t_begin, t_end, n_splits,
                       scale, part_o, part_lse, status, pos_dev, pos_add, stream, nullptr, nullptr, nullptr, 0, 0);
}

extern "C" __attribute__((visibility("default"))) int bgtq_decode_fused(
    const BgtqDecodePlan* plan_host, const BgtqHeadDesc* desc, const void* q_rot, const uint8_t* k_packed,
    int64_t kp_sb, int64_t kp_sh, int64_t kp_st, const void* k_norms, int64_t kn_sb, int64_t kn_sh, int64_t kn_st,
    const uint8_t* v_packed, int64_t vp_sb, int64_t vp_sh, int64_t vp_st, const void* v_norms, int64_t vn_sb,
    int64_t vn_sh, int64_t vn_st, int32_t n_batch, int32_t n_q, int32_t n_kv, int32_t t_begin, int32_t t_end,
    int32_t n_splits, float scale, float* part_o, float* part_lse, int32_t* status, const int32_t* pos_dev,
    int32_t pos_add, const float* v_rot, void* out, int64_t o_sb, int64_t o_sh, int32_t* tickets, void* stream) {
    if (!out || !tickets) return BGTQ_E_BADARG;
    if ((reinterpret_cast<uintptr_t>(out) & 7u) || (o_sb & 3) || (o_sh & 3) || (reinterpret_cast<uintptr_t>(v_rot) & 15u))
        return BGTQ_E_ALIGN;
    return decode_impl(plan_host, desc, q_rot, k_packed, kp_sb, kp_sh, kp_st, k_norms, kn_sb, kn_sh, kn_st, v_packed,
                       vp_sb, vp_sh, vp_st, v_norms, vn_sb, vn_sh, vn_st, n_batch, n_q, n_kv, t_begin, t_end, n_splits,
                       scale, part_o, part_lse, status, pos_dev, pos_add, stream, tickets, v_rot, out, o_sb, o_sh);
}

// ---------------------------------------------------------------------------
// Decode + combine for callers that cannot allocate device memory.
//
// bgtq_decode leaves its per-split partial outputs in a buffer the caller must
// provide.  Some callers have no way to get one: code running inside a CUDA
// graph capture or a stream callback, plugins handed a fixed set of tensors by
// their host framework, and processes whose memory pool is owned by someone
// else.  For them the partials live in the file-scope array below, which every
// GPU that loads this library reserves until the process exits.
// ---------------------------------------------------------------------------
namespace {
constexpr int kNoAllocMaxRows = 8192;    // n_batch * n_q * n_splits
constexpr int kNoAllocMaxDevices = 64;
struct NoAllocScratch {
    float part_o[kNoAllocMaxRows * BGTQ_HEAD_DIM];
    float part_lse[kNoAllocMaxRows];
};
static __device__ __align__(256) NoAllocScratch g_noalloc_scratch;
// Device address of g_noalloc_scratch per device ordinal.  In host code the symbol's name is only a
// handle; the address a kernel can use has to be asked for, with that device current.
NoAllocScratch* g_noalloc_ptr[kNoAllocMaxDevices] = {nullptr};
}  // namespace

extern "C" __attribute__((visibility("default"))) int bgtq_decode_combined_noalloc(
    const BgtqDecodePlan* plan_host, const BgtqHeadDesc* desc, const void* q_rot, const uint8_t* k_packed,
    int64_t kp_sb, int64_t kp_sh, int64_t kp_st, const void* k_norms, int64_t kn_sb, int64_t kn_sh, int64_t kn_st,
    const uint8_t* v_packed, int64_t vp_sb, int64_t vp_sh, int64_t vp_st, const void* v_norms, int64_t vn_sb,
    int64_t vn_sh, int64_t vn_st, int32_t n_batch, int32_t n_q, int32_t n_kv, int32_t t_begin, int32_t t_end,
    int32_t n_splits, float scale, const float* v_rot, void* out, int64_t o_sb, int64_t o_sh, float* lse_out,
    int32_t* status, void* stream) {
    if (n_batch < 1 || n_q < 1 || n_splits < 1 || !out) return BGTQ_E_BADARG;
    if ((int64_t)n_batch * n_q * n_splits > kNoAllocMaxRows) return BGTQ_E_TOOBIG;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices) {
        cudaGetLastError();
        return BGTQ_E_LAUNCH;
    }
    if (!g_noalloc_ptr[dev]) {   // first call on this device: look the array's device address up once
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || !p) {
            cudaGetLastError();
            return BGTQ_E_LAUNCH;
        }
        g_noalloc_ptr[dev] = static_cast<NoAllocScratch*>(p);
    }
    NoAllocScratch* sc = g_noalloc_ptr[dev];
    // Every split of every row is rewritten by the decode kernel (empty splits get zeros and -inf), so
    // nothing left over from the previous call is ever read and nothing needs clearing.
    const int rc = bgtq_decode(plan_host, desc, q_rot, k_packed, kp_sb, kp_sh, kp_st, k_norms, kn_sb, kn_sh, kn_st,
                               v_packed, vp_sb, vp_sh, vp_st, v_norms, vn_sb, vn_sh, vn_st, n_batch, n_q, n_kv,
                               t_begin, t_end, n_splits, scale, sc->part_o, sc->part_lse, status, nullptr, 0, stream);
    if (rc != BGTQ_OK) return rc;
    return bgtq_combine(sc->part_o, sc->part_lse, n_splits, v_rot, nullptr, nullptr, n_batch, n_q, n_kv, out, o_sb,
                        o_sh, nullptr, lse_out, 0, stream);
}
