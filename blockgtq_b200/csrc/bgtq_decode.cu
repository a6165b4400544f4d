// Fused unpack + dequantise + split-KV attention over the packed cache
// (kernel b).  One launch covers every (batch, KV head, token split) of a layer.
//
// Mapping (per CTA = one split of one (batch, KV head)):
//   * a producer warp streams 64-token tiles of the four cache arrays (packed
//     K, K norms, packed V, V norms) into shared memory with 1-D bulk (TMA)
//     copies completed on mbarriers, kStages deep;
//   * four consumer warps each own 16 tokens of a tile.  Codes are expanded
//     straight into tensor-core operand registers through small fp16x2 lookup
//     tables in shared memory (one per K width segment, one for V), replicated
//     per lane so lookups are bank-conflict free:
//        S^T(16 tok x 8 q)  = sum_seg norm_seg[tok] * ( Khat_seg(16 x k) . Qrot_seg^T )
//        O^T(128 dim x 8 q) += Vhat^T(dim x 16 tok) . P^T(16 tok x 8 q)
//     so the GQA group (<= 8 query heads) is the N dimension of m16n8k16 and no
//     tile row is padding.  Softmax state is fp32 and per warp; warps are
//     merged once at the end of the CTA.
//   * rounding points follow the reference kernel
//     (blockgtq/kernels/fused_packed_attention.py:770-873): fp32 logits,
//     p rounded to fp16 for the PV product while the denominator uses fp32 p,
//     vhat = fp16(fp16 centroid * fp16 norm), fp32 accumulation.
#include "bgtq_common.cuh"
#include "bgtq_plan.h"

namespace bgtq {
namespace {

constexpr int kTileTok = 64;
constexpr int kConsumerWarps = 4;
constexpr int kThreads = 32 * (kConsumerWarps + 1);
constexpr int kStages = 4;
constexpr int kMergeStride = 132;  // floats per query row in the end-of-CTA merge buffer

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
    float scale_log2;
    float* part_o;
    float* part_lse;
    int32_t* status;
    uint32_t lut_off, stage_off, stage_bytes, off_kn, off_v, off_vn;  // shared-memory layout
    DecPlanDev plan;
};

template <int VB>
struct VBits;
template <>
struct VBits<1> { using T = uint32_t; static constexpr uint32_t M = 0x55555555u; };
template <>
struct VBits<2> { using T = uint32_t; static constexpr uint32_t M = 0x33333333u; };
template <>
struct VBits<3> { using T = uint64_t; static constexpr uint64_t M = 0x00001C71C71C71C7ull; };
template <>
struct VBits<4> { using T = uint64_t; static constexpr uint64_t M = 0x0F0F0F0F0F0F0F0Full; };

template <int VB>
__device__ __forceinline__ typename VBits<VB>::T load_v16(uint32_t row, uint32_t bitpos) {
    if constexpr (VB <= 2) {
        return lds_bits32(row, bitpos);
    } else {
        uint2 w = lds_bits64(row, bitpos);
        return (static_cast<uint64_t>(w.y) << 32) | w.x;
    }
}

template <int VB>
__global__ void __launch_bounds__(kThreads) decode_kernel(const __grid_constant__ DecParams P) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const DecHeadPlan& hp = P.plan.head[h];

    const int t0 = P.t_begin + split * P.chunk;
    const int t1 = min(P.t_end, t0 + P.chunk);
    const int n_tok = max(0, t1 - t0);
    const int n_tiles = (n_tok + kTileTok - 1) / kTileTok;

    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + kStages;
    uint16_t* cbk = reinterpret_cast<uint16_t*>(smem + 128);  // 512 K entries + 16 V entries
    uint32_t* lut = reinterpret_cast<uint32_t*>(smem + P.lut_off);
    uint8_t* stages = smem + P.stage_off;

    if (tid == 0) {
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], kConsumerWarps);
        }
        mbar_fence_init();
    }
    {
        const BgtqHeadDesc& d = P.desc[h];
        for (int i = tid; i < 528; i += kThreads) cbk[i] = i < 512 ? d.codebook[i] : d.v_lut[i - 512];
    }
    __syncthreads();
    // Expand codebooks into lane-replicated fp16x2 tables.
    for (int s = 0; s < hp.n_seg; ++s) {
        const DecSegTbl tb = hp.seg[s];
        const uint32_t cm = (1u << tb.bw) - 1u, sm = (1u << tb.sbits) - 1u;
        for (uint32_t i = tid; i < tb.n_words; i += kThreads) {
            const uint32_t e = i >> tb.rep_shift;
            uint32_t v;
            if (tb.pair) v = cbk[tb.cb_off + ((e & sm) & cm)] | (uint32_t(cbk[tb.cb_off + ((e >> tb.sbits) & cm)]) << 16);
            else v = cbk[tb.cb_off + (e & cm)];
            lut[tb.word_off + i] = v;
        }
    }
    {
        const uint32_t vm = (1u << P.plan.v_bits) - 1u, sm = (1u << VB) - 1u;
        for (uint32_t i = tid; i < (uint32_t)P.plan.v_n_words; i += kThreads) {
            const uint32_t e = i >> P.plan.v_rep_shift;
            lut[hp.v_word_off + i] = cbk[512 + ((e & sm) & vm)] | (uint32_t(cbk[512 + ((e >> VB) & vm)]) << 16);
        }
    }
    __syncthreads();

    const size_t bh_kp = (size_t)b * P.kp_sb + (size_t)h * P.kp_sh;
    const size_t bh_kn = (size_t)b * P.kn_sb + (size_t)h * P.kn_sh;
    const size_t bh_vp = (size_t)b * P.vp_sb + (size_t)h * P.vp_sh;
    const size_t bh_vn = (size_t)b * P.vn_sb + (size_t)h * P.vn_sh;

    if (warp == kConsumerWarps) {
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            for (int it = 0; it < n_tiles; ++it) {
                const int st = it % kStages, use = it / kStages;
                if (use > 0 && !mbar_wait_bounded(&empty[st], (use - 1) & 1)) {
                    if (P.status) atomicExch(P.status, kStatusWaitTimeout);
                    break;
                }
                const int t = t0 + it * kTileTok;
                const int nt = min(kTileTok, t1 - t);
                uint8_t* sb = stages + (size_t)st * P.stage_bytes;
                const uint8_t* src[4] = {P.kp + bh_kp + (size_t)t * P.kp_st, P.kn + bh_kn + (size_t)t * P.kn_st,
                                         P.vp + bh_vp + (size_t)t * P.vp_st, P.vn + bh_vn + (size_t)t * P.vn_st};
                const uint32_t len[4] = {(uint32_t)nt * P.kp_st, (uint32_t)nt * P.kn_st, (uint32_t)nt * P.vp_st,
                                         (uint32_t)nt * P.vn_st};
                const uint32_t dst[4] = {0, P.off_kn, P.off_v, P.off_vn};
                uint32_t sz[4], total = 0;
                for (int c = 0; c < 4; ++c) {
                    const uint32_t pre = (uint32_t)(reinterpret_cast<uintptr_t>(src[c]) & 15u);
                    sz[c] = (pre + len[c] + 15u) & ~15u;
                    total += sz[c];
                }
                mbar_arrive_expect_tx(&full[st], total);
                for (int c = 0; c < 4; ++c) {
                    const uint8_t* al = src[c] - (reinterpret_cast<uintptr_t>(src[c]) & 15u);
                    bulk_g2s(sb + dst[c], al, sz[c], &full[st]);
                }
            }
        }
        return;
    }

    // -------------------------------- consumers --------------------------------
    const int r = lane >> 2, j = lane & 3;
    const bool q_ok = r < P.gqa;
    uint32_t qf[kMaxSteps][2];
    {
        const __half* qrow = P.q_rot + ((size_t)b * P.n_q + (size_t)h * P.gqa + (q_ok ? r : 0)) * kHD;
#pragma unroll
        for (int s = 0; s < kMaxSteps; ++s) {
            qf[s][0] = qf[s][1] = 0u;
            if (s < hp.n_steps) {
                const uint32_t c = hp.steps[s].c;
                const int qb = c & 0xFF, nv = (c >> 8) & 0xFF;
                const uint32_t* src = reinterpret_cast<const uint32_t*>(qrow + qb + 4 * j);
                if (q_ok && 4 * j < nv) qf[s][0] = __ldg(src);
                if (q_ok && 4 * j + 2 < nv) qf[s][1] = __ldg(src + 1);
            }
        }
    }

    float O[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) O[i][0] = O[i][1] = O[i][2] = O[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    const uint32_t lut_a = smem_u32(lut);
    const uint32_t vtbl = lut_a + (hp.v_word_off << 2) + ((lane << 2) & ((4u << P.plan.v_rep_shift) - 1u));
    const uint32_t v_sh = P.plan.v_rep_shift + 2;
    bool dead = false;

    for (int it = 0; it < n_tiles; ++it) {
        const int st = it % kStages, use = it / kStages;
        if (!mbar_wait_bounded(&full[st], use & 1)) {
            if (P.status && lane == 0) atomicExch(P.status, kStatusWaitTimeout);
            dead = true;
            break;
        }
        const int t = t0 + it * kTileTok;
        const int nt = min(kTileTok, t1 - t);
        const uint32_t sb = smem_u32(stages + (size_t)st * P.stage_bytes);
        const uint32_t k_a = sb + (uint32_t)((reinterpret_cast<uintptr_t>(P.kp) + bh_kp + (size_t)t * P.kp_st) & 15u);
        const uint32_t kn_a =
            sb + P.off_kn + (uint32_t)((reinterpret_cast<uintptr_t>(P.kn) + bh_kn + (size_t)t * P.kn_st) & 15u);
        const uint32_t v_a =
            sb + P.off_v + (uint32_t)((reinterpret_cast<uintptr_t>(P.vp) + bh_vp + (size_t)t * P.vp_st) & 15u);
        const uint32_t vn_a =
            sb + P.off_vn + (uint32_t)((reinterpret_cast<uintptr_t>(P.vn) + bh_vn + (size_t)t * P.vn_st) & 15u);

        if (warp * 16 < nt) {
            // ---------------- S^T = Khat . Qrot^T ----------------
            const int tokA = warp * 16 + r, tokB = tokA + 8;
            const bool okA = tokA < nt, okB = tokB < nt;
            const uint32_t rowA = k_a + tokA * P.kp_st, rowB = k_a + tokB * P.kp_st;
            const uint32_t nrA = kn_a + tokA * P.kn_st, nrB = kn_a + tokB * P.kn_st;
            float S[4] = {0.f, 0.f, 0.f, 0.f};
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int s = 0; s < kMaxSteps; ++s) {
                if (s < hp.n_steps) {
                    const uint32_t sa = hp.steps[s].a, sbw = hp.steps[s].b;
                    const uint32_t sbits = sbw & 15u, rsh = ((sbw >> 4) & 15u) + 2u;
                    const uint32_t mask = sbw >> 16;
                    const uint32_t bitpos = (sa & 0xFFFFu) + j * 4u * sbits;
                    const uint32_t tb = lut_a + ((sa >> 16) << 2) + ((lane << 2) & ((1u << rsh) - 1u));
                    const uint32_t FA = lds_bits32(rowA, bitpos), FB = lds_bits32(rowB, bitpos);
                    uint32_t a[4];
                    if (sbw & 0x100u) {  // two codes per lookup
                        const uint32_t w2 = 2u * sbits;
                        a[0] = lds32(tb + ((FA & mask) << rsh));
                        a[1] = lds32(tb + ((FB & mask) << rsh));
                        a[2] = lds32(tb + (((FA >> w2) & mask) << rsh));
                        a[3] = lds32(tb + (((FB >> w2) & mask) << rsh));
                    } else {             // raw bytes, one code per lookup
                        a[0] = lds32(tb + ((FA & mask) << rsh)) | (lds32(tb + (((FA >> 8) & mask) << rsh)) << 16);
                        a[1] = lds32(tb + ((FB & mask) << rsh)) | (lds32(tb + (((FB >> 8) & mask) << rsh)) << 16);
                        a[2] = lds32(tb + (((FA >> 16) & mask) << rsh)) | (lds32(tb + (((FA >> 24) & mask) << rsh)) << 16);
                        a[3] = lds32(tb + (((FB >> 16) & mask) << rsh)) | (lds32(tb + (((FB >> 24) & mask) << rsh)) << 16);
                    }
                    mma_16816(acc, a, qf[s]);
                    if (sbw & 0x200u) {  // last k-tile of the segment: apply its norm
                        const uint32_t sg = (sbw >> 12) & 15u;
                        const float nA = __half2float(__ushort_as_half((unsigned short)lds16(nrA + 2u * sg)));
                        const float nB = __half2float(__ushort_as_half((unsigned short)lds16(nrB + 2u * sg)));
                        S[0] = fmaf(nA, acc[0], S[0]);
                        S[1] = fmaf(nA, acc[1], S[1]);
                        S[2] = fmaf(nB, acc[2], S[2]);
                        S[3] = fmaf(nB, acc[3], S[3]);
                        acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
                    }
                }
            }
            // ---------------- online softmax (log2 domain) ----------------
            float s0 = okA ? S[0] * P.scale_log2 : -INFINITY, s1 = okA ? S[1] * P.scale_log2 : -INFINITY;
            float s2 = okB ? S[2] * P.scale_log2 : -INFINITY, s3 = okB ? S[3] * P.scale_log2 : -INFINITY;
            float x0 = fmaxf(s0, s2), x1 = fmaxf(s1, s3);
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) {
                x0 = fmaxf(x0, __shfl_xor_sync(0xffffffffu, x0, o));
                x1 = fmaxf(x1, __shfl_xor_sync(0xffffffffu, x1, o));
            }
            const float n0 = fmaxf(m0, x0), n1 = fmaxf(m1, x1);
            const float z0 = n0 == -INFINITY ? 0.f : n0, z1 = n1 == -INFINITY ? 0.f : n1;
            const float al0 = exp2f(m0 - z0), al1 = exp2f(m1 - z1);
            const float p0 = exp2f(s0 - z0), p1 = exp2f(s1 - z1), p2 = exp2f(s2 - z0), p3 = exp2f(s3 - z1);
            l0 = fmaf(l0, al0, p0 + p2);
            l1 = fmaf(l1, al1, p1 + p3);
            m0 = n0;
            m1 = n1;
            if (__any_sync(0xffffffffu, al0 != 1.f || al1 != 1.f)) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    O[i][0] *= al0;
                    O[i][1] *= al1;
                    O[i][2] *= al0;
                    O[i][3] *= al1;
                }
            }
            uint32_t pf[2];
            pf[0] = movmatrix_trans(pack_half2(p0, p1));
            pf[1] = movmatrix_trans(pack_half2(p2, p3));

            // ---------------- O^T += Vhat^T . P^T ----------------
            const int tk = warp * 16 + 2 * j;
            using VT = typename VBits<VB>::T;
            const uint32_t vbit = 16u * VB * r;
            const VT fA = load_v16<VB>(v_a + (tk + 0) * P.vp_st, vbit), fB = load_v16<VB>(v_a + (tk + 1) * P.vp_st, vbit);
            const VT fC = load_v16<VB>(v_a + (tk + 8) * P.vp_st, vbit), fD = load_v16<VB>(v_a + (tk + 9) * P.vp_st, vbit);
            constexpr VT M = VBits<VB>::M;
            const VT xab = (fA & M) | ((fB & M) << VB), yab = ((fA >> VB) & M) | (fB & (M << VB));
            const VT xcd = (fC & M) | ((fD & M) << VB), ycd = ((fC >> VB) & M) | (fD & (M << VB));
            const uint32_t hA = tk + 0 < nt ? lds16(vn_a + (tk + 0) * P.vn_st) : 0u;
            const uint32_t hB = tk + 1 < nt ? lds16(vn_a + (tk + 1) * P.vn_st) : 0u;
            const uint32_t hC = tk + 8 < nt ? lds16(vn_a + (tk + 8) * P.vn_st) : 0u;
            const uint32_t hD = tk + 9 < nt ? lds16(vn_a + (tk + 9) * P.vn_st) : 0u;
            const uint32_t nab = hA | (hB << 16), ncd = hC | (hD << 16);
            constexpr uint32_t IM = (1u << (2 * VB)) - 1u;
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                uint32_t a[4];
                a[0] = hmul2_u32(lds32(vtbl + (((uint32_t)(xab >> (2 * VB * mt)) & IM) << v_sh)), nab);
                a[1] = hmul2_u32(lds32(vtbl + (((uint32_t)(yab >> (2 * VB * mt)) & IM) << v_sh)), nab);
                a[2] = hmul2_u32(lds32(vtbl + (((uint32_t)(xcd >> (2 * VB * mt)) & IM) << v_sh)), ncd);
                a[3] = hmul2_u32(lds32(vtbl + (((uint32_t)(ycd >> (2 * VB * mt)) & IM) << v_sh)), ncd);
                mma_16816(O[mt], a, pf);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[st]);
    }
    (void)dead;

    // ---------------- merge the four warps, write the split's partial ----------------
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
        const int q = tid >> 4, d0 = (tid & 15) * 8;
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
            float o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < kConsumerWarps; ++w) v = fmaf(mo[(w * 8 + q) * kMergeStride + d0 + i], wgt[w], v);
                o[i] = v * inv;
            }
            const size_t row = ((size_t)b * P.n_q + (size_t)h * P.gqa + q) * P.n_splits + split;
            float4* dst = reinterpret_cast<float4*>(P.part_o + row * kHD + d0);
            dst[0] = make_float4(o[0], o[1], o[2], o[3]);
            dst[1] = make_float4(o[4], o[5], o[6], o[7]);
            if ((tid & 15) == 0)
                P.part_lse[row] = den > 0.f ? (mx + log2f(den)) * 0.6931471805599453f : -INFINITY;
        }
    }
}

// Shared-memory size of the per-head table region: K tables + V table, but at
// least the end-of-CTA merge buffer that reuses the same bytes.
uint32_t lut_region_bytes(const DecPlanDev& pl) {
    uint32_t w = 0;
    for (int h = 0; h < pl.n_heads; ++h) w = max(w, (uint32_t)(pl.head[h].v_word_off + pl.v_n_words));
    const uint32_t merge = (kConsumerWarps * 8 * kMergeStride + 2 * kConsumerWarps * 8) * 4;
    return ((max(w * 4u, merge) + 127u) / 128u) * 128u;
}

}  // namespace
}  // namespace bgtq

using namespace bgtq;

extern "C" __attribute__((visibility("default"))) int bgtq_decode_plan(const BgtqHeadDesc* desc_host, int32_t n_kv, int32_t flags, BgtqDecodePlan* out) {
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
    {
        const uint32_t entries = 1u << (2 * pl.v_sbits);
        uint32_t rep = kLutTableBytes / 4 / entries;
        rep = rep < 1 ? 1 : (rep > 32 ? 32 : rep);
        pl.v_rep_shift = 31 - __builtin_clz(rep);
        pl.v_n_words = entries << pl.v_rep_shift;
    }
    for (int h = 0; h < n_kv; ++h) {
        const BgtqHeadDesc& d = desc_host[h];
        if (d.v_bits != pl.v_bits) return BGTQ_E_UNSUPPORTED;
        if (d.n_seg < 1 || d.n_seg > BGTQ_MAX_SEGMENTS) return BGTQ_E_BADARG;
        DecHeadPlan& hp = pl.head[h];
        hp.n_seg = d.n_seg;
        uint32_t word = 0;
        int step = 0;
        for (int s = 0; s < d.n_seg; ++s) {
            const int bw = d.seg_bw[s], len = d.seg_len[s], start = d.seg_start[s];
            if (bw < 1 || bw > 8 || len < 2 || (len & 1) || start + len > kHD) return BGTQ_E_BADARG;
            int sbits;
            uint32_t bitbase;
            if (flags & BGTQ_DEC_K_MIXED) {
                sbits = bw <= 4 ? 4 : 8;
                bitbase = bw <= 4 ? start * 4u : 8u * (d.nopack_start / 2 + (start - d.nopack_start));
            } else {
                sbits = bw <= 4 ? bw : 8;
                bitbase = 8u * d.seg_pack_off[s];
            }
            const bool pair = sbits <= 4;
            const uint32_t entries = pair ? 1u << (2 * sbits) : 1u << bw;
            uint32_t rep = kLutTableBytes / 4 / entries;
            rep = rep < 1 ? 1 : (rep > 32 ? 32 : rep);
            DecSegTbl& tb = hp.seg[s];
            tb.word_off = word;
            tb.cb_off = d.seg_lut_off[s];
            tb.sbits = sbits;
            tb.bw = bw;
            tb.rep_shift = 31 - __builtin_clz(rep);
            tb.pair = pair;
            tb.n_words = entries << tb.rep_shift;
            const int n_kt = (len + 15) / 16;
            for (int kt = 0; kt < n_kt; ++kt) {
                if (step >= kMaxSteps) return BGTQ_E_UNSUPPORTED;
                DecStep& stp = hp.steps[step++];
                const uint32_t bb = bitbase + kt * 16u * sbits;
                const uint32_t mask = pair ? (1u << (2 * sbits)) - 1u : (1u << bw) - 1u;
                stp.a = (bb & 0xFFFFu) | (word << 16);
                stp.b = sbits | (tb.rep_shift << 4) | (pair ? 0x100u : 0u) | (kt == n_kt - 1 ? 0x200u : 0u) |
                        ((uint32_t)s << 12) | (mask << 16);
                const int nv = len - 16 * kt < 16 ? len - 16 * kt : 16;
                stp.c = (uint32_t)(start + 16 * kt) | ((uint32_t)nv << 8);
            }
            word += tb.n_words;
            if (word > 0xFFFFu) return BGTQ_E_TOOBIG;
        }
        hp.n_steps = step;
        hp.v_word_off = word;
    }
    memcpy(out, &pl, sizeof(pl));
    return BGTQ_OK;
}

extern "C" __attribute__((visibility("default"))) int bgtq_decode_default_splits(int32_t n_batch, int32_t n_kv, int32_t n_tokens) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int pairs = n_batch * n_kv > 0 ? n_batch * n_kv : 1;
    const int by_len = (n_tokens + 255) / 256;  // keep at least 256 tokens per split
    int want = (2 * sms + pairs - 1) / pairs;   // two CTAs per SM
    if (want > by_len) want = by_len;
    return want < 1 ? 1 : want;
}

extern "C" __attribute__((visibility("default"))) int bgtq_decode(const BgtqDecodePlan* plan_host, const BgtqHeadDesc* desc, const void* q_rot,
                           const uint8_t* k_packed, int64_t kp_sb, int64_t kp_sh, int64_t kp_st,
                           const void* k_norms, int64_t kn_sb, int64_t kn_sh, int64_t kn_st,
                           const uint8_t* v_packed, int64_t vp_sb, int64_t vp_sh, int64_t vp_st,
                           const void* v_norms, int64_t vn_sb, int64_t vn_sh, int64_t vn_st, int32_t n_batch,
                           int32_t n_q, int32_t n_kv, int32_t t_begin, int32_t t_end, int32_t n_splits, float scale,
                           float* part_o, float* part_lse, int32_t* status, void* stream) {
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
    int chunk = (n_tok + n_splits - 1) / n_splits;
    chunk = ((chunk + kTileTok - 1) / kTileTok) * kTileTok;
    P.chunk = chunk < kTileTok ? kTileTok : chunk;
    P.scale_log2 = scale * 1.4426950408889634f;
    P.part_o = part_o; P.part_lse = part_lse; P.status = status;

    auto r16 = [](uint32_t x) { return (x + 15u) & ~15u; };
    // each array: 64 rows + 15 bytes of leading phase + rounding + slack for the bit-field over-read
    const uint32_t sz_k = r16(kTileTok * P.kp_st + 48), sz_kn = r16(kTileTok * P.kn_st + 48);
    const uint32_t sz_v = r16(kTileTok * P.vp_st + 48), sz_vn = r16(kTileTok * P.vn_st + 48);
    P.off_kn = sz_k; P.off_v = sz_k + sz_kn; P.off_vn = sz_k + sz_kn + sz_v;
    P.stage_bytes = sz_k + sz_kn + sz_v + sz_vn;
    P.lut_off = 128 + 1152;
    P.stage_off = P.lut_off + lut_region_bytes(P.plan);
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
    kern<<<grid, kThreads, smem, static_cast<cudaStream_t>(stream)>>>(P);
    return cudaGetLastError() == cudaSuccess ? BGTQ_OK : BGTQ_E_LAUNCH;
}
