// Shared by the two prefill-attention kernels (mma.sync and tcgen05): launch parameters, the per-head list of
// dequantisation tasks (8 consecutive codes of one width) and the dequantisers themselves.
#pragma once
#include "bgtq_common.cuh"

namespace bgtq {

constexpr int kPfTok = 64;        // cache tokens per tile
constexpr int kPfMaxTasks = 32;

struct PfParams {
    const BgtqHeadDesc* desc;
    const __half* q;
    int64_t q_sb, q_sh, q_ss;
    const uint8_t *kp, *kn, *vp, *vn;
    int64_t kp_sb, kp_sh, kn_sb, kn_sh, vp_sb, vp_sh, vn_sb, vn_sh;
    int32_t kp_st, kn_st, vp_st, vn_st;      // bytes between token rows
    int32_t n_q, n_kv, gqa, s_q, n_tok, q_pos_offset, causal, flags;
    float scale_log2;
    float* out;
    int32_t* status;                         // tcgen05 kernel: set to 1 when a bounded wait gave up
};

// Dequantisation tasks of one head.  ktask.x: first code | count << 8 | stored bits << 12 | segment << 16 |
// fp16-round << 20; .y: byte offset in the packed row | codebook offset << 16.  Written by one thread.
__device__ inline void pf_build_tasks(const PfParams& P, const BgtqHeadDesc& d, uint2* ktask, uint2* vtask, int32_t* n_ktask,
                                      int32_t* n_vtask) {
    const bool mixed = P.flags & BGTQ_DEC_K_MIXED;
    int nt = 0;
    for (int s = 0; s < d.n_seg; ++s) {
        const int bw = d.seg_bw[s], st = d.seg_start[s], len = d.seg_len[s];
        const int sb = mixed ? (bw <= 4 ? 4 : 8) : (bw <= 4 ? bw : 8);
        // nibble-layout numerics of the reference (fused_packed_attention.py:1449-1452), as in the decode
        // plan: long low-width segments round centroid * norm to fp16
        const int fold = (mixed && len >= 16 && s < 5) ? 1 : 0;
        const int base = mixed ? (bw <= 4 ? st / 2 : d.nopack_start / 2 + (st - d.nopack_start)) : d.seg_pack_off[s];
        for (int c = 0; c < len; c += 8) {
            const int n = len - c < 8 ? len - c : 8;
            ktask[nt] = make_uint2((uint32_t)(st + c) | (uint32_t)n << 8 | (uint32_t)sb << 12 | (uint32_t)s << 16 | (uint32_t)fold << 20,
                                   (uint32_t)(base + (c * sb) / 8) | (uint32_t)d.seg_lut_off[s] << 16);
            ++nt;
        }
    }
    *n_ktask = nt;
    const int vsb = (P.flags & BGTQ_DEC_V_NIBBLE) ? 4 : d.v_bits;
    for (int c = 0; c < kHD; c += 8)
        vtask[c / 8] = make_uint2((uint32_t)c | 8u << 8 | (uint32_t)vsb << 12, (uint32_t)((c * vsb) / 8) | 512u << 16);
    *n_vtask = kHD / 8;
}

// Up to 8 codes of `sb` bits starting at byte p -> fp16 values (optionally times an fp16 norm) at dst.
__device__ __forceinline__ void pf_dequant8(const uint8_t* p, int n, int sb, const uint16_t* cb, bool fold, __half nrm,
                                            __half* dst) {
    const int nbytes = (n * sb + 7) >> 3;
    uint64_t w = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i)
        if (i < nbytes) w |= (uint64_t)p[i] << (8 * i);
    const uint32_t m = (1u << sb) - 1u;
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
        if (i < n) {
            __half a = __ushort_as_half(cb[(uint32_t)(w >> (i * sb)) & m]);
            __half b = __ushort_as_half(cb[(uint32_t)(w >> ((i + 1) * sb)) & m]);
            if (fold) {
                a = __hmul(a, nrm);
                b = __hmul(b, nrm);
            }
            *reinterpret_cast<__half2*>(dst + i) = __halves2half2(a, b);
        }
    }
}

// K variant: value = fp16 centroid * fp16 norm, exact in fp32 (22 significant bits), stored as the sum of
// two fp16 numbers so that the tensor-core product with fp32 accumulation keeps the fp32 norm scaling of
// the decode kernel without a per-segment accumulator.
__device__ __forceinline__ void pf_dequant8_k(const uint8_t* p, int n, int sb, const uint16_t* cb, float nrm,
                                              bool round16, __half* dst_hi, __half* dst_lo) {
    const int nbytes = (n * sb + 7) >> 3;
    uint64_t w = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i)
        if (i < nbytes) w |= (uint64_t)p[i] << (8 * i);
    const uint32_t m = (1u << sb) - 1u;
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
        if (i < n) {
            const float a = __half2float(__ushort_as_half(cb[(uint32_t)(w >> (i * sb)) & m])) * nrm;
            const float b = __half2float(__ushort_as_half(cb[(uint32_t)(w >> ((i + 1) * sb)) & m])) * nrm;
            const __half2 hi = __floats2half2_rn(a, b);
            const float2 hf = __half22float2(hi);
            *reinterpret_cast<__half2*>(dst_hi + i) = hi;
            *reinterpret_cast<__half2*>(dst_lo + i) = round16 ? __floats2half2_rn(0.f, 0.f) : __floats2half2_rn(a - hf.x, b - hf.y);
        }
    }
}

}  // namespace bgtq
