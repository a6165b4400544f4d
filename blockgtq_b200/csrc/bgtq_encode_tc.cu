// Bulk (prefill) encoder on tensor cores.
//
// Same arithmetic contract as encode_kernel (bgtq_encode.cu), organised for throughput:
//   * a CTA serves one (KV head, K or V) role: the 128x128 fp32 rotation is staged in shared memory
//     once, split into hi = fp16(W) and lo = fp16((W - hi) * 2^10);  y = (x . lo) * 2^-10 + x . hi with
//     fp32 accumulation carries about 22 bits of W, the same order as fp32 summation noise (the fp16
//     inputs x are exact);
//   * each of the 16 warps runs its own loop over 16-row slabs, start to finish, with no CTA barrier:
//     load rows (K gathered into packed-position order, which keeps its rotation block diagonal so that
//     k-tiles outside the blocks of a 16-column strip are skipped), group norms, A fragments into
//     registers, then the slab's shared memory is reused for the codes and the packed rows;
//   * dividing by the group norm happens after the product (norm groups are the diagonal blocks);
//   * packing is table driven: one task = up to 8 consecutive codes of one width -> up to 8 bytes;
//   * packed rows of a slab are one contiguous byte range in the cache and leave as 32-bit stores.
#include "bgtq_common.cuh"
#include "bgtq_encode_params.cuh"

namespace bgtq {
namespace {

constexpr int kTcWarps = 16;
constexpr int kSlab = 16;                       // rows per warp iteration
constexpr int kLd = 136;                        // halfs per shared row (128 + 8 pad): conflict-free ldmatrix
constexpr int kSlabBytes = kSlab * kLd * 2;     // 4352
constexpr int kCodeLd = 132;                    // bytes per code row (bank-conflict-free row walks)
constexpr int kStageOff = kSlab * kCodeLd;      // packed-row staging follows the code rows
constexpr int kMaxTasks = 32;
constexpr float kLoScale = 1024.0f;
static_assert(kStageOff + 4 + kSlab * 128 <= kSlabBytes, "codes + staged rows must fit in the slab");

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

struct TcSmem {
    __half w_hi[kHD * kLd];                     // [output position n][input position k]
    __half w_lo[kHD * kLd];
    __align__(16) uint8_t slab[kTcWarps][kSlabBytes];
    float gn[kTcWarps][kSlab][BGTQ_MAX_SEGMENTS];     // group norms (V: [.][0] = raw row norm)
    float rinv[kTcWarps][kSlab][BGTQ_MAX_SEGMENTS];   // 1 / norm, or 1 where the norm is below the floor
    float4 colp[kHD / 2];                       // per column pair: {lut_off, lut_inv, bits(group), bits(group * 256)}
    float kcent[512];
    uint8_t code_lut[BGTQ_MAX_SEGMENTS][BGTQ_N_BINS];
    float vbounds[16], vcents[16];
    uint32_t tasks[kMaxTasks];                  // first code | count << 8 | width << 12 | byte offset << 16
    int32_t n_tasks, row_bytes, n_seg;
    int32_t seg_start[BGTQ_MAX_SEGMENTS], seg_len[BGTQ_MAX_SEGMENTS], seg_lut_off[BGTQ_MAX_SEGMENTS];
    uint8_t kt_lo[8], kt_hi[8];                 // k-tile range per 16-column strip
    __align__(8) uint8_t inv_perm[kHD];
};

// bits of up to four byte-held codes (in the bytes of w) squeezed together, `bw` bits each
__device__ __forceinline__ uint32_t squeeze4(uint32_t w, int bw) {
    switch (bw) {
        case 1: return ((w & 0x01010101u) * 0x10204080u) >> 28;
        case 2: return ((w & 0x03030303u) * 0x01041040u) >> 24;
        case 3: return (w & 7u) | ((w >> 5) & 0x38u) | ((w >> 10) & 0x1C0u) | ((w >> 15) & 0xE00u);
        default: return (w & 0xFu) | ((w >> 4) & 0xF0u) | ((w >> 8) & 0xF00u) | ((w >> 12) & 0xF000u);
    }
}

// Per-CTA tables: rotation split, bin tables, pack tasks.
__device__ void tc_setup(TcSmem& S, const EncParams& P, const BgtqHeadDesc& d, bool is_v, int h) {
    const int tid = threadIdx.x;
    const float* W = (is_v ? P.rot_v : P.rot_k) + (size_t)h * kHD * kHD;
    for (int i = tid; i < kHD * kHD; i += kTcWarps * 32) {
        const int k = i >> 7, n = i & 127;          // coalesced over n
        const float w = __ldg(W + i);
        const __half hi = __float2half_rn(w);
        S.w_hi[n * kLd + k] = hi;
        S.w_lo[n * kLd + k] = __float2half_rn((w - __half2float(hi)) * kLoScale);
    }
    for (int i = tid; i < BGTQ_MAX_SEGMENTS * BGTQ_N_BINS; i += kTcWarps * 32) S.code_lut[i >> 8][i & 255] = d.code_lut[i >> 8][i & 255];
    if (tid < 512) S.kcent[tid] = d.k_cents[tid];
    if (tid < kHD) S.inv_perm[d.head_perm[tid]] = (uint8_t)tid;
    if (tid < kHD / 2) {
        const int g = d.group_of[2 * tid];
        S.colp[tid] = make_float4(d.lut_off[g], d.lut_inv[g], __int_as_float(g), __int_as_float(g * BGTQ_N_BINS));
    }
    if (tid < 16) {
        S.vbounds[tid] = d.v_bounds[tid];
        S.vcents[tid] = d.v_cents[tid];
    }
    if (tid < BGTQ_MAX_SEGMENTS) {
        S.seg_start[tid] = d.seg_start[tid];
        S.seg_len[tid] = d.seg_len[tid];
        S.seg_lut_off[tid] = d.seg_lut_off[tid];
    }
    if (tid < 8) {     // k-tiles a 16-column strip needs: the blocks its columns belong to (V: all)
        int lo = 0, hi = 8;
        if (!is_v) {
            const int g0 = d.group_of[16 * tid], g1 = d.group_of[16 * tid + 15];
            lo = d.seg_start[g0] / 16;
            hi = (d.seg_start[g1] + d.seg_len[g1] + 15) / 16;
        }
        S.kt_lo[tid] = (uint8_t)lo;
        S.kt_hi[tid] = (uint8_t)hi;
    }
    if (tid == 0) {
        int nt = 0;
        auto add_run = [&](int first, int len, int bw, int out) {
            for (int c = 0; c < len; c += 8) {
                const int n = len - c < 8 ? len - c : 8;
                S.tasks[nt++] = (uint32_t)(first + c) | (uint32_t)n << 8 | (uint32_t)bw << 12 | (uint32_t)(out + (bw >= 5 ? c : (c / 8) * bw)) << 16;
            }
        };
        if (is_v) {
            const int vb = (P.flags & BGTQ_ENC_V_NIBBLE) ? 4 : d.v_bits;
            add_run(0, kHD, vb, 0);
            S.row_bytes = seg_storage_bytes(vb, kHD);
        } else if (P.flags & BGTQ_ENC_K_MIXED) {
            add_run(0, d.nopack_start, 4, 0);
            add_run(d.nopack_start, d.nopack_len, 8, d.nopack_start / 2);
            S.row_bytes = P.kp_row_bytes;
        } else {
            for (int s = 0; s < d.n_seg; ++s) add_run(d.seg_start[s], d.seg_len[s], d.seg_bw[s], d.seg_pack_off[s]);
            S.row_bytes = P.kp_row_bytes;
        }
        S.n_tasks = nt;
        S.n_seg = is_v ? 1 : d.n_seg;
    }
}

// Copy `n_bytes` staged bytes (shared, same address phase mod 4 as dst) to global memory.
__device__ __forceinline__ void flat_store(uint8_t* dst, const uint8_t* stg, int n_bytes, int lane) {
    const int head = (int)((4u - (uint32_t)(reinterpret_cast<uintptr_t>(dst) & 3u)) & 3u);
    const int h = head < n_bytes ? head : n_bytes;
    if (lane < h) dst[lane] = stg[lane];
    const int n_words = (n_bytes - h) >> 2;
    const uint32_t* sw = reinterpret_cast<const uint32_t*>(stg + h);
    uint32_t* dw = reinterpret_cast<uint32_t*>(dst + h);
    for (int i = lane; i < n_words; i += 32) dw[i] = sw[i];
    const int done = h + 4 * n_words;
    if (lane < n_bytes - done) dst[done + lane] = stg[done + lane];
}

template <bool IS_V>
__device__ __forceinline__ void tc_role(TcSmem& S, const EncParams& P, const int h, const int role_cta, const int role_ctas) {
    constexpr bool is_v = IS_V;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_rows = P.n_batch * P.n_tok;                  // the launcher checks that this fits
    const int n_slabs = (n_rows + kSlab - 1) / kSlab;
    const int t0 = P.pos_dev ? *P.pos_dev : P.t0;

    const int r = lane >> 2, j = lane & 3;
    uint8_t* const slab = S.slab[warp];
    const uint32_t slab_u32 = smem_u32(slab), whi_base = smem_u32(S.w_hi), wlo_base = smem_u32(S.w_lo);
    const int n_seg = S.n_seg, n_tasks = S.n_tasks, rb = S.row_bytes;
    const bool mixed = !is_v && (P.flags & BGTQ_ENC_K_MIXED);
    const bool f16n = P.flags & BGTQ_ENC_K_NORMS_F16;
    const __half* const src_base = is_v ? P.v + h * P.v_sh : P.k + h * P.k_sh;
    const int64_t s_sb = is_v ? P.v_sb : P.k_sb, s_ss = is_v ? P.v_ss : P.k_ss;
    uint8_t* const out_base = is_v ? P.vp + h * P.vp_sh : P.kp + h * P.kp_sh;
    const int64_t o_sb = is_v ? P.vp_sb : P.kp_sb, o_st = is_v ? P.vp_st : P.kp_st;

    for (int sl = role_cta * kTcWarps + warp; sl < n_slabs; sl += role_ctas * kTcWarps) {
        const int n0 = sl * kSlab;
        const int n_valid = n_rows - n0 < kSlab ? n_rows - n0 : kSlab;
        const int b0 = (int)((uint32_t)n0 / (uint32_t)P.n_tok), s0 = n0 - b0 * P.n_tok;   // n_tok >= kSlab: a slab wraps at most once
        // ---- load 16 rows: lane -> 16-byte column chunk (lane & 15) of rows 2q + (lane >> 4) ----
        {
            uint4 v[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const int row = 2 * q + (lane >> 4);
                v[q] = make_uint4(0, 0, 0, 0);
                if (row < n_valid) {
                    int b = b0, s = s0 + row;
                    if (s >= P.n_tok) { s -= P.n_tok; ++b; }
                    v[q] = __ldg(reinterpret_cast<const uint4*>(src_base + b * s_sb + s * s_ss) + (lane & 15));
                }
            }
            uint32_t dpos[8];       // packed positions of this lane's 8 input columns
            if (!is_v) {
                const uint2 ip = *reinterpret_cast<const uint2*>(&S.inv_perm[(lane & 15) * 8]);
#pragma unroll
                for (int c = 0; c < 8; ++c) dpos[c] = ((c < 4 ? ip.x : ip.y) >> (8 * (c & 3))) & 0xFFu;
            }
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const int row = 2 * q + (lane >> 4);
                __half* xr = reinterpret_cast<__half*>(slab) + row * kLd;
                if (is_v) {
                    *reinterpret_cast<uint4*>(xr + (lane & 15) * 8) = v[q];
                } else {
                    const __half* e = reinterpret_cast<const __half*>(&v[q]);
#pragma unroll
                    for (int c = 0; c < 8; ++c) xr[dpos[c]] = e[c];
                }
            }
        }
        __syncwarp();
        // ---- group norms: lane (row = lane & 15, parity = lane >> 4) walks half2 pairs ----
        {
            const int row = lane & 15, par = lane >> 4;
            const __half2* xr = reinterpret_cast<const __half2*>(slab) + row * (kLd / 2);
            for (int s = 0; s < n_seg; ++s) {
                const int st = is_v ? 0 : S.seg_start[s] >> 1, en = is_v ? kHD / 2 : st + (S.seg_len[s] >> 1);
                float acc = 0.f;
                int p2 = st + par;
                for (; p2 + 6 < en; p2 += 8) {
                    const float2 x0 = __half22float2(xr[p2]), x1 = __half22float2(xr[p2 + 2]);
                    const float2 x2 = __half22float2(xr[p2 + 4]), x3 = __half22float2(xr[p2 + 6]);
                    acc = fmaf(x0.x, x0.x, acc); acc = fmaf(x0.y, x0.y, acc);
                    acc = fmaf(x1.x, x1.x, acc); acc = fmaf(x1.y, x1.y, acc);
                    acc = fmaf(x2.x, x2.x, acc); acc = fmaf(x2.y, x2.y, acc);
                    acc = fmaf(x3.x, x3.x, acc); acc = fmaf(x3.y, x3.y, acc);
                }
                for (; p2 < en; p2 += 2) {
                    const float2 xv = __half22float2(xr[p2]);
                    acc = fmaf(xv.x, xv.x, acc);
                    acc = fmaf(xv.y, xv.y, acc);
                }
                acc += __shfl_xor_sync(0xffffffffu, acc, 16);
                if (par == 0) {
                    const float nr = sqrtf(acc + 1e-30f);
                    S.gn[warp][row][s] = nr;
                    S.rinv[warp][row][s] = nr > (is_v ? 1e-8f : 1e-10f) ? 1.0f / nr : 1.0f;
                }
            }
        }
        // ---- A fragments of the 16 rows into registers; the slab memory is free afterwards ----
        uint32_t a[8][4];
#pragma unroll
        for (int kt = 0; kt < 8; ++kt)
            ldmatrix_x4(a[kt], slab_u32 + 2u * (((lane & 7) + ((lane >> 3) & 1) * 8) * kLd + kt * 16 + (lane >> 4) * 8));
        __syncwarp();
        const float rvA = S.rinv[warp][r][0], rvB = S.rinv[warp][r + 8][0];
        float csqA = 0.f, csqB = 0.f;       // V: running sum of squared levels of this lane's columns
        // ---- rotation + quantisation, one 16-column strip at a time ----
#pragma unroll 1
        for (int np = 0; np < 8; ++np) {
            float acc0[4] = {0, 0, 0, 0}, acc1[4] = {0, 0, 0, 0}, lo0[4] = {0, 0, 0, 0}, lo1[4] = {0, 0, 0, 0};
            const uint32_t kmask = is_v ? 0xFFu : ((1u << S.kt_hi[np]) - (1u << S.kt_lo[np]));
            const uint32_t boff = 2u * ((np * 16 + (lane & 7) + (lane >> 4) * 8) * kLd + ((lane >> 3) & 1) * 8);
#pragma unroll
            for (int kt = 0; kt < 8; ++kt) {
                if (is_v || (kmask >> kt & 1u)) {
                    uint32_t bl[4], bh[4];
                    ldmatrix_x4(bl, wlo_base + boff + 32u * kt);
                    ldmatrix_x4(bh, whi_base + boff + 32u * kt);
                    const uint32_t bl0[2] = {bl[0], bl[1]}, bl1[2] = {bl[2], bl[3]};
                    const uint32_t bh0[2] = {bh[0], bh[1]}, bh1[2] = {bh[2], bh[3]};
                    mma_16816(lo0, a[kt], bl0);
                    mma_16816(lo1, a[kt], bl1);
                    mma_16816(acc0, a[kt], bh0);
                    mma_16816(acc1, a[kt], bh1);
                }
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                acc0[e] = fmaf(lo0[e], 1.0f / kLoScale, acc0[e]);
                acc1[e] = fmaf(lo1[e], 1.0f / kLoScale, acc1[e]);
            }
            // this lane: rows r / r+8, column pairs (16np + 2j) and (16np + 8 + 2j)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const float* ac = half ? acc1 : acc0;
                const int col = np * 16 + half * 8 + 2 * j;
                uint32_t cA, cB;      // two codes of row r / row r+8
                if (!is_v) {
                    const float4 cp = S.colp[col >> 1];
                    const int g = __float_as_int(cp.z);
                    const uint8_t* lut = &S.code_lut[0][0] + __float_as_int(cp.w);
                    const float ra = S.rinv[warp][r][g], rb2 = S.rinv[warp][r + 8][g];
                    uint32_t c[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float y = ac[e] * ((e & 2) ? rb2 : ra);
                        float u = (y - cp.x) * cp.y;
                        u = fminf(fmaxf(u, 0.f), 255.f);
                        c[e] = lut[(int)u];
                    }
                    cA = c[0] | c[1] << 8;
                    cB = c[2] | c[3] << 8;
                } else {
                    uint32_t c[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float y = ac[e] * ((e & 2) ? rvB : rvA);
                        int cc = 0;      // boundaries are sorted and padded with +inf: four fixed halving steps
#pragma unroll
                        for (int st = 3; st >= 0; --st) cc += y > S.vbounds[cc + (1 << st) - 1] ? (1 << st) : 0;
                        c[e] = (uint32_t)cc;
                        const float cv = S.vcents[cc];
                        if (e & 2) csqB = fmaf(cv, cv, csqB); else csqA = fmaf(cv, cv, csqA);
                    }
                    cA = c[0] | c[1] << 8;
                    cB = c[2] | c[3] << 8;
                }
                *reinterpret_cast<uint16_t*>(slab + r * kCodeLd + col) = (uint16_t)cA;
                *reinterpret_cast<uint16_t*>(slab + (r + 8) * kCodeLd + col) = (uint16_t)cB;
            }
        }
        if (is_v) {    // squared level norms: add the four lanes of a quad
            csqA += __shfl_xor_sync(0xffffffffu, csqA, 1);
            csqA += __shfl_xor_sync(0xffffffffu, csqA, 2);
            csqB += __shfl_xor_sync(0xffffffffu, csqB, 1);
            csqB += __shfl_xor_sync(0xffffffffu, csqB, 2);
            if (j == 0) {
                S.rinv[warp][r][1] = csqA;
                S.rinv[warp][r + 8][1] = csqB;
            }
        }
        // byte phase of the staged rows = phase of their cache address, so both sides move as words
        int bfirst = b0, sfirst = s0;
        uint8_t* const dst0 = out_base + bfirst * o_sb + (int64_t)(t0 + sfirst) * o_st;
        const bool flat = o_st == rb && s0 + n_valid <= P.n_tok;
        uint8_t* const stg = slab + kStageOff + (flat ? (int)(reinterpret_cast<uintptr_t>(dst0) & 3u) : 0);
        for (int i = lane; i < (kSlab * rb + 3) / 4 + 1; i += 32) reinterpret_cast<uint32_t*>(slab + kStageOff)[i] = 0u;
        __syncwarp();
        // ---- norms ----
        if (!is_v) {
            if (mixed) {   // norm correction: divide by the norm of the chosen levels, per group
                const int row = lane & 15, par = lane >> 4;
                for (int s = 0; s < n_seg; ++s) {
                    const int st = S.seg_start[s], en = st + S.seg_len[s];
                    const float* cent = S.kcent + S.seg_lut_off[s];
                    float acc = 0.f;
                    for (int p = st + par; p < en; p += 2) {
                        const float cv = cent[slab[row * kCodeLd + p]];
                        acc = fmaf(cv, cv, acc);
                    }
                    acc += __shfl_xor_sync(0xffffffffu, acc, 16);
                    if (par == 0) S.gn[warp][row][s] = S.gn[warp][row][s] / fmaxf(sqrtf(acc), 1e-10f);
                }
                __syncwarp();
            }
            // lane -> (group = lane & 7, row = 4 * pass + (lane >> 3))
            for (int pass = 0; pass < 4; ++pass) {
                const int row = 4 * pass + (lane >> 3), s = lane & 7;
                if (row < n_valid && s < P.kn_count) {
                    int b = b0, t = s0 + row;
                    if (t >= P.n_tok) { t -= P.n_tok; ++b; }
                    const float val = s < n_seg ? S.gn[warp][row][s] : 0.f;
                    const size_t o = b * P.kn_sb + h * P.kn_sh + (size_t)(t0 + t) * P.kn_st + s;
                    if (f16n) static_cast<__half*>(P.kn)[o] = __float2half_rn(val);
                    else static_cast<float*>(P.kn)[o] = val;
                }
            }
        } else if (lane < n_valid) {
            int b = b0, t = s0 + lane;
            if (t >= P.n_tok) { t -= P.n_tok; ++b; }
            const float cnorm = sqrtf(S.rinv[warp][lane][1] + 1e-20f);
            P.vn[b * P.vn_sb + h * P.vn_sh + (size_t)(t0 + t) * P.vn_st] =
                __float2half_rn(S.gn[warp][lane][0] / (cnorm > 1e-10f ? cnorm : 1.0f));
        }
        // ---- pack: one task = up to 8 codes of one width ----
        // lane -> row (lane & 15); the two half-warps take alternate tasks, so a warp runs at most two widths at a time
        for (int ti = lane >> 4; ti < n_tasks; ti += 2) {
            const int row = lane & 15;
            const uint32_t tk = S.tasks[ti];
            const int first = tk & 0xFF, n = (tk >> 8) & 0xF, bw = (tk >> 12) & 0xF, out = tk >> 16;
            const uint16_t* cs = reinterpret_cast<const uint16_t*>(slab + row * kCodeLd + first);
            uint32_t lo = cs[0] | (uint32_t)cs[1] << 16, hi = cs[2] | (uint32_t)cs[3] << 16;
            if (n < 8) {        // codes past the run belong to the next segment
                if (n <= 4) { hi = 0; lo &= n == 4 ? 0xFFFFFFFFu : (1u << (8 * n)) - 1u; }
                else hi &= (1u << (8 * (n - 4))) - 1u;
            }
            uint8_t* o = stg + row * rb + out;
            if (bw >= 5) {
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    if (c < n) o[c] = (uint8_t)((c < 4 ? lo >> (8 * c) : hi >> (8 * (c - 4))) & 0xFFu);
            } else {
                const uint32_t word = squeeze4(lo, bw) | squeeze4(hi, bw) << (4 * bw);
                const int nb = bw == 3 ? 3 : (n * bw + 7) >> 3;
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    if (c < nb) o[c] = (uint8_t)(word >> (8 * c));
            }
        }
        __syncwarp();
        // ---- rows out ----
        if (flat) {
            flat_store(dst0, stg, n_valid * rb, lane);
        } else {
            for (int row = 0; row < n_valid; ++row) {
                int b = b0, t = s0 + row;
                if (t >= P.n_tok) { t -= P.n_tok; ++b; }
                uint8_t* dst = out_base + b * o_sb + (int64_t)(t0 + t) * o_st;
                for (int p = lane; p < rb; p += 32) dst[p] = stg[row * rb + p];
            }
        }
        uint8_t* const codes_out = is_v ? P.v_codes : P.k_codes;
        if (codes_out) {
            for (int row = 0; row < n_valid; ++row) {
                int b = b0, t = s0 + row;
                if (t >= P.n_tok) { t -= P.n_tok; ++b; }
                uint32_t* cd = reinterpret_cast<uint32_t*>(codes_out + (((size_t)b * P.n_kv + h) * P.n_tok + t) * kHD);
                cd[lane] = *reinterpret_cast<const uint32_t*>(slab + row * kCodeLd + 4 * lane);
            }
        }
        __syncwarp();       // the slab is reloaded next
    }
}

__global__ void __launch_bounds__(kTcWarps * 32, 1) encode_tc_kernel(const EncParams P, const int n_k_ctas) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    TcSmem& S = *reinterpret_cast<TcSmem*>(smem_raw);
    const int h = blockIdx.y;
    if (P.pos_dev && !enc_range_ok(P, *P.pos_dev, P.n_tok)) return;      // whole launch, before any set-up
    if (n_k_ctas < 0) {      // bulk: every CTA takes its share of the K slabs, then of the V slabs
        if (!(P.flags & BGTQ_ENC_SKIP_K)) {
            tc_setup(S, P, P.desc[h], false, h);
            __syncthreads();
            tc_role<false>(S, P, h, blockIdx.x, gridDim.x);
            __syncthreads();
        }
        if (!(P.flags & BGTQ_ENC_SKIP_V)) {
            tc_setup(S, P, P.desc[h], true, h);
            __syncthreads();
            tc_role<true>(S, P, h, blockIdx.x, gridDim.x);
        }
        return;
    }
    const bool is_v = (int)blockIdx.x >= n_k_ctas;     // few rows: K and V in separate CTAs, side by side
    tc_setup(S, P, P.desc[h], is_v, h);
    __syncthreads();
    if (is_v) tc_role<true>(S, P, h, blockIdx.x - n_k_ctas, gridDim.x - n_k_ctas);
    else tc_role<false>(S, P, h, blockIdx.x, n_k_ctas);
}

}  // namespace

int launch_encode_tc(const EncParams& P, cudaStream_t stream) {
    const int64_t n_rows = (int64_t)P.n_batch * P.n_tok;
    if (n_rows > (1LL << 30)) return BGTQ_E_TOOBIG;
    const int n_slabs = (int)((n_rows + kSlab - 1) / kSlab);
    const bool do_k = !(P.flags & BGTQ_ENC_SKIP_K), do_v = !(P.flags & BGTQ_ENC_SKIP_V);
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // CTAs per head: fill the SMs once; K and V roles share them in proportion to their cost
    int per = sms / P.n_kv;
    if (per < 2) per = 2;
    const int useful = (n_slabs + kTcWarps - 1) / kTcWarps;     // CTAs of one role that still get a slab per warp
    const int fill = per < useful ? per : useful;
    int n_k, grid_x;        // n_k < 0: every CTA runs the K role, then the V role
    if (do_k && do_v && 2 * useful <= per) { n_k = useful; grid_x = 2 * useful; }
    else if (do_k && do_v) { n_k = -1; grid_x = fill; }
    else if (do_k) { n_k = fill; grid_x = fill; }
    else { n_k = 0; grid_x = fill; }
    const int smem = (int)sizeof(TcSmem);
    // the attribute is per device: set it on every launch (cheap, and legal under stream capture)
    if (cudaFuncSetAttribute(encode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
        cudaGetLastError();
        return BGTQ_E_LAUNCH;
    }
    encode_tc_kernel<<<dim3(grid_x, P.n_kv), kTcWarps * 32, smem, stream>>>(P, n_k);
    return cudaGetLastError() == cudaSuccess ? BGTQ_OK : BGTQ_E_LAUNCH;
}

}  // namespace bgtq
