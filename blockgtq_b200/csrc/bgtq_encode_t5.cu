// Bulk (prefill) encoder with the 128x128 rotation on the fifth-generation tensor cores
// (tcgen05.mma, operands read from shared memory, accumulators in tensor memory).
//
// Same arithmetic contract as the warp-MMA bulk encoder (bgtq_encode_tc.cu); what changes is who does
// the matrix product and how the rest of the work is laid out around it:
//   * a CTA serves one (KV head, K or V) role and works through 128-row tiles.  The rotation W is staged
//     once per CTA as hi = fp16(W), lo = fp16((W - hi) * 2^10); a tile's rows are staged as the A operand
//     (K rows gathered into packed-position order).  Both use the no-swizzle K-major canonical layout:
//     8-row x 16-byte core matrices, 128 B apart along k and 2048 B apart along rows;
//   * one thread issues 16 tcgen05.mma (M = 128, N = 128, K = 16): x . hi into tensor-memory columns
//     [0, 128) and x . lo into [128, 256), then commits them to an mbarrier;
//   * tensor-memory lane r holds the 128 rotated values of row r.  Two threads serve a row (threads r and
//     r + 128: warps w and w + 4 may read the same 32 lanes): each reads half of the columns with
//     tcgen05.ld, scales by 1 / group norm, bins through the code tables and writes code bytes; the pack
//     tasks of the row are shared between the pair the same way.  Loads, norms and the copy of the packed
//     rows to the cache are warp-cooperative over 16 rows per warp;
//   * 110 KB of shared memory and 256 tensor-memory columns per CTA: two CTAs (16 warps) per SM, so one
//     CTA's loads and product overlap the other's quantisation.
// Every wait is bounded; tensor memory is released on every path out of the kernel.
#include "bgtq_common.cuh"
#include "bgtq_encode_params.cuh"

namespace bgtq {
// Sticky error word: set when a wait for the tensor cores ran out (read by bgtq_encode_tcgen05_status).
__device__ int g_t5_status = 0;

namespace {

constexpr int kT5Rows = 128;                  // rows per tile = tensor-memory lanes; two threads per row
constexpr int kT5CodeLd = 132;                // bytes per code row: rows of consecutive lanes fall in distinct banks
constexpr int kT5StageOff = kT5Rows * kT5CodeLd;
constexpr int kT5TileBytes = kT5Rows * kHD * 2;
constexpr int kT5MaxRowBytes = (kT5TileBytes - kT5StageOff) / kT5Rows;     // packed row bytes that fit next to the codes
constexpr uint32_t kT5TmemCols = 256;
constexpr float kT5LoScale = 1024.0f;
constexpr int kT5MaxTasks = 32;

// Byte offset of element (row, k) of a 128 x 128 fp16 operand in the canonical no-swizzle K-major layout.
__device__ __forceinline__ uint32_t canon_off(int row, int k) {
    return (uint32_t)((row >> 3) * 2048 + (k >> 3) * 128 + (row & 7) * 16 + (k & 7) * 2);
}

struct T5Smem {
    __align__(128) uint8_t w_hi[kHD * kHD * 2];
    __align__(128) uint8_t w_lo[kHD * kHD * 2];
    __align__(128) uint8_t tile[kT5TileBytes];      // A operand; after the product: code rows, then staged packed rows
    float gn[BGTQ_MAX_SEGMENTS][kT5Rows];           // group norms (V: [0] = raw row norm)
    float rinv[BGTQ_MAX_SEGMENTS][kT5Rows];         // 1 / norm, or 1 where the norm is below the floor
    float4 colp[kHD / 2];                           // per column pair: {lut_off, lut_inv, bits(group), bits(group * 256)}
    float kcent[512];
    uint8_t code_lut[BGTQ_MAX_SEGMENTS][BGTQ_N_BINS];
    float vbounds[16], vcents[16];
    uint32_t tasks[kT5MaxTasks];                    // first code | count << 8 | width << 12 | byte offset << 16
    int32_t n_tasks, row_bytes, n_seg;
    int32_t seg_start[BGTQ_MAX_SEGMENTS], seg_len[BGTQ_MAX_SEGMENTS], seg_lut_off[BGTQ_MAX_SEGMENTS];
    __align__(8) uint8_t inv_perm[kHD];
    __align__(8) uint64_t mma_bar;
    uint32_t tmem_base;
};
static_assert(sizeof(T5Smem) <= 113 * 1024, "two CTAs per SM");

// ---- tcgen05 wrappers --------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {     // whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t cols) {         // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// shared-memory matrix descriptor: no swizzle, K-major, 128 B between the two k chunks of a step, 2048 B between 8-row groups
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)(128u >> 4) << 16) | ((uint64_t)(2048u >> 4) << 32) |
           (1ull << 46);
}
// D(tmem, 128 x 128 fp32) (+)= A(smem, 128 x 16 fp16) . B(smem, 128 x 16 fp16)^T      (one thread)
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {                          // one thread
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 consecutive fp32 columns of this thread's tensor-memory lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// instruction descriptor: D fp32, A and B fp16, both K-major, N = 128, M = 128
constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(kHD >> 3) << 17) | ((uint32_t)(kT5Rows >> 4) << 24);

// bits of up to four byte-held codes (in the bytes of w) squeezed together, `bw` bits each
__device__ __forceinline__ uint32_t t5_squeeze4(uint32_t w, int bw) {
    switch (bw) {
        case 1: return ((w & 0x01010101u) * 0x10204080u) >> 28;
        case 2: return ((w & 0x03030303u) * 0x01041040u) >> 24;
        case 3: return (w & 7u) | ((w >> 5) & 0x38u) | ((w >> 10) & 0x1C0u) | ((w >> 15) & 0xE00u);
        default: return (w & 0xFu) | ((w >> 4) & 0xF0u) | ((w >> 8) & 0xF00u) | ((w >> 12) & 0xF000u);
    }
}

// Per-CTA tables: rotation split into the operand layout, bin tables, pack tasks.
__device__ void t5_setup(T5Smem& S, const EncParams& P, const BgtqHeadDesc& d, bool is_v, int h) {
    const int tid = threadIdx.x;
    const float* W = (is_v ? P.rot_v : P.rot_k) + (size_t)h * kHD * kHD;
    for (int i = tid; i < kHD * kHD; i += 2 * kT5Rows) {
        const int k = i >> 7, n = i & 127;          // W[k][n], coalesced over n; operand row = output position n
        const float w = __ldg(W + i);
        const __half hi = __float2half_rn(w);
        const uint32_t o = canon_off(n, k);
        *reinterpret_cast<__half*>(S.w_hi + o) = hi;
        *reinterpret_cast<__half*>(S.w_lo + o) = __float2half_rn((w - __half2float(hi)) * kT5LoScale);
    }
    for (int i = tid; i < BGTQ_MAX_SEGMENTS * BGTQ_N_BINS; i += 2 * kT5Rows) S.code_lut[i >> 8][i & 255] = d.code_lut[i >> 8][i & 255];
    for (int i = tid; i < 512; i += 2 * kT5Rows) S.kcent[i] = d.k_cents[i];
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

template <bool IS_V>
__device__ __forceinline__ void t5_role(T5Smem& S, const EncParams& P, const int h, const int role_cta, const int role_ctas,
                                        int64_t* row_src, int64_t* row_dst) {
    constexpr bool is_v = IS_V;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row = tid & (kT5Rows - 1), half = tid >> 7;    // two threads per row: the halves split columns and tasks
    const int n_rows = P.n_batch * P.n_tok;                  // the launcher checks that this fits
    const int n_tiles = (n_rows + kT5Rows - 1) / kT5Rows;
    const int t0 = P.pos_dev ? *P.pos_dev : P.t0;

    const int n_seg = S.n_seg, n_tasks = S.n_tasks, rb = S.row_bytes;
    const int stg_ld = (rb + 3) & ~3;                        // staged rows start on word boundaries
    const bool mixed = !is_v && (P.flags & BGTQ_ENC_K_MIXED);
    const bool f16n = P.flags & BGTQ_ENC_K_NORMS_F16;
    const __half* const src_base = is_v ? P.v + h * P.v_sh : P.k + h * P.k_sh;
    const int64_t s_sb = is_v ? P.v_sb : P.k_sb, s_ss = is_v ? P.v_ss : P.k_ss;
    uint8_t* const out_base = is_v ? P.vp + h * P.vp_sh : P.kp + h * P.kp_sh;
    const int64_t o_sb = is_v ? P.vp_sb : P.kp_sb, o_st = is_v ? P.vp_st : P.kp_st;
    const uint32_t tile_u32 = smem_u32(S.tile), whi_u32 = smem_u32(S.w_hi), wlo_u32 = smem_u32(S.w_lo);
    // warps w and w + 4 read the same 32 tensor-memory lanes (rows), different columns
    const uint32_t tmem_lane = S.tmem_base + ((uint32_t)((warp & 3) * 32) << 16);

    // packed positions of the 8 input columns this lane moves during the load (K only)
    uint32_t koff[8];
    if (!is_v) {
        const uint2 ip = *reinterpret_cast<const uint2*>(&S.inv_perm[(lane & 15) * 8]);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const uint32_t dp = ((c < 4 ? ip.x : ip.y) >> (8 * (c & 3))) & 0xFFu;
            koff[c] = (dp >> 3) * 128u + (dp & 7u) * 2u;
        }
    }
    // V with at most 7 boundaries (1-3 bits): boundaries live in registers, code = number of boundaries below y
    float vb[7];
    bool v_small = false;
    if (is_v) {
        v_small = !(S.vbounds[7] < INFINITY);
#pragma unroll
        for (int i = 0; i < 7; ++i) vb[i] = S.vbounds[i];
    }

    int it = 0;
    for (int tl = role_cta; tl < n_tiles; tl += role_ctas, ++it) {
        const int n0 = tl * kT5Rows;
        // ---- a warp loads and reduces its own 16 rows ----
        if (lane < 16) {   // source / destination offsets of row 16 warp + lane; -1 past the end
            const int rr = 16 * warp + lane, n = n0 + rr;
            int64_t so = -1, dof = -1;
            if (n < n_rows) {
                const int b = n / P.n_tok, s = n - b * P.n_tok;
                so = b * s_sb + s * s_ss;
                dof = b * o_sb + (int64_t)(t0 + s) * o_st;
            }
            row_src[rr] = so;
            row_dst[rr] = dof;
        }
        __syncwarp();
        // V: lane -> row (lane & 7) of an 8-row group, chunk 4 (q & 3) + (lane >> 3): eight lanes fill one 128-byte
        //    core matrix, so the shared stores are conflict free and a row is read 64 bytes at a time.
        // K: lane -> chunk (lane & 15) of rows 2q + (lane >> 4): the lane's eight packed positions stay fixed.
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const int rr = 16 * warp + (is_v ? (q >> 2) * 8 + (lane & 7) : 2 * q + (lane >> 4));
            const int chunk = is_v ? 4 * (q & 3) + (lane >> 3) : (lane & 15);
            const int64_t so = row_src[rr];
            uint4 v = make_uint4(0, 0, 0, 0);
            if (so >= 0) v = __ldg(reinterpret_cast<const uint4*>(src_base + so) + chunk);
            uint8_t* xr = S.tile + (rr >> 3) * 2048 + (rr & 7) * 16;
            if (is_v) {
                *reinterpret_cast<uint4*>(xr + chunk * 128) = v;
            } else {
                const __half* e = reinterpret_cast<const __half*>(&v);
#pragma unroll
                for (int c = 0; c < 8; ++c) *reinterpret_cast<__half*>(xr + koff[c]) = e[c];
            }
        }
        __syncwarp();
        // ---- group norms: lane -> row 16 warp + (lane & 15); the two half-warps take alternate pairs ----
        {
            const int rr = 16 * warp + (lane & 15), par = lane >> 4;
            const uint8_t* xr = S.tile + (rr >> 3) * 2048 + (rr & 7) * 16;
            for (int s = 0; s < n_seg; ++s) {
                const int st = is_v ? 0 : S.seg_start[s], en = is_v ? kHD : st + S.seg_len[s];
                float acc = 0.f;
                for (int p = st + 2 * par; p < en; p += 4) {
                    const float2 x = __half22float2(*reinterpret_cast<const __half2*>(xr + (p >> 3) * 128 + (p & 7) * 2));
                    acc = fmaf(x.x, x.x, acc);
                    acc = fmaf(x.y, x.y, acc);
                }
                acc += __shfl_xor_sync(0xffffffffu, acc, 16);
                if (par == 0) {
                    const float nr = sqrtf(acc + 1e-30f);
                    S.gn[s][rr] = nr;
                    S.rinv[s][rr] = nr > (is_v ? 1e-8f : 1e-10f) ? 1.0f / nr : 1.0f;
                }
            }
        }
        // ---- product: the tile is complete in shared memory; one thread issues, everybody waits ----
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // generic-proxy stores -> tensor-core reads
        tc_fence_before_sync();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after_sync();
#pragma unroll
            for (int ks = 0; ks < kHD / 16; ++ks)
                umma_f16(S.tmem_base, umma_desc(tile_u32 + 256u * ks), umma_desc(whi_u32 + 256u * ks), kIdesc, ks > 0);
#pragma unroll
            for (int ks = 0; ks < kHD / 16; ++ks)
                umma_f16(S.tmem_base + kHD, umma_desc(tile_u32 + 256u * ks), umma_desc(wlo_u32 + 256u * ks), kIdesc, ks > 0);
            umma_commit(&S.mma_bar);
        }
        const int ok = mbar_wait_bounded(&S.mma_bar, it & 1) ? 1 : 0;
        if (!__syncthreads_and(ok)) {           // same verdict for the whole CTA
            if (tid == 0) atomicExch(&g_t5_status, kStatusWaitTimeout);
            break;
        }
        tc_fence_after_sync();
        // ---- quantise this thread's half row: 32 columns at a time out of tensor memory ----
        float csq = 0.f;                        // V: sum of squared levels
        uint8_t* const crow = S.tile + row * kT5CodeLd;
        uint8_t* const srow = S.tile + kT5StageOff + row * stg_ld;
        {   // the staged row starts out zero: this thread clears its half of the words
            const int nw = stg_ld >> 2, w0 = half ? nw >> 1 : 0, w1 = half ? nw : nw >> 1;
            for (int i = w0; i < w1; ++i) reinterpret_cast<uint32_t*>(srow)[i] = 0u;
        }
        const float rv0 = S.rinv[0][row];
#pragma unroll 1
        for (int cc32 = 0; cc32 < 2; ++cc32) {
            const int c32 = 2 * half + cc32;
            float hi[32], lo[32];
            tmem_ld32(tmem_lane + 32u * c32, hi);
            tmem_ld32(tmem_lane + kHD + 32u * c32, lo);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
                uint32_t word = 0;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int col = c32 * 32 + i + e;
                    const float acc = fmaf(lo[i + e], 1.0f / kT5LoScale, hi[i + e]);
                    uint32_t code;
                    if (!is_v) {
                        const float4 cp = S.colp[col >> 1];
                        const float y = acc * S.rinv[__float_as_int(cp.z)][row];
                        float u = (y - cp.x) * cp.y;
                        u = fminf(fmaxf(u, 0.f), 255.f);
                        code = (&S.code_lut[0][0])[__float_as_int(cp.w) + (int)u];
                    } else {
                        const float y = acc * rv0;
                        int cc = 0;
                        if (v_small) {
#pragma unroll
                            for (int b = 0; b < 7; ++b) cc += y > vb[b] ? 1 : 0;
                        } else {         // boundaries are sorted and padded with +inf: four fixed halving steps
#pragma unroll
                            for (int st = 3; st >= 0; --st) cc += y > S.vbounds[cc + (1 << st) - 1] ? (1 << st) : 0;
                        }
                        code = (uint32_t)cc;
                        const float cv = S.vcents[cc];
                        csq = fmaf(cv, cv, csq);
                    }
                    word |= code << (8 * e);
                }
                *reinterpret_cast<uint32_t*>(crow + c32 * 32 + i) = word;
            }
        }
        if (is_v) S.gn[1 + half][row] = csq;    // V uses only group 0 of the norm arrays: park the partial sums here
        tc_fence_before_sync();                 // orders the tensor-memory reads before the barriers below
        __syncthreads();                        // all codes of the tile written, staged rows cleared
        // ---- norms out (first thread of the pair) ----
        if (half == 0) {
            const int n = n0 + row;
            if (!is_v) {
                if (mixed) {   // norm correction: divide by the norm of the chosen levels, per group
                    for (int s = 0; s < n_seg; ++s) {
                        const int st = S.seg_start[s], en = st + S.seg_len[s];
                        const float* cent = S.kcent + S.seg_lut_off[s];
                        float acc = 0.f;
                        for (int p = st; p < en; ++p) {
                            const float cv = cent[crow[p]];
                            acc = fmaf(cv, cv, acc);
                        }
                        S.gn[s][row] = S.gn[s][row] / fmaxf(sqrtf(acc), 1e-10f);
                    }
                }
                if (n < n_rows) {
                    const int b = n / P.n_tok, sq = n - b * P.n_tok;
                    const size_t o = b * P.kn_sb + h * P.kn_sh + (size_t)(t0 + sq) * P.kn_st;
                    for (int s = 0; s < P.kn_count; ++s) {
                        const float val = s < n_seg ? S.gn[s][row] : 0.f;
                        if (f16n) static_cast<__half*>(P.kn)[o + s] = __float2half_rn(val);
                        else static_cast<float*>(P.kn)[o + s] = val;
                    }
                }
            } else if (n < n_rows) {
                const int b = n / P.n_tok, sq = n - b * P.n_tok;
                const float cnorm = sqrtf(S.gn[1][row] + S.gn[2][row] + 1e-20f);
                P.vn[b * P.vn_sb + h * P.vn_sh + (size_t)(t0 + sq) * P.vn_st] =
                    __float2half_rn(S.gn[0][row] / (cnorm > 1e-10f ? cnorm : 1.0f));
            }
        }
        // ---- pack this row: one task = up to 8 codes of one width; the pair takes alternate tasks ----
        for (int ti = half; ti < n_tasks; ti += 2) {
            const uint32_t tk = S.tasks[ti];
            const int first = tk & 0xFF, n = (tk >> 8) & 0xF, bw = (tk >> 12) & 0xF, out = tk >> 16;
            const uint16_t* cs = reinterpret_cast<const uint16_t*>(crow + first);
            uint32_t lo = cs[0] | (uint32_t)cs[1] << 16, hi = cs[2] | (uint32_t)cs[3] << 16;
            if (n < 8) {        // codes past the run belong to the next segment
                if (n <= 4) { hi = 0; lo &= n == 4 ? 0xFFFFFFFFu : (1u << (8 * n)) - 1u; }
                else hi &= (1u << (8 * (n - 4))) - 1u;
            }
            uint8_t* o = srow + out;
            if (bw >= 5) {
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    if (c < n) o[c] = (uint8_t)((c < 4 ? lo >> (8 * c) : hi >> (8 * (c - 4))) & 0xFFu);
            } else {
                const uint32_t word = t5_squeeze4(lo, bw) | t5_squeeze4(hi, bw) << (4 * bw);
                const int nb = bw == 3 ? 3 : (n * bw + 7) >> 3;
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    if (c < nb) o[c] = (uint8_t)(word >> (8 * c));
            }
        }
        __syncthreads();
        // ---- rows out: a warp copies 16 staged rows, 32 bytes per store ----
        for (int r16 = 0; r16 < 16; ++r16) {
            const int rr = 16 * warp + r16;
            const int64_t dof = row_dst[rr];
            if (dof < 0) break;
            const uint8_t* src = S.tile + kT5StageOff + rr * stg_ld;
            for (int p = lane; p < rb; p += 32) out_base[dof + p] = src[p];
        }
        uint8_t* const codes_out = is_v ? P.v_codes : P.k_codes;
        if (codes_out && n0 + row < n_rows) {
            const int n = n0 + row, b = n / P.n_tok, sq = n - b * P.n_tok;
            uint32_t* cd = reinterpret_cast<uint32_t*>(codes_out + (((size_t)b * P.n_kv + h) * P.n_tok + sq) * kHD) + 16 * half;
            for (int i = 0; i < kHD / 8; ++i) cd[i] = *reinterpret_cast<const uint32_t*>(crow + 64 * half + 4 * i);
        }
        __syncthreads();    // tile memory and tensor memory are reused by the next tile
    }
}

constexpr int kT5Threads = 2 * kT5Rows;

__global__ void __launch_bounds__(kT5Threads, 2) encode_t5_kernel(const EncParams P) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    T5Smem& S = *reinterpret_cast<T5Smem*>(smem_raw);
    __shared__ int64_t row_src[kT5Rows], row_dst[kT5Rows];
    const int h = blockIdx.y, tid = threadIdx.x;
    const bool is_v = blockIdx.z != 0 || (P.flags & BGTQ_ENC_SKIP_K);
    if (tid == 0) {
        mbar_init(&S.mma_bar, 1);
        mbar_fence_init();
    }
    if (tid < 32) tmem_alloc(&S.tmem_base, kT5TmemCols);
    t5_setup(S, P, P.desc[h], is_v, h);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");          // W operand: generic stores -> tensor-core reads
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (is_v) t5_role<true>(S, P, h, blockIdx.x, gridDim.x, row_src, row_dst);
    else t5_role<false>(S, P, h, blockIdx.x, gridDim.x, row_src, row_dst);
    tc_fence_before_sync();
    __syncthreads();
    if (tid < 32) tmem_dealloc(S.tmem_base, kT5TmemCols);
}

}  // namespace

// The launcher checks: every input row 16-byte aligned (as for the warp-MMA bulk path).
int launch_encode_t5(const EncParams& P, cudaStream_t stream) {
    const int64_t n_rows = (int64_t)P.n_batch * P.n_tok;
    if (n_rows > (1LL << 30)) return BGTQ_E_TOOBIG;
    const bool do_k = !(P.flags & BGTQ_ENC_SKIP_K), do_v = !(P.flags & BGTQ_ENC_SKIP_V);
    if (!do_k && !do_v) return BGTQ_OK;
    const int n_tiles = (int)((n_rows + kT5Rows - 1) / kT5Rows);
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int roles = (do_k && do_v) ? 2 : 1;
    int per = 2 * sms / (P.n_kv * roles);       // two CTAs per SM, one wave
    if (per < 1) per = 1;
    const int grid_x = per < n_tiles ? per : n_tiles;
    const int smem = (int)sizeof(T5Smem);
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(encode_t5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
            cudaGetLastError();
            return BGTQ_E_LAUNCH;
        }
        attr_set = true;
    }
    encode_t5_kernel<<<dim3(grid_x, P.n_kv, roles), kT5Threads, smem, stream>>>(P);
    return cudaGetLastError() == cudaSuccess ? BGTQ_OK : BGTQ_E_LAUNCH;
}

int encode_t5_max_row_bytes() { return kT5MaxRowBytes & ~3; }

}  // namespace bgtq

extern "C" __attribute__((visibility("default"))) int bgtq_encode_tcgen05_status(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, bgtq::g_t5_status, sizeof(v)) != cudaSuccess) {
        cudaGetLastError();
        return BGTQ_E_LAUNCH;
    }
    return v;
}
