// Bulk (prefill) encoder: the warp-cooperative pipeline of the warp-MMA encoder (bgtq_encode_tc.cu) around
// a tcgen05 product.
//
//   * a CTA of 16 warps serves one (KV head, K or V) role.  The rotation W is staged once as
//     hi = fp16(W), lo = fp16((W - hi) * 2^10) in the no-swizzle K-major canonical operand layout;
//   * the warps form two groups of eight.  A group works on one 128-row tile at a time: each warp loads
//     and reduces ITS 16 rows (a 4 KB piece of the group's A operand), the group meets at a named
//     barrier, one thread issues 16 tcgen05.mma (x . hi and x . lo into 2 x 128 tensor-memory columns) and
//     commits them to the group's mbarrier;
//   * every warp then reads back only its own 16 rows with tcgen05.ld.16x256b, which delivers them in
//     the register layout of mma.sync accumulator tiles, so quantisation, packing and the stores are the
//     warp-MMA encoder's, working out of the warp's own 4 KB of the (now dead) operand tile;
//   * one barrier and one mbarrier wait per tile and group; the two groups run out of phase, so one
//     group's loads overlap the other's quantisation.  217 KB of shared memory, all 512 tensor-memory
//     columns, one CTA per SM;
//   * a warp's input rows for its NEXT tile are fetched with cp.async into a raw buffer while it works on
//     the current one.
// Every wait is bounded; tensor memory is released on every path out of the kernel.
#include "bgtq_common.cuh"
#include "bgtq_encode_params.cuh"
#include "bgtq_tcgen05.cuh"

namespace bgtq {
// Sticky error word of this kernel: set when a wait for the tensor cores ran out.
__device__ int g_t5w_status = 0;

namespace {

constexpr int kWarps = 16;
constexpr int kGroupWarps = 8;
constexpr int kSlab = 16;                       // rows per warp
constexpr int kTileRows = kGroupWarps * kSlab;  // 128 = tensor-memory lanes
constexpr int kSlabBytes = kSlab * kHD * 2;     // 4096: a warp's rows of the operand tile = its scratch afterwards
constexpr int kCodeLd = 132;                    // bytes per code row (bank-conflict-free row walks)
constexpr int kStageOff = kSlab * kCodeLd;      // packed-row staging follows the code rows
constexpr int kMaxRowBytes = (kSlabBytes - kStageOff - 8) / kSlab;   // 123
constexpr int kMaxTasks = 32;
constexpr float kLoScale = 1024.0f;
constexpr uint32_t kTmemCols = 512;             // per group: hi accumulator 128 columns + lo accumulator 128 columns
// instruction descriptor: D fp32, A and B fp16, both K-major, N = 128, M = 128
constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(kHD >> 3) << 17) | ((uint32_t)(kTileRows >> 4) << 24);

struct WSmem {
    __align__(128) uint8_t w_hi[kHD * kHD * 2];
    __align__(128) uint8_t w_lo[kHD * kHD * 2];
    __align__(128) uint8_t tile[2][kTileRows * kHD * 2];    // A operand of each group; per-warp scratch after the product
    __align__(128) uint8_t raw[kWarps][kSlabBytes];         // next tile's input rows per warp, fetched with cp.async (16-byte chunks XOR-swizzled by row)
    float gn[kWarps][kSlab][BGTQ_MAX_SEGMENTS];     // group norms (V: [.][0] = raw row norm)
    float rinv[kWarps][kSlab][BGTQ_MAX_SEGMENTS];   // 1 / norm, or 1 where the norm is below the floor
    float4 colp[kHD / 2];                           // per column pair: {lut_off, lut_inv, bits(group), bits(group * 256)}
    float kcent[512];
    uint8_t code_lut[BGTQ_MAX_SEGMENTS][BGTQ_N_BINS];
    float vbounds[16], vcents[16];
    uint32_t tasks[kMaxTasks];                      // first code | count << 8 | width << 12 | byte offset << 16
    int32_t n_tasks, row_bytes, n_seg;
    int32_t seg_start[BGTQ_MAX_SEGMENTS], seg_len[BGTQ_MAX_SEGMENTS], seg_lut_off[BGTQ_MAX_SEGMENTS];
    __align__(8) uint8_t inv_perm[kHD];
    __align__(8) uint64_t mma_bar[2];
    uint32_t tmem_base;
};
static_assert(sizeof(WSmem) > 114 * 1024 && sizeof(WSmem) <= 227 * 1024, "exactly one CTA per SM (it takes all tensor memory)");

// bits of up to four byte-held codes (in the bytes of w) squeezed together, `bw` bits each
__device__ __forceinline__ uint32_t w_squeeze4(uint32_t w, int bw) {
    switch (bw) {
        case 1: return ((w & 0x01010101u) * 0x10204080u) >> 28;
        case 2: return ((w & 0x03030303u) * 0x01041040u) >> 24;
        case 3: return (w & 7u) | ((w >> 5) & 0x38u) | ((w >> 10) & 0x1C0u) | ((w >> 15) & 0xE00u);
        default: return (w & 0xFu) | ((w >> 4) & 0xF0u) | ((w >> 8) & 0xF00u) | ((w >> 12) & 0xF000u);
    }
}

// Copy `n_bytes` staged bytes (shared, same address phase mod 4 as dst) to global memory.
__device__ __forceinline__ void w_flat_store(uint8_t* dst, const uint8_t* stg, int n_bytes, int lane) {
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

// Per-CTA tables: rotation split into the operand layout, bin tables, pack tasks.
__device__ void w_setup(WSmem& S, const EncParams& P, const BgtqHeadDesc& d, bool is_v, int h) {
    const int tid = threadIdx.x;
    const float* W = (is_v ? P.rot_v : P.rot_k) + (size_t)h * kHD * kHD;
    for (int i = tid; i < kHD * kHD; i += kWarps * 32) {
        const int k = i >> 7, n = i & 127;          // W[k][n], coalesced over n; operand row = output position n
        const float w = __ldg(W + i);
        const __half hi = __float2half_rn(w);
        const uint32_t o = (uint32_t)((n >> 3) * 2048 + (k >> 3) * 128 + (n & 7) * 16 + (k & 7) * 2);
        *reinterpret_cast<__half*>(S.w_hi + o) = hi;
        *reinterpret_cast<__half*>(S.w_lo + o) = __float2half_rn((w - __half2float(hi)) * kLoScale);
    }
    for (int i = tid; i < BGTQ_MAX_SEGMENTS * BGTQ_N_BINS; i += kWarps * 32) S.code_lut[i >> 8][i & 255] = d.code_lut[i >> 8][i & 255];
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
__device__ __forceinline__ void w_role(WSmem& S, const EncParams& P, const int h, const int role_cta, const int role_ctas) {
    constexpr bool is_v = IS_V;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int grp = warp >> 3, wg = warp & 7;
    // A warp may read tensor-memory lanes [32 (warp % 4), +32) only: warp wg of a group takes the 16-row slab
    // 2 (wg % 4) + wg / 4 of the tile.
    const int slab_i = 2 * (wg & 3) + (wg >> 2);
    const int n_rows = P.n_batch * P.n_tok;                  // the launcher checks that this fits
    const int n_tiles = (n_rows + kTileRows - 1) / kTileRows;
    const int t0 = P.pos_dev ? *P.pos_dev : P.t0;

    const int r = lane >> 2, j = lane & 3;
    uint8_t* const slab = S.tile[grp] + slab_i * kSlabBytes;     // rows 16 slab_i .. +15: two 8-row groups of 2048 B
    const uint32_t tile_u32 = smem_u32(S.tile[grp]), whi_u32 = smem_u32(S.w_hi), wlo_u32 = smem_u32(S.w_lo);
    const uint32_t tmem_acc = S.tmem_base + 256u * grp;
    const uint32_t tmem_rows = tmem_acc + ((uint32_t)(16 * slab_i) << 16);
    uint64_t* const bar = &S.mma_bar[grp];
    const int n_seg = S.n_seg, n_tasks = S.n_tasks, rb = S.row_bytes;
    const bool mixed = !is_v && (P.flags & BGTQ_ENC_K_MIXED);
    const bool f16n = P.flags & BGTQ_ENC_K_NORMS_F16;
    const __half* const src_base = is_v ? P.v + h * P.v_sh : P.k + h * P.k_sh;
    const int64_t s_sb = is_v ? P.v_sb : P.k_sb, s_ss = is_v ? P.v_ss : P.k_ss;
    uint8_t* const out_base = is_v ? P.vp + h * P.vp_sh : P.kp + h * P.kp_sh;
    const int64_t o_sb = is_v ? P.vp_sb : P.kp_sb, o_st = is_v ? P.vp_st : P.kp_st;

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

    // Input rows of tile `tl` -> this warp's raw buffer, asynchronously: lane -> chunk (lane & 15) of rows
    // 2q + (lane >> 4); rows past the end are zero-filled.  Chunk c of row rr sits at rr * 256 + ((c ^ (rr & 7)) * 16.
    uint8_t* const raw = S.raw[warp];
    const uint32_t raw_u32 = smem_u32(raw);
    auto prefetch = [&](int tl) {
        const int n0 = tl * kTileRows + slab_i * kSlab;
        const int b0 = (int)((uint32_t)n0 / (uint32_t)P.n_tok), s0 = n0 - b0 * P.n_tok;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const int row = 2 * q + (lane >> 4), chunk = lane & 15;
            int b = b0, s = s0 + row;
            if (s >= P.n_tok) { s -= P.n_tok; ++b; }
            const bool valid = tl < n_tiles && n0 + row < n_rows;
            const __half* src = valid ? src_base + b * s_sb + s * s_ss + chunk * 8 : src_base;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(raw_u32 + row * 256 + ((chunk ^ (row & 7)) << 4)),
                         "l"(src), "r"(valid ? 16 : 0)
                         : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    prefetch(2 * role_cta + grp);

    int it = 0;
    for (int tl = 2 * role_cta + grp; tl < n_tiles; tl += 2 * role_ctas, ++it) {
        const int n0 = tl * kTileRows + slab_i * kSlab;
        const int n_valid = n_rows - n0 < kSlab ? (n_rows - n0 > 0 ? n_rows - n0 : 0) : kSlab;
        const int b0 = (int)((uint32_t)n0 / (uint32_t)P.n_tok), s0 = n0 - b0 * P.n_tok;   // n_tok >= kSlab: a slab wraps at most once
        // ---- the prefetched rows -> operand layout (row rr: (rr >> 3) * 2048 + (rr & 7) * 16; chunk c: + 128 c) ----
        // V: lane -> row (lane & 7) of an 8-row group, chunk 4 (q & 3) + (lane >> 3): eight lanes fill one 128-byte
        //    core matrix; K: lane -> chunk (lane & 15) of rows 2q + (lane >> 4): the lane's eight packed positions
        //    stay fixed.  Both read patterns are conflict free in the swizzled raw buffer.
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncwarp();
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const int row = is_v ? (q >> 2) * 8 + (lane & 7) : 2 * q + (lane >> 4);
            const int chunk = is_v ? 4 * (q & 3) + (lane >> 3) : (lane & 15);
            const uint4 v = *reinterpret_cast<const uint4*>(raw + row * 256 + ((chunk ^ (row & 7)) << 4));
            uint8_t* xr = slab + (row >> 3) * 2048 + (row & 7) * 16;
            if (is_v) {
                *reinterpret_cast<uint4*>(xr + chunk * 128) = v;
            } else {
                const __half* e = reinterpret_cast<const __half*>(&v);
#pragma unroll
                for (int c = 0; c < 8; ++c) *reinterpret_cast<__half*>(xr + koff[c]) = e[c];
            }
        }
        __syncwarp();
        prefetch(tl + 2 * role_ctas);       // the raw buffer is free again: the next tile's rows arrive during this tile's work
        __syncwarp();
        // ---- group norms: lane -> row (lane & 15); the two half-warps take alternate element pairs ----
        {
            const int row = lane & 15, par = lane >> 4;
            const uint8_t* xr = slab + (row >> 3) * 2048 + (row & 7) * 16;
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
                    S.gn[warp][row][s] = nr;
                    S.rinv[warp][row][s] = nr > (is_v ? 1e-8f : 1e-10f) ? 1.0f / nr : 1.0f;
                }
            }
        }
        // ---- product: the group's tile is complete; one thread issues, the group waits ----
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // generic-proxy stores -> tensor-core reads
        tc_fence_before_sync();     // also orders this warp's tensor-memory reads of the previous tile
        asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "n"(kGroupWarps * 32) : "memory");
        if (wg == 0 && lane == 0) {
            tc_fence_after_sync();
#pragma unroll
            for (int ks = 0; ks < kHD / 16; ++ks)
                umma_f16(tmem_acc, umma_desc(tile_u32 + 256u * ks), umma_desc(whi_u32 + 256u * ks), kIdesc, ks > 0);
#pragma unroll
            for (int ks = 0; ks < kHD / 16; ++ks)
                umma_f16(tmem_acc + kHD, umma_desc(tile_u32 + 256u * ks), umma_desc(wlo_u32 + 256u * ks), kIdesc, ks > 0);
            umma_commit(bar);
        }
        __syncwarp();
        const bool ok = mbar_wait_bounded(bar, it & 1);
        if (!bar_and(3 + grp, kGroupWarps * 32, ok)) {      // same verdict for the whole group
            if (wg == 0 && lane == 0) atomicExch(&g_t5w_status, kStatusWaitTimeout);
            break;
        }
        tc_fence_after_sync();
        // ---- quantise the warp's 16 rows, one 16-column strip at a time; codes go to the warp's scratch ----
        const float rvA = S.rinv[warp][r][0], rvB = S.rinv[warp][r + 8][0];
        float csqA = 0.f, csqB = 0.f;       // V: running sum of squared levels of this lane's columns
#pragma unroll 2
        for (int np = 0; np < 8; ++np) {
            float hi8[8], lo8[8];
            tmem_ld_16x16(tmem_rows + 16u * np, hi8);
            tmem_ld_16x16(tmem_rows + kHD + 16u * np, lo8);
            tmem_ld_wait();
            // this lane: rows r / r+8, column pairs (16np + 2j) and (16np + 8 + 2j)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                float ac[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) ac[e] = fmaf(lo8[4 * half + e], 1.0f / kLoScale, hi8[4 * half + e]);
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
        uint8_t* const dst0 = out_base + b0 * o_sb + (int64_t)(t0 + s0) * o_st;
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
                const uint32_t word = w_squeeze4(lo, bw) | w_squeeze4(hi, bw) << (4 * bw);
                const int nb = bw == 3 ? 3 : (n * bw + 7) >> 3;
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    if (c < nb) o[c] = (uint8_t)(word >> (8 * c));
            }
        }
        __syncwarp();
        // ---- rows out ----
        if (flat) {
            w_flat_store(dst0, stg, n_valid * rb, lane);
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
        __syncwarp();       // the warp's rows are reloaded next
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");     // the last prefetch (past the end: zero fill) lands before the CTA leaves
}

__global__ void __launch_bounds__(kWarps * 32, 1) encode_t5w_kernel(const EncParams P) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    WSmem& S = *reinterpret_cast<WSmem*>(smem_raw);
    const int h = blockIdx.y, tid = threadIdx.x;
    const bool is_v = blockIdx.z != 0 || (P.flags & BGTQ_ENC_SKIP_K);
    // whole launch, before barriers or tensor memory exist
    if (P.pos_dev && !enc_range_ok(P, *P.pos_dev, P.n_tok)) return;
    if (tid == 0) {
        mbar_init(&S.mma_bar[0], 1);
        mbar_init(&S.mma_bar[1], 1);
        mbar_fence_init();
    }
    if (tid < 32) tmem_alloc(&S.tmem_base, kTmemCols);
    w_setup(S, P, P.desc[h], is_v, h);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");          // W operand: generic stores -> tensor-core reads
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (is_v) w_role<true>(S, P, h, blockIdx.x, gridDim.x);
    else w_role<false>(S, P, h, blockIdx.x, gridDim.x);
    tc_fence_before_sync();
    __syncthreads();
    if (tid < 32) tmem_dealloc(S.tmem_base, kTmemCols);
}

}  // namespace

// The launcher checks: every input row 16-byte aligned and n_tok >= 16 (as for the warp-MMA bulk path).
int launch_encode_t5w(const EncParams& P, cudaStream_t stream) {
    const int64_t n_rows = (int64_t)P.n_batch * P.n_tok;
    if (n_rows > (1LL << 30)) return BGTQ_E_TOOBIG;
    const bool do_k = !(P.flags & BGTQ_ENC_SKIP_K), do_v = !(P.flags & BGTQ_ENC_SKIP_V);
    if (!do_k && !do_v) return BGTQ_OK;
    const int n_tiles = (int)((n_rows + kTileRows - 1) / kTileRows);
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int roles = (do_k && do_v) ? 2 : 1;
    int per = sms / (P.n_kv * roles);           // one CTA per SM, one wave
    if (per < 1) per = 1;
    const int useful = (n_tiles + 1) / 2;       // a CTA works on two tiles at a time
    const int grid_x = per < useful ? per : useful;
    const int smem = (int)sizeof(WSmem);
    // the attribute is per device: set it on every launch (cheap, and legal under stream capture)
    if (cudaFuncSetAttribute(encode_t5w_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
        cudaGetLastError();
        return BGTQ_E_LAUNCH;
    }
    encode_t5w_kernel<<<dim3(grid_x, P.n_kv, roles), kWarps * 32, smem, stream>>>(P);
    return cudaGetLastError() == cudaSuccess ? BGTQ_OK : BGTQ_E_LAUNCH;
}

int encode_t5w_max_row_bytes() { return kMaxRowBytes & ~3; }

}  // namespace bgtq

extern "C" __attribute__((visibility("default"))) int bgtq_encode_tcgen05_status(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, bgtq::g_t5w_status, sizeof(v)) != cudaSuccess) {
        cudaGetLastError();
        return BGTQ_E_LAUNCH;
    }
    return v;
}
