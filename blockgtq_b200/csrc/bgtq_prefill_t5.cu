// Packed-cache prefill attention on the fifth-generation tensor cores (tcgen05) with accumulators in tensor
// memory.  Same contract and arithmetic as prefill_kernel in bgtq_prefill.cu; this is the form for sm_100a.
//
// One CTA owns 256 query rows of one (batch, KV head) (row = position * gqa + head of the group), as two blocks
// of 128 = the M of every product; both blocks multiply the same dequantised tile.  Cache tokens are walked in
// tiles of 64:
//   1. the tile's packed rows (fetched with cp.async while the previous tile was multiplied) are
//      dequantised ONCE into shared memory, directly in the tensor cores' operand layout: khat = fp16 centroid
//      * fp16 norm held exactly as a high and a low fp16 tile [token][dim], vhat = fp16(centroid * norm)
//      transposed [dim][token];
//   2. one thread issues S = Q . Khat_hi^T + Q . Khat_lo^T per block: 16 tcgen05.mma (M 128, N 64, K 16), fp32
//      accumulator in 64 tensor-memory columns;
//   3. 256 threads, one per query row, read their row of S with tcgen05.ld, apply the causal limit, keep the
//      running maximum and denominator, and write P (fp16) to shared memory as the next product's A operand.
//      The accumulator O is only rescaled when a row's maximum grew by more than 2^8 since the value the row
//      scales by was set (the final division undoes either scale): tcgen05.ld / st of the row;
//   4. the same thread issues O += P . Vhat per block: 4 tcgen05.mma (M 128, N 128, K 16) into 128 more columns.
// Dequantisation is table driven: per segment a table of fp16x2 centroid pairs indexed by two codes at once,
// hi = centroid * norm and lo = fma(centroid, norm, -hi) as packed fp16 operations (the same two numbers the
// fp32 product splits into), packed rows read as aligned words.
// The phases of a CTA run one after the other (one CTA of 16 warps per SM: all of them dequantise, eight own the
// rows); what the tensor cores buy is that the products no longer pass operands through the register file.
// Every wait is bounded: a wait that gives up is recorded in a sticky status word, the CTA leaves its loop
// together, releases its tensor memory and returns.
#include "bgtq_prefill_common.cuh"
#include "bgtq_tcgen05.cuh"

namespace bgtq {

__device__ int g_pf5_status = 0;

namespace {

constexpr int kT5Rows = 128;            // M of every product
constexpr int kT5Blocks = 2;            // 128-row blocks per CTA: both read the same dequantised tile
constexpr int kT5Tok = 128;             // cache tokens per tile = N of the S product, K of the O product
constexpr int kT5Threads = 512;
constexpr uint32_t kT5TmemCols = 512;   // S of block m: columns [128 m, 128 m + 128); O of block m: [256 + 128 m, 384 + 128 m)
constexpr uint32_t kColS = 0, kColO = 256;
// instruction descriptors: D fp32, A and B fp16, both K-major, M = 128, N = 64 / 128
constexpr uint32_t kIdescS = (1u << 4) | ((uint32_t)(kT5Tok >> 3) << 17) | ((uint32_t)(kT5Rows >> 4) << 24);
constexpr uint32_t kIdescO = (1u << 4) | ((uint32_t)(kHD >> 3) << 17) | ((uint32_t)(kT5Rows >> 4) << 24);
constexpr float kLazyLog2 = 8.0f;       // a row rescales O only when its maximum grew by more than 2^8
constexpr int kPtWords = BGTQ_MAX_SEGMENTS * 256 + 256;
static_assert(kT5Rows * kT5Tok * 2 <= kT5Tok * kHD * 2, "P fits the K tile it replaces");

// Operand layout (no swizzle, K-major): 8 x 8 core matrices of 128 B (8 rows of 16 B); along K they follow each
// other 128 B apart, 8-row groups are `sbo` apart: element (row, k) at
//     (row / 8) * sbo + (k / 8) * 128 + (row % 8) * 16 + (k % 8) * 2.
// All four operands are 128 deep (dims for Q and Khat, tokens for P and Vhat^T): sbo = 2048.
struct T5Smem {
    __align__(128) uint8_t q[kT5Blocks][kT5Rows * kHD * 2];
    __align__(128) uint8_t kh[kT5Tok * kHD * 2];
    __align__(128) uint8_t kl[kT5Tok * kHD * 2];
    __align__(128) uint8_t vt[kHD * kT5Tok * 2];
    // (P, 128 rows x 128 tokens per block, is written over the K tiles once the S products have completed:
    // block 0 over `kl`, block 1 over `kh`)
    __align__(16) uint32_t pt[kPtWords];            // pair tables: (code, code) -> fp16x2, per K segment of <= 4 stored bits, then V
    uint16_t seg_pt[BGTQ_MAX_SEGMENTS + 1];         // first word of each segment's pair table; last entry: V's
    uint16_t cb[528];                               // 512 K entries + 16 V entries (fp16 bits)
    uint2 ktask[kPfMaxTasks];
    uint2 vtask[16];
    int32_t n_ktask, n_vtask;
    __align__(8) uint64_t bar_s, bar_o;
    uint32_t tmem_base;
};

struct T5Raw {      // byte offsets of the tile's packed rows behind T5Smem (each region 16-byte aligned, + 4 bytes of phase)
    uint32_t k, kn, v, vn, total;
};

__device__ __forceinline__ void t5_stage(uint8_t* dst, const uint8_t* src, int n_bytes, int tid) {
    // dst[(src & 3) + i] = src[i]: whole 32-bit words asynchronously, the ragged tail byte by byte
    const uint32_t ph = (uint32_t)(reinterpret_cast<uintptr_t>(src) & 3u);
    const uint8_t* s4 = src - ph;
    const uint32_t d4 = smem_u32(dst);
    const int n_words = (int)((ph + n_bytes) >> 2);
    for (int i = tid; i < n_words; i += kT5Threads)
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d4 + 4u * i), "l"(s4 + 4 * i) : "memory");
    const int tail = (int)((ph + n_bytes) & 3u);
    if (tid < tail) dst[4 * n_words + tid] = __ldg(s4 + 4 * n_words + tid);
}

// The 32 (or, for raw-byte codes, 64) bits that start at byte p, from aligned 32-bit loads.  Reads up to 11
// bytes past p + 4: inside the staging buffer (its regions carry that much slack or are followed by another).
__device__ __forceinline__ void t5_words(const uint8_t* p, bool two, uint32_t& w0, uint32_t& w1) {
    const uint32_t a = smem_u32(p), al = a & ~3u, sh = (a & 3u) * 8u;
    const uint32_t x0 = lds32(al), x1 = lds32(al + 4u);
    w0 = __funnelshift_r(x0, x1, sh);
    w1 = 0u;
    if (two) w1 = __funnelshift_r(x1, lds32(al + 8u), sh);
}
__device__ __forceinline__ float t5_exp2(float x) {      // hardware 2^x; ex2(-inf) = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// One K task of TWO tokens (lane and lane + 32 of the tile: two independent chains per lane): up to 8 codes of SB
// stored bits at src[e] -> khat = centroid * norm as a high and a low fp16 tile.  hi = fp16(centroid * norm);
// lo = fp16(centroid * norm - hi) with one rounding (fused), i.e. the two fp16 numbers the exact fp32 product
// splits into.  A token past the tile's end stores zeros.
// FAST: a full task (8 codes) of two live tokens whose low part is kept: no per-pair checks.
template <int SB, bool FAST>
__device__ __forceinline__ void t5_k_task(uint8_t* kh, uint8_t* kl, const uint8_t* const (&src)[2], const uint32_t* pt,
                                          const uint16_t* cb, const __half2 (&n2)[2], bool round16, int first, int n,
                                          const uint32_t (&trow)[2], uint32_t rot, const bool (&live)[2]) {
    uint32_t w0[2] = {0u, 0u}, w1[2] = {0u, 0u};
#pragma unroll
    for (int e = 0; e < 2; ++e)
        if (FAST || live[e]) t5_words(src[e], SB == 8, w0[e], w1[e]);
#pragma unroll
    for (int pi0 = 0; pi0 < 4; ++pi0) {
        const uint32_t c = 2u * ((pi0 + rot) & 3u);
        if (FAST || (int)c < n) {
            const int dd = first + (int)c;
            const uint32_t doff = (uint32_t)((dd >> 3) * 128 + (dd & 7) * 2);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                uint32_t cc;       // the two centroids as fp16x2
                if constexpr (SB == 8) {
                    const uint32_t two = (c < 4u ? w0[e] : w1[e]) >> ((c & 2u) * 8u);
                    cc = (uint32_t)cb[two & 0xFFu] | (uint32_t)cb[(two >> 8) & 0xFFu] << 16;
                } else {
                    cc = pt[(w0[e] >> (c * SB)) & ((1u << (2 * SB)) - 1u)];
                }
                const __half2 c2 = *reinterpret_cast<const __half2*>(&cc);
                const __half2 h2 = __hmul2(c2, n2[e]);
                const __half2 l2 = __hfma2(c2, n2[e], __hneg2(h2));
                uint32_t hi = *reinterpret_cast<const uint32_t*>(&h2), lo = *reinterpret_cast<const uint32_t*>(&l2);
                if (!FAST) {
                    if (round16) lo = 0u;
                    if (!live[e]) hi = lo = 0u;
                }
                *reinterpret_cast<uint32_t*>(kh + trow[e] + doff) = hi;
                *reinterpret_cast<uint32_t*>(kl + trow[e] + doff) = lo;
            }
        }
    }
}
// One V task of two tokens: 8 codes each -> vhat = fp16(centroid * norm), stored down each token's column of the
// transposed tile (`col` = the task's first dim, token `lane`; token lane + 32 sits 4 k-chunks = 512 B further).
template <int SB, bool FAST>
__device__ __forceinline__ void t5_v_task(uint8_t* col, const uint8_t* const (&src)[2], const uint32_t* vpt, const __half2 (&n2)[2],
                                          uint32_t rot, const bool (&live)[2]) {
    uint32_t w0[2] = {0u, 0u}, w1 = 0u;
#pragma unroll
    for (int e = 0; e < 2; ++e)
        if (FAST || live[e]) t5_words(src[e], false, w0[e], w1);
#pragma unroll
    for (int pi0 = 0; pi0 < 4; ++pi0) {
        const uint32_t c = 2u * ((pi0 + rot) & 3u);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const uint32_t cc = vpt[(w0[e] >> (c * SB)) & ((1u << (2 * SB)) - 1u)];
            const __half2 v2 = __hmul2(*reinterpret_cast<const __half2*>(&cc), n2[e]);
            uint32_t v = *reinterpret_cast<const uint32_t*>(&v2);
            if (!FAST && !live[e]) v = 0u;
            *reinterpret_cast<uint16_t*>(col + e * 512 + c * 16u) = (uint16_t)v;
            *reinterpret_cast<uint16_t*>(col + e * 512 + (c + 1u) * 16u) = (uint16_t)(v >> 16);
        }
    }
}

__global__ void __launch_bounds__(kT5Threads, 1) prefill_t5_kernel(const PfParams P, const T5Raw R) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    T5Smem& S = *reinterpret_cast<T5Smem*>(smem_raw);
    uint8_t* const raw0 = smem_raw + sizeof(T5Smem);      // two staging buffers of R.total bytes
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.y, b = blockIdx.z;
    const int bq = kT5Rows * kT5Blocks / P.gqa;      // query positions per CTA
    const int q0 = (int)(gridDim.x - 1 - blockIdx.x) * bq;      // latest positions (most tiles under the causal mask) first
    const BgtqHeadDesc& d = P.desc[h];

    for (int i = tid; i < 528; i += kT5Threads) S.cb[i] = i < 512 ? d.codebook[i] : d.v_lut[i - 512];
    if (tid == 0) {
        pf_build_tasks(P, d, S.ktask, S.vtask, &S.n_ktask, &S.n_vtask);
        mbar_init(&S.bar_s, 1);
        mbar_init(&S.bar_o, 1);
        mbar_fence_init();
    }
    // pair tables: entry i of a table for `sb` stored bits = (centroid[i & m], centroid[(i >> sb) & m])
    {
        const bool mixed = P.flags & BGTQ_DEC_K_MIXED;
        int base = 0;
        for (int sg = 0; sg <= d.n_seg; ++sg) {
            const bool is_v = sg == d.n_seg;
            const int bw = is_v ? d.v_bits : d.seg_bw[sg];
            const int sb = is_v ? ((P.flags & BGTQ_DEC_V_NIBBLE) ? 4 : d.v_bits) : (mixed ? (bw <= 4 ? 4 : 8) : (bw <= 4 ? bw : 8));
            if (tid == 0) S.seg_pt[is_v ? BGTQ_MAX_SEGMENTS : sg] = (uint16_t)base;
            if (sb <= 4) {
                const uint32_t m = (1u << sb) - 1u;
                const uint16_t* src = is_v ? d.v_lut : d.codebook + d.seg_lut_off[sg];
                for (int i = tid; i < (1 << (2 * sb)); i += kT5Threads)
                    S.pt[base + i] = (uint32_t)src[i & m] | (uint32_t)src[(i >> sb) & m] << 16;
                base += 1 << (2 * sb);
            }
        }
    }
    if (warp == 0) tmem_alloc(&S.tmem_base, kT5TmemCols);
    // the CTA's query rows -> the A operand (16-byte chunks of 8 dims); rows past the end are zero
    for (int i = tid; i < kT5Rows * kT5Blocks * 16; i += kT5Threads) {
        const int row = i >> 4, kc = i & 15;
        const int qi_ = row / P.gqa, hq_ = h * P.gqa + row % P.gqa;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (q0 + qi_ < P.s_q) {
            const __half* src = P.q + b * P.q_sb + hq_ * P.q_sh + (int64_t)(q0 + qi_) * P.q_ss + kc * 8;
            if ((reinterpret_cast<uintptr_t>(src) & 15u) == 0) v = __ldg(reinterpret_cast<const uint4*>(src));
            else {
                const uint32_t* s32 = reinterpret_cast<const uint32_t*>(src);
                v = make_uint4(__ldg(s32), __ldg(s32 + 1), __ldg(s32 + 2), __ldg(s32 + 3));
            }
        }
        *reinterpret_cast<uint4*>(S.q[row >> 7] + ((row & 127) >> 3) * 2048 + kc * 128 + (row & 7) * 16) = v;
    }
    // this thread's query row (threads 0..255: warps 0-3 own block 0, warps 4-7 block 1)
    const int row = tid & (kT5Rows * kT5Blocks - 1), mb = row >> 7, r128 = row & 127;
    const int qi = row / P.gqa, hq = h * P.gqa + row % P.gqa;
    const bool rok = q0 + qi < P.s_q;
    const int lim = !rok ? 0 : (P.causal ? min(P.n_tok, P.q_pos_offset + q0 + qi + 1) : P.n_tok);
    const int last_q = min(q0 + bq, P.s_q) - 1;
    const int t_max = P.causal ? min(P.n_tok, P.q_pos_offset + last_q + 1) : P.n_tok;

    const size_t bh_kp = (size_t)b * P.kp_sb + (size_t)h * P.kp_sh, bh_kn = (size_t)b * P.kn_sb + (size_t)h * P.kn_sh;
    const size_t bh_vp = (size_t)b * P.vp_sb + (size_t)h * P.vp_sh, bh_vn = (size_t)b * P.vn_sb + (size_t)h * P.vn_sh;
    const uint32_t q_u32 = smem_u32(S.q[0]), kh_u32 = smem_u32(S.kh), kl_u32 = smem_u32(S.kl), vt_u32 = smem_u32(S.vt),
                   p_u32 = smem_u32(S.kl), p1_u32 = smem_u32(S.kh);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // Q: generic-proxy stores -> tensor-core reads
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = S.tmem_base;
    const uint32_t tlane = tmem + ((uint32_t)((warp & 3) * 32) << 16);   // this warp's quarter of the lanes
    const uint32_t colS = kColS + 128u * mb, colO = kColO + 128u * mb;      // this row's block
    const int n_ktask = S.n_ktask, n_vtask = S.n_vtask;

    auto stage_tile = [&](int t0, int buf) {
        uint8_t* const raw = raw0 + (size_t)buf * R.total;
        const int nt = min(kT5Tok, t_max - t0);
        t5_stage(raw + R.k, P.kp + bh_kp + (size_t)t0 * P.kp_st, nt * P.kp_st, tid);
        t5_stage(raw + R.kn, P.kn + bh_kn + (size_t)t0 * P.kn_st, nt * P.kn_st, tid);
        t5_stage(raw + R.v, P.vp + bh_vp + (size_t)t0 * P.vp_st, nt * P.vp_st, tid);
        t5_stage(raw + R.vn, P.vn + bh_vn + (size_t)t0 * P.vn_st, nt * P.vn_st, tid);
    };
    if (t_max > 0) stage_tile(0, 0);

    float m_used = -INFINITY, lsum = 0.f;    // the maximum this row scales by (log2 domain), its denominator
    bool ok = true;
    int it = 0;
    for (int t0 = 0; t0 < t_max; t0 += kT5Tok, ++it) {
        const int nt = min(kT5Tok, t_max - t0);
        // ---- 1. the tile's packed rows have landed; dequantise them into the operand tiles ----
        asm volatile("cp.async.wait_all;" ::: "memory");
        __syncthreads();
        if (t0 + kT5Tok < t_max) stage_tile(t0 + kT5Tok, (it + 1) & 1);     // the next tile's rows, a whole tile ahead
        const uint8_t* const raw = raw0 + (size_t)(it & 1) * R.total;
        const uint8_t* rk = raw + R.k + (reinterpret_cast<uintptr_t>(P.kp + bh_kp + (size_t)t0 * P.kp_st) & 3u);
        const uint8_t* rn = raw + R.kn + (reinterpret_cast<uintptr_t>(P.kn + bh_kn + (size_t)t0 * P.kn_st) & 3u);
        const uint8_t* rv = raw + R.v + (reinterpret_cast<uintptr_t>(P.vp + bh_vp + (size_t)t0 * P.vp_st) & 3u);
        const uint8_t* rw = raw + R.vn + (reinterpret_cast<uintptr_t>(P.vn + bh_vn + (size_t)t0 * P.vn_st) & 3u);
        // One warp per task: the task's fields are uniform; lane l dequantises tokens l and l + 32.  The four 8-token
        // groups of a warp walk a task's four pairs in different order, so that their stores (same banks, 2048 /
        // 128 B apart) do not collide.
        const uint32_t rot = (uint32_t)lane >> 3;
        for (int u = warp; u < 2 * n_ktask; u += kT5Threads / 32) {      // (task, 64-token half)
            const uint2 tk = S.ktask[u >> 1];
            const int tb = (u & 1) * 64 + lane;                            // this lane's tokens: tb and tb + 32
            const bool live[2] = {tb < nt, tb + 32 < nt};
            const int first = tk.x & 0xFF, n = (tk.x >> 8) & 0xF, sg = (tk.x >> 16) & 0xF;
            const uint32_t sb = (tk.x >> 12) & 0xF;
            const bool round16 = (tk.x >> 20) & 1u;
            const uint32_t trow[2] = {(uint32_t)((tb >> 3) * 2048 + (tb & 7) * 16), (uint32_t)(((tb >> 3) + 4) * 2048 + (tb & 7) * 16)};
            const uint8_t* const src[2] = {rk + tb * P.kp_st + (tk.y & 0xFFFFu), rk + (tb + 32) * P.kp_st + (tk.y & 0xFFFFu)};
            const __half2 n2[2] = {
                __half2half2(__ushort_as_half(*reinterpret_cast<const uint16_t*>(rn + tb * P.kn_st + 2 * sg))),
                __half2half2(__ushort_as_half(*reinterpret_cast<const uint16_t*>(rn + (tb + 32) * P.kn_st + 2 * sg)))};
            const uint32_t* pt = S.pt + S.seg_pt[sg];
            const uint16_t* cb = S.cb + (tk.y >> 16);
            if (nt == kT5Tok && n == 8 && !round16) {       // (uniform over the warp)
                switch (sb) {
                    case 1: t5_k_task<1, true>(S.kh, S.kl, src, pt, cb, n2, round16, first, n, trow, rot, live); break;
                    case 2: t5_k_task<2, true>(S.kh, S.kl, src, pt, cb, n2, round16, first, n, trow, rot, live); break;
                    case 3: t5_k_task<3, true>(S.kh, S.kl, src, pt, cb, n2, round16, first, n, trow, rot, live); break;
                    case 4: t5_k_task<4, true>(S.kh, S.kl, src, pt, cb, n2, round16, first, n, trow, rot, live); break;
                    default: t5_k_task<8, true>(S.kh, S.kl, src, pt, cb, n2, round16, first, n, trow, rot, live); break;
                }
            } else {
                switch (sb) {
                    case 1: t5_k_task<1, false>(S.kh, S.kl, src, pt, cb, n2, round16, first, n, trow, rot, live); break;
                    case 2: t5_k_task<2, false>(S.kh, S.kl, src, pt, cb, n2, round16, first, n, trow, rot, live); break;
                    case 3: t5_k_task<3, false>(S.kh, S.kl, src, pt, cb, n2, round16, first, n, trow, rot, live); break;
                    case 4: t5_k_task<4, false>(S.kh, S.kl, src, pt, cb, n2, round16, first, n, trow, rot, live); break;
                    default: t5_k_task<8, false>(S.kh, S.kl, src, pt, cb, n2, round16, first, n, trow, rot, live); break;
                }
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
        // ---- 2. S = Q . Khat^T ----
        if (tid == 0) {
            tc_fence_after_sync();
#pragma unroll
            for (int m = 0; m < kT5Blocks; ++m) {
                const uint32_t qa = q_u32 + (uint32_t)m * (kT5Rows * kHD * 2);
#pragma unroll
                for (int ks = 0; ks < kHD / 16; ++ks)
                    umma_f16(tmem + kColS + 128u * m, umma_desc(qa + 256u * ks), umma_desc(kl_u32 + 256u * ks), kIdescS, ks > 0);
#pragma unroll
                for (int ks = 0; ks < kHD / 16; ++ks)
                    umma_f16(tmem + kColS + 128u * m, umma_desc(qa + 256u * ks), umma_desc(kh_u32 + 256u * ks), kIdescS, 1u);
            }
            umma_commit(&S.bar_s);
        }
        // ---- 3. softmax of the tile, one thread per query row ----
        if (warp < 4 * kT5Blocks) {
            if (!mbar_wait_bounded(&S.bar_s, it & 1)) ok = false;
            tc_fence_after_sync();
            const bool masked = !__all_sync(0xffffffffu, t0 + kT5Tok <= lim);     // only tiles that reach a row's causal limit
            uint8_t* const prow = (mb ? S.kh : S.kl) + (r128 >> 3) * 2048 + (r128 & 7) * 16;
            float ps = 0.f;
#pragma unroll 1
            for (int hf = 0; hf < kT5Tok / 64; ++hf) {      // 64 columns of the row at a time
                float sv[64];
                {
                    float (&s0)[32] = *reinterpret_cast<float (*)[32]>(&sv[0]);
                    float (&s1)[32] = *reinterpret_cast<float (*)[32]>(&sv[32]);
                    tmem_ld32(tlane + colS + 64u * hf, s0);
                    tmem_ld32(tlane + colS + 64u * hf + 32u, s1);
                    tmem_ld_wait();
                }
                float mx = -INFINITY;
                if (masked) {
#pragma unroll
                    for (int c = 0; c < 64; ++c) sv[c] = t0 + 64 * hf + c < lim ? sv[c] : -INFINITY;
                }
#pragma unroll
                for (int c = 0; c < 64; ++c) mx = fmaxf(mx, sv[c]);
                const float m_new = fmaxf(m_used, mx * P.scale_log2);
                float alpha = 1.f;
                if (m_used == -INFINITY) m_used = m_new;                 // nothing accumulated for this row yet
                else if (m_new > m_used + kLazyLog2) {
                    alpha = t5_exp2(m_used - m_new);
                    m_used = m_new;
                }
                if (__any_sync(0xffffffffu, alpha != 1.f)) {             // (the previous tile's product has completed)
                    lsum *= alpha;
                    ps *= alpha;                                          // (the first half of this tile, already in P)
                    if (hf > 0) {                                         // rescale what this row put into P so far
#pragma unroll 1
                        for (int kc = 0; kc < 8 * hf; ++kc) {
                            uint4 v = *reinterpret_cast<uint4*>(prow + kc * 128);
                            const __half2 a2 = __float2half2_rn(alpha);
                            __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
                            for (int e = 0; e < 4; ++e) h[e] = __hmul2(h[e], a2);
                            *reinterpret_cast<uint4*>(prow + kc * 128) = v;
                        }
                    }
                    if (it > 0) {
#pragma unroll 1
                        for (int ch = 0; ch < kHD / 32; ++ch) {
                            float o[32];
                            tmem_ld32(tlane + colO + 32u * ch, o);
                            tmem_ld_wait();
#pragma unroll
                            for (int c = 0; c < 32; ++c) o[c] *= alpha;
                            tmem_st32(tlane + colO + 32u * ch, o);
                        }
                        tmem_st_wait();
                    }
                }
                const float z = m_used == -INFINITY ? 0.f : m_used;
#pragma unroll
                for (int kc = 0; kc < 8; ++kc) {
                    uint32_t pk[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float p0 = t5_exp2(fmaf(sv[kc * 8 + 2 * e], P.scale_log2, -z));
                        const float p1 = t5_exp2(fmaf(sv[kc * 8 + 2 * e + 1], P.scale_log2, -z));
                        ps += p0 + p1;
                        pk[e] = pack_half2(p0, p1);
                    }
                    *reinterpret_cast<uint4*>(prow + (8 * hf + kc) * 128) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                }
            }
            lsum += ps;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tc_fence_before_sync();
        }
        if (warp >= 4 * kT5Blocks) {     // ---- 3b. meanwhile the other warps dequantise V for the second product ----
            const uint32_t* vpt = S.pt + S.seg_pt[BGTQ_MAX_SEGMENTS];
            const uint32_t vsb = (S.vtask[0].x >> 12) & 0xF;
            for (int u = warp - 4 * kT5Blocks; u < 2 * n_vtask; u += kT5Threads / 32 - 4 * kT5Blocks) {      // (task, 64-token half)
                const uint2 tk = S.vtask[u >> 1];
                const int first = tk.x & 0xFF;
                const int tb = (u & 1) * 64 + lane;
                const bool live[2] = {tb < nt, tb + 32 < nt};
                uint8_t* const col = S.vt + (first >> 3) * 2048 + (tb >> 3) * 128 + (tb & 7) * 2;
                const uint8_t* const src[2] = {rv + tb * P.vp_st + (tk.y & 0xFFFFu), rv + (tb + 32) * P.vp_st + (tk.y & 0xFFFFu)};
                const __half2 n2[2] = {__half2half2(__ushort_as_half(*reinterpret_cast<const uint16_t*>(rw + tb * P.vn_st))),
                                       __half2half2(__ushort_as_half(*reinterpret_cast<const uint16_t*>(rw + (tb + 32) * P.vn_st)))};
                if (nt == kT5Tok) {
                    switch (vsb) {
                        case 1: t5_v_task<1, true>(col, src, vpt, n2, rot, live); break;
                        case 2: t5_v_task<2, true>(col, src, vpt, n2, rot, live); break;
                        case 3: t5_v_task<3, true>(col, src, vpt, n2, rot, live); break;
                        default: t5_v_task<4, true>(col, src, vpt, n2, rot, live); break;
                    }
                } else {
                    switch (vsb) {
                        case 1: t5_v_task<1, false>(col, src, vpt, n2, rot, live); break;
                        case 2: t5_v_task<2, false>(col, src, vpt, n2, rot, live); break;
                        case 3: t5_v_task<3, false>(col, src, vpt, n2, rot, live); break;
                        default: t5_v_task<4, false>(col, src, vpt, n2, rot, live); break;
                    }
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        __syncthreads();
        // ---- 4. O += P . Vhat ----
        if (tid == 0) {
            tc_fence_after_sync();
#pragma unroll
            for (int m = 0; m < kT5Blocks; ++m)
#pragma unroll
                for (int ks = 0; ks < kT5Tok / 16; ++ks)
                    umma_f16(tmem + kColO + 128u * m, umma_desc((m ? p1_u32 : p_u32) + 256u * ks), umma_desc(vt_u32 + 256u * ks), kIdescO,
                             (it > 0 || ks > 0) ? 1u : 0u);
            umma_commit(&S.bar_o);
        }
        // the product reads the tile buffers and P: everyone waits for it before the next tile overwrites them
        if (!mbar_wait_bounded(&S.bar_o, it & 1)) ok = false;
        tc_fence_after_sync();
        ok = __syncthreads_and(ok ? 1 : 0) != 0;
        if (!ok) break;
    }

    // ---- normalise and write (fp32, V's rotated basis) ----
    if (warp < 4 * kT5Blocks && ok) {
        const float inv = lsum > 0.f ? 1.0f / lsum : 0.f;
        float* dst = P.out + (((size_t)b * P.n_q + hq) * P.s_q + (q0 + qi)) * kHD;
#pragma unroll 1
        for (int ch = 0; ch < kHD / 32; ++ch) {
            float o[32];
            if (t_max > 0) {
                tmem_ld32(tlane + colO + 32u * ch, o);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int c = 0; c < 32; ++c) o[c] = 0.f;
            }
            if (rok) {
#pragma unroll
                for (int c = 0; c < 32; c += 4)
                    *reinterpret_cast<float4*>(dst + 32 * ch + c) =
                        make_float4(o[c] * inv, o[c + 1] * inv, o[c + 2] * inv, o[c + 3] * inv);
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kT5TmemCols);
    if (!ok && tid == 0) atomicExch(&g_pf5_status, kStatusWaitTimeout);
}

}  // namespace

// Launch the tcgen05 form if the shape fits it (group size divides 128; the tile's packed rows fit next to the
// operand tiles); returns false otherwise, without touching *err.
bool launch_prefill_t5(const PfParams& P, int n_batch, cudaStream_t stream, cudaError_t* err) {
    if ((kT5Rows * kT5Blocks) % P.gqa) return false;
    auto r16 = [](uint32_t x) { return (x + 15u) & ~15u; };
    T5Raw R;
    R.k = 0;
    R.kn = R.k + r16((uint32_t)kT5Tok * P.kp_st + 8u);
    R.v = R.kn + r16((uint32_t)kT5Tok * P.kn_st + 8u);
    R.vn = R.v + r16((uint32_t)kT5Tok * P.vp_st + 8u);
    R.total = R.vn + r16((uint32_t)kT5Tok * P.vn_st + 8u);
    const size_t smem = sizeof(T5Smem) + 2u * (size_t)R.total;      // two staging buffers
    if (smem > 227u * 1024u) return false;
    const int bq = kT5Rows * kT5Blocks / P.gqa;
    const int64_t q_blocks = ((int64_t)P.s_q + bq - 1) / bq;
    *err = cudaFuncSetAttribute(prefill_t5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (*err != cudaSuccess) return true;
    prefill_t5_kernel<<<dim3((unsigned)q_blocks, P.n_kv, n_batch), kT5Threads, smem, stream>>>(P, R);
    *err = cudaGetLastError();
    return true;
}

}  // namespace bgtq

extern "C" __attribute__((visibility("default"))) int bgtq_prefill_tcgen05_status(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, bgtq::g_pf5_status, sizeof(v)) != cudaSuccess) {
        cudaGetLastError();
        return BGTQ_E_LAUNCH;
    }
    return v;
}
