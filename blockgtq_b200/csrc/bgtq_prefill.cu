// Packed-cache prefill attention: many query positions per KV head against the quantised cache, causal.
//
// One CTA owns 256 query rows of one (batch, KV head): 256 / gqa consecutive positions x the gqa query
// heads of the group (row = position * gqa + head), one m16 MMA tile per warp, queries staged in shared memory.  Cache tokens are walked
// in tiles of 64: the packed rows are copied to shared memory, dequantised ONCE per tile into fp16 K and V
// tiles (the cost the decode kernel pays per 8 query rows is shared by 256 here), then
//   S = Q . Khat^T   with khat = fp16 centroid * fp16 segment norm held EXACTLY as a sum of two fp16
//                    tiles (the product has 22 significant bits), so fp32 accumulation reproduces the
//                    decode kernel's "fp32 dot product per segment times norm" without per-segment
//                    accumulators or masked k-tiles: a plain 8-k-tile MMA chain, run twice,
//   online softmax in the log2 domain (causal limit per row), P rounded to fp16,
//   O += P . Vhat    with vhat = fp16(centroid * norm)
// on mma.sync m16n8k16.  The result is written as fp32 in V's rotated basis; the caller applies V's
// rotation as one plain GEMM.
#include "bgtq_prefill_common.cuh"

namespace bgtq {
// the tcgen05 form (bgtq_prefill_t5.cu); returns false when the shape does not fit it
bool launch_prefill_t5(const PfParams& P, int n_batch, cudaStream_t stream, cudaError_t* err);
namespace {

constexpr int kPfRows = 256;      // query rows per CTA
// m16 tiles per warp: every K/V fragment loaded from shared memory feeds this many MMAs.  2 halves the
// ldmatrix traffic but needs 255 registers, i.e. 8 warps per SM: measured 17.7 ms against 14.8 ms with 1
// (16 warps) on 16384 tokens x 32 heads.
constexpr int kPfMt = 1;
constexpr int kPfWarps = kPfRows / (16 * kPfMt);
constexpr int kPfLd = 136;        // halfs per row of the dequantised tiles (conflict-free ldmatrix)

struct PfSmem {
    __half qs[kPfRows * kPfLd];                      // the CTA's query rows (packed-K basis)
    __half kh[kPfTok * kPfLd];                       // khat, high fp16 part
    __half kl[kPfTok * kPfLd];                       // khat, low fp16 part (khat = kh + kl exactly)
    __half vh[kPfTok * kPfLd];
    // packed rows of a tile, as they lie in the cache; two buffers: the next tile streams in (cp.async)
    // while the current one is dequantised and multiplied
    __align__(16) uint8_t raw_k[2][kPfTok * 160 + 16];
    __align__(16) uint8_t raw_kn[2][kPfTok * 32 + 16];
    __align__(16) uint8_t raw_v[2][kPfTok * 128 + 16];
    __align__(16) uint8_t raw_vn[2][kPfTok * 16 + 16];
    uint16_t cb[528];                               // 512 K entries + 16 V entries (fp16 bits)
    uint2 ktask[kPfMaxTasks];   // x: first code | count << 8 | stored bits << 12 | segment << 16 | fp16-round << 20
    uint2 vtask[16];            // y: byte offset | codebook offset << 16
    int32_t n_ktask, n_vtask;
};

__device__ __forceinline__ void pf_ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void pf_ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// Start copying n_bytes from src (any alignment) into dst so that dst[(src & 3) + i] = src[i]:
// whole 32-bit words asynchronously (cp.async), the ragged tail byte by byte.
__device__ __forceinline__ void pf_stage(uint8_t* dst, const uint8_t* src, int n_bytes, int tid) {
    const uint32_t ph = (uint32_t)(reinterpret_cast<uintptr_t>(src) & 3u);
    const uint8_t* s4 = src - ph;
    const uint32_t d4 = smem_u32(dst);
    const int n_words = (int)((ph + n_bytes) >> 2);
    for (int i = tid; i < n_words; i += kPfWarps * 32)
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d4 + 4u * i), "l"(s4 + 4 * i) : "memory");
    const int tail = (int)((ph + n_bytes) & 3u);
    if (tid < tail) dst[4 * n_words + tid] = __ldg(s4 + 4 * n_words + tid);
}
__device__ __forceinline__ void pf_stage_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Tables of one head: codebooks and the dequantisation tasks.
__device__ void pf_setup(PfSmem& S, const PfParams& P, const BgtqHeadDesc& d) {
    const int tid = threadIdx.x;
    for (int i = tid; i < 528; i += kPfWarps * 32) S.cb[i] = i < 512 ? d.codebook[i] : d.v_lut[i - 512];
    if (tid == 0) pf_build_tasks(P, d, S.ktask, S.vtask, &S.n_ktask, &S.n_vtask);
}

__global__ void __launch_bounds__(kPfWarps * 32, 1) prefill_kernel(const PfParams P) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    PfSmem& S = *reinterpret_cast<PfSmem*>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r = lane >> 2, j = lane & 3;
    const int h = blockIdx.y, b = blockIdx.z;
    const int bq = kPfRows / P.gqa;                  // query positions per CTA
    const int q0 = (int)(gridDim.x - 1 - blockIdx.x) * bq;      // latest positions (most tiles under the causal mask) first
    const BgtqHeadDesc& d = P.desc[h];

    pf_setup(S, P, d);

    // the CTA's query rows -> shared memory (16-byte chunks, coalesced); rows past the end are zero
    for (int i = tid; i < kPfRows * 16; i += kPfWarps * 32) {
        const int row = i >> 4, c8 = (i & 15) * 8;
        const int qi_ = row / P.gqa, hq_ = h * P.gqa + row % P.gqa;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < bq * P.gqa && q0 + qi_ < P.s_q) {
            const __half* src = P.q + b * P.q_sb + hq_ * P.q_sh + (int64_t)(q0 + qi_) * P.q_ss + c8;
            if ((reinterpret_cast<uintptr_t>(src) & 15u) == 0) v = __ldg(reinterpret_cast<const uint4*>(src));
            else {
                const uint32_t* s32 = reinterpret_cast<const uint32_t*>(src);
                v = make_uint4(__ldg(s32), __ldg(s32 + 1), __ldg(s32 + 2), __ldg(s32 + 3));
            }
        }
        *reinterpret_cast<uint4*>(&S.qs[row * kPfLd + c8]) = v;
    }
    // this thread's two query rows (accumulator rows r and r + 8 of the warp's tile)
    int qi[kPfMt][2], hq[kPfMt][2], lim[kPfMt][2];      // lim: causal limit (exclusive cache token index) per row
    bool rok[kPfMt][2];
#pragma unroll
    for (int mt = 0; mt < kPfMt; ++mt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int row = (warp * kPfMt + mt) * 16 + r + 8 * e;
            qi[mt][e] = row / P.gqa;
            hq[mt][e] = h * P.gqa + row % P.gqa;
            rok[mt][e] = row < bq * P.gqa && q0 + qi[mt][e] < P.s_q;
            lim[mt][e] = !rok[mt][e] ? 0 : (P.causal ? min(P.n_tok, P.q_pos_offset + q0 + qi[mt][e] + 1) : P.n_tok);
        }
    }
    const int last_q = min(q0 + bq, P.s_q) - 1;
    const int t_max = P.causal ? min(P.n_tok, P.q_pos_offset + last_q + 1) : P.n_tok;

    float O[kPfMt][16][4];
    float mrow[kPfMt][2], lrow[kPfMt][2];
#pragma unroll
    for (int mt = 0; mt < kPfMt; ++mt) {
#pragma unroll
        for (int i = 0; i < 16; ++i) O[mt][i][0] = O[mt][i][1] = O[mt][i][2] = O[mt][i][3] = 0.f;
        mrow[mt][0] = mrow[mt][1] = -INFINITY;
        lrow[mt][0] = lrow[mt][1] = 0.f;
    }

    const size_t bh_kp = (size_t)b * P.kp_sb + (size_t)h * P.kp_sh, bh_kn = (size_t)b * P.kn_sb + (size_t)h * P.kn_sh;
    const size_t bh_vp = (size_t)b * P.vp_sb + (size_t)h * P.vp_sh, bh_vn = (size_t)b * P.vn_sb + (size_t)h * P.vn_sh;
    const uint32_t kh_u32 = smem_u32(S.kh), kl_u32 = smem_u32(S.kl), vh_u32 = smem_u32(S.vh);
    const uint32_t qa_u32 = smem_u32(S.qs) + 2u * ((warp * kPfMt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kPfLd + (lane >> 4) * 8);
    __syncthreads();
    const int n_ktask = S.n_ktask, n_vtask = S.n_vtask;

    auto stage_tile = [&](int t0, int buf) {
        const int nt = min(kPfTok, t_max - t0);
        pf_stage(S.raw_k[buf], P.kp + bh_kp + (size_t)t0 * P.kp_st, nt * P.kp_st, tid);
        pf_stage(S.raw_kn[buf], P.kn + bh_kn + (size_t)t0 * P.kn_st, nt * P.kn_st, tid);
        pf_stage(S.raw_v[buf], P.vp + bh_vp + (size_t)t0 * P.vp_st, nt * P.vp_st, tid);
        pf_stage(S.raw_vn[buf], P.vn + bh_vn + (size_t)t0 * P.vn_st, nt * P.vn_st, tid);
    };
    if (t_max > 0) stage_tile(0, 0);
    int buf = 0;
    for (int t0 = 0; t0 < t_max; t0 += kPfTok, buf ^= 1) {
        const int nt = min(kPfTok, t_max - t0);
        // ---- 1. packed rows of this tile have been streaming in; start the next tile's ----
        pf_stage_wait();
        __syncthreads();
        if (t0 + kPfTok < t_max) stage_tile(t0 + kPfTok, buf ^ 1);
        const uint8_t* rk = S.raw_k[buf] + (reinterpret_cast<uintptr_t>(P.kp + bh_kp + (size_t)t0 * P.kp_st) & 3u);
        const uint8_t* rn = S.raw_kn[buf] + (reinterpret_cast<uintptr_t>(P.kn + bh_kn + (size_t)t0 * P.kn_st) & 3u);
        const uint8_t* rv = S.raw_v[buf] + (reinterpret_cast<uintptr_t>(P.vp + bh_vp + (size_t)t0 * P.vp_st) & 3u);
        const uint8_t* rw = S.raw_vn[buf] + (reinterpret_cast<uintptr_t>(P.vn + bh_vn + (size_t)t0 * P.vn_st) & 3u);
        // ---- 2. dequantise: task index = (task << 6) | token, so a warp works on one width at a time ----
        for (int i = tid; i < kPfTok * n_ktask; i += kPfWarps * 32) {
            const int tok = i & (kPfTok - 1);
            const uint2 tk = S.ktask[i >> 6];
            const int first = tk.x & 0xFF, n = (tk.x >> 8) & 0xF, sb = (tk.x >> 12) & 0xF, sg = (tk.x >> 16) & 0xF;
            __half* dst = S.kh + tok * kPfLd + first;
            __half* dsl = S.kl + tok * kPfLd + first;
            if (tok < nt) {
                const float nrm = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(rn + tok * P.kn_st + 2 * sg)));
                pf_dequant8_k(rk + tok * P.kp_st + (tk.y & 0xFFFFu), n, sb, S.cb + (tk.y >> 16), nrm, (tk.x >> 20) & 1u, dst, dsl);
            } else {
#pragma unroll
                for (int c = 0; c < 8; c += 2)
                    if (c < n) {
                        *reinterpret_cast<uint32_t*>(dst + c) = 0u;
                        *reinterpret_cast<uint32_t*>(dsl + c) = 0u;
                    }
            }
        }
        for (int i = tid; i < kPfTok * n_vtask; i += kPfWarps * 32) {
            const int tok = i & (kPfTok - 1);
            const uint2 tk = S.vtask[i >> 6];
            const int first = tk.x & 0xFF, sb = (tk.x >> 12) & 0xF;
            __half* dst = S.vh + tok * kPfLd + first;
            if (tok < nt) {
                const __half nrm = __ushort_as_half(*reinterpret_cast<const uint16_t*>(rw + tok * P.vn_st));
                pf_dequant8(rv + tok * P.vp_st + (tk.y & 0xFFFFu), 8, sb, S.cb + 512, true, nrm, dst);
            } else {
                *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
            }
        }
        __syncthreads();
        // ---- 3-5. per 32-token half tile: S = Q . Khat^T, online softmax in the log2 domain, O += P . Vhat ----
#pragma unroll 1
        for (int hf = 0; hf < 2; ++hf) {
            if (hf * 32 >= nt) break;
            float Sv[kPfMt][4][4];
#pragma unroll
            for (int mt = 0; mt < kPfMt; ++mt)
#pragma unroll
                for (int i = 0; i < 4; ++i) Sv[mt][i][0] = Sv[mt][i][1] = Sv[mt][i][2] = Sv[mt][i][3] = 0.f;
#pragma unroll
            for (int kt = 0; kt < 8; ++kt) {
                uint32_t a[kPfMt][4];
#pragma unroll
                for (int mt = 0; mt < kPfMt; ++mt) pf_ldmatrix_x4(a[mt], qa_u32 + 2u * (mt * 16 * kPfLd) + 32u * kt);
#pragma unroll
                for (int np = 0; np < 2; ++np) {     // two n-tiles (16 tokens) per ldmatrix.x4
                    uint32_t bm[4];
                    const int tok = hf * 32 + np * 16 + (lane & 7) + (lane >> 4) * 8;
                    const uint32_t off = 2u * (tok * kPfLd + kt * 16 + ((lane >> 3) & 1) * 8);
                    pf_ldmatrix_x4(bm, kl_u32 + off);                 // small part first
                    const uint32_t l0[2] = {bm[0], bm[1]}, l1[2] = {bm[2], bm[3]};
#pragma unroll
                    for (int mt = 0; mt < kPfMt; ++mt) {
                        mma_16816(Sv[mt][2 * np], a[mt], l0);
                        mma_16816(Sv[mt][2 * np + 1], a[mt], l1);
                    }
                    pf_ldmatrix_x4(bm, kh_u32 + off);
                    const uint32_t b0[2] = {bm[0], bm[1]}, b1[2] = {bm[2], bm[3]};
#pragma unroll
                    for (int mt = 0; mt < kPfMt; ++mt) {
                        mma_16816(Sv[mt][2 * np], a[mt], b0);
                        mma_16816(Sv[mt][2 * np + 1], a[mt], b1);
                    }
                }
            }
            // online softmax; rows r (e = 0) and r + 8 (e = 1) of each m-tile
            uint32_t pa[kPfMt][2][4];     // P as A fragments of the two 16-token k-tiles
#pragma unroll
            for (int mt = 0; mt < kPfMt; ++mt) {
                float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int e = c >> 1, tok = t0 + hf * 32 + i * 8 + 2 * j + (c & 1);
                        Sv[mt][i][c] = tok < lim[mt][e] ? Sv[mt][i][c] * P.scale_log2 : -INFINITY;
                        mx[e] = fmaxf(mx[e], Sv[mt][i][c]);
                    }
                }
                float al[2], z[2], ps[2] = {0.f, 0.f};
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 1));
                    mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 2));
                    const float nm = fmaxf(mrow[mt][e], mx[e]);
                    z[e] = nm == -INFINITY ? 0.f : nm;
                    al[e] = exp2f(mrow[mt][e] - z[e]);
                    mrow[mt][e] = nm;
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float p0 = exp2f(Sv[mt][i][0] - z[0]), p1 = exp2f(Sv[mt][i][1] - z[0]);
                    const float p2 = exp2f(Sv[mt][i][2] - z[1]), p3 = exp2f(Sv[mt][i][3] - z[1]);
                    ps[0] += p0 + p1;
                    ps[1] += p2 + p3;
                    pa[mt][i >> 1][(i & 1) * 2] = pack_half2(p0, p1);
                    pa[mt][i >> 1][(i & 1) * 2 + 1] = pack_half2(p2, p3);
                }
#pragma unroll
                for (int e = 0; e < 2; ++e) lrow[mt][e] = fmaf(lrow[mt][e], al[e], ps[e]);
                if (__any_sync(0xffffffffu, al[0] != 1.f || al[1] != 1.f)) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        O[mt][i][0] *= al[0];
                        O[mt][i][1] *= al[0];
                        O[mt][i][2] *= al[1];
                        O[mt][i][3] *= al[1];
                    }
                }
            }
#pragma unroll
            for (int kt = 0; kt < 2; ++kt) {
#pragma unroll
                for (int nd = 0; nd < 8; ++nd) {         // two n-tiles (16 dims) per ldmatrix.x4.trans
                    uint32_t bm[4];
                    const int tok = hf * 32 + kt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                    pf_ldmatrix_x4_trans(bm, vh_u32 + 2u * (tok * kPfLd + nd * 16 + (lane >> 4) * 8));
                    const uint32_t b0[2] = {bm[0], bm[1]}, b1[2] = {bm[2], bm[3]};
#pragma unroll
                    for (int mt = 0; mt < kPfMt; ++mt) {
                        mma_16816(O[mt][2 * nd], pa[mt][kt], b0);
                        mma_16816(O[mt][2 * nd + 1], pa[mt][kt], b1);
                    }
                }
            }
        }
    }

    // ---- normalise and write (fp32, V's rotated basis) ----
#pragma unroll
    for (int mt = 0; mt < kPfMt; ++mt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            float l = lrow[mt][e];
            l += __shfl_xor_sync(0xffffffffu, l, 1);
            l += __shfl_xor_sync(0xffffffffu, l, 2);
            if (!rok[mt][e]) continue;
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            float* dst = P.out + (((size_t)b * P.n_q + hq[mt][e]) * P.s_q + (q0 + qi[mt][e])) * kHD;
#pragma unroll
            for (int i = 0; i < 16; ++i)
                *reinterpret_cast<float2*>(dst + i * 8 + 2 * j) = make_float2(O[mt][i][2 * e] * inv, O[mt][i][2 * e + 1] * inv);
        }
    }
}

}  // namespace
}  // namespace bgtq

using namespace bgtq;

extern "C" __attribute__((visibility("default"))) int bgtq_prefill_attention(
    const BgtqHeadDesc* desc, const void* q_rot, int64_t q_sb, int64_t q_sh, int64_t q_ss, const uint8_t* k_packed,
    int64_t kp_sb, int64_t kp_sh, int64_t kp_st, const void* k_norms, int64_t kn_sb, int64_t kn_sh, int64_t kn_st,
    const uint8_t* v_packed, int64_t vp_sb, int64_t vp_sh, int64_t vp_st, const void* v_norms, int64_t vn_sb,
    int64_t vn_sh, int64_t vn_st, int32_t n_batch, int32_t n_q, int32_t n_kv, int32_t s_q, int32_t n_tokens,
    int32_t q_pos_offset, int32_t causal, float scale, int32_t flags, float* out_rot, void* stream) {
    if (!desc || !q_rot || !k_packed || !k_norms || !v_packed || !v_norms || !out_rot) return BGTQ_E_BADARG;
    if (n_batch < 1 || n_kv < 1 || n_q < n_kv || n_q % n_kv || s_q < 1 || n_tokens < 0 || q_pos_offset < 0)
        return BGTQ_E_BADARG;
    const int gqa = n_q / n_kv;
    if (gqa > 16) return BGTQ_E_UNSUPPORTED;
    if (kp_st < 1 || kp_st > 160 || vp_st < 1 || vp_st > 128 || kn_st < 1 || kn_st > 16 || vn_st < 1 || vn_st > 8)
        return BGTQ_E_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(q_rot) & 3u) || (q_sb & 1) || (q_sh & 1) || (q_ss & 1) ||
        (reinterpret_cast<uintptr_t>(out_rot) & 7u) || (reinterpret_cast<uintptr_t>(k_norms) & 1u) ||
        (reinterpret_cast<uintptr_t>(v_norms) & 1u))
        return BGTQ_E_ALIGN;
    const int bq = kPfRows / gqa;
    const int64_t q_blocks = ((int64_t)s_q + bq - 1) / bq;
    if (q_blocks > 0x7FFFFFFF || n_kv > 65535 || n_batch > 65535) return BGTQ_E_TOOBIG;
    PfParams P;
    P.desc = desc;
    P.q = static_cast<const __half*>(q_rot);
    P.q_sb = q_sb; P.q_sh = q_sh; P.q_ss = q_ss;
    P.kp = k_packed; P.kn = static_cast<const uint8_t*>(k_norms);
    P.vp = v_packed; P.vn = static_cast<const uint8_t*>(v_norms);
    P.kp_sb = kp_sb; P.kp_sh = kp_sh; P.kp_st = (int32_t)kp_st;
    P.kn_sb = 2 * kn_sb; P.kn_sh = 2 * kn_sh; P.kn_st = (int32_t)(2 * kn_st);
    P.vp_sb = vp_sb; P.vp_sh = vp_sh; P.vp_st = (int32_t)vp_st;
    P.vn_sb = 2 * vn_sb; P.vn_sh = 2 * vn_sh; P.vn_st = (int32_t)(2 * vn_st);
    P.n_q = n_q; P.n_kv = n_kv; P.gqa = gqa; P.s_q = s_q; P.n_tok = n_tokens;
    P.q_pos_offset = q_pos_offset; P.causal = causal ? 1 : 0; P.flags = flags;
    P.scale_log2 = scale * 1.4426950408889634f;
    P.out = out_rot;
    P.status = nullptr;
    if (!(flags & BGTQ_PF_NO_TCGEN05)) {     // the tensor-memory form, when the shape fits it
        cudaError_t e = cudaSuccess;
        if (launch_prefill_t5(P, n_batch, static_cast<cudaStream_t>(stream), &e)) {
            if (e != cudaSuccess) {
                cudaGetLastError();
                return BGTQ_E_LAUNCH;
            }
            return BGTQ_OK;
        }
    }
    const int smem = (int)sizeof(PfSmem);
    if (cudaFuncSetAttribute(prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
        cudaGetLastError();
        return BGTQ_E_LAUNCH;
    }
    prefill_kernel<<<dim3((unsigned)q_blocks, n_kv, n_batch), kPfWarps * 32, smem, static_cast<cudaStream_t>(stream)>>>(P);
    return cudaGetLastError() == cudaSuccess ? BGTQ_OK : BGTQ_E_LAUNCH;
}
