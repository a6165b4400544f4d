// Bulk (prefill) encoder on tensor cores.
//
// Same arithmetic contract as encode_kernel (bgtq_encode.cu) but organised for throughput:
//   * persistent CTAs: one CTA owns (KV head, K or V) and loops over 64-row tiles, so the 128x128
//     rotation is staged in shared memory once;
//   * the rotation y = x_unit . W runs as fp16 m16n8k16 MMAs with fp32 accumulation.  The inputs are
//     fp16 already, so x is exact; W (fp32) is split while staging into hi = fp16(W) and
//     lo = fp16((W - hi) * 2^10), two MMAs per tile, y = acc_hi + acc_lo * 2^-10 (about 22 bits of W,
//     the same order as fp32 summation noise).  Dividing by the group norm happens after the product;
//     norm groups coincide with the diagonal blocks of the K rotation, so this equals normalising first;
//   * K rows are gathered into packed-position order when the tile is loaded, which keeps the K
//     rotation block diagonal: k-tiles outside the blocks of a 16-column output strip are skipped;
//   * the epilogue bins / counts boundaries straight from the accumulators, writes codes to a shared
//     tile, then packs bytes and stores rows.
#include "bgtq_common.cuh"
#include "bgtq_encode_params.cuh"

namespace bgtq {
namespace {

constexpr int kTileRows = 64;
constexpr int kWarps = 4;
constexpr int kLd = 136;                 // halfs per shared row (128 + 8 pad): conflict-free ldmatrix
constexpr float kLoScale = 1024.0f;

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

struct TcSmem {
    __half w_hi[kHD * kLd];              // [output position n][input position k]
    __half w_lo[kHD * kLd];
    __half x[kTileRows * kLd];           // [row][packed input position]
    uint8_t codes[kTileRows][kHD];
    float gn[kTileRows][BGTQ_MAX_SEGMENTS];   // group norms (V: [.][0] raw norm)
    float gc[kTileRows][BGTQ_MAX_SEGMENTS];   // sum of squared chosen levels per group (V: [.][0])
    uint8_t code_lut[BGTQ_MAX_SEGMENTS][BGTQ_N_BINS];
    uint8_t kt_lo[8], kt_hi[8];          // k-tile range per 16-column strip
    uint8_t inv_perm[kHD];
    uint8_t grp[kHD];
    float loff[BGTQ_MAX_SEGMENTS], linv[BGTQ_MAX_SEGMENTS];
    float vbounds[16], vcents[16];
};

__global__ void __launch_bounds__(kWarps * 32, 2) encode_tc_kernel(const EncParams P) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    TcSmem& S = *reinterpret_cast<TcSmem*>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.y;
    const bool is_v = blockIdx.z == 1;
    if (is_v ? (P.flags & BGTQ_ENC_SKIP_V) : (P.flags & BGTQ_ENC_SKIP_K)) return;
    const BgtqHeadDesc& d = P.desc[h];
    const int64_t n_rows = (int64_t)P.n_batch * P.n_tok;
    const int n_tiles = (int)((n_rows + kTileRows - 1) / kTileRows);
    const int t0 = P.pos_dev ? *P.pos_dev : P.t0;

    // ---- stage the rotation once: Wt[n][k] = W[k][n], split into hi / scaled lo ----
    {
        const float* W = (is_v ? P.rot_v : P.rot_k) + (size_t)h * kHD * kHD;
        for (int i = tid; i < kHD * kHD; i += kWarps * 32) {
            const int k = i >> 7, n = i & 127;          // coalesced over n
            const float w = __ldg(W + i);
            const __half hi = __float2half_rn(w);
            S.w_hi[n * kLd + k] = hi;
            S.w_lo[n * kLd + k] = __float2half_rn((w - __half2float(hi)) * kLoScale);
        }
        for (int i = tid; i < BGTQ_MAX_SEGMENTS * BGTQ_N_BINS; i += kWarps * 32)
            S.code_lut[i >> 8][i & 255] = d.code_lut[i >> 8][i & 255];
        if (tid < kHD) {
            S.inv_perm[d.head_perm[tid]] = (uint8_t)tid;
            S.grp[tid] = d.group_of[tid];
        }
        if (tid < BGTQ_MAX_SEGMENTS) {
            S.loff[tid] = d.lut_off[tid];
            S.linv[tid] = d.lut_inv[tid];
        }
        if (tid < 16) {
            S.vbounds[tid] = d.v_bounds[tid];
            S.vcents[tid] = d.v_cents[tid];
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
    }
    __syncthreads();

    const int r = lane >> 2, j = lane & 3;
    const uint32_t x_base = smem_u32(S.x), whi_base = smem_u32(S.w_hi), wlo_base = smem_u32(S.w_lo);
    const int n_seg = is_v ? 1 : d.n_seg;
    const bool mixed = !is_v && (P.flags & BGTQ_ENC_K_MIXED);
    const int v_nb = (1 << d.v_bits) - 1;

    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int64_t row0 = (int64_t)tile * kTileRows;
        // ---- load 64 rows (K: gathered into packed order) ----
        for (int i = tid; i < kTileRows * 16; i += kWarps * 32) {
            const int row = i >> 4, c8 = (i & 15) * 8;
            const int64_t n = row0 + row;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (n < n_rows) {
                const int b = (int)(n / P.n_tok), s = (int)(n % P.n_tok);
                const __half* src = is_v ? P.v + b * P.v_sb + h * P.v_sh + s * P.v_ss : P.k + b * P.k_sb + h * P.k_sh + s * P.k_ss;
                v = *reinterpret_cast<const uint4*>(src + c8);
            }
            if (is_v) {
                *reinterpret_cast<uint4*>(&S.x[row * kLd + c8]) = v;
            } else {
                const __half* e = reinterpret_cast<const __half*>(&v);
#pragma unroll
                for (int q = 0; q < 8; ++q) S.x[row * kLd + S.inv_perm[c8 + q]] = e[q];
            }
        }
        __syncthreads();
        // ---- group norms: lane (row = lane & 15, parity) walks its warp's 16 rows ----
        {
            const int row = warp * 16 + (lane & 15), par = lane >> 4;
            for (int s = 0; s < n_seg; ++s) {
                const int st = is_v ? 0 : d.seg_start[s], en = is_v ? kHD : st + d.seg_len[s];
                float acc = 0.f;
                for (int p = st + par; p < en; p += 2) {
                    const float xv = __half2float(S.x[row * kLd + p]);
                    acc = fmaf(xv, xv, acc);
                }
                acc += __shfl_xor_sync(0xffffffffu, acc, 16);
                if (par == 0) {
                    S.gn[row][s] = sqrtf(acc + 1e-30f);
                    S.gc[row][s] = 0.f;
                }
            }
        }
        __syncwarp();
        // ---- rotation + quantisation, one 16-column strip at a time ----
        const int rowA = warp * 16 + r, rowB = rowA + 8;
        float csqA = 0.f, csqB = 0.f;       // V: running sum of squared levels of this lane's columns
        for (int np = 0; np < 8; ++np) {
            float hi0[4] = {0, 0, 0, 0}, hi1[4] = {0, 0, 0, 0}, lo0[4] = {0, 0, 0, 0}, lo1[4] = {0, 0, 0, 0};
            const int k0 = S.kt_lo[np], k1 = S.kt_hi[np];
            for (int kt = k0; kt < k1; ++kt) {
                uint32_t a[4], bh[4], bl[4];
                ldmatrix_x4(a, x_base + 2u * ((warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kLd + kt * 16 + (lane >> 4) * 8));
                const uint32_t boff = 2u * ((np * 16 + (lane & 7) + (lane >> 4) * 8) * kLd + kt * 16 + ((lane >> 3) & 1) * 8);
                ldmatrix_x4(bh, whi_base + boff);
                ldmatrix_x4(bl, wlo_base + boff);
                const uint32_t bh0[2] = {bh[0], bh[1]}, bh1[2] = {bh[2], bh[3]};
                const uint32_t bl0[2] = {bl[0], bl[1]}, bl1[2] = {bl[2], bl[3]};
                mma_16816(hi0, a, bh0);
                mma_16816(hi1, a, bh1);
                mma_16816(lo0, a, bl0);
                mma_16816(lo1, a, bl1);
            }
            // this lane: rows rowA / rowB, columns c, c+1 (strip half 0) and c+8, c+9 (half 1)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const float* ah = half ? hi1 : hi0;
                const float* al = half ? lo1 : lo0;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int col = np * 16 + half * 8 + 2 * j + (e & 1);
                    const int row = (e & 2) ? rowB : rowA;
                    const float acc = ah[e] + al[e] * (1.0f / kLoScale);
                    uint8_t code;
                    float cv = 0.f;
                    (void)cv;
                    if (!is_v) {
                        const int g = S.grp[col];
                        const float nr = S.gn[row][g];
                        const float y = acc / (nr > 1e-10f ? nr : 1.0f);
                        float u = (y - S.loff[g]) * S.linv[g];
                        u = fminf(fmaxf(u, 0.f), 255.f);
                        code = S.code_lut[g][(int)u];
                    } else {
                        const float nr = S.gn[row][0];
                        const float y = acc / (nr > 1e-8f ? nr : 1.0f);
                        int c = 0;
                        for (int i = 0; i < v_nb; ++i) c += y > S.vbounds[i] ? 1 : 0;
                        code = (uint8_t)c;
                        cv = S.vcents[c];
                        if (e & 2) csqB = fmaf(cv, cv, csqB); else csqA = fmaf(cv, cv, csqA);
                    }
                    S.codes[row][col] = code;
                }
            }
        }
        if (is_v) {    // squared level norms: add the four lanes of a quad
            csqA += __shfl_xor_sync(0xffffffffu, csqA, 1);
            csqA += __shfl_xor_sync(0xffffffffu, csqA, 2);
            csqB += __shfl_xor_sync(0xffffffffu, csqB, 1);
            csqB += __shfl_xor_sync(0xffffffffu, csqB, 2);
            if (j == 0) {
                S.gc[rowA][0] = csqA;
                S.gc[rowB][0] = csqB;
            }
        }
        __syncwarp();
        // ---- outputs of this warp's 16 rows ----
        for (int rr = 0; rr < 16; ++rr) {
            const int row = warp * 16 + rr;
            const int64_t n = row0 + row;
            if (n >= n_rows) break;
            const int b = (int)(n / P.n_tok), s = (int)(n % P.n_tok);
            const size_t slot = (size_t)(t0 + s);
            if (!is_v) {
                if (lane < P.kn_count) {
                    float val = lane < d.n_seg ? S.gn[row][lane] : 0.f;
                    if (mixed && lane < d.n_seg) {   // norm correction: divide by the norm of the chosen levels
                        float csq = 0.f;
                        for (int p = d.seg_start[lane]; p < d.seg_start[lane] + d.seg_len[lane]; ++p) {
                            const float c1 = d.k_cents[d.seg_lut_off[lane] + S.codes[row][p]];
                            csq += c1 * c1;
                        }
                        val = val / fmaxf(sqrtf(csq), 1e-10f);
                    }
                    const size_t o = b * P.kn_sb + h * P.kn_sh + slot * P.kn_st + lane;
                    if (P.flags & BGTQ_ENC_K_NORMS_F16) static_cast<__half*>(P.kn)[o] = __float2half_rn(val);
                    else static_cast<float*>(P.kn)[o] = val;
                }
                uint8_t* dst = P.kp + b * P.kp_sb + h * P.kp_sh + slot * P.kp_st;
                for (int p = lane; p < P.kp_row_bytes; p += 32) {
                    uint32_t byte = 0;
                    if (mixed) {
                        const int nib = d.nopack_start / 2;
                        if (p < nib) byte = (S.codes[row][2 * p] & 15u) | ((S.codes[row][2 * p + 1] & 15u) << 4);
                        else if (p < nib + d.nopack_len) byte = S.codes[row][d.nopack_start + (p - nib)];
                    } else {
                        for (int sg = 0; sg < d.n_seg; ++sg) {
                            const int bw = d.seg_bw[sg], nb = seg_storage_bytes(bw, d.seg_len[sg]);
                            if (p >= d.seg_pack_off[sg] && p < d.seg_pack_off[sg] + nb) {
                                const int st = p - d.seg_pack_off[sg];
                                byte = bw >= 5 ? S.codes[row][d.seg_start[sg] + st]
                                               : enc_pack_byte(&S.codes[row][d.seg_start[sg]], d.seg_len[sg], bw, st);
                            }
                        }
                    }
                    dst[p] = (uint8_t)byte;
                }
                if (P.k_codes) {
                    uint8_t* cd = P.k_codes + (((size_t)b * P.n_kv + h) * P.n_tok + s) * kHD;
                    for (int p = lane; p < kHD; p += 32) cd[p] = S.codes[row][p];
                }
            } else {
                if (lane == 0) {
                    const float cnorm = sqrtf(S.gc[row][0] + 1e-20f);
                    P.vn[b * P.vn_sb + h * P.vn_sh + slot * P.vn_st] =
                        __float2half_rn(S.gn[row][0] / (cnorm > 1e-10f ? cnorm : 1.0f));
                }
                const int vb = (P.flags & BGTQ_ENC_V_NIBBLE) ? 4 : d.v_bits;
                uint8_t* dst = P.vp + b * P.vp_sb + h * P.vp_sh + slot * P.vp_st;
                for (int p = lane; p < seg_storage_bytes(vb, kHD); p += 32)
                    dst[p] = (uint8_t)enc_pack_byte(&S.codes[row][0], kHD, vb, p);
                if (P.v_codes) {
                    uint8_t* cd = P.v_codes + (((size_t)b * P.n_kv + h) * P.n_tok + s) * kHD;
                    for (int p = lane; p < kHD; p += 32) cd[p] = S.codes[row][p];
                }
            }
        }
        __syncthreads();    // tile buffers are reused
    }
}

}  // namespace

int launch_encode_tc(const EncParams& P, cudaStream_t stream) {
    const int64_t n_rows = (int64_t)P.n_batch * P.n_tok;
    const int n_tiles = (int)((n_rows + kTileRows - 1) / kTileRows);
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int per = (2 * sms + 2 * P.n_kv - 1) / (2 * P.n_kv);        // CTAs per (head, side): fill two per SM
    if (per > n_tiles) per = n_tiles;
    if (per < 1) per = 1;
    const int smem = (int)sizeof(TcSmem);
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(encode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
            cudaGetLastError();
            return BGTQ_E_LAUNCH;
        }
        attr_set = true;
    }
    encode_tc_kernel<<<dim3(per, P.n_kv, 2), kWarps * 32, smem, stream>>>(P);
    return cudaGetLastError() == cudaSuccess ? BGTQ_OK : BGTQ_E_LAUNCH;
}

}  // namespace bgtq
