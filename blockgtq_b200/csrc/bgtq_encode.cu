// Prefill / append encoder (kernel a): rotate, quantise against the per-position
// codebooks, bit-pack and write K and V rows straight into their cache slots.
//
// Arithmetic follows the reference encoders step by step
// (blockgtq/quantizer.py:800-850 for K, :560-590 for V): group norms
// sqrt(sum x^2 + 1e-30), x / norm (skipped below 1e-10 / 1e-8), fp32 rotation,
// (y - off) * inv clamped to [0,255] and truncated, 256-bin code LUT for K;
// boundary count for V with the norm divided by the norm of the chosen levels.
// The packed bytes then follow quantizer.py:861-990 (LSB-first streams for
// 1-4 bits, raw bytes for 5-8).
//
// One CTA = kRows rows of one KV head, 128 threads = one per packed position.
// The rotation is a register-blocked fp32 product: a thread owns one output
// position for kRows rows and only walks the input positions of its own
// width group (the K rotation is block diagonal); V's rotation is dense.
#include "bgtq_common.cuh"
#include "bgtq_encode_params.cuh"

namespace bgtq {
namespace {

constexpr int kRows = 8;

__device__ __forceinline__ uint32_t pack_byte(const uint8_t* codes, int n, int bw, int t) {
    return enc_pack_byte(codes, n, bw, t);
}

// Copy one 128x128 fp32 rotation into shared memory with every load independent (the matrix is
// usually cold in L2 after a decode step streamed the cache, so latency, not bandwidth, matters).
__device__ __forceinline__ void stage_rotation(float* dst, const float* src, int tid) {
    const float4* s4 = reinterpret_cast<const float4*>(src);
    float4* d4 = reinterpret_cast<float4*>(dst);
    float4 buf[8];
#pragma unroll
    for (int base = 0; base < kHD * kHD / 4; base += 8 * 128) {
#pragma unroll
        for (int i = 0; i < 8; ++i) buf[i] = __ldg(s4 + base + i * 128 + tid);
#pragma unroll
        for (int i = 0; i < 8; ++i) d4[base + i * 128 + tid] = buf[i];
    }
}

__global__ void __launch_bounds__(128) encode_kernel(const EncParams P) {
    extern __shared__ __align__(16) float wsm[];            // staged rotation, [input position][output position]
    __shared__ __align__(16) float xs[kHD][kRows];          // [packed position][row]
    __shared__ float gn[BGTQ_MAX_SEGMENTS][kRows];
    __shared__ float gc[BGTQ_MAX_SEGMENTS][kRows];
    __shared__ float red[4][kRows];
    __shared__ float rawn[kRows];
    __shared__ uint8_t codes[kRows][kHD];

    const int p = threadIdx.x;
    const int h = blockIdx.y;
    const bool is_v = blockIdx.z == 1;
    const int t0 = P.pos_dev ? *P.pos_dev : P.t0;   // first destination token slot
    if (P.pos_dev && !enc_range_ok(P, t0, P.n_tok)) return;
    if (is_v ? (P.flags & BGTQ_ENC_SKIP_V) : (P.flags & BGTQ_ENC_SKIP_K)) return;
    const BgtqHeadDesc& d = P.desc[h];
    const int64_t n_rows = (int64_t)P.n_batch * P.n_tok;
    const int64_t row0 = (int64_t)blockIdx.x * kRows;

    int rb[kRows], rs[kRows];
    bool rok[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        const int64_t n = row0 + r;
        rok[r] = n < n_rows;
        rb[r] = rok[r] ? (int)(n / P.n_tok) : 0;
        rs[r] = rok[r] ? (int)(n % P.n_tok) : 0;
    }

    stage_rotation(wsm, (is_v ? P.rot_v : P.rot_k) + (size_t)h * kHD * kHD, p);
    if (!is_v) {
        // ------------------------------- K -------------------------------
        const int src_dim = d.head_perm[p];
        const int g = d.group_of[p];
#pragma unroll
        for (int r = 0; r < kRows; ++r)
            xs[p][r] = rok[r] ? __half2float(P.k[rb[r] * P.k_sb + h * P.k_sh + rs[r] * P.k_ss + src_dim]) : 0.f;
        __syncthreads();
        if (p < BGTQ_MAX_SEGMENTS * kRows) {
            const int r = p % kRows, s = p / kRows;
            if (s < d.n_seg) {
                float acc = 0.f;
                for (int i = d.seg_start[s]; i < d.seg_start[s] + d.seg_len[s]; ++i) acc = fmaf(xs[i][r], xs[i][r], acc);
                gn[s][r] = sqrtf(acc + 1e-30f);
            }
        }
        __syncthreads();
        float xn[kRows];
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            const float nr = gn[g][r];
            xn[r] = xs[p][r] / (nr > 1e-10f ? nr : 1.0f);
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < kRows; ++r) xs[p][r] = xn[r];
        __syncthreads();
        float y[kRows];
#pragma unroll
        for (int r = 0; r < kRows; ++r) y[r] = 0.f;
        const float* W = wsm + p;
        const int js = d.seg_start[g], je = js + d.seg_len[g];
        for (int jj = js; jj < je; ++jj) {
            const float w = W[jj * kHD];
            const float4 a = *reinterpret_cast<const float4*>(&xs[jj][0]);
            const float4 b = *reinterpret_cast<const float4*>(&xs[jj][4]);
            y[0] = fmaf(a.x, w, y[0]); y[1] = fmaf(a.y, w, y[1]); y[2] = fmaf(a.z, w, y[2]); y[3] = fmaf(a.w, w, y[3]);
            y[4] = fmaf(b.x, w, y[4]); y[5] = fmaf(b.y, w, y[5]); y[6] = fmaf(b.z, w, y[6]); y[7] = fmaf(b.w, w, y[7]);
        }
        const float off = d.lut_off[g], inv = d.lut_inv[g];
        const int lo = d.seg_lut_off[g];
        const bool mixed = P.flags & BGTQ_ENC_K_MIXED;
        float c2[kRows];
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            float u = (y[r] - off) * inv;
            u = fminf(fmaxf(u, 0.f), 255.f);
            const uint8_t c = d.code_lut[g][(int)u];
            codes[r][p] = c;
            const float cv = d.k_cents[lo + c];
            c2[r] = cv * cv;
            if (P.k_codes && rok[r])
                P.k_codes[(((size_t)rb[r] * P.n_kv + h) * P.n_tok + rs[r]) * kHD + p] = c;
        }
        __syncthreads();
        if (mixed) {   // norm correction: divide by the norm of the chosen levels per group
#pragma unroll
            for (int r = 0; r < kRows; ++r) xs[p][r] = c2[r];
            __syncthreads();
            if (p < BGTQ_MAX_SEGMENTS * kRows) {
                const int r = p % kRows, s = p / kRows;
                if (s < d.n_seg) {
                    float acc = 0.f;
                    for (int i = d.seg_start[s]; i < d.seg_start[s] + d.seg_len[s]; ++i) acc += xs[i][r];
                    gc[s][r] = fmaxf(sqrtf(acc), 1e-10f);
                }
            }
            __syncthreads();
        }
        // norms
        if (p < P.kn_count * kRows) {
            const int r = p % kRows, s = p / kRows;
            if (rok[r]) {
                float val = s < d.n_seg ? gn[s][r] : 0.f;
                if (mixed && s < d.n_seg) val = val / gc[s][r];
                const size_t o = rb[r] * P.kn_sb + h * P.kn_sh + (size_t)(t0 + rs[r]) * P.kn_st + s;
                if (P.flags & BGTQ_ENC_K_NORMS_F16) static_cast<__half*>(P.kn)[o] = __float2half_rn(val);
                else static_cast<float*>(P.kn)[o] = val;
            }
        }
        // bytes
        if (p < P.kp_row_bytes) {
            int mode = 0, s_bw = 0, s_first = 0, s_n = 0, s_t = 0;   // mode 0: zero, 1: bit stream, 2: raw, 3: nibble pair
            if (mixed) {
                const int nib = d.nopack_start / 2;
                if (p < nib) { mode = 3; s_first = 2 * p; }
                else if (p < nib + d.nopack_len) { mode = 2; s_first = d.nopack_start + (p - nib); }
            } else {
                for (int s = 0; s < d.n_seg; ++s) {
                    const int bw = d.seg_bw[s], nb = seg_storage_bytes(bw, d.seg_len[s]);
                    if (p >= d.seg_pack_off[s] && p < d.seg_pack_off[s] + nb) {
                        s_t = p - d.seg_pack_off[s];
                        if (bw >= 5) { mode = 2; s_first = d.seg_start[s] + s_t; }
                        else { mode = 1; s_bw = bw; s_first = d.seg_start[s]; s_n = d.seg_len[s]; }
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                if (!rok[r]) continue;
                uint32_t byte = 0;
                if (mode == 1) byte = pack_byte(&codes[r][s_first], s_n, s_bw, s_t);
                else if (mode == 2) byte = codes[r][s_first];
                else if (mode == 3) byte = (codes[r][s_first] & 15u) | ((codes[r][s_first + 1] & 15u) << 4);
                P.kp[rb[r] * P.kp_sb + h * P.kp_sh + (size_t)(t0 + rs[r]) * P.kp_st + p] = (uint8_t)byte;
            }
        }
    } else {
        // ------------------------------- V -------------------------------
        float x[kRows];
#pragma unroll
        for (int r = 0; r < kRows; ++r)
            x[r] = rok[r] ? __half2float(P.v[rb[r] * P.v_sb + h * P.v_sh + rs[r] * P.v_ss + p]) : 0.f;
        auto block_sum = [&](float (&val)[kRows], float* out) {
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                float s = val[r];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                if ((p & 31) == 0) red[p >> 5][r] = s;
            }
            __syncthreads();
            if (p < kRows) out[p] = red[0][p] + red[1][p] + red[2][p] + red[3][p];
            __syncthreads();
        };
        float sq[kRows];
#pragma unroll
        for (int r = 0; r < kRows; ++r) sq[r] = x[r] * x[r];
        block_sum(sq, rawn);
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            const float raw = sqrtf(rawn[r] + 1e-30f);
            xs[p][r] = x[r] / (raw > 1e-8f ? raw : 1.0f);
        }
        __syncthreads();
        float y[kRows];
#pragma unroll
        for (int r = 0; r < kRows; ++r) y[r] = 0.f;
        const float* W = wsm + p;
#pragma unroll 4
        for (int jj = 0; jj < kHD; ++jj) {
            const float w = W[jj * kHD];
            const float4 a = *reinterpret_cast<const float4*>(&xs[jj][0]);
            const float4 b = *reinterpret_cast<const float4*>(&xs[jj][4]);
            y[0] = fmaf(a.x, w, y[0]); y[1] = fmaf(a.y, w, y[1]); y[2] = fmaf(a.z, w, y[2]); y[3] = fmaf(a.w, w, y[3]);
            y[4] = fmaf(b.x, w, y[4]); y[5] = fmaf(b.y, w, y[5]); y[6] = fmaf(b.z, w, y[6]); y[7] = fmaf(b.w, w, y[7]);
        }
        const int nb = (1 << d.v_bits) - 1;
        float c2[kRows];
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            int c = 0;
            for (int i = 0; i < nb; ++i) c += y[r] > d.v_bounds[i] ? 1 : 0;
            codes[r][p] = (uint8_t)c;
            const float cv = d.v_cents[c];
            c2[r] = cv * cv;
            if (P.v_codes && rok[r])
                P.v_codes[(((size_t)rb[r] * P.n_kv + h) * P.n_tok + rs[r]) * kHD + p] = (uint8_t)c;
        }
        __shared__ float cn[kRows];
        block_sum(c2, cn);
        if (p < kRows && rok[p]) {
            const float raw = sqrtf(rawn[p] + 1e-30f);
            const float cnorm = sqrtf(cn[p] + 1e-20f);
            const float val = raw / (cnorm > 1e-10f ? cnorm : 1.0f);
            P.vn[rb[p] * P.vn_sb + h * P.vn_sh + (size_t)(t0 + rs[p]) * P.vn_st] = __float2half_rn(val);
        }
        const bool nibble = P.flags & BGTQ_ENC_V_NIBBLE;
        const int vb = nibble ? 4 : d.v_bits;
        const int n_bytes = seg_storage_bytes(vb, kHD);
        if (p < n_bytes) {
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                if (!rok[r]) continue;
                const uint32_t byte = pack_byte(&codes[r][0], kHD, vb, p);
                P.vp[rb[r] * P.vp_sb + h * P.vp_sh + (size_t)(t0 + rs[r]) * P.vp_st + p] = (uint8_t)byte;
            }
        }
    }
}


// ---------------------------------------------------------------------------
// Single-token step preparation: query rotation and K/V append in ONE launch,
// organised for latency (a decode step appends n_batch x n_kv rows only).
// One CTA of 512 threads per work item; thread (p = tid % 128, c = tid / 128)
// prefetches 32 entries of column p of the rotation before the inputs arrive and
// produces a quarter of the dot product; the four quarters are added in order.
// Work items: [0, n_rot) query rows (b, hq); then K rows (b, h); then V rows (b, h).
// With rot_group == 4 (four or a multiple of four query heads per KV head) a query item is four consecutive
// query heads of one KV head: quarter c of the CTA fetches row c, every thread applies its 32 rotation entries
// to all four rows, and quarter c adds up and stores row c.  Same sums in the same order as one row per CTA,
// a quarter of the rotation reads and of the CTAs.
// ---------------------------------------------------------------------------
struct PrepParams {
    EncParams e;            // n_tok == 1
    const __half* q;
    int64_t q_sb, q_sh;
    __half* q_rot;
    int32_t n_q, do_rot, rot_group;
    const __half* rope_cos;   // optional (n_batch, 128) fp16 tables of the step's position: q and k arrive pre-RoPE
    const __half* rope_sin;
    int64_t rope_sb;
    // three-region mode (optional): fp16 sink + recent ring per (batch, KV head); the step's token is written
    // into its ring (or sink) slot and the token that leaves the recent window is the one that gets encoded
    __half* k_buf;
    __half* v_buf;
    int64_t kb_sb, kb_sh;
    int32_t n_sink, window;
};

// Element `dim` of a row after rotary embedding in the split-half convention, with the rounding points of
// the fp16 reference expression (x * cos) + (rotate_half(x) * sin): two rounded products, one rounded sum.
__device__ __forceinline__ float rope_element(const __half* row, int dim, const __half* cs, const __half* sn) {
    const __half x = row[dim];
    if (cs == nullptr) return __half2float(x);
    const __half xr = dim < kHD / 2 ? __hneg(row[dim + kHD / 2]) : row[dim - kHD / 2];
    return __half2float(__hadd_rn(__hmul_rn(x, cs[dim]), __hmul_rn(xr, sn[dim])));
}

__global__ void __launch_bounds__(512) prep_kernel(const PrepParams P) {
    __shared__ float xs[kHD];
    __shared__ float xn[kHD];
    __shared__ float part[4][kHD];
    __shared__ float gn[BGTQ_MAX_SEGMENTS];
    __shared__ float gc[BGTQ_MAX_SEGMENTS];
    __shared__ float red[4];
    __shared__ uint8_t codes[kHD];
    const EncParams& E = P.e;
    const int tid = threadIdx.x, p = tid & 127, c = tid >> 7, warp = tid >> 5, lane = tid & 31;
    const int n_rot = P.do_rot ? E.n_batch * P.n_q / P.rot_group : 0;
    const int n_rows = E.n_batch * E.n_kv;
    int item = blockIdx.x, kind;   // 0 rotate, 1 K, 2 V
    int b, h, hq = 0;
    bool skip = false;
    if (item < n_rot) {
        const int per_b = P.n_q / P.rot_group;
        kind = 0; b = item / per_b; hq = (item % per_b) * P.rot_group; h = hq / (P.n_q / E.n_kv);
    } else {
        item -= n_rot;
        kind = 1 + item / n_rows;
        item %= n_rows;
        b = item / E.n_kv; h = item % E.n_kv;
        skip = (kind == 1 && (E.flags & BGTQ_ENC_SKIP_K)) || (kind == 2 && (E.flags & BGTQ_ENC_SKIP_V));
        if (skip && P.k_buf == nullptr) return;
    }
    const BgtqHeadDesc& d = E.desc[h];
    // rotation column p, rows 32c .. 32c+31: independent loads issued before anything else
    const float* W = (kind == 2 ? E.rot_v : E.rot_k) + (size_t)h * kHD * kHD + (size_t)(32 * c) * kHD + p;
    float w[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) w[i] = __ldg(W + (size_t)i * kHD);
    // static tables of the head, fetched before the dependency wait so their latency is off the critical path
    __shared__ __align__(16) uint8_t s_lut[BGTQ_MAX_SEGMENTS][BGTQ_N_BINS];
    __shared__ float s_cent[512];
    reinterpret_cast<uint32_t*>(&s_lut[0][0])[tid] = reinterpret_cast<const uint32_t*>(&d.code_lut[0][0])[tid];
    s_cent[tid] = d.k_cents[tid];
    __shared__ float s_vb[16], s_vc[16];
    if (tid < 16) {
        s_vb[tid] = d.v_bounds[tid];
        s_vc[tid] = d.v_cents[tid];
    }
    const int perm_p = d.head_perm[p];
    const int g_p = d.group_of[p];
    const float lut_off_p = d.lut_off[g_p], lut_inv_p = d.lut_inv[g_p];
    const int cent_off_p = d.seg_lut_off[g_p];
    grid_launch_dependents();
    grid_dependency_wait();       // inputs and the slot position come from earlier work in the stream
    int t0 = E.pos_dev ? *E.pos_dev : E.t0;
    if (P.k_buf != nullptr && kind != 0) {
        // three-region mode: the step's token enters the sink (first n_sink tokens) or its ring slot, copied by
        // the last quarter of the CTA; the token this CTA encodes below sits in another slot of the ring
        if (c == 3) {
            const int ring = P.window + 1;
            const int slot = t0 < P.n_sink ? t0 : P.n_sink + (t0 - P.n_sink) % ring;
            const __half* src = kind == 1 ? E.k + b * E.k_sb + h * E.k_sh : E.v + b * E.v_sb + h * E.v_sh;
            __half* dst = (kind == 1 ? P.k_buf : P.v_buf) + b * P.kb_sb + h * P.kb_sh + (int64_t)slot * kHD;
            dst[p] = src[p];
        }
        if (skip) return;
    }
    if (E.pos_dev && kind != 0 && P.k_buf == nullptr && !enc_range_ok(E, t0, 1)) return;
    const __half* k_src = E.k + b * E.k_sb + h * E.k_sh;
    const __half* v_src = E.v + b * E.v_sb + h * E.v_sh;
    if (P.k_buf != nullptr && kind != 0) {
        // Three-region policy with one-token blocks (blockgtq/unaccelerated.py:226-233): t0 tokens exist before
        // this step.  Of the a0 non-sink tokens, f0 = max(0, a0 - window) are packed already; the step's token
        // makes a0 + 1, and if that leaves more than `window` + 1 unpacked ones, token f0 is encoded into
        // packed row f0 from its ring slot.
        const int a0 = max(0, t0 - P.n_sink), a1 = max(0, t0 + 1 - P.n_sink);
        const int f0 = max(0, a0 - P.window), f1 = max(0, a1 - P.window);
        if (f1 <= f0) return;
        const int64_t slot = P.n_sink + f0 % (P.window + 1);
        k_src = P.k_buf + b * P.kb_sb + h * P.kb_sh + slot * kHD;
        v_src = P.v_buf + b * P.kb_sb + h * P.kb_sh + slot * kHD;
        t0 = f0;
        if (E.pos_dev && !enc_range_ok(E, t0, 1)) return;
    }

    const __half* cs = P.rope_cos ? P.rope_cos + b * P.rope_sb : nullptr;
    const __half* sn = P.rope_cos ? P.rope_sin + b * P.rope_sb : nullptr;
    if (kind == 0 && P.rot_group == 4) {
        __shared__ float xg[4][kHD];
        __shared__ float pg[4][4][kHD];
        xg[c][p] = rope_element(P.q + b * P.q_sb + (hq + c) * P.q_sh, perm_p, cs, sn);
        __syncthreads();
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            a0 = fmaf(xg[0][32 * c + i], w[i], a0);
            a1 = fmaf(xg[1][32 * c + i], w[i], a1);
            a2 = fmaf(xg[2][32 * c + i], w[i], a2);
            a3 = fmaf(xg[3][32 * c + i], w[i], a3);
        }
        pg[0][c][p] = a0; pg[1][c][p] = a1; pg[2][c][p] = a2; pg[3][c][p] = a3;
        __syncthreads();
        const float yq = (pg[c][0][p] + pg[c][1][p]) + (pg[c][2][p] + pg[c][3][p]);
        P.q_rot[((size_t)b * P.n_q + hq + c) * kHD + p] = __float2half_rn(yq);
        return;
    }
    float x = 0.f;
    int g = 0;
    if (c == 0) {
        if (kind == 0) x = rope_element(P.q + b * P.q_sb + hq * P.q_sh, perm_p, cs, sn);
        else if (kind == 1) x = rope_element(k_src, perm_p, cs, sn);
        else x = __half2float(v_src[p]);
        xs[p] = x;
        g = g_p;
    }
    __syncthreads();
    float raw_v = 0.f;
    if (kind == 1) {            // group norms: warp s reduces segment s
        if (warp < d.n_seg) {
            float acc = 0.f;
            for (int i = d.seg_start[warp] + lane; i < d.seg_start[warp] + d.seg_len[warp]; i += 32) acc = fmaf(xs[i], xs[i], acc);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (lane == 0) gn[warp] = sqrtf(acc + 1e-30f);
        }
    } else if (kind == 2) {
        if (c == 0) {
            float acc = x * x;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (lane == 0) red[warp] = acc;
        }
    }
    __syncthreads();
    if (c == 0) {
        if (kind == 0) xn[p] = x;
        else if (kind == 1) { const float nr = gn[g]; xn[p] = x / (nr > 1e-10f ? nr : 1.0f); }
        else { raw_v = sqrtf(red[0] + red[1] + red[2] + red[3] + 1e-30f); xn[p] = x / (raw_v > 1e-8f ? raw_v : 1.0f); }
    }
    __syncthreads();
    {
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) acc = fmaf(xn[32 * c + i], w[i], acc);
        part[c][p] = acc;
    }
    __syncthreads();
    if (c != 0 && kind != 2) { if (kind == 0) return; }
    const float y = (part[0][p] + part[1][p]) + (part[2][p] + part[3][p]);
    if (kind == 0) {
        if (c == 0) P.q_rot[((size_t)b * P.n_q + hq) * kHD + p] = __float2half_rn(y);
        return;
    }
    if (kind == 1) {
        const bool mixed = E.flags & BGTQ_ENC_K_MIXED;
        float c2 = 0.f;
        if (c == 0) {
            float u = (y - lut_off_p) * lut_inv_p;
            u = fminf(fmaxf(u, 0.f), 255.f);
            const uint8_t cd = s_lut[g][(int)u];
            codes[p] = cd;
            const float cv = s_cent[cent_off_p + cd];
            c2 = cv * cv;
            if (E.k_codes) E.k_codes[((size_t)b * E.n_kv + h) * kHD + p] = cd;
            xs[p] = c2;
        }
        __syncthreads();
        if (mixed && warp < d.n_seg) {
            float acc = 0.f;
            for (int i = d.seg_start[warp] + lane; i < d.seg_start[warp] + d.seg_len[warp]; i += 32) acc += xs[i];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (lane == 0) gc[warp] = fmaxf(sqrtf(acc), 1e-10f);
        }
        __syncthreads();
        if (c != 0) return;
        if (p < E.kn_count) {
            float val = p < d.n_seg ? gn[p] : 0.f;
            if (mixed && p < d.n_seg) val = val / gc[p];
            const size_t o = b * E.kn_sb + h * E.kn_sh + (size_t)t0 * E.kn_st + p;
            if (E.flags & BGTQ_ENC_K_NORMS_F16) static_cast<__half*>(E.kn)[o] = __float2half_rn(val);
            else static_cast<float*>(E.kn)[o] = val;
        }
        if (p < E.kp_row_bytes) {
            uint32_t byte = 0;
            if (mixed) {
                const int nib = d.nopack_start / 2;
                if (p < nib) byte = (codes[2 * p] & 15u) | ((codes[2 * p + 1] & 15u) << 4);
                else if (p < nib + d.nopack_len) byte = codes[d.nopack_start + (p - nib)];
            } else {
                for (int s = 0; s < d.n_seg; ++s) {
                    const int bw = d.seg_bw[s], nb = seg_storage_bytes(bw, d.seg_len[s]);
                    if (p >= d.seg_pack_off[s] && p < d.seg_pack_off[s] + nb) {
                        const int st = p - d.seg_pack_off[s];
                        byte = bw >= 5 ? codes[d.seg_start[s] + st] : pack_byte(&codes[d.seg_start[s]], d.seg_len[s], bw, st);
                    }
                }
            }
            E.kp[b * E.kp_sb + h * E.kp_sh + (size_t)t0 * E.kp_st + p] = (uint8_t)byte;
        }
        return;
    }
    // ---- V ----
    float c2 = 0.f;
    if (c == 0) {
        const int nb = (1 << d.v_bits) - 1;
        int cd = 0;
        for (int i = 0; i < nb; ++i) cd += y > s_vb[i] ? 1 : 0;
        codes[p] = (uint8_t)cd;
        const float cv = s_vc[cd];
        c2 = cv * cv;
        if (E.v_codes) E.v_codes[((size_t)b * E.n_kv + h) * kHD + p] = (uint8_t)cd;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) c2 += __shfl_xor_sync(0xffffffffu, c2, o);
        if (lane == 0) gn[warp] = c2;
    }
    __syncthreads();
    if (c != 0) return;
    if (p == 0) {
        const float cnorm = sqrtf(gn[0] + gn[1] + gn[2] + gn[3] + 1e-20f);
        E.vn[b * E.vn_sb + h * E.vn_sh + (size_t)t0 * E.vn_st] = __float2half_rn(raw_v / (cnorm > 1e-10f ? cnorm : 1.0f));
    }
    const int vb = (E.flags & BGTQ_ENC_V_NIBBLE) ? 4 : d.v_bits;
    if (p < seg_storage_bytes(vb, kHD))
        E.vp[b * E.vp_sb + h * E.vp_sh + (size_t)t0 * E.vp_st + p] = (uint8_t)pack_byte(&codes[0], kHD, vb, p);
}

}  // namespace
}  // namespace bgtq

using namespace bgtq;

extern "C" __attribute__((visibility("default"))) int bgtq_encode(const BgtqHeadDesc* desc, const float* rot_k, const float* rot_v, const void* k,
                           int64_t k_sb, int64_t k_sh, int64_t k_ss, const void* v, int64_t v_sb, int64_t v_sh,
                           int64_t v_ss, int32_t n_batch, int32_t n_kv, int32_t n_tok, int32_t t0, uint8_t* k_packed,
                           int64_t kp_sb, int64_t kp_sh, int64_t kp_st, int32_t kp_row_bytes, void* k_norms,
                           int64_t kn_sb, int64_t kn_sh, int64_t kn_st, int32_t kn_count, uint8_t* v_packed,
                           int64_t vp_sb, int64_t vp_sh, int64_t vp_st, void* v_norms, int64_t vn_sb, int64_t vn_sh,
                           int64_t vn_st, uint8_t* k_codes, uint8_t* v_codes, int32_t flags, const int32_t* pos_dev,
                           int32_t t_capacity, int32_t* status, void* stream) {
    const bool do_k = !(flags & BGTQ_ENC_SKIP_K), do_v = !(flags & BGTQ_ENC_SKIP_V);
    if (!desc || n_batch < 1 || n_kv < 1 || n_tok < 0 || t0 < 0 || t_capacity < 0) return BGTQ_E_BADARG;
    if (!pos_dev && t_capacity > 0 && (int64_t)t0 + n_tok > t_capacity) return BGTQ_E_BADARG;
    if (do_k && (!rot_k || !k || !k_packed || !k_norms)) return BGTQ_E_BADARG;
    if (do_v && (!rot_v || !v || !v_packed || !v_norms)) return BGTQ_E_BADARG;
    if (do_k && (kp_row_bytes < 1 || kp_row_bytes > kHD || kn_count < 1 || kn_count > BGTQ_MAX_SEGMENTS))
        return BGTQ_E_BADARG;
    if (n_tok == 0 || (!do_k && !do_v)) return BGTQ_OK;
    EncParams P;
    P.desc = desc; P.rot_k = rot_k; P.rot_v = rot_v;
    P.k = static_cast<const __half*>(k); P.v = static_cast<const __half*>(v);
    P.k_sb = k_sb; P.k_sh = k_sh; P.k_ss = k_ss; P.v_sb = v_sb; P.v_sh = v_sh; P.v_ss = v_ss;
    P.n_batch = n_batch; P.n_kv = n_kv; P.n_tok = n_tok; P.t0 = t0; P.pos_dev = pos_dev;
    P.kp = k_packed; P.kp_sb = kp_sb; P.kp_sh = kp_sh; P.kp_st = kp_st; P.kp_row_bytes = kp_row_bytes;
    P.kn = k_norms; P.kn_sb = kn_sb; P.kn_sh = kn_sh; P.kn_st = kn_st; P.kn_count = kn_count;
    P.vp = v_packed; P.vp_sb = vp_sb; P.vp_sh = vp_sh; P.vp_st = vp_st;
    P.vn = static_cast<__half*>(v_norms); P.vn_sb = vn_sb; P.vn_sh = vn_sh; P.vn_st = vn_st;
    P.k_codes = k_codes; P.v_codes = v_codes; P.flags = flags; P.capacity = t_capacity; P.status = status;
    const int64_t n_rows = (int64_t)n_batch * n_tok;
    {   // bulk row counts go to the tensor-core kernel when every input row is 16-byte aligned
        auto al16 = [](const void* ptr, int64_t a, int64_t b2, int64_t c) {
            return ptr == nullptr || (((reinterpret_cast<uintptr_t>(ptr) & 15u) == 0) && a % 8 == 0 && b2 % 8 == 0 && c % 8 == 0);
        };
        if (n_rows >= 64 && n_tok >= 16 && kn_count <= BGTQ_MAX_SEGMENTS && !(flags & BGTQ_ENC_FORCE_SIMT) && al16(do_k ? k : nullptr, k_sb, k_sh, k_ss) &&
            al16(do_v ? v : nullptr, v_sb, v_sh, v_ss)) {
            if (!(flags & BGTQ_ENC_NO_TCGEN05) && n_rows >= 128 && (!do_k || kp_row_bytes <= encode_t5w_max_row_bytes()))
                return launch_encode_t5w(P, static_cast<cudaStream_t>(stream));
            return launch_encode_tc(P, static_cast<cudaStream_t>(stream));
        }
    }
    const int64_t gx = (n_rows + kRows - 1) / kRows;
    if (gx > 0x7fffffffLL || n_kv > 65535) return BGTQ_E_TOOBIG;
    dim3 grid((unsigned)gx, n_kv, 2);
    constexpr int kWsmBytes = kHD * kHD * (int)sizeof(float);
    // the attribute is per device: set it on every launch (cheap, and legal under stream capture)
    if (cudaFuncSetAttribute(encode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kWsmBytes) != cudaSuccess) {
        cudaGetLastError();
        return BGTQ_E_LAUNCH;
    }
    encode_kernel<<<grid, 128, kWsmBytes, static_cast<cudaStream_t>(stream)>>>(P);
    return cudaGetLastError() == cudaSuccess ? BGTQ_OK : BGTQ_E_LAUNCH;
}

static int step_prepare_impl(
    const BgtqHeadDesc* desc, const float* rot_k, const float* rot_v, const void* q, int64_t q_sb, int64_t q_sh,
    void* q_rot, int32_t n_q, const void* k, int64_t k_sb, int64_t k_sh, const void* v, int64_t v_sb, int64_t v_sh,
    int32_t n_batch, int32_t n_kv, int32_t t0, uint8_t* k_packed, int64_t kp_sb, int64_t kp_sh, int64_t kp_st,
    int32_t kp_row_bytes, void* k_norms, int64_t kn_sb, int64_t kn_sh, int64_t kn_st, int32_t kn_count,
    uint8_t* v_packed, int64_t vp_sb, int64_t vp_sh, int64_t vp_st, void* v_norms, int64_t vn_sb, int64_t vn_sh,
    int64_t vn_st, int32_t flags, const int32_t* pos_dev, int32_t t_capacity, int32_t* status, void* stream,
    const void* rope_cos, const void* rope_sin, int64_t rope_sb, void* k_buf = nullptr, void* v_buf = nullptr, int64_t kb_sb = 0, int64_t kb_sh = 0,
    int32_t n_sink = 0, int32_t window = 0) {
    if (!desc || !rot_k || !rot_v || !k || !v || !k_packed || !k_norms || !v_packed || !v_norms) return BGTQ_E_BADARG;
    if (n_batch < 1 || n_kv < 1 || t0 < 0 || kp_row_bytes < 1 || kp_row_bytes > kHD || kn_count < 1 ||
        kn_count > BGTQ_MAX_SEGMENTS || t_capacity < 0)
        return BGTQ_E_BADARG;
    if (!pos_dev && !k_buf && t_capacity > 0 && t0 >= t_capacity) return BGTQ_E_BADARG;
    const bool do_rot = q != nullptr && q_rot != nullptr;
    if (do_rot && (n_q < n_kv || n_q % n_kv)) return BGTQ_E_BADARG;
    PrepParams P;
    EncParams& E = P.e;
    E.desc = desc; E.rot_k = rot_k; E.rot_v = rot_v;
    E.k = static_cast<const __half*>(k); E.v = static_cast<const __half*>(v);
    E.k_sb = k_sb; E.k_sh = k_sh; E.k_ss = 0; E.v_sb = v_sb; E.v_sh = v_sh; E.v_ss = 0;
    E.n_batch = n_batch; E.n_kv = n_kv; E.n_tok = 1; E.t0 = t0; E.pos_dev = pos_dev;
    E.kp = k_packed; E.kp_sb = kp_sb; E.kp_sh = kp_sh; E.kp_st = kp_st; E.kp_row_bytes = kp_row_bytes;
    E.kn = k_norms; E.kn_sb = kn_sb; E.kn_sh = kn_sh; E.kn_st = kn_st; E.kn_count = kn_count;
    E.vp = v_packed; E.vp_sb = vp_sb; E.vp_sh = vp_sh; E.vp_st = vp_st;
    E.vn = static_cast<__half*>(v_norms); E.vn_sb = vn_sb; E.vn_sh = vn_sh; E.vn_st = vn_st;
    E.k_codes = nullptr; E.v_codes = nullptr; E.flags = flags; E.capacity = t_capacity; E.status = status;
    P.q = static_cast<const __half*>(q); P.q_sb = q_sb; P.q_sh = q_sh; P.q_rot = static_cast<__half*>(q_rot);
    P.n_q = n_q; P.do_rot = do_rot ? 1 : 0;
    P.rot_group = do_rot && (n_q / n_kv) % 4 == 0 ? 4 : 1;
    P.rope_cos = static_cast<const __half*>(rope_cos); P.rope_sin = static_cast<const __half*>(rope_sin);
    P.rope_sb = rope_sb;
    P.k_buf = static_cast<__half*>(k_buf); P.v_buf = static_cast<__half*>(v_buf);
    P.kb_sb = kb_sb; P.kb_sh = kb_sh; P.n_sink = n_sink; P.window = window;
    const int64_t items = (int64_t)(do_rot ? n_batch * n_q / P.rot_group : 0) + 2LL * n_batch * n_kv;
    if (items > 0x7fffffffLL) return BGTQ_E_TOOBIG;
    return launch_kernel(prep_kernel, dim3((unsigned)items), dim3(512), 0, static_cast<cudaStream_t>(stream),
                         (flags & BGTQ_ENC_PROGRAMMATIC) != 0, P) == cudaSuccess ? BGTQ_OK : BGTQ_E_LAUNCH;
}

extern "C" __attribute__((visibility("default"))) int bgtq_step_prepare(
    const BgtqHeadDesc* desc, const float* rot_k, const float* rot_v, const void* q, int64_t q_sb, int64_t q_sh,
    void* q_rot, int32_t n_q, const void* k, int64_t k_sb, int64_t k_sh, const void* v, int64_t v_sb, int64_t v_sh,
    int32_t n_batch, int32_t n_kv, int32_t t0, uint8_t* k_packed, int64_t kp_sb, int64_t kp_sh, int64_t kp_st,
    int32_t kp_row_bytes, void* k_norms, int64_t kn_sb, int64_t kn_sh, int64_t kn_st, int32_t kn_count,
    uint8_t* v_packed, int64_t vp_sb, int64_t vp_sh, int64_t vp_st, void* v_norms, int64_t vn_sb, int64_t vn_sh,
    int64_t vn_st, int32_t flags, const int32_t* pos_dev, int32_t t_capacity, int32_t* status, void* stream) {
    return step_prepare_impl(desc, rot_k, rot_v, q, q_sb, q_sh, q_rot, n_q, k, k_sb, k_sh, v, v_sb, v_sh, n_batch, n_kv, t0, k_packed,
                             kp_sb, kp_sh, kp_st, kp_row_bytes, k_norms, kn_sb, kn_sh, kn_st, kn_count, v_packed, vp_sb, vp_sh,
                             vp_st, v_norms, vn_sb, vn_sh, vn_st, flags, pos_dev, t_capacity, status, stream, nullptr, nullptr, 0);
}

extern "C" __attribute__((visibility("default"))) int bgtq_step_prepare_rope(
    const BgtqHeadDesc* desc, const float* rot_k, const float* rot_v, const void* q, int64_t q_sb, int64_t q_sh,
    void* q_rot, int32_t n_q, const void* k, int64_t k_sb, int64_t k_sh, const void* v, int64_t v_sb, int64_t v_sh,
    int32_t n_batch, int32_t n_kv, int32_t t0, uint8_t* k_packed, int64_t kp_sb, int64_t kp_sh, int64_t kp_st,
    int32_t kp_row_bytes, void* k_norms, int64_t kn_sb, int64_t kn_sh, int64_t kn_st, int32_t kn_count,
    uint8_t* v_packed, int64_t vp_sb, int64_t vp_sh, int64_t vp_st, void* v_norms, int64_t vn_sb, int64_t vn_sh,
    int64_t vn_st, int32_t flags, const int32_t* pos_dev, int32_t t_capacity, int32_t* status, const void* rope_cos,
    const void* rope_sin, int64_t rope_sb, void* stream) {
    if (!rope_cos || !rope_sin) return BGTQ_E_BADARG;
    return step_prepare_impl(desc, rot_k, rot_v, q, q_sb, q_sh, q_rot, n_q, k, k_sb, k_sh, v, v_sb, v_sh, n_batch, n_kv, t0, k_packed,
                             kp_sb, kp_sh, kp_st, kp_row_bytes, k_norms, kn_sb, kn_sh, kn_st, kn_count, v_packed, vp_sb, vp_sh,
                             vp_st, v_norms, vn_sb, vn_sh, vn_st, flags, pos_dev, t_capacity, status, stream, rope_cos, rope_sin, rope_sb);
}

extern "C" __attribute__((visibility("default"))) int bgtq_step_prepare_ring(
    const BgtqHeadDesc* desc, const float* rot_k, const float* rot_v, const void* q, int64_t q_sb, int64_t q_sh,
    void* q_rot, int32_t n_q, const void* k, int64_t k_sb, int64_t k_sh, const void* v, int64_t v_sb, int64_t v_sh,
    int32_t n_batch, int32_t n_kv, int32_t t0, uint8_t* k_packed, int64_t kp_sb, int64_t kp_sh, int64_t kp_st,
    int32_t kp_row_bytes, void* k_norms, int64_t kn_sb, int64_t kn_sh, int64_t kn_st, int32_t kn_count,
    uint8_t* v_packed, int64_t vp_sb, int64_t vp_sh, int64_t vp_st, void* v_norms, int64_t vn_sb, int64_t vn_sh,
    int64_t vn_st, int32_t flags, const int32_t* pos_dev, int32_t t_capacity, int32_t* status, void* k_buf, void* v_buf,
    int64_t kb_sb, int64_t kb_sh, int32_t n_sink,
    int32_t window, void* stream) {
    if (!k_buf || !v_buf || n_sink < 0 || window < 1) return BGTQ_E_BADARG;
    return step_prepare_impl(desc, rot_k, rot_v, q, q_sb, q_sh, q_rot, n_q, k, k_sb, k_sh, v, v_sb, v_sh, n_batch, n_kv, t0, k_packed,
                             kp_sb, kp_sh, kp_st, kp_row_bytes, k_norms, kn_sb, kn_sh, kn_st, kn_count, v_packed, vp_sb, vp_sh,
                             vp_st, v_norms, vn_sb, vn_sh, vn_st, flags, pos_dev, t_capacity, status, stream, nullptr, nullptr, 0, k_buf, v_buf, kb_sb, kb_sh,
                             n_sink, window);
}
