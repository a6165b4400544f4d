// Small kernels around the fused decode: query rotation, split-KV combine
// (kernel c) and attention over the fp16 sink / recent-window tokens (kernel d).
#include "bgtq_common.cuh"

namespace bgtq {
namespace {

// ---------------------------------------------------------------------------
// q_rot[p] = fp16( sum_j q[head_perm[j]] * rot_k[j][p] ), fp32 accumulate.
// The rotation is block diagonal, so only the inputs of p's own segment count.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128) rotate_q_kernel(const BgtqHeadDesc* desc, const float* rot_k,
                                                        const __half* q, int64_t q_sb, int64_t q_sh,
                                                        __half* q_rot, int n_q, int n_kv) {
    __shared__ float qs[kHD];
    const int p = threadIdx.x, hq = blockIdx.x, b = blockIdx.y;
    const int h = hq / (n_q / n_kv);
    const BgtqHeadDesc& d = desc[h];
    qs[p] = __half2float(q[b * q_sb + hq * q_sh + d.head_perm[p]]);
    __syncthreads();
    const int g = d.group_of[p];
    const int js = d.seg_start[g], je = js + d.seg_len[g];
    const float* W = rot_k + (size_t)h * kHD * kHD + p;
    float acc = 0.f;
#pragma unroll 8
    for (int j = js; j < je; ++j) acc = fmaf(qs[j], __ldg(W + (size_t)j * kHD), acc);
    q_rot[((size_t)b * n_q + hq) * kHD + p] = __float2half_rn(acc);
}

// Optional last step of the combine on a sequence-sharded cache: the row's fp32 result and LSE go straight
// into this rank's slot of EVERY rank's exchange buffer (plain peer stores over NVLink), and the last CTA of
// the grid raises this rank's flag on every rank.  Layout and protocol: see the exchange kernels below.
struct PublishArgs {
    float* const* peer_bufs;
    int32_t* const* peer_flags;
    int64_t slot_off, parity_stride, rows;
    const int32_t* seq_dev;
    int32_t* ticket;
    int32_t rank, n_ranks;
};

// ---------------------------------------------------------------------------
// combine: merge split partials (and optionally the fp16-buffer partial).
// One CTA per (query head, batch), one thread per output dim.
// kPrefetch: every thread holds its 32 rotation entries in registers and requests them before the partials
// exist, which takes their latency off a single wave of CTAs but leaves room for one CTA per SM.  With more
// rows than SMs the CTAs queue up instead, so that variant reads the entries where it uses them and fits
// three CTAs per SM, whose latency chains overlap.
// ---------------------------------------------------------------------------
template <bool kPrefetch>
__global__ void __launch_bounds__(512, kPrefetch ? 1 : 3) combine_kernel(const float* part_o, const float* part_lse, int n_splits,
                                                       const float* v_rot, const float* buf_o, const float* buf_lse,
                                                       int n_q, int n_kv, __half* out, int64_t o_sb, int64_t o_sh,
                                                       float* out_f32, float* lse_out, int64_t rank_stride,
                                                       const PublishArgs pub) {
    // rank_stride == 0: partial s of row r at part_o[(r * n_splits + s) * 128], part_lse[r * n_splits + s];
    // rank_stride  > 0: partial s is a whole (rows, 128) block + (rows) block, rank_stride floats apart
    // (the receive buffer of an all-gather of per-rank results)
    // thread (d = tid % 128, c = tid / 128): output dim d; quarter c of the splits and of the rotation rows
    __shared__ float pnum[4][kHD];
    __shared__ float pden[4];
    __shared__ float merged[kHD];
    const int tid = threadIdx.x, d = tid & 127, c = tid >> 7;
    const int hq = blockIdx.x, b = blockIdx.y;
    const size_t row = (size_t)b * n_q + hq;
    // rows 32c .. 32c+31 of column d of the head's rotation
    const float* R = v_rot ? v_rot + (size_t)(hq / (n_q / n_kv)) * kHD * kHD + (size_t)(32 * c) * kHD + d : nullptr;
    float w[kPrefetch ? 32 : 1];
    if (kPrefetch && v_rot) {   // requested before anything depends on them
#pragma unroll
        for (int i = 0; i < 32; ++i) w[i] = __ldg(R + (size_t)i * kHD);
    }
    grid_launch_dependents();
    grid_dependency_wait();       // the partials come from the preceding kernel
    const float* lse = rank_stride ? part_lse + row : part_lse + row * n_splits;
    const float* po = rank_stride ? part_o + row * kHD + d : part_o + row * n_splits * kHD + d;
    const int64_t sl = rank_stride ? rank_stride : 1, so = rank_stride ? rank_stride : kHD;
    // The slot count only sets the granularity of the decode launch's work split: most slots hold no partial
    // (LSE = -inf).  The block finds the maximum and the live slots together (each thread looks at one slot per
    // 512), keeps them in slot order, and only then walks the live ones: no thread scans the whole row alone.
    __shared__ float s_red[16];
    __shared__ int s_cnt[16];
    __shared__ int s_slot[512];
    __shared__ float s_w[512];
    const int warp = tid >> 5, lane = tid & 31;
    float mx = -INFINITY;
    for (int s = tid; s < n_splits; s += 512) mx = fmaxf(mx, lse[s * sl]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) s_red[warp] = mx;
    __syncthreads();
    mx = s_red[0];
#pragma unroll
    for (int i = 1; i < 16; ++i) mx = fmaxf(mx, s_red[i]);
    float num = 0.f, den = 0.f;
    if (mx > -INFINITY) {
        for (int base = 0; base < n_splits; base += 512) {
            const int s = base + tid;
            const float l = s < n_splits ? lse[s * sl] : -INFINITY;
            const bool live = l > -INFINITY;
            const unsigned bal = __ballot_sync(0xffffffffu, live);
            __syncthreads();                               // the previous chunk's list has been consumed
            if (lane == 0) s_cnt[warp] = __popc(bal);
            __syncthreads();
            int off = 0, total = 0;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int n = s_cnt[i];
                off += i < warp ? n : 0;
                total += n;
            }
            if (live) {
                const int pos = off + __popc(bal & ((1u << lane) - 1u));
                s_slot[pos] = s;
                s_w[pos] = expf(l - mx);
            }
            __syncthreads();
            // quarter c of the live slots, four of its partials requested before the first is used (a slot past
            // the end contributes exact zeros)
            for (int i0 = c; i0 < total; i0 += 16) {
                float a[4], x[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int i = i0 + 4 * u;
                    const bool ok = i < total;
                    a[u] = ok ? s_w[i] : 0.f;
                    x[u] = ok ? po[(int64_t)s_slot[i] * so] : 0.f;
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    den += a[u];
                    num = fmaf(a[u], x[u], num);
                }
            }
        }
    }
    pnum[c][d] = num;
    if (d == 0) pden[c] = den;
    __syncthreads();
    den = (pden[0] + pden[1]) + (pden[2] + pden[3]);
    float o = den > 0.f ? ((pnum[0][d] + pnum[1][d]) + (pnum[2][d] + pnum[3][d])) / den : 0.f;
    float tot = den > 0.f ? mx + logf(den) : -INFINITY;
    if (v_rot) {
        if (c == 0) merged[d] = o;
        __syncthreads();
        float acc = 0.f;
        if (kPrefetch) {
#pragma unroll
            for (int i = 0; i < 32; ++i) acc = fmaf(merged[32 * c + i], w[i], acc);
        } else {
#pragma unroll 8
            for (int i = 0; i < 32; ++i) acc = fmaf(merged[32 * c + i], __ldg(R + (size_t)i * kHD), acc);
        }
        __syncthreads();
        pnum[c][d] = acc;
        __syncthreads();
        o = (pnum[0][d] + pnum[1][d]) + (pnum[2][d] + pnum[3][d]);
    }
    if (c == 0) {
        if (buf_o) {
            const float lb = buf_lse[row];
            const float m2 = fmaxf(tot, lb);
            if (m2 > -INFINITY) {
                const float wp = tot == -INFINITY ? 0.f : expf(tot - m2);
                const float wb = lb == -INFINITY ? 0.f : expf(lb - m2);
                o = (wp * o + wb * buf_o[row * kHD + d]) / (wp + wb);
                tot = m2 + logf(wp + wb);
            }
        }
        if (out) out[b * o_sb + hq * o_sh + d] = __float2half_rn(o);
        if (out_f32) out_f32[row * kHD + d] = o;
        if (lse_out && d == 0) lse_out[row] = tot;
        if (pub.n_ranks > 0) {
            const int seq = *pub.seq_dev;
            for (int p = 0; p < pub.n_ranks; ++p) {
                float* dst = pub.peer_bufs[p] + (seq & 1) * pub.parity_stride + pub.slot_off;
                dst[row * kHD + d] = o;
                if (d == 0) dst[pub.rows * kHD + row] = tot;
            }
            __threadfence_system();
        }
    }
    if (pub.n_ranks == 0) return;
    __syncthreads();
    if (threadIdx.x == 0) {
        const int seq = *pub.seq_dev;
        const int t = atomicAdd(pub.ticket, 1);
        if (t == (int)(gridDim.x * gridDim.y) - 1) {    // every CTA's stores are fenced: raise the flag everywhere
            *pub.ticket = 0;
            __threadfence_system();
            for (int p = 0; p < pub.n_ranks; ++p) {
                volatile int32_t* f = pub.peer_flags[p] + pub.rank;
                *f = seq + 1;
            }
        }
    }
}

// ---------------------------------------------------------------------------
// combine for many rows: one CTA per FOUR consecutive query heads of one KV head (and batch element).  Quarter c
// of the CTA (128 threads, one per output dim) merges the live partial slots of row c; every thread then applies
// its 32 rotation entries to all four merged rows, and quarter c adds up, merges the fp16-region partial and
// stores row c.  A quarter of the CTAs and of the rotation reads of the one-row kernel, which is what bounds a
// launch of a thousand rows.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(512) combine4_kernel(const float* part_o, const float* part_lse, int n_splits,
                                                        const float* v_rot, const float* buf_o, const float* buf_lse,
                                                        int n_q, int n_kv, __half* out, int64_t o_sb, int64_t o_sh,
                                                        float* out_f32, float* lse_out, const PublishArgs pub) {
    __shared__ float merged[4][kHD];
    __shared__ float pnum[4][4][kHD];
    __shared__ float s_red[16];
    __shared__ int s_cnt[16];
    __shared__ int s_slot[4][128];
    __shared__ float s_w[4][128];
    const int tid = threadIdx.x, d = tid & 127, c = tid >> 7, warp = tid >> 5, lane = tid & 31;
    const int hq0 = blockIdx.x * 4, hq = hq0 + c, b = blockIdx.y;
    const size_t row = (size_t)b * n_q + hq;
    const float* R = v_rot + (size_t)(hq0 / (n_q / n_kv)) * kHD * kHD + (size_t)(32 * c) * kHD + d;
    float w[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) w[i] = __ldg(R + (size_t)i * kHD);
    grid_launch_dependents();
    grid_dependency_wait();       // the partials come from the preceding kernel
    const float* lse = part_lse + row * n_splits;
    const float* po = part_o + row * n_splits * kHD + d;
    float mx = -INFINITY;
    for (int s = d; s < n_splits; s += 128) mx = fmaxf(mx, lse[s]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) s_red[warp] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(s_red[4 * c], s_red[4 * c + 1]), fmaxf(s_red[4 * c + 2], s_red[4 * c + 3]));
    float num = 0.f, den = 0.f;
    for (int base = 0; base < n_splits; base += 128) {     // the same trip count in every quarter
        const int s = base + d;
        const float l = s < n_splits ? lse[s] : -INFINITY;
        const bool live = l > -INFINITY;
        const unsigned bal = __ballot_sync(0xffffffffu, live);
        __syncthreads();                                   // the previous chunk's lists have been consumed
        if (lane == 0) s_cnt[warp] = __popc(bal);
        __syncthreads();
        int off = 0, total = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int n = s_cnt[4 * c + i];
            off += 4 * c + i < warp ? n : 0;
            total += n;
        }
        if (live) {
            const int pos = off + __popc(bal & ((1u << lane) - 1u));
            s_slot[c][pos] = s;
            s_w[c][pos] = expf(l - mx);
        }
        __syncthreads();
#pragma unroll 4
        for (int i = 0; i < total; ++i) {                  // live slots of row c, in slot order
            const float a = s_w[c][i];
            den += a;
            num = fmaf(a, po[(int64_t)s_slot[c][i] * kHD], num);
        }
    }
    float o = den > 0.f ? num / den : 0.f;
    float tot = den > 0.f ? mx + logf(den) : -INFINITY;
    merged[c][d] = o;
    __syncthreads();
    {
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            a0 = fmaf(merged[0][32 * c + i], w[i], a0);
            a1 = fmaf(merged[1][32 * c + i], w[i], a1);
            a2 = fmaf(merged[2][32 * c + i], w[i], a2);
            a3 = fmaf(merged[3][32 * c + i], w[i], a3);
        }
        pnum[0][c][d] = a0; pnum[1][c][d] = a1; pnum[2][c][d] = a2; pnum[3][c][d] = a3;
    }
    __syncthreads();
    o = (pnum[c][0][d] + pnum[c][1][d]) + (pnum[c][2][d] + pnum[c][3][d]);
    if (buf_o) {
        const float lb = buf_lse[row];
        const float m2 = fmaxf(tot, lb);
        if (m2 > -INFINITY) {
            const float wp = tot == -INFINITY ? 0.f : expf(tot - m2);
            const float wb = lb == -INFINITY ? 0.f : expf(lb - m2);
            o = (wp * o + wb * buf_o[row * kHD + d]) / (wp + wb);
            tot = m2 + logf(wp + wb);
        }
    }
    if (out) out[b * o_sb + hq * o_sh + d] = __float2half_rn(o);
    if (out_f32) out_f32[row * kHD + d] = o;
    if (lse_out && d == 0) lse_out[row] = tot;
    if (pub.n_ranks == 0) return;
    {
        const int seq = *pub.seq_dev;
        for (int p = 0; p < pub.n_ranks; ++p) {
            float* dst = pub.peer_bufs[p] + (seq & 1) * pub.parity_stride + pub.slot_off;
            dst[row * kHD + d] = o;
            if (d == 0) dst[pub.rows * kHD + row] = tot;
        }
        __threadfence_system();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const int seq = *pub.seq_dev;
        const int t = atomicAdd(pub.ticket, 1);
        if (t == (int)(gridDim.x * gridDim.y) - 1) {    // every CTA's stores are fenced: raise the flag everywhere
            *pub.ticket = 0;
            __threadfence_system();
            for (int p = 0; p < pub.n_ranks; ++p) {
                volatile int32_t* f = pub.peer_flags[p] + pub.rank;
                *f = seq + 1;
            }
        }
    }
}

// ---------------------------------------------------------------------------
// fp16 buffer attention: plain softmax(q k^T) v over a few hundred tokens.
// One CTA of 256 threads per (query head, batch): one thread per token scores it, then thread (column pair,
// quarter) adds up every fourth token.  The kernel is a chain of memory latencies (a few hundred tokens per
// row): the width and the unroll depths below set how many loads of the chain are in flight at once.
// ---------------------------------------------------------------------------
constexpr int kBufThreads = 256;
__global__ void __launch_bounds__(kBufThreads) buffer_attn_kernel(const __half* q, int64_t q_sb, int64_t q_sh,
                                                           const __half* kb, const __half* vb, int64_t kb_sb,
                                                           int64_t kb_sh, int n_sink_tok, int n_ring_tok,
                                                           int sink_cap, int ring_first, int ring_size, int n_q,
                                                           int n_kv, float scale, float* buf_o, float* buf_lse,
                                                           const int32_t* pos_dev, int sc_cap) {
    // shared memory: sc_cap logits / probabilities, 16 floats of scratch, the query (128 floats), 3 x 128 partial outputs
    extern __shared__ __align__(16) float sc[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (pos_dev) {      // region sizes from the device-side token count (one-token blocks, window = ring_size - 1)
        const int avail = *pos_dev + 1;                // tokens including the one appended this step
        const int a0 = max(0, avail - 1 - sink_cap), a1 = max(0, avail - sink_cap);
        const int f0 = max(0, a0 - (ring_size - 1));
        n_sink_tok = min(avail, sink_cap);
        n_ring_tok = a1 - f0;
        ring_first = f0 % ring_size;
    }
    const int hq = blockIdx.x, b = blockIdx.y;
    const int h = hq / (n_q / n_kv);
    const size_t row = (size_t)b * n_q + hq;
    const int n_tok = n_sink_tok + n_ring_tok;
    // logical token i -> buffer slot: sink prefix, then a ring starting at ring_first
    auto slot = [&](int i) {
        if (i < n_sink_tok) return i;
        const int x = ring_first + (i - n_sink_tok);
        return sink_cap + (x >= ring_size ? x - ring_size : x);
    };
    if (n_tok <= 0) {
        if (tid < kHD) buf_o[row * kHD + tid] = 0.f;
        if (tid == 0) buf_lse[row] = -INFINITY;
        return;
    }
    float* red = sc + sc_cap;
    float* qs = red + 16;
    float* po = qs + kHD;
    if (tid < kHD) qs[tid] = __half2float(q[b * q_sb + hq * q_sh + tid]);
    __syncthreads();
    const __half* kbase = kb + b * kb_sb + h * kb_sh;
    const __half* vbase = vb + b * kb_sb + h * kb_sh;
    // logits: one thread per token walks the 256-byte key row (16-byte loads, the query is broadcast from shared memory)
    for (int i = tid; i < n_tok; i += kBufThreads) {
        const uint4* kr = reinterpret_cast<const uint4*>(kbase + (size_t)slot(i) * kHD);
        float s0 = 0.f, s1 = 0.f;
#pragma unroll 8
        for (int c = 0; c < kHD / 8; ++c) {
            const uint4 kv = __ldg(kr + c);
            const float4 qa = *reinterpret_cast<const float4*>(qs + 8 * c), qb = *reinterpret_cast<const float4*>(qs + 8 * c + 4);
            const float2 k0 = __half22float2(*reinterpret_cast<const __half2*>(&kv.x));
            const float2 k1 = __half22float2(*reinterpret_cast<const __half2*>(&kv.y));
            const float2 k2 = __half22float2(*reinterpret_cast<const __half2*>(&kv.z));
            const float2 k3 = __half22float2(*reinterpret_cast<const __half2*>(&kv.w));
            s0 = fmaf(qa.x, k0.x, s0); s1 = fmaf(qa.y, k0.y, s1);
            s0 = fmaf(qa.z, k1.x, s0); s1 = fmaf(qa.w, k1.y, s1);
            s0 = fmaf(qb.x, k2.x, s0); s1 = fmaf(qb.y, k2.y, s1);
            s0 = fmaf(qb.z, k3.x, s0); s1 = fmaf(qb.w, k3.y, s1);
        }
        sc[i] = (s0 + s1) * scale;
    }
    __syncthreads();
    float mx = -INFINITY;
    for (int i = tid; i < n_tok; i += kBufThreads) mx = fmaxf(mx, sc[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3])), fmaxf(fmaxf(red[4], red[5]), fmaxf(red[6], red[7])));
    float sum = 0.f;
    for (int i = tid; i < n_tok; i += kBufThreads) {
        const float pv = expf(sc[i] - mx);
        sc[i] = pv;
        sum += pv;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) red[8 + warp] = sum;
    __syncthreads();
    sum = ((red[8] + red[9]) + (red[10] + red[11])) + ((red[12] + red[13]) + (red[14] + red[15]));
    // output: thread -> dims (2 d2, 2 d2 + 1) of every fourth token; the quarters add up through shared memory
    // (sixteen threads per row with 16-byte loads and eight rows in flight measured slower than this)
    const int d2 = tid & 63, par = tid >> 6;
    float a0 = 0.f, a1 = 0.f;
#pragma unroll 8
    for (int i = par; i < n_tok; i += 4) {
        const float2 v = __half22float2(*reinterpret_cast<const __half2*>(vbase + (size_t)slot(i) * kHD + 2 * d2));
        const float pr = sc[i];
        a0 = fmaf(pr, v.x, a0);
        a1 = fmaf(pr, v.y, a1);
    }
    if (par) *reinterpret_cast<float2*>(po + (par - 1) * kHD + 2 * d2) = make_float2(a0, a1);
    __syncthreads();
    if (!par) {
        const float inv = 1.0f / sum;
        const float2 p1 = *reinterpret_cast<const float2*>(po + 2 * d2), p2 = *reinterpret_cast<const float2*>(po + kHD + 2 * d2),
                     p3 = *reinterpret_cast<const float2*>(po + 2 * kHD + 2 * d2);
        *reinterpret_cast<float2*>(buf_o + row * kHD + 2 * d2) =
            make_float2(((a0 + p1.x) + (p2.x + p3.x)) * inv, ((a1 + p1.y) + (p2.y + p3.y)) * inv);
    }
    if (tid == 0) buf_lse[row] = mx + logf(sum);
}

// ---------------------------------------------------------------------------
// fp16 buffer attention for grouped query heads: one CTA per (KV head, batch) serves its NREP query heads.  The
// live key and value rows are first copied into shared memory with cp.async (all of them in flight at once: the
// kernel's time is otherwise a chain of dependent memory latencies, and a row crosses L2 -> SM once instead of
// NREP times); the arithmetic then runs out of shared memory, the same sums in the same order as
// buffer_attn_kernel, head by head.  Rows are kBufRowLd bytes apart so that a warp's 16-byte reads of 32
// different rows do not collide.
// Shared memory: key rows, value rows (cap_rows x kBufRowLd bytes each, indexed by buffer slot), then
// NREP x (sc_cap logits / probabilities, 16 floats of scratch, the query, 3 x 128 partial outputs).
// ---------------------------------------------------------------------------
constexpr int kBufRowLd = 2 * kHD + 16;
template <int NREP>
__global__ void __launch_bounds__(kBufThreads) buffer_attn_group_kernel(const __half* q, int64_t q_sb, int64_t q_sh,
                                                                         const __half* kb, const __half* vb, int64_t kb_sb,
                                                                         int64_t kb_sh, int n_sink_tok, int n_ring_tok,
                                                                         int sink_cap, int ring_first, int ring_size, int n_q,
                                                                         float scale, float* buf_o, float* buf_lse,
                                                                         const int32_t* pos_dev, int sc_cap, int cap_rows) {
    extern __shared__ __align__(16) uint8_t smem_rows[];
    uint8_t* const ks = smem_rows;
    uint8_t* const vs = smem_rows + (size_t)cap_rows * kBufRowLd;
    float* const sc = reinterpret_cast<float*>(smem_rows + 2 * (size_t)cap_rows * kBufRowLd);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (pos_dev) {      // region sizes from the device-side token count (one-token blocks, window = ring_size - 1)
        const int avail = *pos_dev + 1;                // tokens including the one appended this step
        const int a0 = max(0, avail - 1 - sink_cap), a1 = max(0, avail - sink_cap);
        const int f0 = max(0, a0 - (ring_size - 1));
        n_sink_tok = min(avail, sink_cap);
        n_ring_tok = a1 - f0;
        ring_first = f0 % ring_size;
    }
    const int h = blockIdx.x, b = blockIdx.y;
    const int hq0 = h * NREP;
    const size_t row0 = (size_t)b * n_q + hq0;
    const int n_tok = n_sink_tok + n_ring_tok;
    auto slot = [&](int i) {
        if (i < n_sink_tok) return i;
        const int x = ring_first + (i - n_sink_tok);
        return sink_cap + (x >= ring_size ? x - ring_size : x);
    };
    if (n_tok <= 0) {
        for (int e = tid; e < NREP * kHD; e += kBufThreads) buf_o[row0 * kHD + e] = 0.f;
        if (tid < NREP) buf_lse[row0 + tid] = -INFINITY;
        return;
    }
    float* red = sc + NREP * sc_cap;        // [2][8 warps][NREP]
    float* qs = red + 16 * NREP;            // [NREP][128]
    float* po = qs + NREP * kHD;            // [3][NREP][128]
    const __half* kbase = kb + b * kb_sb + h * kb_sh;
    const __half* vbase = vb + b * kb_sb + h * kb_sh;
    // live rows -> shared memory, 16 bytes per request: first all key rows (one group), then all value rows
    for (int which = 0; which < 2; ++which) {
        const __half* src = which ? vbase : kbase;
        const uint32_t dst = smem_u32(which ? vs : ks);
        for (int e = tid; e < n_tok * 16; e += kBufThreads) {
            const int sl = slot(e >> 4), c = e & 15;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + sl * kBufRowLd + c * 16),
                         "l"(src + (size_t)sl * kHD + c * 8)
                         : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int e = tid; e < NREP * kHD; e += kBufThreads)
        qs[e] = __half2float(q[b * q_sb + (hq0 + (e >> 7)) * q_sh + (e & 127)]);
    asm volatile("cp.async.wait_group 1;" ::: "memory");      // the key rows have landed
    __syncthreads();
    // logits: one thread per token, its key row used for every head
    for (int i = tid; i < n_tok; i += kBufThreads) {
        const uint4* kr = reinterpret_cast<const uint4*>(ks + (size_t)slot(i) * kBufRowLd);
        float s0[NREP], s1[NREP];
#pragma unroll
        for (int g = 0; g < NREP; ++g) s0[g] = s1[g] = 0.f;
#pragma unroll
        for (int c = 0; c < kHD / 8; ++c) {
            const uint4 kv = kr[c];
            const float2 k0 = __half22float2(*reinterpret_cast<const __half2*>(&kv.x));
            const float2 k1 = __half22float2(*reinterpret_cast<const __half2*>(&kv.y));
            const float2 k2 = __half22float2(*reinterpret_cast<const __half2*>(&kv.z));
            const float2 k3 = __half22float2(*reinterpret_cast<const __half2*>(&kv.w));
#pragma unroll
            for (int g = 0; g < NREP; ++g) {
                const float4 qa = *reinterpret_cast<const float4*>(qs + g * kHD + 8 * c);
                const float4 qb = *reinterpret_cast<const float4*>(qs + g * kHD + 8 * c + 4);
                s0[g] = fmaf(qa.x, k0.x, s0[g]); s1[g] = fmaf(qa.y, k0.y, s1[g]);
                s0[g] = fmaf(qa.z, k1.x, s0[g]); s1[g] = fmaf(qa.w, k1.y, s1[g]);
                s0[g] = fmaf(qb.x, k2.x, s0[g]); s1[g] = fmaf(qb.y, k2.y, s1[g]);
                s0[g] = fmaf(qb.z, k3.x, s0[g]); s1[g] = fmaf(qb.w, k3.y, s1[g]);
            }
        }
#pragma unroll
        for (int g = 0; g < NREP; ++g) sc[g * sc_cap + i] = (s0[g] + s1[g]) * scale;
    }
    __syncthreads();
    float mx[NREP];
#pragma unroll
    for (int g = 0; g < NREP; ++g) {
        float m = -INFINITY;
        for (int i = tid; i < n_tok; i += kBufThreads) m = fmaxf(m, sc[g * sc_cap + i]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) red[warp * NREP + g] = m;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < NREP; ++g) {
        float m = red[g];
#pragma unroll
        for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w * NREP + g]);
        mx[g] = m;
        float sm = 0.f;
        for (int i = tid; i < n_tok; i += kBufThreads) {
            const float pv = expf(sc[g * sc_cap + i] - m);
            sc[g * sc_cap + i] = pv;
            sm += pv;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sm += __shfl_xor_sync(0xffffffffu, sm, o);
        if (lane == 0) red[(8 + warp) * NREP + g] = sm;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");      // the value rows have landed
    __syncthreads();
    // the eight warps' sums of head g, added in a fixed order (read again after the value phase: red stays as it is)
    auto head_sum = [&](int g) {
        const float* r8 = red + 8 * NREP + g;
        return ((r8[0] + r8[NREP]) + (r8[2 * NREP] + r8[3 * NREP])) + ((r8[4 * NREP] + r8[5 * NREP]) + (r8[6 * NREP] + r8[7 * NREP]));
    };
#pragma unroll
    for (int g = 0; g < NREP; ++g)
        if (tid == g) buf_lse[row0 + g] = mx[g] + logf(head_sum(g));
    // output: thread -> dims (2 d2, 2 d2 + 1) of every fourth token for all heads
    const int d2 = tid & 63, par = tid >> 6;
    float a0[NREP], a1[NREP];
#pragma unroll
    for (int g = 0; g < NREP; ++g) a0[g] = a1[g] = 0.f;
#pragma unroll 2
    for (int i = par; i < n_tok; i += 4) {
        const float2 v = __half22float2(*reinterpret_cast<const __half2*>(vs + (size_t)slot(i) * kBufRowLd + 4 * d2));
#pragma unroll
        for (int g = 0; g < NREP; ++g) {
            const float pr = sc[g * sc_cap + i];
            a0[g] = fmaf(pr, v.x, a0[g]);
            a1[g] = fmaf(pr, v.y, a1[g]);
        }
    }
    if (par) {
#pragma unroll
        for (int g = 0; g < NREP; ++g)
            *reinterpret_cast<float2*>(po + ((par - 1) * NREP + g) * kHD + 2 * d2) = make_float2(a0[g], a1[g]);
    }
    __syncthreads();
    if (!par) {
#pragma unroll
        for (int g = 0; g < NREP; ++g) {
            const float inv = 1.0f / head_sum(g);
            const float2 p1 = *reinterpret_cast<const float2*>(po + g * kHD + 2 * d2),
                         p2 = *reinterpret_cast<const float2*>(po + (NREP + g) * kHD + 2 * d2),
                         p3 = *reinterpret_cast<const float2*>(po + (2 * NREP + g) * kHD + 2 * d2);
            *reinterpret_cast<float2*>(buf_o + (row0 + g) * kHD + 2 * d2) =
                make_float2(((a0[g] + p1.x) + (p2.x + p3.x)) * inv, ((a1[g] + p1.y) + (p2.y + p3.y)) * inv);
        }
    }
}

// The combine variant for a launch of n_q x n_batch rows: one row per CTA with its rotation entries in registers
// while all CTAs fit the GPU at once; beyond that four rows of one KV head per CTA where the head grouping
// allows it, else the lean one-row variant.
cudaError_t launch_combine(int n_batch, cudaStream_t stream, bool programmatic, const float* part_o, const float* part_lse,
                           int n_splits, const float* v_rot, const float* buf_o, const float* buf_lse, int n_q, int n_kv,
                           __half* out, int64_t o_sb, int64_t o_sh, float* out_f32, float* lse_out, int64_t rank_stride,
                           const PublishArgs& pub) {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        sms = n > 0 ? n : 148;
    }
    const bool single_wave = (int64_t)n_q * n_batch <= sms;
    if (!single_wave && v_rot && rank_stride == 0 && (n_q / n_kv) % 4 == 0)
        return launch_kernel(combine4_kernel, dim3(n_q / 4, n_batch), dim3(512), 0, stream, programmatic, part_o, part_lse,
                             n_splits, v_rot, buf_o, buf_lse, n_q, n_kv, out, o_sb, o_sh, out_f32, lse_out, pub);
    return launch_kernel(single_wave ? combine_kernel<true> : combine_kernel<false>, dim3(n_q, n_batch), dim3(512), 0,
                         stream, programmatic, part_o, part_lse, n_splits, v_rot, buf_o, buf_lse, n_q, n_kv, out, o_sb,
                         o_sh, out_f32, lse_out, rank_stride, pub);
}

const char* const kErrNames[] = {"ok", "bad argument", "unsupported shape or mode", "misaligned pointer",
                                 "kernel launch failed", "size exceeds a library limit"};

}  // namespace
}  // namespace bgtq

using namespace bgtq;

extern "C" __attribute__((visibility("default"))) int bgtq_abi_version(void) { return BGTQ_ABI_VERSION; }
extern "C" __attribute__((visibility("default"))) int bgtq_desc_size(void) { return (int)sizeof(BgtqHeadDesc); }
extern "C" __attribute__((visibility("default"))) const char* bgtq_error_string(int code) {
    const int i = -code;
    return (i >= 0 && i < (int)(sizeof(kErrNames) / sizeof(kErrNames[0]))) ? kErrNames[i] : "unknown error";
}

extern "C" __attribute__((visibility("default"))) int bgtq_rotate_q(const BgtqHeadDesc* desc, const float* rot_k, const void* q, int64_t q_sb, int64_t q_sh,
                             void* q_rot, int32_t n_batch, int32_t n_q, int32_t n_kv, void* stream) {
    if (!desc || !rot_k || !q || !q_rot || n_batch < 1 || n_kv < 1 || n_q < n_kv || n_q % n_kv) return BGTQ_E_BADARG;
    if (n_batch > 65535) return BGTQ_E_TOOBIG;
    rotate_q_kernel<<<dim3(n_q, n_batch), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        desc, rot_k, static_cast<const __half*>(q), q_sb, q_sh, static_cast<__half*>(q_rot), n_q, n_kv);
    return cudaGetLastError() == cudaSuccess ? BGTQ_OK : BGTQ_E_LAUNCH;
}

extern "C" __attribute__((visibility("default"))) int bgtq_combine(const float* part_o, const float* part_lse, int32_t n_splits, const float* v_rot,
                            const float* buf_o, const float* buf_lse, int32_t n_batch, int32_t n_q, int32_t n_kv,
                            void* out, int64_t o_sb, int64_t o_sh, float* out_f32, float* lse_out, int32_t flags, void* stream) {
    if (!part_o || !part_lse || n_splits < 1 || n_batch < 1 || n_kv < 1 || n_q < n_kv || n_q % n_kv)
        return BGTQ_E_BADARG;
    if ((buf_o == nullptr) != (buf_lse == nullptr)) return BGTQ_E_BADARG;
    if (!out && !out_f32) return BGTQ_E_BADARG;
    if (n_batch > 65535) return BGTQ_E_TOOBIG;
    return launch_combine(n_batch, static_cast<cudaStream_t>(stream),
                         (flags & BGTQ_COMBINE_PROGRAMMATIC) != 0, part_o, part_lse, n_splits, v_rot, buf_o, buf_lse,
                         n_q, n_kv, static_cast<__half*>(out), o_sb, o_sh, out_f32, lse_out, (int64_t)0,
                         PublishArgs{}) == cudaSuccess
               ? BGTQ_OK : BGTQ_E_LAUNCH;
}

extern "C" __attribute__((visibility("default"))) int bgtq_combine_publish(
    const float* part_o, const float* part_lse, int32_t n_splits, const float* v_rot, int32_t n_batch, int32_t n_q,
    int32_t n_kv, float* const* peer_bufs, int64_t slot_off, int64_t parity_stride, int32_t* const* peer_flags,
    int32_t rank, int32_t n_ranks, const int32_t* seq_dev, int32_t* ticket, int32_t flags, void* stream) {
    if (!part_o || !part_lse || n_splits < 1 || n_batch < 1 || n_kv < 1 || n_q < n_kv || n_q % n_kv)
        return BGTQ_E_BADARG;
    if (!peer_bufs || !peer_flags || !seq_dev || !ticket || n_ranks < 1 || rank < 0 || rank >= n_ranks)
        return BGTQ_E_BADARG;
    if (n_batch > 65535) return BGTQ_E_TOOBIG;
    PublishArgs pub;
    pub.peer_bufs = peer_bufs; pub.peer_flags = peer_flags; pub.slot_off = slot_off; pub.parity_stride = parity_stride;
    pub.rows = (int64_t)n_batch * n_q; pub.seq_dev = seq_dev; pub.ticket = ticket; pub.rank = rank; pub.n_ranks = n_ranks;
    return launch_combine(n_batch, static_cast<cudaStream_t>(stream),
                         (flags & BGTQ_COMBINE_PROGRAMMATIC) != 0, part_o, part_lse, n_splits, v_rot,
                         static_cast<const float*>(nullptr), static_cast<const float*>(nullptr), n_q, n_kv,
                         static_cast<__half*>(nullptr), (int64_t)0, (int64_t)0, static_cast<float*>(nullptr),
                         static_cast<float*>(nullptr), (int64_t)0, pub) == cudaSuccess
               ? BGTQ_OK : BGTQ_E_LAUNCH;
}

extern "C" __attribute__((visibility("default"))) int bgtq_combine_ranks(const float* gathered, int32_t n_ranks, int64_t rank_stride,
                                  int32_t n_batch, int32_t n_q, void* out, int64_t o_sb, int64_t o_sh, int32_t flags,
                                  void* stream) {
    if (!gathered || !out || n_ranks < 1 || n_batch < 1 || n_q < 1) return BGTQ_E_BADARG;
    const int64_t rows = (int64_t)n_batch * n_q;
    if (rank_stride < rows * (kHD + 1)) return BGTQ_E_BADARG;
    if (n_batch > 65535) return BGTQ_E_TOOBIG;
    return launch_combine(n_batch, static_cast<cudaStream_t>(stream),
                         (flags & BGTQ_COMBINE_PROGRAMMATIC) != 0, gathered, gathered + rows * kHD, n_ranks,
                         static_cast<const float*>(nullptr), static_cast<const float*>(nullptr),
                         static_cast<const float*>(nullptr), n_q, 1, static_cast<__half*>(out), o_sb, o_sh,
                         static_cast<float*>(nullptr), static_cast<float*>(nullptr), rank_stride,
                         PublishArgs{}) == cudaSuccess
               ? BGTQ_OK : BGTQ_E_LAUNCH;
}

extern "C" int bgtq_buffer_attn_pos(const void* q, int64_t q_sb, int64_t q_sh, const void* k_buf, const void* v_buf,
                                int64_t kb_sb, int64_t kb_sh, int32_t n_sink_tokens, int32_t n_ring_tokens,
                                int32_t sink_cap, int32_t ring_first, int32_t ring_size, int32_t n_batch, int32_t n_q,
                                int32_t n_kv, float scale, float* buf_o, float* buf_lse, const int32_t* pos_dev,
                                void* stream);

extern "C" __attribute__((visibility("default"))) int bgtq_buffer_attn(const void* q, int64_t q_sb, int64_t q_sh, const void* k_buf, const void* v_buf,
                                int64_t kb_sb, int64_t kb_sh, int32_t n_sink_tokens, int32_t n_ring_tokens,
                                int32_t sink_cap, int32_t ring_first, int32_t ring_size, int32_t n_batch, int32_t n_q,
                                int32_t n_kv, float scale, float* buf_o, float* buf_lse, void* stream) {
    return bgtq_buffer_attn_pos(q, q_sb, q_sh, k_buf, v_buf, kb_sb, kb_sh, n_sink_tokens, n_ring_tokens, sink_cap,
                                ring_first, ring_size, n_batch, n_q, n_kv, scale, buf_o, buf_lse, nullptr, stream);
}

extern "C" __attribute__((visibility("default"))) int bgtq_buffer_attn_pos(const void* q, int64_t q_sb, int64_t q_sh, const void* k_buf, const void* v_buf,
                                int64_t kb_sb, int64_t kb_sh, int32_t n_sink_tokens, int32_t n_ring_tokens,
                                int32_t sink_cap, int32_t ring_first, int32_t ring_size, int32_t n_batch, int32_t n_q,
                                int32_t n_kv, float scale, float* buf_o, float* buf_lse, const int32_t* pos_dev,
                                void* stream) {
    if (!q || !buf_o || !buf_lse || n_batch < 1 || n_kv < 1 || n_q < n_kv || n_q % n_kv || n_sink_tokens < 0 ||
        n_ring_tokens < 0 || n_sink_tokens > sink_cap || n_ring_tokens > ring_size || ring_first < 0 ||
        (n_ring_tokens > 0 && ring_first >= ring_size))
        return BGTQ_E_BADARG;
    // with a device-side position the region sizes are computed in the kernel: size the scratch for the most
    const int32_t n_buf_tokens = pos_dev ? sink_cap + ring_size : n_sink_tokens + n_ring_tokens;
    if (n_buf_tokens > 0 && (!k_buf || !v_buf)) return BGTQ_E_BADARG;
    if (pos_dev && ring_size < 2) return BGTQ_E_BADARG;
    if (n_buf_tokens > 8192 || n_batch > 65535) return BGTQ_E_TOOBIG;
    if (n_buf_tokens > 0 && ((reinterpret_cast<uintptr_t>(k_buf) & 15u) || (reinterpret_cast<uintptr_t>(v_buf) & 15u) ||
                             (kb_sb & 7) || (kb_sh & 7) || (reinterpret_cast<uintptr_t>(buf_o) & 7u)))
        return BGTQ_E_ALIGN;
    const int sc_cap = (n_buf_tokens + 3) & ~3;       // keeps the query block 16-byte aligned
    const int n_rep = n_q / n_kv;
    const int cap_rows = sink_cap + (ring_size > 0 ? ring_size : 1);      // buffer slots a live token can sit in
    const size_t smem_group = 2 * (size_t)cap_rows * kBufRowLd + (size_t)n_rep * (sc_cap + 16 + 4 * kHD) * sizeof(float);
    if ((n_rep == 2 || n_rep == 4 || n_rep == 8) && n_buf_tokens > 0 && smem_group <= 200 * 1024) {
        // grouped heads with the rows staged in shared memory: one CTA per KV head
        auto kern = n_rep == 2 ? buffer_attn_group_kernel<2> : n_rep == 4 ? buffer_attn_group_kernel<4> : buffer_attn_group_kernel<8>;
        // the attribute is per device: set it on every launch (cheap, and legal under stream capture)
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) {
            cudaGetLastError();
            return BGTQ_E_LAUNCH;
        }
        kern<<<dim3(n_kv, n_batch), kBufThreads, smem_group, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const __half*>(q), q_sb, q_sh, static_cast<const __half*>(k_buf), static_cast<const __half*>(v_buf),
            kb_sb, kb_sh, n_sink_tokens, n_ring_tokens, sink_cap, ring_first, ring_size > 0 ? ring_size : 1, n_q, scale,
            buf_o, buf_lse, pos_dev, sc_cap, cap_rows);
        return cudaGetLastError() == cudaSuccess ? BGTQ_OK : BGTQ_E_LAUNCH;
    }
    const size_t smem = (size_t)(sc_cap + 16 + 4 * kHD) * sizeof(float);
    buffer_attn_kernel<<<dim3(n_q, n_batch), kBufThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(q), q_sb, q_sh, static_cast<const __half*>(k_buf),
        static_cast<const __half*>(v_buf), kb_sb, kb_sh, n_sink_tokens, n_ring_tokens, sink_cap, ring_first,
        ring_size > 0 ? ring_size : 1, n_q, n_kv, scale, buf_o, buf_lse, pos_dev, sc_cap);
    return cudaGetLastError() == cudaSuccess ? BGTQ_OK : BGTQ_E_LAUNCH;
}

// ---------------------------------------------------------------------------
// Sequence-sharded cache: exchange of the per-rank [O | LSE] messages over peer memory (NVLink) instead of
// a library all-gather.  Every rank owns one exchange buffer [2 parities][n_ranks][stride] fp32 and one
// flag word per rank, all mapped into every peer (symmetric memory).  Step number s (a device counter, so
// a captured graph can be replayed):
//   publish : copy the local message into slot [s & 1][my rank] of EVERY rank's buffer with plain peer
//             stores, fence at system scope, then (last block of the grid) store s + 1 into flag[my rank]
//             of every rank;
//   merge   : wait (bounded) until flag[r] >= s + 1 for all r, merge the n_ranks messages of parity s & 1
//             from the LOCAL buffer, and (last block) advance the counter.
// Two parities are enough: a rank can be at most one step ahead of the slowest one, because its next
// publish needs every peer's flag of the step before.
// ---------------------------------------------------------------------------
namespace bgtq {
namespace {

constexpr int kStatusPeerTimeout = 3;

__global__ void __launch_bounds__(256) publish_kernel(const float* msg, int n_vec4, float* const* peer_bufs,
                                                      int64_t slot_off, int64_t parity_stride, int32_t* const* peer_flags,
                                                      int rank, int n_ranks, const int32_t* seq_dev, int32_t* ticket) {
    const int seq = *seq_dev;
    const float4* src = reinterpret_cast<const float4*>(msg);
    for (int p = 0; p < n_ranks; ++p) {
        float4* dst = reinterpret_cast<float4*>(peer_bufs[p] + (seq & 1) * parity_stride + slot_off);
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_vec4; i += gridDim.x * blockDim.x) dst[i] = src[i];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int t = atomicAdd(ticket, 1);
        if (t == (int)gridDim.x - 1) {          // every block's stores are fenced: raise the flag everywhere
            *ticket = 0;
            __threadfence_system();
            for (int p = 0; p < n_ranks; ++p) {
                volatile int32_t* f = peer_flags[p] + rank;
                *f = seq + 1;
            }
        }
    }
}

__global__ void __launch_bounds__(128) merge_ranks_kernel(const float* local_buf, int n_ranks, int64_t rank_stride,
                                                          int64_t parity_stride, const int32_t* flags, int32_t* seq_dev,
                                                          int n_q, int64_t rows, __half* out, int64_t o_sb, int64_t o_sh,
                                                          int32_t* status, int32_t* ticket) {
    __shared__ int ok;
    const int d = threadIdx.x, hq = blockIdx.x, b = blockIdx.y;
    grid_launch_dependents();
    grid_dependency_wait();       // the step counter and the local message come from the stream's earlier kernels
    const int seq = *seq_dev;
    if (d == 0) {
        int good = 1;
        for (int r = 0; r < n_ranks && good; ++r) {
            const volatile int32_t* f = flags + r;
            int spins = 0;
            while (*f < seq + 1) {
                if (++spins > (1 << 20)) { good = 0; break; }      // give up: report, do not hang
                __nanosleep(200);
            }
        }
        __threadfence_system();
        ok = good;
        if (!good && status) atomicExch(status, kStatusPeerTimeout);
    }
    __syncthreads();
    const size_t row = (size_t)b * n_q + hq;
    const float* base = local_buf + (seq & 1) * parity_stride;
    float o = 0.f;
    if (ok) {
        float mx = -INFINITY;
        for (int r = 0; r < n_ranks; ++r) mx = fmaxf(mx, __ldcg(base + r * rank_stride + rows * kHD + row));
        float num = 0.f, den = 0.f;
        if (mx > -INFINITY) {
            for (int r = 0; r < n_ranks; ++r) {
                const float l = __ldcg(base + r * rank_stride + rows * kHD + row);
                if (l == -INFINITY) continue;
                const float a = expf(l - mx);
                den += a;
                num = fmaf(a, __ldcg(base + r * rank_stride + row * kHD + d), num);
            }
        }
        o = den > 0.f ? num / den : 0.f;
    }
    out[b * o_sb + hq * o_sh + d] = __float2half_rn(o);
    __syncthreads();
    if (d == 0) {
        const int t = atomicAdd(ticket, 1);
        if (t == (int)(gridDim.x * gridDim.y) - 1) {    // all blocks have read the flags and the messages
            *ticket = 0;
            *seq_dev = seq + 1;
        }
    }
}

}  // namespace
}  // namespace bgtq

extern "C" __attribute__((visibility("default"))) int bgtq_exchange_publish(
    const float* msg, int64_t n_floats, float* const* peer_bufs, int64_t slot_off, int64_t parity_stride,
    int32_t* const* peer_flags, int32_t rank, int32_t n_ranks, const int32_t* seq_dev, int32_t* ticket, void* stream) {
    if (!msg || !peer_bufs || !peer_flags || !seq_dev || !ticket || n_ranks < 1 || rank < 0 || rank >= n_ranks || n_floats < 4)
        return BGTQ_E_BADARG;
    if ((n_floats & 3) || (slot_off & 3) || (parity_stride & 3) || (reinterpret_cast<uintptr_t>(msg) & 15u)) return BGTQ_E_ALIGN;
    const int n_vec4 = (int)(n_floats / 4);
    int blocks = (n_vec4 + 255) / 256;
    blocks = blocks > 32 ? 32 : blocks;
    publish_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(msg, n_vec4, peer_bufs, slot_off, parity_stride,
                                                                            peer_flags, rank, n_ranks, seq_dev, ticket);
    return cudaGetLastError() == cudaSuccess ? BGTQ_OK : BGTQ_E_LAUNCH;
}

extern "C" __attribute__((visibility("default"))) int bgtq_exchange_merge(
    const float* local_buf, int32_t n_ranks, int64_t rank_stride, int64_t parity_stride, const int32_t* flags,
    int32_t* seq_dev, int32_t n_batch, int32_t n_q, void* out, int64_t o_sb, int64_t o_sh, int32_t* status,
    int32_t* ticket, void* stream) {
    if (!local_buf || !flags || !seq_dev || !out || !ticket || n_ranks < 1 || n_batch < 1 || n_q < 1) return BGTQ_E_BADARG;
    const int64_t rows = (int64_t)n_batch * n_q;
    if (rank_stride < rows * (kHD + 1) || parity_stride < rank_stride * n_ranks) return BGTQ_E_BADARG;
    if (n_batch > 65535) return BGTQ_E_TOOBIG;
    // launched as a programmatic dependent: its blocks may become resident while the step's previous kernel
    // drains; they wait for it on the device before reading anything
    return launch_kernel(merge_ranks_kernel, dim3(n_q, n_batch), dim3(128), 0, static_cast<cudaStream_t>(stream), true,
                         local_buf, n_ranks, rank_stride, parity_stride, flags, seq_dev, n_q, rows,
                         static_cast<__half*>(out), o_sb, o_sh, status, ticket) == cudaSuccess
               ? BGTQ_OK : BGTQ_E_LAUNCH;
}
