// Host side of the decode kernel: the launch plan of a layer's KV heads, the
// prebuilt lookup-table image the kernel copies into shared memory, and the
// suggested split count.  No GPU work happens here.
#include <string.h>

#include "bgtq_common.cuh"
#include "bgtq_plan.h"

using namespace bgtq;

namespace {

struct TableDims {
    uint32_t entries, ent_log2, rep_log2;
    uint32_t bytes() const { return (entries << ent_log2) << rep_log2; }
};

TableDims k_table_dims(int kind, int bw, uint32_t boost) {
    switch (kind) {
        case 1: return {16u, 3u, kRep1};
        case 2: return {16u, 2u, kRep2};
        case 3: return {64u, 2u, kRep3};
        case 4: return {256u, 2u, kRep4 + boost};
        default: return {1u << bw, 2u, bw <= 6 ? 5u : (bw == 7 ? 4u : 3u)};
    }
}

uint32_t v_rep_log2_for(int sbits) { return sbits <= 3 ? 5u : 3u; }

}  // namespace

extern "C" __attribute__((visibility("default"))) int bgtq_decode_plan(const BgtqHeadDesc* desc_host, int32_t n_kv,
                                                                       int32_t flags, BgtqDecodePlan* out) {
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
    pl.v_rep_log2 = v_rep_log2_for(pl.v_sbits);
    const uint32_t v_bytes = ((1u << (2 * pl.v_sbits)) << 2) << pl.v_rep_log2;
    // Shared memory left for the tables once two stages of 512-token tiles of the live row sizes are set aside
    // (launches with wider, padded rows fall back to 256-token tiles on their own).
    uint32_t row_bytes = 0;
    for (int h = 0; h < n_kv; ++h) {
        const BgtqHeadDesc& d = desc_host[h];
        const uint32_t kb = (flags & BGTQ_DEC_K_MIXED) ? (uint32_t)d.k_mixed_bytes : (uint32_t)d.k_row_bytes;
        const uint32_t vb = (flags & BGTQ_DEC_V_NIBBLE) ? kHD / 2u : (uint32_t)d.v_row_bytes;
        const uint32_t rb = kb + 2u * 8u + vb + 2u;
        row_bytes = rb > row_bytes ? rb : row_bytes;
    }
    const uint32_t stage_est = 2u * (512u * row_bytes + 4u * 64u + 128u);
    const uint32_t fixed_est = 7168u + kLutAlign + stage_est;
    const uint32_t lut_budget = fixed_est < 227u * 1024u ? 227u * 1024u - fixed_est : 0u;
    uint32_t lut_bytes = 0;
    for (uint32_t boost = 1;; --boost) {        // more replicas of the 256-entry table when they fit
    lut_bytes = 0;
    for (int h = 0; h < n_kv; ++h) {
        const BgtqHeadDesc& d = desc_host[h];
        if (d.v_bits != pl.v_bits) return BGTQ_E_UNSUPPORTED;
        if (d.n_seg < 1 || d.n_seg > BGTQ_MAX_SEGMENTS) return BGTQ_E_BADARG;
        DecHeadPlan& hp = pl.head[h];
        hp.n_seg = d.n_seg;
        uint32_t bytes_of[BGTQ_MAX_SEGMENTS + 1];
        int step = 0;
        for (int s = 0; s < d.n_seg; ++s) {
            const int bw = d.seg_bw[s], len = d.seg_len[s], start = d.seg_start[s];
            if (bw < 1 || bw > 8 || len < 2 || (len & 1) || start < 0 || start + len > kHD) return BGTQ_E_BADARG;
            DecSeg& sg = hp.seg[s];
            uint32_t bit0;
            if (flags & BGTQ_DEC_K_MIXED) {
                sg.kind = bw <= 4 ? 4 : 8;
                bit0 = bw <= 4 ? start * 4u : 8u * (d.nopack_start / 2 + (start - d.nopack_start));
            } else {
                sg.kind = bw <= 4 ? bw : 8;
                bit0 = 8u * d.seg_pack_off[s];
            }
            const TableDims td = k_table_dims(sg.kind, bw, boost);
            sg.bw = (uint8_t)bw;
            sg.q = (uint8_t)(2 * ((len + 7) / 8));
            // reference: only segments 0..4 of at least 16 dims take the tensor-core (fp16 operand) path
            sg.f16_norm = ((flags & BGTQ_DEC_K_MIXED) && len >= 16 && s < 5) ? 1 : 0;
            sg.lane_bits = (uint16_t)(sg.q * sg.kind);
            if (bit0 + 3u * sg.lane_bits + 64u > 0xFFFFu) return BGTQ_E_UNSUPPORTED;
            sg.bit0 = (uint16_t)bit0;
            sg.ent_log2 = (uint8_t)td.ent_log2;
            sg.rep_log2 = (uint8_t)td.rep_log2;
            sg.esh = (uint8_t)(td.ent_log2 + td.rep_log2);
            sg.norm_idx = (uint8_t)s;
            bytes_of[s] = td.bytes();
            if (bytes_of[s] > kLutAlign) return BGTQ_E_UNSUPPORTED;
            for (int c4 = 0; c4 < sg.q; c4 += 4) {
                if (step >= kMaxSteps) return BGTQ_E_UNSUPPORTED;
                DecStepQ& st = hp.steps[step++];
                st.pos = (uint8_t)(start + c4);
                st.q = sg.q;
                st.end = (uint8_t)(start + len);
                st.c4 = (uint8_t)c4;
            }
        }
        hp.n_steps = step;
        bytes_of[d.n_seg] = v_bytes;
        // Place tables largest first: every size is a power of two, so each lands on a multiple of its size.
        uint32_t off = 0;
        bool placed[BGTQ_MAX_SEGMENTS + 1] = {false};
        for (int n = 0; n <= d.n_seg; ++n) {
            int best = -1;
            for (int s = 0; s <= d.n_seg; ++s)
                if (!placed[s] && (best < 0 || bytes_of[s] > bytes_of[best])) best = s;
            placed[best] = true;
            if (best < d.n_seg) hp.seg[best].tbl = off;
            else hp.v_tbl = off;
            off += bytes_of[best];
        }
        hp.image_bytes = off;
        lut_bytes = off > lut_bytes ? off : lut_bytes;
    }
    if (boost == 0 || lut_bytes <= lut_budget) break;
    }
    pl.lut_bytes = (lut_bytes + 127u) / 128u * 128u;
    pl.image = nullptr;
    memcpy(out, &pl, sizeof(pl));
    return BGTQ_OK;
}

extern "C" __attribute__((visibility("default"))) int64_t bgtq_decode_image_bytes(const BgtqDecodePlan* plan_host) {
    if (!plan_host) return BGTQ_E_BADARG;
    DecPlanDev pl;
    memcpy(&pl, plan_host, sizeof(pl));
    if (pl.n_heads < 1 || pl.n_heads > kMaxPlanHeads) return BGTQ_E_BADARG;
    return (int64_t)pl.n_heads * pl.lut_bytes;
}

extern "C" __attribute__((visibility("default"))) int bgtq_decode_build_image(const BgtqDecodePlan* plan_host,
                                                                              const BgtqHeadDesc* desc_host,
                                                                              uint8_t* image_host, int64_t bytes) {
    if (!plan_host || !desc_host || !image_host) return BGTQ_E_BADARG;
    DecPlanDev pl;
    memcpy(&pl, plan_host, sizeof(pl));
    if (pl.n_heads < 1 || pl.n_heads > kMaxPlanHeads) return BGTQ_E_BADARG;
    if (bytes < (int64_t)pl.n_heads * pl.lut_bytes) return BGTQ_E_BADARG;
    memset(image_host, 0, (size_t)pl.n_heads * pl.lut_bytes);
    for (int h = 0; h < pl.n_heads; ++h) {
        const BgtqHeadDesc& d = desc_host[h];
        const DecHeadPlan& hp = pl.head[h];
        uint8_t* img = image_host + (size_t)h * pl.lut_bytes;
        auto put = [&](uint32_t off, uint32_t word) { memcpy(img + off, &word, 4); };
        for (int s = 0; s < hp.n_seg; ++s) {
            const DecSeg& sg = hp.seg[s];
            const uint16_t* cb = d.codebook + d.seg_lut_off[s];
            const uint32_t cm = (1u << sg.bw) - 1u, reps = 1u << sg.rep_log2;
            const uint32_t sb = sg.kind == 8 ? 8u : sg.kind, smk = (1u << sb) - 1u;
            const uint32_t entries = sg.kind <= 2 ? 16u : sg.kind == 3 ? 64u : sg.kind == 8 ? (1u << sg.bw) : 256u;
            for (uint32_t e = 0; e < entries; ++e) {
                uint32_t w0, w1 = 0;
                if (sg.kind == 8) {
                    w0 = cb[e & cm] | ((uint32_t)cb[e & cm] << 16);
                } else {
                    auto code = [&](int k) { return ((e >> (k * sb)) & smk) & cm; };
                    w0 = cb[code(0)] | ((uint32_t)cb[code(1)] << 16);
                    if (sg.ent_log2 == 3) w1 = cb[code(2)] | ((uint32_t)cb[code(3)] << 16);
                }
                for (uint32_t r = 0; r < reps; ++r) {
                    const uint32_t off = sg.tbl + (e << sg.esh) + (r << sg.ent_log2);
                    put(off, w0);
                    if (sg.ent_log2 == 3) put(off + 4, w1);
                }
            }
        }
        const uint32_t vb = (uint32_t)pl.v_sbits, vm = (1u << pl.v_bits) - 1u, smk = (1u << vb) - 1u;
        const uint32_t vesh = 2u + pl.v_rep_log2;
        for (uint32_t e = 0; e < (1u << (2 * vb)); ++e) {
            const uint32_t w = d.v_lut[(e & smk) & vm] | ((uint32_t)d.v_lut[(e >> vb) & vm] << 16);
            for (uint32_t r = 0; r < (1u << pl.v_rep_log2); ++r) put(hp.v_tbl + (e << vesh) + (r << 2), w);
        }
    }
    return BGTQ_OK;
}

extern "C" __attribute__((visibility("default"))) int bgtq_decode_plan_set_image(BgtqDecodePlan* plan_host,
                                                                                 const uint8_t* image_dev) {
    if (!plan_host) return BGTQ_E_BADARG;
    if (reinterpret_cast<uintptr_t>(image_dev) & 15u) return BGTQ_E_ALIGN;
    DecPlanDev pl;
    memcpy(&pl, plan_host, sizeof(pl));
    pl.image = image_dev;
    memcpy(plan_host, &pl, sizeof(pl));
    return BGTQ_OK;
}

extern "C" __attribute__((visibility("default"))) int bgtq_decode_plan_set_row_strides(BgtqDecodePlan* plan_host,
                                                                                       int32_t kp_st, int32_t kn_st,
                                                                                       int32_t vp_st, int32_t vn_st) {
    if (!plan_host) return BGTQ_E_BADARG;
    const bool clear = kp_st == 0 && kn_st == 0 && vp_st == 0 && vn_st == 0;
    if (!clear && (kp_st < 1 || kp_st > 160 || vp_st < 1 || vp_st > 128 || kn_st < 1 || kn_st > 16 || vn_st < 1 || vn_st > 8))
        return BGTQ_E_UNSUPPORTED;
    DecPlanDev pl;
    memcpy(&pl, plan_host, sizeof(pl));
    if (pl.jit_kernel) return BGTQ_E_BADARG;       // already specialised: the strides are part of that kernel
    pl.row_st[0] = kp_st;
    pl.row_st[1] = 2 * kn_st;                      // bytes, like the kernel's own parameters
    pl.row_st[2] = vp_st;
    pl.row_st[3] = 2 * vn_st;
    memcpy(plan_host, &pl, sizeof(pl));
    return BGTQ_OK;
}

extern "C" __attribute__((visibility("default"))) int bgtq_decode_plan_set_early_fetch(BgtqDecodePlan* plan_host,
                                                                                      int32_t fresh_rows) {
    if (!plan_host || fresh_rows < 0) return BGTQ_E_BADARG;
    DecPlanDev pl;
    memcpy(&pl, plan_host, sizeof(pl));
    pl.early_fresh = fresh_rows;
    memcpy(plan_host, &pl, sizeof(pl));
    return BGTQ_OK;
}

extern "C" __attribute__((visibility("default"))) int bgtq_decode_plan_set_partition(BgtqDecodePlan* plan_host,
                                                                                     const int32_t* partition_dev) {
    if (!plan_host) return BGTQ_E_BADARG;
    if (reinterpret_cast<uintptr_t>(partition_dev) & 3u) return BGTQ_E_ALIGN;
    DecPlanDev pl;
    memcpy(&pl, plan_host, sizeof(pl));
    pl.partition = partition_dev;
    memcpy(plan_host, &pl, sizeof(pl));
    return BGTQ_OK;
}

extern "C" __attribute__((visibility("default"))) int bgtq_decode_grid_size(int32_t n_batch, int32_t n_kv,
                                                                           int32_t n_splits) {
    if (n_batch < 1 || n_kv < 1 || n_splits < 1) return BGTQ_E_BADARG;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    else cudaGetLastError();
    const int64_t items = (int64_t)n_batch * n_kv * n_splits;
    return (int)(items < sms ? items : sms);
}

// Item ranges per CTA that even out what the CTAs spend, not what they stream: a CTA pays kRunCostUnits for
// every run it starts (prologue, merge of its sixteen warps, one more partial), so one whose range straddles
// a pair boundary gets fewer items than one that stays inside a pair.  Greedy fill under a cost cap, the
// smallest cap that needs no more than n_cta CTAs found by bisection.  Any non-decreasing table from 0 to the
// item count gives the same attention result; this one only moves the boundaries.
extern "C" __attribute__((visibility("default"))) int bgtq_decode_partition(int32_t n_batch, int32_t n_kv,
                                                                           int32_t n_tokens, int32_t n_splits,
                                                                           int32_t n_cta, int32_t* table_host,
                                                                           int32_t table_len) {
    if (!table_host || n_batch < 1 || n_kv < 1 || n_splits < 1 || n_cta < 1 || n_tokens < 0) return BGTQ_E_BADARG;
    if (table_len < kPartHeader + n_cta + 1) return BGTQ_E_BADARG;
    const int64_t units = ((int64_t)n_tokens + 31) / 32;
    const int64_t c_units = units == 0 ? 1 : (units + n_splits - 1) / n_splits;
    const int64_t n_live = (units + c_units - 1) / c_units;
    const int64_t n_pairs = (int64_t)n_batch * n_kv, n_items = n_pairs * n_live;
    if (n_items * ((int64_t)n_cta + 1) > 0xFFFFFFFFll) return BGTQ_E_TOOBIG;
    table_host[0] = (int32_t)n_live;
    table_host[1] = (int32_t)n_pairs;
    table_host[2] = n_cta;
    table_host[3] = (int32_t)c_units;
    int32_t* off = table_host + kPartHeader;
    const int64_t last_units = units - (n_live - 1) * c_units;     // the last item of a pair may be shorter
    // What streaming a run of `u` units costs: whole 512-token tiles, and a last partial tile that keeps fewer
    // warps busy but takes at least half the time of a full one (a tile's time is mostly the latency of one
    // warp's share of it, which fewer neighbours shorten only so far).
    auto stream_cost = [](int64_t u) -> int64_t {
        const int64_t part = u % 16;
        return u - part + (part ? (part < 8 ? 8 : part) : 0);
    };
    // CTAs the greedy fill needs under cost cap `cap` (units); fills `off` when `write`
    auto fill = [&](int64_t cap, bool write) -> int64_t {
        int64_t cta = 0, closed = 0, run = 0;        // cost of this CTA's finished runs; units of its open run
        if (write) off[0] = 0;
        for (int64_t p = 0; p < n_pairs; ++p) {
            for (int64_t s = 0; s < n_live; ++s) {
                const int64_t u = s + 1 == n_live ? last_units : c_units;
                if (closed + kRunCostUnits + stream_cost(run + u) > cap) {
                    if (closed == 0 && run == 0) return INT64_MAX;     // not even one item fits a fresh CTA
                    ++cta;
                    if (write && cta <= n_cta) off[cta] = (int32_t)(p * n_live + s);
                    closed = run = 0;
                    if (kRunCostUnits + stream_cost(u) > cap) return INT64_MAX;
                }
                run += u;
            }
            if (run) {                               // the pair ends: so does the CTA's run
                closed += kRunCostUnits + stream_cost(run);
                run = 0;
            }
        }
        const int64_t used = n_items ? cta + 1 : 0;
        if (write)
            for (int64_t c = used; c <= n_cta; ++c) off[c] = (int32_t)n_items;
        return used;
    };
    int64_t lo = kRunCostUnits + 1, hi = n_items * (c_units + 8) + n_pairs * kRunCostUnits + kRunCostUnits;
    while (lo < hi) {
        const int64_t mid = lo + (hi - lo) / 2;
        if (fill(mid, false) <= n_cta) hi = mid;
        else lo = mid + 1;
    }
    // What the equal-count split costs under the same model; the table is only worth using when it is cheaper.
    int64_t equal_max = 0;
    for (int64_t c = 0; c < n_cta; ++c) {
        int64_t cost = 0;
        for (int64_t it = c * n_items / n_cta, end = (c + 1) * n_items / n_cta; it < end;) {
            const int64_t s0 = it % n_live, cnt = (n_live - s0 < end - it) ? n_live - s0 : end - it;
            const int64_t u = cnt * c_units - (s0 + cnt == n_live ? c_units - last_units : 0);
            cost += kRunCostUnits + stream_cost(u);
            it += cnt;
        }
        equal_max = cost > equal_max ? cost : equal_max;
    }
    if (lo >= equal_max) {
        table_host[0] = -1;          // matches no launch: the kernel keeps its equal-count split
        for (int64_t c = 0; c <= n_cta; ++c) off[c] = (int32_t)(c * n_items / n_cta);
        return BGTQ_OK;
    }
    fill(lo, true);
    return BGTQ_OK;
}

extern "C" __attribute__((visibility("default"))) int bgtq_decode_default_splits(int32_t n_batch, int32_t n_kv,
                                                                                 int32_t n_tokens) {
    // The launch cuts every (batch, KV head) pair into n_splits equal items of whole 32-token warp units and
    // hands each of its CTAs (one per SM) a contiguous run of items; consecutive items of one pair inside a
    // CTA become ONE partial.  So the split count only sets the granularity at which work is balanced.  Items
    // of one 512-token tile keep every run a whole number of tiles (a finer cut leaves each run a partial last
    // tile, which costs more than it balances); below that, aim at four items per CTA; at most 256 slots.
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    else cudaGetLastError();
    const long pairs = (long)n_batch * n_kv > 0 ? (long)n_batch * n_kv : 1;
    const long units = ((long)(n_tokens > 0 ? n_tokens : 0) + 31) / 32;
    if (units <= 1) return 1;
    long c = (pairs * units + 4L * sms - 1) / (4L * sms);
    c = c < 1 ? 1 : (c > 16 ? 16 : c);
    const long c_min = (units + 255) / 256;
    c = c < c_min ? c_min : c;
    return (int)((units + c - 1) / c);
}
