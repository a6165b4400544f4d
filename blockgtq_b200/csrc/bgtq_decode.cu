// C entry points of the fused decode (kernel b): argument checks, shared-memory layout and launch.
// The kernel itself lives in bgtq_decode_kernel.cuh (one translation unit per stored V width), the
// plan / table-image builders in bgtq_decode_plan.cu.
#include "bgtq_decode_kernel.cuh"

using namespace bgtq;

static int decode_impl(
    const BgtqDecodePlan* plan_host, const void* q_rot, const uint8_t* k_packed,
    int64_t kp_sb, int64_t kp_sh, int64_t kp_st, const void* k_norms, int64_t kn_sb, int64_t kn_sh, int64_t kn_st,
    const uint8_t* v_packed, int64_t vp_sb, int64_t vp_sh, int64_t vp_st, const void* v_norms, int64_t vn_sb,
    int64_t vn_sh, int64_t vn_st, int32_t n_batch, int32_t n_q, int32_t n_kv, int32_t t_begin, int32_t t_end,
    int32_t n_splits, float scale, float* part_o, float* part_lse, int32_t* status, const int32_t* pos_dev,
    int32_t pos_add, void* stream) {
    if (!plan_host || !q_rot || !k_packed || !k_norms || !v_packed || !v_norms || !part_o || !part_lse)
        return BGTQ_E_BADARG;
    if (n_batch < 1 || n_kv < 1 || n_q < n_kv || n_q % n_kv || n_splits < 1 || t_end < t_begin || t_begin < 0)
        return BGTQ_E_BADARG;
    DecParams P;
    memcpy(&P.plan, plan_host, sizeof(DecPlanDev));
    if (P.plan.n_heads != n_kv) return BGTQ_E_BADARG;
    if (!P.plan.image) return BGTQ_E_BADARG;          // bgtq_decode_plan_set_image has not been called
    const int gqa = n_q / n_kv;
    if (gqa > 8) return BGTQ_E_UNSUPPORTED;
    if (kp_st < 1 || kp_st > 160 || vp_st < 1 || vp_st > 128 || kn_st < 1 || kn_st > 16 || vn_st < 1 || vn_st > 8)
        return BGTQ_E_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(part_o) & 7u) || (reinterpret_cast<uintptr_t>(q_rot) & 3u)) return BGTQ_E_ALIGN;
    if (n_batch > 65535 || n_splits > 65535) return BGTQ_E_TOOBIG;

    P.q_rot = static_cast<const uint16_t*>(q_rot);
    P.kp = k_packed;
    P.kn = static_cast<const uint8_t*>(k_norms);
    P.vp = v_packed;
    P.vn = static_cast<const uint8_t*>(v_norms);
    P.kp_sb = kp_sb; P.kp_sh = kp_sh; P.kp_st = (int32_t)kp_st;
    P.kn_sb = 2 * kn_sb; P.kn_sh = 2 * kn_sh; P.kn_st = (int32_t)(2 * kn_st);
    P.vp_sb = vp_sb; P.vp_sh = vp_sh; P.vp_st = (int32_t)vp_st;
    P.vn_sb = 2 * vn_sb; P.vn_sh = 2 * vn_sh; P.vn_st = (int32_t)(2 * vn_st);
    P.n_batch = n_batch; P.n_q = n_q; P.n_kv = n_kv; P.gqa = gqa;
    P.t_begin = t_begin; P.t_end = t_end; P.n_splits = n_splits;
    P.scale_log2 = scale * 1.4426950408889634f;
    P.part_o = part_o; P.part_lse = part_lse; P.status = status;
    P.pos_dev = pos_dev; P.pos_add = pos_add;

    // Tiles of 16 warps x 32 tokens, two stages; rows too wide for that (padded strides, the nibble layout with
    // large tables) fall back to 16 tokens per warp.
    int nu = 2;
    size_t smem = 0;
    for (;; --nu) {
        if (nu == 0) return BGTQ_E_TOOBIG;
        const StageLayout sl = stage_layout(kDecWarps * 16u * nu, P.kp_st, P.kn_st, P.vp_st, P.vn_st);
        P.off_kn = sl.off_kn; P.off_v = sl.off_v; P.off_vn = sl.off_vn;
        P.stage_bytes = sl.stage_bytes;
        P.stage_off = kOffStagesMin + P.plan.lut_bytes;
        const uint32_t region = kDecStages * P.stage_bytes > kMergeBytes ? kDecStages * P.stage_bytes : kMergeBytes;
        smem = (size_t)P.stage_off + region;
        if (smem <= 227 * 1024) break;
    }

    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        cudaGetLastError();
        return BGTQ_E_LAUNCH;
    }
    const int64_t max_items = (int64_t)n_batch * n_kv * n_splits;
    // the kernel cuts the item range among its CTAs in 32-bit arithmetic: (CTA index + 1) * items must fit
    if (max_items * ((int64_t)sms + 1) > 0xFFFFFFFFll) return BGTQ_E_TOOBIG;
    dim3 grid((unsigned)(max_items < sms ? max_items : sms));
    const cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool pdl = (P.plan.flags & BGTQ_DEC_PROGRAMMATIC) != 0;
    cudaError_t e;
    // the kernel specialised for this layer's heads, when the plan carries one (it exists for the wide tile only)
    bool jit = P.plan.jit_kernel != nullptr && nu == 2 && !(P.plan.flags & BGTQ_DEC_GENERIC);
    if (jit && P.plan.row_st[0] > 0) {
        // compiled for fixed row strides and for arrays whose every (batch, head) slice and first row start on a
        // 16-byte boundary: any other launch takes the general kernel
        const int32_t* rs = P.plan.row_st;
        auto al16 = [&](const void* p, int64_t sb, int64_t sh, int64_t st) {
            return ((reinterpret_cast<uintptr_t>(p) | (uint64_t)sb | (uint64_t)sh | (uint64_t)((int64_t)t_begin * st)) & 15u) == 0;
        };
        jit = rs[0] == P.kp_st && rs[1] == P.kn_st && rs[2] == P.vp_st && rs[3] == P.vn_st &&
              al16(P.kp, P.kp_sb, P.kp_sh, P.kp_st) && al16(P.kn, P.kn_sb, P.kn_sh, P.kn_st) &&
              al16(P.vp, P.vp_sb, P.vp_sh, P.vp_st) && al16(P.vn, P.vn_sb, P.vn_sh, P.vn_st);
    }
    if (jit) e = launch_decode_jit(P, grid, smem, st, pdl);
    else switch (P.plan.v_sbits) {
        case 1: e = launch_decode_vb1(P, nu, grid, smem, st, pdl); break;
        case 2: e = launch_decode_vb2(P, nu, grid, smem, st, pdl); break;
        case 3: e = launch_decode_vb3(P, nu, grid, smem, st, pdl); break;
        case 4: e = launch_decode_vb4(P, nu, grid, smem, st, pdl); break;
        default: return BGTQ_E_UNSUPPORTED;
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        return BGTQ_E_LAUNCH;
    }
    return BGTQ_OK;
}

extern "C" __attribute__((visibility("default"))) int bgtq_decode(
    const BgtqDecodePlan* plan_host, const BgtqHeadDesc* desc, const void* q_rot, const uint8_t* k_packed,
    int64_t kp_sb, int64_t kp_sh, int64_t kp_st, const void* k_norms, int64_t kn_sb, int64_t kn_sh, int64_t kn_st,
    const uint8_t* v_packed, int64_t vp_sb, int64_t vp_sh, int64_t vp_st, const void* v_norms, int64_t vn_sb,
    int64_t vn_sh, int64_t vn_st, int32_t n_batch, int32_t n_q, int32_t n_kv, int32_t t_begin, int32_t t_end,
    int32_t n_splits, float scale, float* part_o, float* part_lse, int32_t* status, const int32_t* pos_dev,
    int32_t pos_add, void* stream) {
    (void)desc;      // the kernel reads its tables from the plan's image
    return decode_impl(plan_host, q_rot, k_packed, kp_sb, kp_sh, kp_st, k_norms, kn_sb, kn_sh, kn_st, v_packed,
                       vp_sb, vp_sh, vp_st, v_norms, vn_sb, vn_sh, vn_st, n_batch, n_q, n_kv, t_begin, t_end, n_splits,
                       scale, part_o, part_lse, status, pos_dev, pos_add, stream);
}

// ---------------------------------------------------------------------------
// Decode + combine for callers that cannot allocate device memory.
//
// bgtq_decode leaves its per-split partial outputs in a buffer the caller must
// provide.  Some callers have no way to get one: code running inside a CUDA
// graph capture or a stream callback, plugins handed a fixed set of tensors by
// their host framework, and processes whose memory pool is owned by someone
// else.  For them the partials live in the file-scope array below, which every
// GPU that loads this library reserves until the process exits.
// ---------------------------------------------------------------------------
namespace {
constexpr int kNoAllocMaxRows = 8192;    // n_batch * n_q * n_splits
constexpr int kNoAllocMaxDevices = 64;
struct NoAllocScratch {
    float part_o[kNoAllocMaxRows * BGTQ_HEAD_DIM];
    float part_lse[kNoAllocMaxRows];
};
static __device__ __align__(256) NoAllocScratch g_noalloc_scratch;
// Device address of g_noalloc_scratch per device ordinal.  In host code the symbol's name is only a
// handle; the address a kernel can use has to be asked for, with that device current.
NoAllocScratch* g_noalloc_ptr[kNoAllocMaxDevices] = {nullptr};
}  // namespace

extern "C" __attribute__((visibility("default"))) int bgtq_decode_combined_noalloc(
    const BgtqDecodePlan* plan_host, const BgtqHeadDesc* desc, const void* q_rot, const uint8_t* k_packed,
    int64_t kp_sb, int64_t kp_sh, int64_t kp_st, const void* k_norms, int64_t kn_sb, int64_t kn_sh, int64_t kn_st,
    const uint8_t* v_packed, int64_t vp_sb, int64_t vp_sh, int64_t vp_st, const void* v_norms, int64_t vn_sb,
    int64_t vn_sh, int64_t vn_st, int32_t n_batch, int32_t n_q, int32_t n_kv, int32_t t_begin, int32_t t_end,
    int32_t n_splits, float scale, const float* v_rot, void* out, int64_t o_sb, int64_t o_sh, float* lse_out,
    int32_t* status, void* stream) {
    if (n_batch < 1 || n_q < 1 || n_splits < 1 || !out) return BGTQ_E_BADARG;
    if ((int64_t)n_batch * n_q * n_splits > kNoAllocMaxRows) return BGTQ_E_TOOBIG;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices) {
        cudaGetLastError();
        return BGTQ_E_LAUNCH;
    }
    // First call on this device: look the array's device address up once.  The cached pointer is written
    // without host-side ordering; two threads racing here both store the same value, which is harmless.
    if (!g_noalloc_ptr[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || !p) {
            cudaGetLastError();
            return BGTQ_E_LAUNCH;
        }
        g_noalloc_ptr[dev] = static_cast<NoAllocScratch*>(p);
    }
    NoAllocScratch* sc = g_noalloc_ptr[dev];
    // The decode kernel writes the LSE of every slot of every row (-inf for slots that hold no partial) and
    // the combine never reads the output of a slot whose LSE is -inf, so nothing left over from the previous
    // call is ever read and nothing needs clearing.
    const int rc = bgtq_decode(plan_host, desc, q_rot, k_packed, kp_sb, kp_sh, kp_st, k_norms, kn_sb, kn_sh, kn_st,
                               v_packed, vp_sb, vp_sh, vp_st, v_norms, vn_sb, vn_sh, vn_st, n_batch, n_q, n_kv,
                               t_begin, t_end, n_splits, scale, sc->part_o, sc->part_lse, status, nullptr, 0, stream);
    if (rc != BGTQ_OK) return rc;
    return bgtq_combine(sc->part_o, sc->part_lse, n_splits, v_rot, nullptr, nullptr, n_batch, n_q, n_kv, out, o_sb,
                        o_sh, nullptr, lse_out, 0, stream);
}
