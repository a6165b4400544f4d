// Launch parameters and helpers shared by the encoder kernels.
#pragma once
#include "bgtq_common.cuh"

namespace bgtq {

struct EncParams {
    const BgtqHeadDesc* desc;
    const float* rot_k;
    const float* rot_v;
    const __half* k;
    const __half* v;
    int64_t k_sb, k_sh, k_ss, v_sb, v_sh, v_ss;
    int32_t n_batch, n_kv, n_tok, t0;
    const int32_t* pos_dev;
    uint8_t* kp; int64_t kp_sb, kp_sh, kp_st; int32_t kp_row_bytes;
    void* kn; int64_t kn_sb, kn_sh, kn_st; int32_t kn_count;
    uint8_t* vp; int64_t vp_sb, vp_sh, vp_st;
    __half* vn; int64_t vn_sb, vn_sh, vn_st;
    uint8_t* k_codes;
    uint8_t* v_codes;
    int32_t flags;
    int32_t capacity;   // token slots per (batch, head) in the destination arrays, 0 = unknown
    int32_t* status;    // optional device word for kStatusOverflow
};

// With a device-side position the host cannot check the destination range: a launch whose rows would land
// outside [0, capacity) stores nothing and reports it.  Uniform over the launch (every thread sees the same slot).
__device__ __forceinline__ bool enc_range_ok(const EncParams& P, int t0, int n_tok) {
    if (P.capacity > 0 && (t0 < 0 || t0 + n_tok > P.capacity)) {
        if (P.status && threadIdx.x == 0) atomicExch(P.status, kStatusOverflow);
        return false;
    }
    return true;
}

// Byte `t` of a bit-packed run: codes of width bw (1..4) starting at codes[0].
__device__ __forceinline__ uint32_t enc_pack_byte(const uint8_t* codes, int n, int bw, int t) {
    const int bit0 = t * 8;
    uint32_t out = 0;
    int i = bit0 / bw;
    for (int pos = i * bw; pos < bit0 + 8; pos += bw, ++i) {
        if (i >= n) break;
        const uint32_t c = codes[i] & ((1u << bw) - 1u);
        const int sh = pos - bit0;
        out |= sh >= 0 ? (c << sh) : (c >> (-sh));
    }
    return out & 0xFFu;
}

// Tensor-core bulk path (bgtq_encode_tc.cu).  Rows must be 16-byte aligned.
int launch_encode_tc(const EncParams& P, cudaStream_t stream);

// tcgen05 bulk path (bgtq_encode_t5w.cu): same requirements, n_tok >= 16, and packed K rows of at most
// encode_t5w_max_row_bytes() bytes.
int launch_encode_t5w(const EncParams& P, cudaStream_t stream);
int encode_t5w_max_row_bytes();

}  // namespace bgtq
