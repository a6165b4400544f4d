// Host-computed launch plan of the decode kernel, passed by value in the
// kernel parameters (constant bank), so per-head segment layouts are read with
// uniform loads instead of occupying registers or shared-memory bandwidth.
//
// Code ownership inside a warp: the four lanes of a quad share one token.  For
// a K segment of `len` codes, lane j (0..3) owns the contiguous run of
// q = 2*ceil(len/8) codes starting at code j*q; the run is consumed four codes
// (one m16n8k16 k-tile) at a time, and one unaligned 32-bit shared-memory load
// (a "unit") feeds 32/16/8/8/4 codes for stored widths 1/2/3/4/8 bits.  Codes
// of a lane's run that lie beyond the segment (q rounds up) meet a zero in the
// query fragment, so whatever bits they pick up contribute nothing.
//
// Lookup tables arrive as a prebuilt, lane-replicated image (one per KV head,
// made on the host next to the plan and kept in device memory by the caller);
// a CTA copies its head's image into shared memory with bulk copies.  Each
// table is aligned to its own size inside the image, so the address of an
// entry is (rotate(unit_word, r) & mask) | table_base: the index lands
// pre-scaled by the entry stride and ORs into the base.
//
//   stored width   entry                      index        replicas  bytes
//   1 bit          4 codes -> 2 x fp16x2      4 bits       32        4096
//   2 bits         2 codes -> fp16x2          4 bits       32        2048
//   3 bits         2 codes -> fp16x2          6 bits       32        8192
//   4 bits         2 codes -> fp16x2          8 bits       8 or 16   8192 / 16384
//   8 bits (5..8)  1 code  -> fp16 (twice)    bw bits      32..8     4096/8192
//   V (pair of tokens, one dim) -> fp16x2     2*vb bits    32..8     <= 8192
// (the larger replica count halves the bank conflicts of the 256-entry table; the plan uses it when the
// tables of every head of the layer still leave room for two stages of 512-token tiles.  A quad table for
// 2-bit codes would halve their lookups but, at the 8 replicas that fit, each 64-bit lookup costs twice the
// wavefronts of two conflict-free 32-bit ones.)
#pragma once
#ifndef BGTQ_JIT
#include <stdint.h>
#endif

namespace bgtq {

constexpr int kMaxSteps = 20;        // m16n8k16 k-tiles per token tile and head: sum over segments of ceil(q/4)
constexpr int kMaxPlanHeads = 8;     // KV heads per launch
constexpr uint32_t kLutAlign = 16384; // largest table; the LUT region starts on a multiple of it

// log2 of the replica count per stored width (kind 8: by code width); kind 4 takes one more when it fits
constexpr uint32_t kRep1 = 5, kRep2 = 5, kRep3 = 5, kRep4 = 3;

// One K width segment = one lookup table = one norm group.
struct DecSeg {
    uint8_t kind;        // stored bits per code: 1, 2, 3, 4, or 8 (raw byte, code widths 5..8)
    uint8_t bw;          // codebook width (entries = 2^bw)
    uint8_t q;           // codes per lane (even)
    uint8_t f16_norm;    // 1: fold the norm into each value as fp16(centroid * norm) (nibble-layout numerics)
    uint16_t bit0;       // bit offset of lane 0's run inside a packed row
    uint16_t lane_bits;  // q * stored bits: distance between the runs of neighbouring lanes
    uint32_t tbl;        // byte offset of the table inside the LUT image (a multiple of the table size)
    uint8_t esh;         // log2(bytes between consecutive entries)
    uint8_t rep_log2;    // log2(replicas)
    uint8_t ent_log2;    // log2(entry bytes): 2 or 3
    uint8_t norm_idx;    // which of the token's norms scales this segment
};
static_assert(sizeof(DecSeg) == 16, "DecSeg layout is mirrored by language bindings");

// Query fragment of one k-tile: lane (g, j) holds q[g][pos + j*q .. +1] and q[g][pos + j*q + 2 .. +3].
struct DecStepQ {
    uint8_t pos;   // packed position of lane 0's first code in this k-tile
    uint8_t q;     // codes per lane in the segment
    uint8_t end;   // first packed position past the segment (positions >= end read as zero)
    uint8_t c4;    // offset of the k-tile inside the lane's run (codes c4 .. c4+3; c4 + 2 >= q: second half is zero)
};

struct DecHeadPlan {
    int32_t n_steps;
    int32_t n_seg;
    uint32_t v_tbl;        // byte offset of the V table inside the LUT image
    uint32_t image_bytes;  // bytes of this head's image (multiple of 16)
    DecSeg seg[8];
    DecStepQ steps[kMaxSteps];
};

struct DecPlanDev {
    int32_t n_heads;
    int32_t flags;
    int32_t v_bits;       // codebook width of V
    int32_t v_sbits;      // stored bits per V code
    uint32_t v_rep_log2;
    uint32_t lut_bytes;   // bytes reserved per head in the image and in shared memory (max over heads, multiple of 128)
    const uint8_t* image; // device memory: n_heads images, lut_bytes apart (set with bgtq_decode_plan_set_image)
    const void* jit_kernel;  // host-side handle of the kernel specialised for these heads (bgtq_decode_plan_specialize), or null
    const int32_t* partition;  // device memory: item ranges per CTA (bgtq_decode_partition), or null: equal item counts
    int32_t early_fresh;       // > 0: rows below (live length - early_fresh) and *pos_dev may be read BEFORE the
                               // programmatic dependency wait (bgtq_decode_plan_set_early_fetch); 0: nothing is
    int32_t row_st[4];         // bytes per token of packed K, K norms, packed V, V norms the specialised kernel was
                               // compiled for (bgtq_decode_plan_set_row_strides), or zeros: strides read at run time
    DecHeadPlan head[kMaxPlanHeads];
};

// Layout of one stage (a tile of each of the four arrays) in shared memory: byte offsets of the K norms, packed V
// and V norms behind the packed K, and the stage size.  Each array: one tile of rows + 15 bytes of leading phase
// + rounding + slack for the bit-field over-read.
struct StageLayout {
    uint32_t off_kn, off_v, off_vn, stage_bytes;
};
#ifdef BGTQ_JIT
__device__
#endif
constexpr StageLayout stage_layout(uint32_t tile_tokens, uint32_t kp_st, uint32_t kn_st, uint32_t vp_st, uint32_t vn_st) {
    const uint32_t sz_k = (tile_tokens * kp_st + 48u + 15u) & ~15u, sz_kn = (tile_tokens * kn_st + 48u + 15u) & ~15u;
    const uint32_t sz_v = (tile_tokens * vp_st + 48u + 15u) & ~15u, sz_vn = (tile_tokens * vn_st + 48u + 15u) & ~15u;
    return StageLayout{sz_k, sz_k + sz_kn, sz_k + sz_kn + sz_v, (sz_k + sz_kn + sz_v + sz_vn + 127u) & ~127u};
}

// Item-range table of a launch (bgtq_decode_partition): kPartHeader key words the kernel compares with the
// values it derives itself (items per pair, pairs, CTAs, units per item), then n_cta + 1 item offsets.
constexpr int kPartHeader = 4;
// What starting a run costs a CTA (its prologue and the merge of its warps), in 32-token units of streaming.
constexpr int kRunCostUnits = 16;

}  // namespace bgtq
