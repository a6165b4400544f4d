// Host-computed launch plan of the decode kernel, passed by value in the
// kernel parameters (constant bank), so per-head segment layouts are read with
// uniform loads instead of occupying registers or shared-memory bandwidth.
//
// Code ownership inside a warp: the four lanes of a quad share one token.  For
// a K segment of `len` codes, n_kt = ceil(len/16) MMA k-tiles are issued and
// lane j (0..3) owns the contiguous run of q = 4*n_kt codes starting at code
// j*q, so ONE unaligned 32-bit shared-memory load ("unit") feeds up to eight
// k-tiles of that lane (32/16/8/8/4 codes for stored widths 1/2/3/4/8 bits).
//
// Lookup tables are aligned to their own size inside the LUT region, so the
// address of an entry is (rotate(unit_word, r) & mask) | table_base: the index
// lands pre-scaled by the entry stride and ORs into the base.
#pragma once
#include <stdint.h>

namespace bgtq {

constexpr int kMaxSteps = 16;        // MMA k-tiles per token tile: at most 8 + 7 per head
constexpr int kMaxPlanHeads = 8;     // KV heads per launch
constexpr uint32_t kLutTableBytes = 4096;  // size cap (and alignment) of one lookup table incl. lane replication

// One lookup table (= one K width segment).
struct DecSegTbl {
    uint16_t word_off;   // first 32-bit word of the table inside the (aligned) LUT region
    uint16_t cb_off;     // first codebook entry of the segment
    uint8_t sbits;       // stored bits per code (1..4, or 8 for raw bytes)
    uint8_t bw;          // codebook width (entries = 2^bw)
    uint8_t rep_shift;   // log2 of the per-lane replication
    uint8_t pair;        // 1: entry = two codes -> fp16x2, 0: one code -> fp16
    uint32_t n_words;
    uint8_t n_kt;        // MMA k-tiles of the segment
    uint8_t kt_per_unit; // k-tiles fed by one 32-bit unit load
    uint8_t f16_norm;    // 1: fold the norm into each value as fp16(centroid * norm) (nibble-layout numerics)
    uint8_t pad;
};

// One m16n8k16 k-tile.
struct DecStep {
    uint32_t a;  // [11:0] bit offset of the unit in a packed row (lane 0), [21:12] bits between lanes' runs,
                 // [22] load a new unit, [23] pair table, [24] first k-tile of a segment (fetch its norm)
    uint32_t b;  // [4:0] rotate for the first lookup, [9:5] rotate for the second (pair tables),
                 // [14:10] log2(bytes per table entry incl. replication), [18:15] segment index
    uint32_t c;  // [15:0] index mask already shifted by the entry stride, [31:16] table byte offset
    uint32_t q;  // [7:0] first packed position of lane 0, [13:8] codes per lane in the segment, [21:14] segment end
};

struct DecHeadPlan {
    int32_t n_steps;
    int32_t n_seg;
    uint32_t v_word_off;
    uint32_t pad;
    DecSegTbl seg[8];
    DecStep steps[kMaxSteps];
};

struct DecPlanDev {
    int32_t n_heads;
    int32_t flags;
    int32_t v_bits;       // codebook width of V
    int32_t v_sbits;      // stored bits per V code
    uint32_t v_rep_shift;
    uint32_t v_n_words;
    uint32_t lut_bytes;   // size of the LUT region (max over heads), multiple of 128
    uint32_t pad;
    DecHeadPlan head[kMaxPlanHeads];
};

}  // namespace bgtq
