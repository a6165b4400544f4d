// Host-computed launch plan of the decode kernel, passed by value in the
// kernel parameters (constant bank), so per-head segment layouts are read with
// uniform loads instead of occupying registers or shared-memory bandwidth.
#pragma once
#include <stdint.h>

namespace bgtq {

constexpr int kMaxSteps = 16;        // k-tiles of 16 packed positions: at most 8 + 7 per head
constexpr int kMaxPlanHeads = 8;     // KV heads per launch
constexpr uint32_t kLutTableBytes = 4096;  // cap per lookup table incl. lane replication

// One lookup table (= one K width segment).
struct DecSegTbl {
    uint16_t word_off;   // first 32-bit word of the table inside the LUT region
    uint16_t cb_off;     // first codebook entry of the segment
    uint8_t sbits;       // stored bits per code (1..4, or 8 for raw bytes)
    uint8_t bw;          // codebook width (entries = 2^bw)
    uint8_t rep_shift;   // log2 of the per-lane replication
    uint8_t pair;        // 1: entry = two codes -> fp16x2, 0: one code -> fp16
    uint32_t n_words;
};

// One m16n8k16 k-tile: 16 consecutive packed positions of one segment.
struct DecStep {
    uint32_t a;  // [15:0] bit offset of the tile inside a packed row, [31:16] table word offset
    uint32_t b;  // [3:0] sbits, [7:4] rep_shift, [8] pair, [9] last tile of segment, [15:12] segment, [31:16] index mask
    uint32_t c;  // [7:0] first packed position, [15:8] valid positions in the tile
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
    uint32_t pad[2];
    DecHeadPlan head[kMaxPlanHeads];
};

}  // namespace bgtq
