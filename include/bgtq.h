/*
 * bgtq.h -- C ABI of the B200 (sm_100a) packed-KV-cache kernels for Block-GTQ.
 *
 * The library replaces the GPU side of the reference's packed-cache decode
 * path (all of which is Triton there).  Each entry point cites the reference
 * operator it stands in for, by the file's path inside the reference project.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless the comment says "host";
 *   - the caller owns all memory; no entry point allocates, frees or
 *     synchronises (bgtq_*_noalloc: see its own comment);
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*);
 *   - return value: BGTQ_OK or a negative BGTQ_E_* code; nothing throws;
 *   - strides are in ELEMENTS of the pointed-to type unless stated in bytes;
 *   - head_dim is fixed at 128 (every configuration of the reference's
 *     benchmarks); other sizes return BGTQ_E_UNSUPPORTED.
 */
#ifndef BGTQ_H_
#define BGTQ_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BGTQ_ABI_VERSION 1
#define BGTQ_HEAD_DIM 128
#define BGTQ_MAX_SEGMENTS 8
#define BGTQ_N_BINS 256

#define BGTQ_OK 0
#define BGTQ_E_BADARG (-1)
#define BGTQ_E_UNSUPPORTED (-2)
#define BGTQ_E_ALIGN (-3)
#define BGTQ_E_LAUNCH (-4)
#define BGTQ_E_TOOBIG (-5)

/* Static tables of one (layer, KV head).  The host fills an array of these
 * (one per KV head of a layer) and uploads it; kernels index it by KV head.
 * Source of every field: BlockGTQQuantizer.calibrate / build_kernel_args /
 * init_v_quantizer and build_batched_encode_args
 * (blockgtq/quantizer.py:1024-1148, 1478-1497, 1598-1747).
 *
 * "packed position" p = index of a dim after head_perm (dims sorted by bit
 * width); segment s = run of packed positions sharing one width = one norm
 * group = one codebook. */
typedef struct BgtqHeadDesc {
    int32_t n_seg;                 /* 1..8 */
    int32_t k_row_bytes;           /* live packed K bytes per token (bit-packed layout) */
    int32_t v_bits;                /* 1..4 */
    int32_t v_row_bytes;           /* packed V bytes per token */
    int32_t nopack_start;          /* first packed position held as a raw byte (128 if none) */
    int32_t nopack_len;
    int32_t k_mixed_bytes;         /* nopack_start/2 + nopack_len (nibble/raw layout) */
    int32_t reserved0;
    int32_t seg_bw[BGTQ_MAX_SEGMENTS];        /* code width 1..8 */
    int32_t seg_start[BGTQ_MAX_SEGMENTS];     /* first packed position */
    int32_t seg_len[BGTQ_MAX_SEGMENTS];       /* number of positions (even) */
    int32_t seg_pack_off[BGTQ_MAX_SEGMENTS];  /* byte offset inside a packed K row */
    int32_t seg_lut_off[BGTQ_MAX_SEGMENTS];   /* offset into codebook[] / k_cents[] */
    float lut_off[BGTQ_MAX_SEGMENTS];         /* bin = (y - lut_off) * lut_inv, clamp 0..255 */
    float lut_inv[BGTQ_MAX_SEGMENTS];
    float v_cents[16];
    float v_bounds[16];            /* 2^v_bits - 1 used; rest +inf */
    uint16_t v_lut[16];            /* fp16 bit patterns of v_cents */
    uint16_t codebook[512];        /* fp16 bit patterns, segment s at seg_lut_off[s] */
    float k_cents[512];            /* same entries in fp32 (norm correction) */
    uint8_t head_perm[BGTQ_HEAD_DIM];         /* packed position -> original dim */
    uint8_t group_of[BGTQ_HEAD_DIM];          /* packed position -> segment index */
    uint8_t code_lut[BGTQ_MAX_SEGMENTS][BGTQ_N_BINS];
} BgtqHeadDesc;

/* Build-time identity checks for language bindings. */
int bgtq_abi_version(void);
int bgtq_desc_size(void);                      /* sizeof(BgtqHeadDesc) */
const char* bgtq_error_string(int code);       /* host pointer to a static string */

/* ---- encoder flags ------------------------------------------------------- */
#define BGTQ_ENC_K_NORMS_F16 1    /* write K norms as fp16 (cache) instead of fp32 (operator API) */
#define BGTQ_ENC_K_MIXED 2        /* K rows in the nibble/raw "mixed" layout + corrected norms */
#define BGTQ_ENC_V_NIBBLE 4       /* V rows as 4-bit nibbles regardless of v_bits */
#define BGTQ_ENC_SKIP_K 8
#define BGTQ_ENC_SKIP_V 16
#define BGTQ_ENC_FORCE_SIMT 32  /* always use the small-batch fp32 kernel (>= 64 rows normally use tensor cores) */
#define BGTQ_ENC_PROGRAMMATIC 64  /* bgtq_step_prepare only: programmatic dependent launch, see below */
#define BGTQ_ENC_NO_TCGEN05 128   /* bulk encode: keep the rotation on mma.sync (bulk row counts of >= 128 rows and packed
                                   * K rows of <= 120 bytes normally use tcgen05.mma with tensor-memory accumulators) */

/* Programmatic dependent launch (BGTQ_ENC_PROGRAMMATIC, BGTQ_DEC_PROGRAMMATIC,
 * BGTQ_COMBINE_PROGRAMMATIC).  The kernel is launched with CUDA's programmatic
 * stream-serialization attribute: its blocks may become resident while the
 * preceding kernel of the stream is still running, set up their static tables,
 * and wait on the device for that kernel to complete before they touch any
 * per-call input or output.  Results are identical; the launch latency and the
 * set-up of each kernel of a decode step overlap the previous kernel's tail.
 * Safe after any kind of preceding work; capturable in a CUDA graph. */

/* Encode K and V rows of all KV heads of one layer and write them straight
 * into their cache slots.
 *
 * Replaces compress_k_packed_batched / compress_v_packed_batched
 * (blockgtq/quantizer.py:2104-2172, 1979-2029; kernels :712-990, :517-706),
 * their "mixed"/"nibble" variants (:1843-1976, :2032-2101), the unpacked-code
 * output of BlockGTQQuantizer.compress (blockgtq/kernels/quant_kernels.py:470-565)
 * and the strided cache writes of BlockGTQKVManager._encode_kv
 * (blockgtq/packed_kv_manager.py:176-180).
 *
 * Rows form a (n_batch, n_kv, n_tok) grid.  Input element (b,h,s,d) is at
 * k + b*k_sb + h*k_sh + s*k_ss + d (same for v).  Output row (b,h,s) lands at
 * token slot t0+s: k_packed + b*kp_sb + h*kp_sh + (t0+s)*kp_st bytes, etc.
 * Each packed K row is written for kp_row_bytes bytes (bytes past the head's
 * live size are zero); K norms are written for kn_count groups (groups the
 * head does not have are zero).
 *
 * rot_k / rot_v: (n_kv, 128, 128) fp32.  rot_k[h][j][p] = block_rot_T (row j =
 * packed input position, column p = packed output position); rot_v[h][i][j] =
 * R^T so that y = v_unit @ rot_v[h].
 * k_codes / v_codes: optional (may be NULL) outputs of the unpacked indices,
 * (n_batch, n_kv, n_tok, 128) contiguous uint8, K in packed-position order.
 * pos_dev: optional device int32; when non-NULL the first destination slot is
 * *pos_dev instead of t0, read when the kernel runs (lets a captured CUDA graph
 * append at a position that advances between replays).
 * t_capacity: token slots every (b,h) has in the destination arrays (0 = not
 * checked).  With t0 given on the host a range that leaves it is refused with
 * BGTQ_E_BADARG; with pos_dev the kernel checks: a launch whose rows would land
 * outside [0, t_capacity) stores NOTHING and sets *status (optional device
 * int32) to 2, so a step replayed past the end of the cache cannot overwrite
 * its neighbours.
 */
int bgtq_encode(const BgtqHeadDesc* desc, const float* rot_k, const float* rot_v,
                const void* k, int64_t k_sb, int64_t k_sh, int64_t k_ss,
                const void* v, int64_t v_sb, int64_t v_sh, int64_t v_ss,
                int32_t n_batch, int32_t n_kv, int32_t n_tok, int32_t t0,
                uint8_t* k_packed, int64_t kp_sb, int64_t kp_sh, int64_t kp_st, int32_t kp_row_bytes,
                void* k_norms, int64_t kn_sb, int64_t kn_sh, int64_t kn_st, int32_t kn_count,
                uint8_t* v_packed, int64_t vp_sb, int64_t vp_sh, int64_t vp_st,
                void* v_norms, int64_t vn_sb, int64_t vn_sh, int64_t vn_st,
                uint8_t* k_codes, uint8_t* v_codes,
                int32_t flags, const int32_t* pos_dev, int32_t t_capacity, int32_t* status, void* stream);

/* Sticky device-side status of the tcgen05 bulk encoder on the current device: 0, or 1 after a wait for
 * the tensor cores ran out (the rows of that launch are then incomplete).  Synchronises the device. */
int bgtq_encode_tcgen05_status(void);

/* Rotate decode queries into the packed-K basis:
 * q_rot[b, hq, p] = fp16( sum_j fp32(q[b, hq, head_perm[j]]) * rot_k[h][j][p] ),
 * h = hq / (n_q / n_kv).
 * Replaces BlockGTQQuantizer.rotate_q_for_packed_kernel
 * (blockgtq/quantizer.py:1160-1187) for all heads of a layer in one launch.
 * q element (b,hq,d) at q + b*q_sb + hq*q_sh + d; q_rot is (n_batch, n_q, 128)
 * contiguous fp16. */
int bgtq_rotate_q(const BgtqHeadDesc* desc, const float* rot_k,
                  const void* q, int64_t q_sb, int64_t q_sh,
                  void* q_rot, int32_t n_batch, int32_t n_q, int32_t n_kv, void* stream);

/* One decode step's preparation in a single latency-oriented launch: the query
 * rotation of bgtq_rotate_q and the append of ONE new token per (batch, KV head)
 * of bgtq_encode (same arguments, n_tok = 1, no code outputs).  q / q_rot may be
 * NULL to skip the rotation (queries baked into q_proj).  Replaces, per layer
 * and step, the n_kv rotate_q_for_packed_kernel calls and the CUDA-graphed T=1
 * encode of the reference (blockgtq/packed_kv_manager.py:221-257, 318-329).
 * The rotation sums are formed in a different order than in bgtq_encode, so a
 * coordinate sitting exactly on a bin edge may land on the neighbouring code.
 * t_capacity / status: as for bgtq_encode (the query rotation still runs when
 * the append is refused). */
int bgtq_step_prepare(const BgtqHeadDesc* desc, const float* rot_k, const float* rot_v,
                      const void* q, int64_t q_sb, int64_t q_sh, void* q_rot, int32_t n_q,
                      const void* k, int64_t k_sb, int64_t k_sh,
                      const void* v, int64_t v_sb, int64_t v_sh,
                      int32_t n_batch, int32_t n_kv, int32_t t0,
                      uint8_t* k_packed, int64_t kp_sb, int64_t kp_sh, int64_t kp_st, int32_t kp_row_bytes,
                      void* k_norms, int64_t kn_sb, int64_t kn_sh, int64_t kn_st, int32_t kn_count,
                      uint8_t* v_packed, int64_t vp_sb, int64_t vp_sh, int64_t vp_st,
                      void* v_norms, int64_t vn_sb, int64_t vn_sh, int64_t vn_st,
                      int32_t flags, const int32_t* pos_dev, int32_t t_capacity, int32_t* status, void* stream);

/* bgtq_step_prepare for queries and keys that have NOT been through the rotary embedding yet: the kernel
 * applies it first, x' = x*cos + rotate_half(x)*sin in the split-half convention (dims d and d+64 form a
 * pair), with fp16 tables of the step's position, rope_cos / rope_sin: (n_batch, 128) fp16, row b at
 * + b*rope_sb.  Rounding is that of the fp16 expression evaluated by the reference's caller
 * (transformers' apply_rotary_pos_emb, called in blockgtq/production_decode.py:37-39 and
 * blockgtq/packed_kv_manager.py:429-431): two rounded products and one rounded sum, so codes and q_rot are
 * bit-identical to rotating first and calling bgtq_step_prepare.  V is not rotated. */
int bgtq_step_prepare_rope(const BgtqHeadDesc* desc, const float* rot_k, const float* rot_v,
                      const void* q, int64_t q_sb, int64_t q_sh, void* q_rot, int32_t n_q,
                      const void* k, int64_t k_sb, int64_t k_sh,
                      const void* v, int64_t v_sb, int64_t v_sh,
                      int32_t n_batch, int32_t n_kv, int32_t t0,
                      uint8_t* k_packed, int64_t kp_sb, int64_t kp_sh, int64_t kp_st, int32_t kp_row_bytes,
                      void* k_norms, int64_t kn_sb, int64_t kn_sh, int64_t kn_st, int32_t kn_count,
                      uint8_t* v_packed, int64_t vp_sb, int64_t vp_sh, int64_t vp_st,
                      void* v_norms, int64_t vn_sb, int64_t vn_sh, int64_t vn_st,
                      int32_t flags, const int32_t* pos_dev, int32_t t_capacity, int32_t* status,
                      const void* rope_cos, const void* rope_sin, int64_t rope_sb, void* stream);

/* bgtq_step_prepare for the three-region cache policy (fp16 sink + packed middle + fp16 recent window,
 * blockgtq/unaccelerated.py:163-244) with one-token blocks, everything derived from the device-side token
 * count so that the step can be captured in a CUDA graph: with t = *pos_dev tokens before the step, the new
 * token's k / v are copied into their slot of the fp16 buffers k_buf / v_buf (slot t while t < n_sink, else
 * n_sink + (t - n_sink) % (window + 1); slot j of (b,h) at buf + b*kb_sb + h*kb_sh + j*128), and the token
 * that thereby leaves the recent window (non-sink index f = t - n_sink - window, if >= 0) is read from its
 * ring slot, encoded and written to packed row f.  Queries are rotated as usual. */
int bgtq_step_prepare_ring(const BgtqHeadDesc* desc, const float* rot_k, const float* rot_v,
                      const void* q, int64_t q_sb, int64_t q_sh, void* q_rot, int32_t n_q,
                      const void* k, int64_t k_sb, int64_t k_sh,
                      const void* v, int64_t v_sb, int64_t v_sh,
                      int32_t n_batch, int32_t n_kv, int32_t t0,
                      uint8_t* k_packed, int64_t kp_sb, int64_t kp_sh, int64_t kp_st, int32_t kp_row_bytes,
                      void* k_norms, int64_t kn_sb, int64_t kn_sh, int64_t kn_st, int32_t kn_count,
                      uint8_t* v_packed, int64_t vp_sb, int64_t vp_sh, int64_t vp_st,
                      void* v_norms, int64_t vn_sb, int64_t vn_sh, int64_t vn_st,
                      int32_t flags, const int32_t* pos_dev, int32_t t_capacity, int32_t* status,
                      void* k_buf, void* v_buf, int64_t kb_sb, int64_t kb_sh, int32_t n_sink, int32_t window,
                      void* stream);

/* ---- decode --------------------------------------------------------------- */
#define BGTQ_DEC_K_MIXED 1        /* k_packed rows are in the nibble/raw mixed layout */
#define BGTQ_DEC_V_NIBBLE 2       /* v_packed rows are 4-bit nibbles */
#define BGTQ_DEC_PROGRAMMATIC 4   /* launch bgtq_decode as a programmatic dependent of the preceding kernel */
#define BGTQ_DEC_GENERIC 8        /* always launch the general kernel, even if the plan holds a specialised one */

/* Opaque launch plan of the decode kernel for the KV heads of one layer (host
 * memory, plain bytes, copyable).  Built once per layer from the HOST copy of
 * the head descriptors; at most 8 KV heads per plan (split wider layers into
 * groups of heads).  The reference specialises its decode kernel per head with
 * Triton constexprs (blockgtq/production_cache.py:19-22); here the per-head
 * layout travels in the plan and in a prebuilt lookup-table image.
 *
 * The kernel reads its lookup tables (codebooks expanded into lane-replicated
 * fp16x2 tables, one set per KV head) from an image in DEVICE memory that the
 * caller owns: ask for its size, let the library fill a host buffer, copy that
 * buffer to the device (16-byte aligned) and record the device address in the
 * plan.  The image must stay valid while launches that use the plan run. */
typedef struct BgtqDecodePlan {
    uint8_t opaque[4096];
} BgtqDecodePlan;
int bgtq_decode_plan(const BgtqHeadDesc* desc_host, int32_t n_kv, int32_t flags, BgtqDecodePlan* plan_host);
int64_t bgtq_decode_image_bytes(const BgtqDecodePlan* plan_host);            /* > 0, or a negative error code */
int bgtq_decode_build_image(const BgtqDecodePlan* plan_host, const BgtqHeadDesc* desc_host,
                            uint8_t* image_host, int64_t bytes);             /* host buffers only */
int bgtq_decode_plan_set_image(BgtqDecodePlan* plan_host, const uint8_t* image_dev);

/* Specialise the decode kernel for the heads of this plan: the kernel's source is compiled at run time
 * (NVRTC, found with dlopen; bgtq_jit_set_nvrtc_path or the environment variable BGTQ_NVRTC name it
 * explicitly) with every head's segment layout as compile-time constants, the way the reference
 * specialises its Triton kernel per head (blockgtq/production_cache.py:19-22), and the resulting kernel is
 * recorded in the plan; bgtq_decode then launches it instead of the general kernel (same arguments, same
 * results).  Takes a second or two per distinct layer layout; layouts are cached per process.  Call it
 * once at set-up, outside any stream capture.  compile_only != 0 stops after the compilation (no GPU
 * needed; nothing is recorded).  log (host, may be NULL) receives the compiler's messages.
 * Returns BGTQ_E_UNSUPPORTED when NVRTC cannot be found (the plan stays usable with the general kernel),
 * BGTQ_E_LAUNCH when compiling or loading fails. */
int bgtq_decode_plan_specialize(BgtqDecodePlan* plan_host, int32_t compile_only, char* log, int64_t log_bytes);
/* Before bgtq_decode_plan_specialize: also fix the cache row strides the specialised kernel is compiled for
 * (kp_st, vp_st in bytes, kn_st, vn_st in fp16 elements, as bgtq_decode takes them), so that row offsets fold
 * into its load instructions.  bgtq_decode then launches that kernel only for calls with exactly these row
 * strides whose four arrays, batch strides, head strides and first row (t_begin) all sit on 16-byte
 * boundaries, and the general kernel for any other call.  All zeros: strides stay launch parameters (default). */
int bgtq_decode_plan_set_row_strides(BgtqDecodePlan* plan_host, int32_t kp_st, int32_t kn_st, int32_t vp_st,
                                     int32_t vn_st);
int bgtq_jit_set_nvrtc_path(const char* path_host);

/* Optional, for launches with BGTQ_DEC_PROGRAMMATIC: let the kernel start streaming the cache before its
 * programmatic-dependency wait.  fresh_rows > 0 promises that, when the launch that PRECEDES the decode in the
 * stream starts, (1) the value at pos_dev is final and (2) every cache row below (live length - fresh_rows) is
 * final: the preceding launch writes nothing but the newest fresh_rows rows (the step's append), the query and
 * buffers the decode does not read.  The kernel then reads pos_dev, cuts its ranges and requests its first tiles
 * right away (tiles that reach into the fresh rows are held back), and only waits before it reads the query and
 * before it writes anything.  0 (default): everything waits.  No counterpart in the reference. */
int bgtq_decode_plan_set_early_fetch(BgtqDecodePlan* plan_host, int32_t fresh_rows);

/* Optional item-range table of a launch.  bgtq_decode cuts every (batch, KV head) pair into items and hands
 * each of its CTAs a contiguous range of them; by default every CTA gets the same number.  A CTA whose range
 * straddles two pairs merges its warps and writes a partial twice, so it finishes later than the others:
 * bgtq_decode_partition fills a table (host memory, table_len >= n_cta + 5 words) that gives such CTAs fewer
 * items.  n_cta = bgtq_decode_grid_size(...) for the same shape and n_splits.  The caller copies the table
 * to device memory (4-byte aligned) and records the address with bgtq_decode_plan_set_partition (NULL takes it
 * out again); the kernel uses it only when its first four words match the launch (same number of live items
 * per pair, pairs, CTAs and item size) and falls back to equal counts otherwise, so a stale table costs
 * balance, never correctness.  The kernel reads the table before its programmatic-dependency wait: write it with a
 * copy that is ordered before the launch that precedes the decode, not by that launch.  The table depends on the shape and on the token count through
 * ceil(tokens / 32) only; the reference has no counterpart (its kernel takes one program per split). */
int bgtq_decode_grid_size(int32_t n_batch, int32_t n_kv, int32_t n_splits);
int bgtq_decode_partition(int32_t n_batch, int32_t n_kv, int32_t n_tokens, int32_t n_splits, int32_t n_cta,
                          int32_t* table_host, int32_t table_len);
int bgtq_decode_plan_set_partition(BgtqDecodePlan* plan_host, const int32_t* partition_dev);

/* Number of partial slots per (batch, KV head) pair the library suggests for a
 * (batch, heads, tokens) shape on the current device (host helper, no GPU work):
 * fine enough that every SM gets the same number of token tiles. */
int bgtq_decode_default_splits(int32_t n_batch, int32_t n_kv, int32_t n_tokens);

/* Fused unpack + dequantise + split-KV attention of one decode query per
 * (batch, query head) over cache tokens [t_begin, t_end).
 *
 * Replaces fused_blockgtq_decode_attention's first phase, _packed_decode_kernel
 * (blockgtq/kernels/fused_packed_attention.py:152-894, wrapper :1541-1843), for
 * every KV head of a layer in ONE launch (the reference launches per head).
 *
 * plan_host: from bgtq_decode_plan, with its image set (host memory); desc is
 * unused (the tables come from the image) and may be NULL.  q_rot: (n_batch,
 * n_q, 128) fp16 contiguous, already in the packed-K basis; n_q / n_kv <= 8.
 * Cache row (b,h,t): k_packed + b*kp_sb + h*kp_sh + t*kp_st  (bytes; rows of one
 * (b,h) must be equally spaced), k_norms fp16 at + b*kn_sb + h*kn_sh + t*kn_st
 * (+ segment index), v_packed / v_norms likewise (v_norms: one fp16 per token).
 * Rows need no particular alignment, but tiles are fetched with 16-byte-aligned
 * bulk copies: up to 15 bytes before the first and after the last row of the
 * token range of every (b,h) are READ (never used), so each of the four arrays
 * must have that much addressable memory on either side of a pair's rows (any
 * allocation whose rows do not start or end exactly on its first / last 16-byte
 * boundary qualifies; a cache tensor with a few spare token rows always does).
 *
 * Work split and outputs.  The live tokens of every pair are cut into n_splits
 * equal items of whole 32-token units; each CTA (one per SM) takes a contiguous
 * range of items, and consecutive items of one pair inside a CTA produce ONE
 * partial, stored in the slot of the first of them:
 *   part_o  (n_batch, n_q, n_splits, 128) fp32  softmax-normalised partial
 *           output, still in V's rotated basis (8-byte aligned)
 *   part_lse(n_batch, n_q, n_splits)      fp32  log-sum-exp of the scaled
 *           logits of the partial; -inf for a slot that holds no partial (its
 *           part_o row is then NOT written and must not be read).
 * Every part_lse element is written by every launch.
 * status: optional int32 on the device; set to a non-zero code if a bounded
 * wait inside the kernel gave up (the output is then invalid).
 * pos_dev / pos_add: optional device int32; when non-NULL the range ends at
 * min(t_end, *pos_dev + pos_add), read when the kernel runs (after the
 * programmatic dependency wait), and the items are cut from that live length:
 * t_end then only bounds the range (graph replay). */
int bgtq_decode(const BgtqDecodePlan* plan_host, const BgtqHeadDesc* desc, const void* q_rot,
                const uint8_t* k_packed, int64_t kp_sb, int64_t kp_sh, int64_t kp_st,
                const void* k_norms, int64_t kn_sb, int64_t kn_sh, int64_t kn_st,
                const uint8_t* v_packed, int64_t vp_sb, int64_t vp_sh, int64_t vp_st,
                const void* v_norms, int64_t vn_sb, int64_t vn_sh, int64_t vn_st,
                int32_t n_batch, int32_t n_q, int32_t n_kv,
                int32_t t_begin, int32_t t_end, int32_t n_splits, float scale,
                float* part_o, float* part_lse, int32_t* status,
                const int32_t* pos_dev, int32_t pos_add, void* stream);

/* Attention of the same queries over tokens kept unquantised in fp16 (the
 * sink prefix and the recent window of the three-region cache policy,
 * blockgtq/unaccelerated.py:163-244; the reference has no packed-path kernel
 * for it).  q is the ORIGINAL query (no permutation/rotation), element
 * (b,hq,d) at q + b*q_sb + hq*q_sh + d.  Buffer slot j of (b,h) is at
 * k_buf + b*kb_sb + h*kb_sh + j*128 (fp16).  Slots [0, n_sink_tokens) hold the
 * sink; the recent tokens sit in a ring of ring_size slots that starts at slot
 * sink_cap: recent token i is in slot sink_cap + (ring_first + i) % ring_size,
 * i < n_ring_tokens.
 * Writes one more partial per (b,hq): buf_o (n_batch, n_q, 128) fp32 in the
 * ORIGINAL V basis, buf_lse (n_batch, n_q) fp32 (-inf when there are no tokens).
 * k_buf / v_buf must be 16-byte aligned with kb_sb, kb_sh multiples of 8 elements, buf_o 8-byte aligned
 * (BGTQ_E_ALIGN otherwise). */
int bgtq_buffer_attn(const void* q, int64_t q_sb, int64_t q_sh,
                     const void* k_buf, const void* v_buf, int64_t kb_sb, int64_t kb_sh,
                     int32_t n_sink_tokens, int32_t n_ring_tokens, int32_t sink_cap,
                     int32_t ring_first, int32_t ring_size,
                     int32_t n_batch, int32_t n_q, int32_t n_kv,
                     float scale, float* buf_o, float* buf_lse, void* stream);

/* bgtq_buffer_attn with the region sizes taken from a device-side token count, for captured graphs: with
 * pos_dev non-NULL, *pos_dev + 1 tokens exist (the step's token included), the three-region policy with
 * one-token blocks and a recent window of ring_size - 1 applies (n_sink_tokens / n_ring_tokens / ring_first
 * are computed in the kernel and the three arguments are ignored). */
int bgtq_buffer_attn_pos(const void* q, int64_t q_sb, int64_t q_sh,
                     const void* k_buf, const void* v_buf, int64_t kb_sb, int64_t kb_sh,
                     int32_t n_sink_tokens, int32_t n_ring_tokens, int32_t sink_cap,
                     int32_t ring_first, int32_t ring_size,
                     int32_t n_batch, int32_t n_q, int32_t n_kv,
                     float scale, float* buf_o, float* buf_lse, const int32_t* pos_dev, void* stream);

/* Merge split partials, undo V's rotation, fold in the fp16-buffer partial.
 *
 * Replaces _split_t_merge_kernel (blockgtq/kernels/fused_packed_attention.py:59-103),
 * the per-split V un-rotation (:875-882) and the return_lse log-sum-exp
 * (:1856-1860).  Splits with lse = -inf are skipped; a row whose every partial
 * is empty yields zeros and lse = -inf.
 *   merged_rot = sum_c a_c part_o[c] / sum_c a_c           (a_c = exp(lse_c - max))
 *   packed_out = merged_rot @ v_rot[h]   if v_rot != NULL  (v_rot: (n_kv,128,128) fp32 = R)
 *   out        = LSE-weighted mix of packed_out and buf_o  (buf_o may be NULL)
 * out: fp16 (n_batch, n_q, 128) at out + b*o_sb + hq*o_sh; out_f32 / lse_out
 * optional: the un-rounded result (n_batch, n_q, 128) and total LSE (n_batch, n_q),
 * the pair another rank needs to continue the merge.
 * flags: 0 or BGTQ_COMBINE_PROGRAMMATIC. */
#define BGTQ_COMBINE_PROGRAMMATIC 1
int bgtq_combine(const float* part_o, const float* part_lse, int32_t n_splits,
                 const float* v_rot, const float* buf_o, const float* buf_lse,
                 int32_t n_batch, int32_t n_q, int32_t n_kv,
                 void* out, int64_t o_sb, int64_t o_sh,
                 float* out_f32, float* lse_out, int32_t flags, void* stream);

/* Prefill attention: s_q query positions per (batch, query head) against the packed cache, causal.
 *
 * Replaces _packed_prefill_kernel / fused_blockgtq_prefill_attention
 * (blockgtq/kernels/fused_packed_attention.py:1875-2760) for every KV head of a layer in one launch; the
 * caller is layer_major_prefill (blockgtq/prefill.py:25-125).
 * Query i of (b, hq) sits at q_rot + b*q_sb + hq*q_sh + i*q_ss (fp16, 128 contiguous dims, already in the
 * packed-K basis like bgtq_decode's q_rot) and has absolute position q_pos_offset + i; with causal != 0 it
 * attends cache tokens t <= q_pos_offset + i, t < n_tokens, else all n_tokens.  Cache arguments and
 * flags (BGTQ_DEC_K_MIXED, BGTQ_DEC_V_NIBBLE) are as for bgtq_decode.
 * out_rot: (n_batch, n_q, s_q, 128) fp32 contiguous, softmax-normalised and still in V's rotated basis:
 * multiply each KV head's rows by its R (one plain GEMM) to finish.  A query with no visible token
 * yields zeros.  n_q / n_kv <= 16.
 * Two kernels: the products run on tcgen05 with accumulators in tensor memory when n_q / n_kv divides 128
 * (bgtq_prefill_t5.cu), else, or with BGTQ_PF_NO_TCGEN05 in flags, on mma.sync (bgtq_prefill.cu).  The tcgen05
 * kernel bounds its waits; bgtq_prefill_tcgen05_status() returns 1 (sticky, per process) if one ever gave up,
 * in which case that launch's output is invalid. */
#define BGTQ_PF_NO_TCGEN05 16
int bgtq_prefill_tcgen05_status(void);
int bgtq_prefill_attention(const BgtqHeadDesc* desc, const void* q_rot, int64_t q_sb, int64_t q_sh, int64_t q_ss,
                const uint8_t* k_packed, int64_t kp_sb, int64_t kp_sh, int64_t kp_st,
                const void* k_norms, int64_t kn_sb, int64_t kn_sh, int64_t kn_st,
                const uint8_t* v_packed, int64_t vp_sb, int64_t vp_sh, int64_t vp_st,
                const void* v_norms, int64_t vn_sb, int64_t vn_sh, int64_t vn_st,
                int32_t n_batch, int32_t n_q, int32_t n_kv, int32_t s_q, int32_t n_tokens,
                int32_t q_pos_offset, int32_t causal, float scale, int32_t flags,
                float* out_rot, void* stream);

/* Final merge of per-rank results after an all-gather (sequence-sharded cache: every rank ran
 * bgtq_decode + bgtq_combine over its own token chunk with out_f32 / lse_out pointing into one message
 * [O (n_batch, n_q, 128) fp32 | LSE (n_batch, n_q) fp32]; the messages of all ranks were gathered into
 * `gathered`, rank r's message starting at gathered + r * rank_stride floats).  The reference is
 * single-GPU; the merge itself is _split_t_merge_kernel (blockgtq/kernels/fused_packed_attention.py:59-103)
 * applied across ranks.  The partials are already in V's original basis, so no rotation is applied.
 * Ranks with LSE = -inf (no tokens) are skipped.  out: fp16 (n_batch, n_q, 128) at out + b*o_sb + hq*o_sh.
 * Only local memory is read: pass the all-gather's receive buffer, never a peer pointer. */
int bgtq_combine_ranks(const float* gathered, int32_t n_ranks, int64_t rank_stride,
                       int32_t n_batch, int32_t n_q, void* out, int64_t o_sb, int64_t o_sh,
                       int32_t flags, void* stream);

/* Exchange of the per-rank [O | LSE] messages of a sequence-sharded cache over PEER MEMORY (NVLink loads
 * and stores between the GPUs of one node) instead of a library all-gather; no counterpart in the
 * single-GPU reference.  Every rank owns an exchange buffer [2 parities][n_ranks][rank_stride] fp32
 * (parity_stride floats between the two halves) and n_ranks int32 flags (initially 0), both mapped into
 * every peer, plus a private step counter seq_dev (int32, initially 0) and two private int32 tickets
 * (initially 0).  Per step, on every rank, in stream order:
 *   bgtq_exchange_publish: copies the local message (n_floats, a multiple of 4) into slot
 *     [seq & 1][rank] of every rank's buffer (peer_bufs: device array of n_ranks buffer base pointers,
 *     slot_off = rank * rank_stride) and then stores seq + 1 into flag[rank] of every rank (peer_flags:
 *     device array of n_ranks flag-array pointers);
 *   bgtq_exchange_merge: waits until all n_ranks local flags reach seq + 1 (bounded: after about 0.3 s
 *     it sets *status = 3 and writes zeros instead of hanging), merges the messages like
 *     bgtq_combine_ranks from the LOCAL buffer, writes fp16 out and advances *seq_dev.
 * Only plain loads/stores and system-scope fences are used (no multicast).  All ranks must run the same
 * sequence of steps; each rank's kernels run on its own GPU. */
/* bgtq_combine with bgtq_exchange_publish folded into its last step: each (batch, query head) row's fp32
 * result and LSE are stored straight into this rank's slot [*seq_dev & 1][rank] of every rank's exchange
 * buffer, and the last block raises this rank's flag on every rank -- a sequence-sharded layer step is then
 * decode -> combine+publish -> merge.  Arguments as for bgtq_combine (no fp16-buffer partial, no local
 * output) and bgtq_exchange_publish (rank_stride of the buffers = n_batch * n_q * 129 floats or more). */
int bgtq_combine_publish(const float* part_o, const float* part_lse, int32_t n_splits, const float* v_rot,
                         int32_t n_batch, int32_t n_q, int32_t n_kv,
                         float* const* peer_bufs, int64_t slot_off, int64_t parity_stride,
                         int32_t* const* peer_flags, int32_t rank, int32_t n_ranks,
                         const int32_t* seq_dev, int32_t* ticket, int32_t flags, void* stream);
int bgtq_exchange_publish(const float* msg, int64_t n_floats, float* const* peer_bufs, int64_t slot_off,
                          int64_t parity_stride, int32_t* const* peer_flags, int32_t rank, int32_t n_ranks,
                          const int32_t* seq_dev, int32_t* ticket, void* stream);
int bgtq_exchange_merge(const float* local_buf, int32_t n_ranks, int64_t rank_stride, int64_t parity_stride,
                        const int32_t* flags, int32_t* seq_dev, int32_t n_batch, int32_t n_q,
                        void* out, int64_t o_sb, int64_t o_sh, int32_t* status, int32_t* ticket, void* stream);

/* bgtq_decode followed by bgtq_combine with NO caller-provided scratch: the
 * split partials go to a fixed array inside the library instead of part_o /
 * part_lse.  This entry point has no counterpart in the reference.
 *
 * It exists for callers that cannot allocate device memory at the point of the
 * call: code being captured into or replayed from a stream-ordered sequence that
 * forbids allocation, plugins that only receive the tensors their host
 * framework hands them, and processes whose device memory is owned by another
 * pool.  Inputs are as for bgtq_decode; out / o_sb / o_sh / lse_out / v_rot as
 * for bgtq_combine (out: fp16 (n_batch, n_q, 128); lse_out optional).
 *
 * Limits and rules:
 *   - n_batch * n_q * n_splits <= 8192, else BGTQ_E_TOOBIG (the array holds
 *     8192 partial rows: about 4.2 MB on every GPU that loads the library, kept
 *     until the process exits);
 *   - it calls no cudaMalloc / cudaFree or other allocating routine;
 *   - the FIRST call on each device looks up the array's device address
 *     (cudaGetSymbolAddress) with that device current; make that first call
 *     before starting any stream capture on the device;
 *   - all calls on a device share the one array: two calls whose kernels can
 *     overlap on the GPU (different streams without ordering) race.  Nothing in
 *     the array has to be cleared between calls: every partial that is read was
 *     written by the same call (slots that hold no partial are marked and skipped). */
int bgtq_decode_combined_noalloc(const BgtqDecodePlan* plan_host, const BgtqHeadDesc* desc, const void* q_rot,
                const uint8_t* k_packed, int64_t kp_sb, int64_t kp_sh, int64_t kp_st,
                const void* k_norms, int64_t kn_sb, int64_t kn_sh, int64_t kn_st,
                const uint8_t* v_packed, int64_t vp_sb, int64_t vp_sh, int64_t vp_st,
                const void* v_norms, int64_t vn_sb, int64_t vn_sh, int64_t vn_st,
                int32_t n_batch, int32_t n_q, int32_t n_kv,
                int32_t t_begin, int32_t t_end, int32_t n_splits, float scale,
                const float* v_rot, void* out, int64_t o_sb, int64_t o_sh, float* lse_out,
                int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BGTQ_H_ */
