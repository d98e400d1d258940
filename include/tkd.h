/* tkd.h: C-ABI of libtkd, the B200 (sm_100a) implementation of the dense_reader path of XylolabsInc/tensix-kernels.
 *
 * Plain pointers and sizes only. Unless a comment says "host", every pointer is a device pointer of the current CUDA
 * device, and `stream` is a cudaStream_t passed as void* (NULL: the default stream). Every function returns 0 or a
 * TKD_ERR_* code (tkd_error_string); codes above 1000 are 1000 + a cudaError_t. Nothing here synchronises with the
 * device unless it says so, and none of the functions taking a stream allocates device memory.
 *
 * Each entry point names the piece of the reference it stands in for (file:line within that project).
 */
#ifndef TKD_H
#define TKD_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* weight formats: ttnn.bfloat8_b, ttnn.bfloat4_b, ttnn.bfloat16 (dense_reader/linear.py:49-50) */
#define TKD_FMT_BFP8 0
#define TKD_FMT_BFP4 1
#define TKD_FMT_BF16 2
#define TKD_FMT_INT4 3   /* int4 codes -7..7 with one bf16 scale per column and 32 k (int4/w4a16.py of the reference):
                           m <= 8 only; tkd_pack takes the scales in place of exps, see there */

#define TKD_OK 0
#define TKD_ERR_BAD_ARG 1      /* a shape, pointer or option the path does not take */
#define TKD_ERR_UNSUPPORTED 2  /* a legal request this build has no kernel for */
#define TKD_ERR_TIMEOUT 3      /* written to the status word by a kernel whose bounded wait gave up */
#define TKD_ERR_WORKSPACE 4    /* workspace missing or too small */
#define TKD_ERR_WIDE 5         /* exponents inside one group of 16 columns spread further than the stream encodes */
#define TKD_ERR_FIXED_SCRATCH 6 /* tkd_matmul_noalloc: the call needs more than TKD_NOALLOC_SCRATCH_BYTES of scratch */
#define TKD_ERR_CUDA 1000

/* output stages (dense_reader/kernels/dense_compute.cpp:200-356) */
#define TKD_EPI_PLAIN 0     /* y = bf16(acc * scale) (scale optional)                    :302-356 */
#define TKD_EPI_GLU_IL 1    /* act(gate) * up over an interleave_glu weight, N / 2 wide  :200-257 */
#define TKD_EPI_GLU2 2      /* the same over two weights (w the gate's, w_up), N wide    :200-257, GLU2 */
#define TKD_EPI_RESIDUAL 3  /* y = bf16(acc + bf16 residual)                             :100-120, 258-301 */
#define TKD_EPI_OUT32 4     /* y = acc in float32 (+ a float32 residual, an extension)   :302-332 */

#define TKD_DT_NONE 0
#define TKD_DT_BF16 1
#define TKD_DT_F32 2

int tkd_version(void);
/* The version of the packed streams' bit layout (tkd_pack's output): it changes whenever the layout does, and a cache
 * of packed weights records it (the counterpart of the pack cache's version key, moe/moe8.py:289-346). */
int tkd_layout_version(void);
/* sizeof of a structure of this header as the library was built (0 TkdMatmul, 1 TkdPlan, 2 TkdBlock, 3 TkdMoe): a binding
 * compares it with its own mirror before the first call. */
int tkd_struct_bytes(int which);
const char* tkd_error_string(int code);

/* --- weights: stands in for ttnn.from_torch(dtype=bfloat8_b|bfloat4_b|bfloat16) as native_weight and block_float call
 * it (dense_reader/linear.py:155, :162) and for ttnn.to_torch on such a weight (tests' held(),
 * dense_reader/tests/test_dense_reader.py:47-49). ------------------------------------------------------------------ */

/* N rounded up to the 128 columns of a panel of the stream. */
int64_t tkd_padded_cols(int64_t n);
/* Bytes of the packed stream of a [K, N] weight: K * padded N * (1.0625 | 0.5625 | 2) for K a multiple of 32 (64 for
 * bfloat4_b, whose last super-atom is zero-filled otherwise). */
int64_t tkd_packed_bytes(int fmt, int64_t k, int64_t n);

/* float32 -> the format's numbers, before any re-layout. src: orient 0 a row-major [N, K] matrix (torch [out, in]),
 * orient 1 a row-major [K, N]. col_div (or NULL): [N] divisors applied first (native_weight's col_scale). exps
 * [K, npad / 16] bytes (unused for bf16); codes [K, npad]: bytes sign << mantissa_bits | magnitude, or uint16 bf16 bits
 * for TKD_FMT_BF16. */
int tkd_quantise(int fmt, const float* src, int orient, int64_t k, int64_t n, const float* col_div, uint8_t* exps,
                 void* codes, void* stream);
/* canonical numbers -> the HBM stream. packed: tkd_packed_bytes; emax: npad / 16 bytes (unused for bf16); info: one
 * int32, zeroed by the caller; bit 0 is set when the weight is "wide": inside some group of 16 columns a row with a
 * non-zero code lies more than 48 binades below the group's largest row, further than the stream's exponents reach.
 * tkd_matmul never sees the info word: a caller that finds the bit set must not launch on that stream (the far rows'
 * exponents are clamped in it) and holds the weight as TKD_FMT_BF16 instead, which is exact: tkd_dequantise_bf16 on
 * the same exps and codes, then tkd_pack with TKD_FMT_BF16 (what the Python layer does; TKD_ERR_WIDE is what a binding
 * raises if it chooses to refuse instead).
 * TKD_FMT_INT4 (the reference's int4_weight + group_scales, int4/w4a16.py:70-105): codes [K, npad] bytes
 * sign << 3 | magnitude (magnitude 0..7), exps = the group scales as bf16 bits [ceil(K / 32), npad] (uint16; K a
 * multiple of 32), emax and info unused (NULL). The weight is code * scale exactly; tkd_unpack returns that. */
int tkd_pack(int fmt, int64_t k, int64_t n, const uint8_t* exps, const void* codes, void* packed, uint8_t* emax,
             int32_t* info, void* stream);
/* tkd_quantise's block-float numbers (TKD_FMT_BFP8 or BFP4) as bf16 bits [K, npad] (uint16), the canonical form
 * tkd_pack takes for TKD_FMT_BF16: every such number is a bf16 value exactly, subnormals included. */
int tkd_dequantise_bf16(int fmt, int64_t k, int64_t n, const uint8_t* exps, const void* codes, void* out_bf16, void* stream);
/* the stream back as float32 [K, npad]: the values the weight holds */
int tkd_unpack(int fmt, int64_t k, int64_t n, const void* packed, const uint8_t* emax, float* out, void* stream);

/* --- the op: stands in for ttnn.generic_op on the program dense_reader/linear.py:828-1070 (_launch) builds from
 * plan() (:187-382): dense_reader.cpp + dense_compute.cpp + dense_writer.cpp. --------------------------------------- */

typedef struct {
    const void* w;          /* packed stream (the gate's with TKD_EPI_GLU2) */
    const void* w_up;       /* the up weight's stream with TKD_EPI_GLU2, else NULL */
    const uint8_t* emax;    /* tkd_pack's side array of w (NULL for bf16) */
    const uint8_t* emax_up;
    int64_t n;              /* real columns of w */
    int64_t out_col0;       /* first output column of this block in out, in elements */
} TkdBlock;

typedef struct {
    int32_t fmt;            /* TKD_FMT_* of every block */
    int32_t m;              /* activation rows, 1..32 */
    int64_t k;
    const void* x;          /* bf16 [m, k], ldx elements a row (at most 2^26 for m > 8), 16-byte aligned rows */
    int64_t ldx;
    int32_t nblocks;        /* 1, or 2..4 for a block list (linear.py:615-624) */
    int32_t epilogue;       /* TKD_EPI_* */
    TkdBlock block[4];
    int32_t act;            /* GLU: 0 silu, 1 gelu_tanh (common/kernels/dense_ops.h:44-59) */
    int32_t scale_dtype;    /* TKD_DT_NONE | BF16 (the reference's scale tensor) | F32 (extension) */
    const void* scale;      /* [n] per output column of w */
    const void* scale_up;   /* [n] of w_up (an extension: scales with a GLU) */
    const void* residual;   /* [m, >= n]: bf16 with TKD_EPI_RESIDUAL, float32 with TKD_EPI_OUT32 (or NULL) */
    int64_t ldr;
    int32_t residual_dtype;
    int32_t out_dtype;      /* TKD_DT_BF16, or TKD_DT_F32 with TKD_EPI_OUT32 */
    void* out;              /* [m, ldo] */
    int64_t ldo;
    /* top-k records (dense_reader/kernels/dense_writer.cpp:185-258; record layout linear.py:771-785): one record per
     * topk_unit columns, record slot0 + unit; a record is keys[rows][k] then indices[rows][k], uint32 each. Within a
     * record: key descending, index ascending among equal keys. topk_k 0: none. */
    void* records;
    int32_t topk_k, topk_rows, topk_unit, topk_slot0, topk_write_y;
    uint32_t topk_base;
    int64_t topk_n;
    void* workspace;        /* tkd_matmul_workspace bytes, zeroed once by the caller before its first use */
    uint64_t workspace_bytes;
    int32_t* status;        /* one int32 (or NULL): a kernel writes TKD_ERR_TIMEOUT here if a wait gives up */
    int32_t ks;             /* k per slice, 0: default; a multiple of 256 (128 for bf16) */
    int32_t max_ctas;       /* 0: one per SM */
    /* exchange between the GPUs of a column-sharded weight (nranks 0 or 1: none). The output stage writes every
     * element of out, and every record, also to the same place of each other rank's buffer (peer stores over NVLink:
     * the all-gather of the outputs happens inside the kernel, column by column as they finish). The warp that
     * finishes last orders the call's stores system-wide, counts the call in flags[TKD_FLAG_SEQ] and writes that count
     * to flags[rank] on every rank.
     * peer_out / peer_records: the addresses, in this process, of the other ranks' buffers (NULL entries: that
     * buffer is not exchanged), nranks - 1 of them in rank order with the own rank left out; peer_flags likewise. */
    int32_t nranks, rank;
    void* peer_out[7];
    void* peer_records[7];
    uint32_t* peer_flags[7];
    uint32_t* flags;        /* this rank's TKD_FLAG_WORDS words, zeroed once, written by every rank */
    int32_t exchange_wait;  /* 1: the kernel ends only when every rank's count for this call has arrived in flags
                               (bounded, about a second: then TKD_ERR_TIMEOUT in the status word and tkd_exchange_wait
                               can wait again); 2: the same wait, but for the exchanged call BEFORE this one (the exchange
                               of one call overlaps the next call's run; tkd_exchange_wait flushes the last one); 0: no
                               wait, the caller orders tkd_exchange_wait behind it; 3: the kernel only stores (no
                               counting, no fence, no flags): the caller announces the call with tkd_exchange_publish
                               once the kernel has completed, e.g. from a second stream behind an event, so that the
                               announcement's system-wide fence and the flags' flight overlap the next call */
    int32_t weights_fresh;  /* 0: every weight stream and emax array of the call was complete (by an event or a
                               synchronisation) before this call was enqueued: the kernel is launched as a programmatic
                               dependent of the work before it on the stream, and its first weight loads may run while
                               that work drains. 1: something enqueued earlier on the stream still writes them (tkd_pack,
                               a copy): the launch is ordered behind all of it, at the cost of that overlap. */
    const uint32_t* hadamard; /* or NULL. TKD_FMT_INT4 only (the ternary projections of a rotated checkpoint,
                               ternary_matmul/t2.py:409-495 hadamard=): the activations are rotated first, x' = H_1024
                               (s * x) per block of 1024 inputs, unnormalised, exactly as tkd_hadamard does it (its sign
                               words), inside the kernel's own copy of x: k a multiple of 1024, and x must fit in shared
                               memory beside the ring (TKD_ERR_UNSUPPORTED otherwise: call tkd_hadamard first) */
} TkdMatmul;
#define TKD_MAX_RANKS 8
#define TKD_FLAG_SEQ 8      /* flags[0..7]: calls completed by rank r, as told by r; flags[8]: calls completed here */
#define TKD_FLAG_WORDS 16

/* What the launch of a TkdMatmul looks like: the counterpart of the dict plan() returns (linear.py:360-382). */
typedef struct {
    int32_t ks, nslices, panels, grid, stages, stream_warps, chunk_k, smem_bytes;
    int64_t items, weight_bytes;
} TkdPlan;

int tkd_matmul_plan(const TkdMatmul* a, TkdPlan* plan);
int tkd_matmul_workspace(const TkdMatmul* a, uint64_t* bytes);
/* The launch. Ordering contract: the activations, scales, residual, outputs and workspace are read and written in
 * stream order; the WEIGHT streams and emax arrays are read from the moment the kernel's first CTAs start, which with
 * programmatic dependent launch is before the work enqueued ahead of it has finished. A caller that packs (or copies) a
 * weight and multiplies by it on the same stream without a synchronisation in between sets a->weights_fresh. */
int tkd_matmul(const TkdMatmul* a, void* stream);

/* tkd_matmul with the activations and the result in HOST memory (pinned, for the copies to be asynchronous): copies
 * x_host [m, k] bf16 into a->x, launches, copies a->out [m, ldo] to out_host, all on `stream`; a->x and a->out are the
 * caller's device staging buffers (ldx == k). The counterpart of a caller doing ttnn.from_torch(x) ... ttnn.to_torch(y)
 * around linear.matmul (e.g. examples/dense_reader_example.py:24-26 of the reference). Does not synchronise. */
int tkd_matmul_host(const TkdMatmul* a, const void* x_host, void* out_host, void* stream);

/* tkd_matmul for callers that cannot allocate device memory (no counterpart in the reference: its device buffers
 * all come from ttnn's allocator). Some hosts of this library never get to call cudaMalloc: a plugin running inside
 * another framework's memory pool, a step replayed from a fixed arena, a process whose device memory was handed out
 * entirely at start-up. For them the kernel's workspace comes from an array of TKD_NOALLOC_SCRATCH_BYTES built into
 * the library's device image (every GPU that loads the library holds that much until exit); a->workspace and
 * a->workspace_bytes are ignored, inputs and outputs are still the caller's. The call allocates nothing and frees
 * nothing. A request whose workspace (tkd_matmul_workspace) exceeds the array is refused with TKD_ERR_FIXED_SCRATCH
 * before anything is launched; as a guide, the array holds about 7900 / M panel-slices of sums (a panel is 128
 * columns, a slice 1024 k by default): one row against the 151936-column LM head fits, eight rows do not.
 * The first call on a device looks the array's device address up and clears its counters; make that first call
 * outside any stream capture, and at start-up: under CUDA's lazy module loading it is also the moment the driver
 * backs the array with memory, so a host whose pool has already taken all of the device's memory can see it fail
 * (1000 + cudaError_t) there and nowhere later (CUDA_MODULE_LOADING=EAGER moves that to the library's load). All calls
 * on a device share the one array, which keeps what the last call left in it (the kernel returns its counters to zero
 * itself): two calls that overlap on the GPU, from different streams or processes' threads, race on it, so keep calls
 * on one device in stream order. A kernel that gave up a bounded wait (TKD_ERR_TIMEOUT in the status word) may have
 * left the counters mid-count: call tkd_matmul_noalloc_reset before the next tkd_matmul_noalloc on that device. */
#define TKD_NOALLOC_SCRATCH_BYTES (8u << 20)
int tkd_matmul_noalloc(const TkdMatmul* a, void* stream);
/* Starts the built-in array's counters from zero again, on `stream` (a memset of its first 256 KB; allocates nothing).
 * For use after TKD_ERR_TIMEOUT, ordered after the kernel that reported it and before the next call. No counterpart
 * in the reference. */
int tkd_matmul_noalloc_reset(void* stream);
/* The built-in array's address on the current device (host out-pointer), for diagnostics and tests; resolves it like a
 * first tkd_matmul_noalloc call does, without clearing anything. No counterpart in the reference. */
int tkd_noalloc_scratch_address(void** ptr);

/* The block Hadamard rotation in front of the reference's ternary projections (ternary_matmul/t2.py:262-340 hadamard,
 * kernels/had_reader.cpp, had_compute.cpp, had_writer.cpp; rotate_rows :220-259 for many rows): per row and block of 1024
 * inputs out = H_1024 (s * x), H the +-1 Sylvester matrix, unnormalised (32 times the orthonormal transform), computed in
 * float32 and rounded to bf16 once. x, out: bf16 [rows, k] with ldx, ldo elements a row (multiples of 4, 8-byte aligned
 * bases; out may be x); k a multiple of 1024; signs: k / 2 words, word q with bit 15 set when input 2 q is negated and
 * bit 31 for input 2 q + 1 (the reference's mask, t2.py:185-202). */
int tkd_hadamard(const void* x, int64_t ldx, const uint32_t* signs, int rows, int k, void* out, int64_t ldo, void* stream);

/* --- the mixture-of-experts layer's two matmuls: stand in for moe8.gate_up / down and gate_up_rows / down_rows
 * (moe/moe8.py:710-911, 928-1136 of the reference; kernels/moe_gu_*.cpp, moe_dn_*.cpp, moe8_rows.h). Only the chosen
 * experts' weights are read, and the expert ids are read on the device: nothing goes to the host. ------------------- */

typedef struct {
    const void* w;           /* every expert's packed stream (fmt), expert e at e * expert_bytes: tkd_pack of
                                the expert's [k_in, n] weight. gate_up: n = 2 I columns in the GLU's tile order (32 gate
                                columns, then their 32 up columns: interleave_glu, dense_reader/linear.py:122-130);
                                down: [I, H] */
    const uint8_t* emax;     /* tkd_pack's side arrays, expert e at e * (tkd_padded_cols(n) / 16) */
    int64_t expert_bytes;    /* a multiple of 16 */
    int32_t experts;
    int32_t k_in;            /* inputs of one expert's weight: H (gate_up) or I (down); a multiple of 32 */
    int32_t n;               /* its columns: 2 I (gate_up; a multiple of 64) or H (down) */
    int32_t rows;            /* activation rows R: 1 (decode), or 1..32 with by_union */
    const void* x;           /* bf16. gate_up: [rows, ldx], k_in used; down: gate_up's result, slot q's inputs at q * k_in */
    int64_t ldx;             /* elements a row, a multiple of 8; x 16-byte aligned */
    const void* ids;         /* [rows, ld_ids] expert ids, uint16 (ids32 0) or uint32; an id at or past `experts` counts
                                as no expert (its slot gives zeros) */
    int32_t ids32;
    int32_t k;               /* experts chosen per row, 1..16 */
    int64_t ld_ids;
    const void* route_w;     /* gate_up: [rows, ld_w] bf16 routing weights, one per id */
    int64_t ld_w;
    int32_t by_union;        /* 0: one row; slot s is expert ids[s] (gate_up, down). 1: the work goes by the distinct
                                experts of all rows' ids in increasing order (gate_up_rows, down_rows, moe8_rows.h): slot
                                q is the q-th of them, a row that did not choose it gets zeros there; experts <= 1024 */
    int32_t slots;           /* by_union 0: k; 1: the slots of the result, min(experts, rows * k) (u_max, moe8.py:923) */
    int32_t act;             /* gate_up: 0 silu, 1 gelu_tanh, 2 swiglu_oai (moe8.py:83-85) */
    const void* bias;        /* gate_up, or NULL: bf16 [experts, tkd_padded_cols(n)] in the weight's column order,
                                added to x G and x U before the activation (moe8.py:224-230) */
    void* out;               /* bf16 [rows, ldo]. gate_up: slot q's I values at q * I, each routing weight * act(x G +
                                b) * (x U + b); down: the n columns of y = sum over the slots of h_q @ D_q */
    int64_t ldo;
    void* workspace;         /* down: tkd_moe_workspace bytes, zeroed once by the caller before the first use (the kernel
                                returns its counters to zero); calls that share one must be ordered on one stream */
    uint64_t workspace_bytes;
    int32_t fmt;             /* TKD_FMT_BFP4, or TKD_FMT_BF16: experts whose values no bfloat4_b stream holds (the K-block
                                layout, moe8.py:507-527 kblock: shared exponents along K), kept exactly at 2 bytes a weight;
                                emax is then unused */
} TkdMoe;

int tkd_moe_workspace(const TkdMoe* a, uint64_t* bytes);
/* Rows whose activations do not fit in shared memory together are taken in passes (the experts' weights are read again
 * for each, from L2). TKD_ERR_UNSUPPORTED: not even one row of k_in inputs fits. */
int tkd_moe_gate_up(const TkdMoe* a, void* stream);
int tkd_moe_down(const TkdMoe* a, void* stream);
/* The router's top k and their weights, into the ids and weights the ops above read: stands in for moe8.route
 * (moe/moe8.py:1139-1253; kernels/moe_route.cpp). logits: float32 [rows, ld] (rows <= 32), the experts' columns
 * 0 .. experts - 1 (a multiple of 32, at most 1024). Per row the k picks in decreasing order of their key, the lower id
 * among equal keys, computed in float64:
 *   kind 0 (softmax): key = the logit; weights = the softmax over the k picks' logits;
 *   kind 1 (sigmoid with a bias): key = sigmoid(logit) + bias[e] (bias: float32 [experts]); weights = the picks'
 *          sigmoids over their sum (norm 0: each pick's own sigmoid);
 *   kind 2 (sigmoid without a bias): key = the logit; weights as kind 1's.
 * Every weight times scale (0 < scale < 4), rounded to bf16. n_group > 1 (kind 1; DeepSeek-V3's group-limited routing): the
 * experts in n_group groups in order, a group's score the sum of its two largest keys, the topk_group best groups kept (the
 * lower group among equal scores), the picks among their experts. has_slot: `slot` is written as slot k of every row at
 * weight 1.0 (ids and w then hold k + 1 slots). ids: uint16 (ids32 0) or uint32 [rows, ld_ids]; w: bf16 [rows, ld_w];
 * shared (or NULL): bf16 [rows, ld_shared], column 0 gets sigmoid(logits[:, experts]). */
int tkd_moe_route(const float* logits, int64_t ld, int rows, int experts, int k, int kind, const float* bias, double scale,
                  int norm, int n_group, int topk_group, int has_slot, uint32_t slot, void* ids, int ids32, int64_t ld_ids,
                  void* w, int64_t ld_w, void* shared, int64_t ld_shared, void* stream);

/* The best `top` candidates of every row among `nrecords` top-k records (the record layout above: keys[rows][k] then
 * indices[rows][k]), key descending and index ascending among equal keys; out is one record of the same layout with
 * `top` in place of k (slots beyond the candidates there are: key 0, index 0xFFFFFFFF). Stands in for the `vh.topk(top)`
 * over the decoded records in the reference's LM head (lm_head_topk/lmhead.py:212-239, collect), whose records are one
 * device's; here they may be every rank's, gathered. */
int tkd_topk_merge(const uint32_t* records, int nrecords, int rows, int k, int top, uint32_t* out, void* stream);

/* The LM head's exact rescore and pick on the device: stands in for head_pick.pick (lm_head_topk/head_pick.py:101-220;
 * kernels/head_pick_reader.cpp, head_pick_compute.cpp, head_pick_writer.cpp). Per row r < rows: the best `top` (<= 32)
 * slots of the records in order (record by record, slot by slot; an equal key keeps the earlier; key 0 or an index at
 * or past `vocab`: empty), their logits recomputed from bf16 x [rows, ldx] and the bf16 head rows [>= vocab, ld_head]
 * (float32 sums; rounded to bf16 with round_bf16), and the pick: the largest logit, a NaN counting as the largest, -0
 * equal to +0, the lowest index among equals. out: 32 uint32 words a row: [token, the first candidate by the device's
 * own logit, candidates held, 0 ...]; no candidate: [0, 0xFFFFFFFF, 0]. ids_out (or NULL): row 0's token, one word. */
int tkd_head_pick(const uint32_t* records, int nrecords, int rows, int k, int top, uint32_t vocab, const void* x,
                  int64_t ldx, int dim, const void* head_rows, int64_t ld_head, int round_bf16, uint32_t* out,
                  uint32_t* ids_out, void* stream);
/* The records-only pick: stands in for head_pick.pick_records (lm_head_topk/head_pick.py:243-335;
 * kernels/head_pick_records.cpp). Per row the first slot, in the records' order, of the largest key (a NaN of either
 * sign above every key, -0 equal to +0); its index (below `vocab`) is the token, or token_map[index] with a map
 * (uint32 [>= vocab]). out as tkd_head_pick's, with the count of all valid slots. */
int tkd_head_pick_records(const uint32_t* records, int nrecords, int rows, int k, uint32_t vocab, const uint32_t* token_map,
                          uint32_t* out, uint32_t* ids_out, void* stream);

/* --- exchange between GPUs: stands in for the all-gather of the column shards' outputs (the reference runs on one
 * device and has none; its multi-device callers would gather [M, N_local] outputs or top-k records). ---------------- */

/* Wait on `stream` until every one of the nranks ranks has completed as many exchanged calls as this rank has
 * (flags[r] >= flags[TKD_FLAG_SEQ] for all r, modulo 2^32); bounded (about a second), then TKD_ERR_TIMEOUT in *status. */
int tkd_exchange_wait(uint32_t* flags, int nranks, int32_t* status, void* stream);
/* Announce an exchanged call made with exchange_wait 3, on a stream on which the call's kernel has completed: counts
 * the call in flags[TKD_FLAG_SEQ] and writes that count to flags[rank] on every rank (peer_flags: host array of the
 * nranks - 1 other ranks' flag words, as in TkdMatmul). lag_wait: then wait (bounded) until every rank has announced
 * the call before this one. No counterpart in the reference (one device). */
int tkd_exchange_publish(uint32_t* flags, uint32_t* const* peer_flags, int nranks, int rank, int lag_wait, int32_t* status,
                         void* stream);
/* Device memory other processes on this machine can map: allocates `bytes` (zeroed; synchronises) and writes its
 * 64-byte inter-process handle to handle (host). The owner frees it with tkd_peer_free. */
int tkd_peer_alloc(uint64_t bytes, void** ptr, void* handle);
int tkd_peer_free(void* ptr);
/* Map another process's tkd_peer_alloc memory from its handle (host, 64 bytes) into this process, with peer access
 * between the two GPUs enabled; tkd_peer_close unmaps it. */
int tkd_peer_open(const void* handle, void** ptr);
int tkd_peer_close(void* ptr);

#ifdef __cplusplus
}
#endif
#endif
