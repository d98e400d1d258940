// tkd_internal.h: what the translation units of libtkd share (not part of the C-ABI).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/tkd.h"

// --- packer (tkd_pack.cu) ---
int tkd_launch_quantise(int fmt, const float* src, int orient, int64_t K, int64_t N, int64_t npad,
                        const float* col_div, uint8_t* exps, void* codes, cudaStream_t st);
int tkd_launch_permute(int fmt, int64_t K, int64_t npad, const uint8_t* exps, const void* codes, uint8_t* emax,
                       int* info, void* stream, cudaStream_t st);
int tkd_launch_dequantise_bf16(int fmt, int64_t K, int64_t npad, const uint8_t* exps, const void* codes, void* out,
                               cudaStream_t st);
int tkd_launch_unpack(int fmt, int64_t K, int64_t npad, const void* stream, const uint8_t* emax, float* out,
                      cudaStream_t st);

// --- streaming matmul (tkd_stream.cu) ---
// (the TKD_EPI_* and TKD_DT_* codes are those of include/tkd.h)

#define TKD_STREAM_WARPS 16    // streaming warps: 8 groups of 16 columns x 2 halves of each chunk's super-atoms
#ifndef TKD_STREAM_WARPS_16ROWS
#define TKD_STREAM_WARPS_16ROWS 8  // ... of the kernel for 9 to 16 rows (as for 32: measured faster than 16)
#endif
#ifndef TKD_STREAM_WARPS_32ROWS
#define TKD_STREAM_WARPS_32ROWS 8
#endif
//  // ... of the kernel for 17 to 32 rows: a warp per column group, both halves
#define TKD_THREADS ((1 + TKD_STREAM_WARPS + 4) * 32)  // + 1 producer warp + 4 output warps
#define TKD_PANEL_COLS 128     // columns one work item covers
#define TKD_MAX_STAGES 16
#define TKD_SMEM_HEAD 1024     // barriers, the stage headers, flags
#define TKD_TC_SLOTS 6         // tensor-memory kernel: operand slots (a unit of two 64-k tiles: 64 columns of A, 8 KB of x)

struct TkdSegDev {
    const uint8_t* w;     // packed stream (the gate's with a separate up weight)
    const uint8_t* w2;    // the up weight's stream, or null
    const uint8_t* emax;  // per group of 16 columns (null for bf16)
    const uint8_t* emax2;
    int n_valid;          // real columns of w
    int out_col0;         // first output column of the segment in out (elements)
    int panel0;           // first panel of the segment in the call's panel list
    int pad_;
};

struct TkdParams {
    TkdSegDev seg[4];
    int nseg;
    int fmt, M, K;
    const uint16_t* x;  // bf16 bits, row-major, ldx elements a row
    int64_t ldx;
    int ks;             // k per slice (a multiple of the chunk depth)
    int nslices;        // ceil(K / ks)
    int nstages;
    int64_t panel_bytes;  // bytes of one 128-column panel of the stream
    int total_panels;
    int64_t total_items;
    int small;          // item counts times the grid fit 32 bits: the kernel divides in 32-bit arithmetic
    int epi, act;
    uint32_t mul16, mul128;  // 16 and 128: shifts done as multiplies (see shl_fma)
    const void* scale;   // per output column of w (bf16 or f32), or null
    const void* scale2;  // the up weight's, GLU two-weight form
    int scale_dt;
    const void* res;     // residual, bf16 (reference form) or f32 (with a float32 output)
    int res_dt;
    int64_t ldr;
    void* out;
    int out_dt;
    int64_t ldo;
    // top-k records (output warps)
    uint32_t* records;
    int topk_k, topk_rows, topk_unit, topk_slot0, write_y;
    uint32_t topk_base;
    int64_t topk_n;
    uint16_t* ytmp;      // bf16 outputs of a call that does not write y: [rows][ld_ytmp]
    int64_t ld_ytmp;
    int* unit_counters;
    // slice sums of panels whose slices are spread over several CTAs: [panel][slice][half][row][128] floats
    float* scratch;
    int* counters;
    int* status;
    // exchange with the other GPUs of a column-sharded weight: the output stage repeats its stores of y and of the
    // records into the other ranks' buffers; npeers == 0: none
    int npeers, rank;
    void* peer_out[7];
    uint32_t* peer_records[7];
    uint32_t* peer_flags[7];
    uint32_t* flags;     // this rank's flag words
    int* grid_counter;   // CTAs of this call that have finished their output (returns to zero)
    int exchange_wait;
    int tc;              // 9 to 32 rows: the tensor-memory kernel (tkd_stream_tc.cuh); off_xt is where its operand tiles go
    int x_smem;          // 1 to 8 rows, and all of x (K rounded up to a chunk) fits in shared memory at off_xt
    int x_stride;        // ... bytes from one row of it to the next
    int no_pdl;          // launch without programmatic dependent launch (the weights may still be being written)
    const uint32_t* had;  // TKD_INT4: sign words of the block Hadamard applied to x in shared memory first (or null)
    // shared-memory map (bytes from the start of dynamic shared memory)
    int off_pbuf, off_tbuf, off_xt, off_ring;
    int stage_bytes;
};

int tkd_launch_stream(const TkdParams& p, int grid, size_t smem, cudaStream_t st);
int tkd_launch_hadamard(const void* x, int64_t ldx, const uint32_t* signs, int rows, int K, void* out, int64_t ldo,
                        cudaStream_t st);
int tkd_launch_topk_merge(const uint32_t* records, int nrec, int rows, int k, int top, uint32_t* out, cudaStream_t st);
int tkd_launch_head_pick(const uint32_t* records, int nrec, int rows, int k, int top, uint32_t vocab, const uint16_t* x,
                         int64_t ldx, int dim, const uint16_t* head, int64_t ld_head, int round, uint32_t* out,
                         uint32_t* ids_out, cudaStream_t st);
int tkd_launch_head_pick_records(const uint32_t* records, int nrec, int rows, int k, uint32_t vocab, const uint32_t* tmap,
                                 uint32_t* out, uint32_t* ids_out, cudaStream_t st);
int tkd_launch_exchange_wait(uint32_t* flags, int nranks, int* status, cudaStream_t st);
struct TkdPeerFlags {
    uint32_t* p[7];
};
int tkd_launch_exchange_publish(uint32_t* flags, const TkdPeerFlags& peers, int nranks, int rank, int lag_wait, int* status,
                                cudaStream_t st);
