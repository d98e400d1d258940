// tkd_api.cu: the extern "C" entry points of libtkd (include/tkd.h): argument checks, the launch plan, the launches.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <atomic>

#include "../../include/tkd.h"
#include "tkd_internal.h"
#include "tkd_layout.h"

static_assert(TKD_FMT_BFP8 == TKD_BFP8 && TKD_FMT_BFP4 == TKD_BFP4 && TKD_FMT_BF16 == TKD_BF16 && TKD_FMT_INT4 == TKD_INT4,
              "format codes");

namespace {

constexpr int kMaxSmem = 227 * 1024;  // dynamic shared memory a CTA may take on sm_100
constexpr int kMaxPanels = 48 * 1024;  // panel counters at the start of the workspace (6 M columns a call)
constexpr int kMaxUnits = 16 * 1024;   // then the top-k unit counters; 256 KB together
constexpr int kMaxMisc = 64;           // then the call's finished-CTA counter (exchange between GPUs)
constexpr int64_t kCounterBytes = (int64_t)(kMaxPanels + kMaxUnits + kMaxMisc) * 4;

inline int cuda_err(cudaError_t e) { return e == cudaSuccess ? TKD_OK : TKD_ERR_CUDA + (int)e; }
inline int launch_err(int e) { return e == 0 ? TKD_OK : TKD_ERR_CUDA + e; }
inline bool fmt_ok(int fmt) { return fmt == TKD_BFP8 || fmt == TKD_BFP4 || fmt == TKD_BF16 || fmt == TKD_INT4; }
// (formats whose stream carries biased exponents against a side array of per-group maxima)
inline bool has_emax(int fmt) { return fmt == TKD_BFP8 || fmt == TKD_BFP4; }
inline int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    if (!cached[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
        cached[dev] = n;
    }
    return cached[dev];
}

struct Layout {
    TkdParams p;
    int grid;
    size_t smem;
    int64_t weight_bytes;
    // workspace map
    int64_t off_counters, off_units, off_misc, off_scratch, off_ytmp, ws_bytes;
};

// Everything a launch needs except the device pointers into the workspace. sms 0: ask the device.
int make_layout(const TkdMatmul* a, Layout* L, int sms) {
    if (!a || !fmt_ok(a->fmt)) return TKD_ERR_BAD_ARG;
    if (a->m < 1 || a->m > 32 || a->k < 32 || a->k % 32 || a->k > (1 << 24)) return TKD_ERR_BAD_ARG;
    // (the int4 weight with group scales is the reference's one-token op; more rows go through its dequantised
    // bfloat8_b form, as there: int4/w4a16.py dequantize)
    if (a->fmt == TKD_INT4 && a->m > 8) return TKD_ERR_UNSUPPORTED;
    if (a->nblocks < 1 || a->nblocks > 4) return TKD_ERR_BAD_ARG;
    if (a->epilogue < TKD_EPI_PLAIN || a->epilogue > TKD_EPI_OUT32) return TKD_ERR_BAD_ARG;
    const bool glu = a->epilogue == TKD_EPI_GLU_IL || a->epilogue == TKD_EPI_GLU2;
    if (a->nblocks > 1 && !(a->epilogue == TKD_EPI_PLAIN || a->epilogue == TKD_EPI_GLU2)) return TKD_ERR_BAD_ARG;
    if (a->nblocks > 1 && (a->scale_dtype != TKD_DT_NONE || a->topk_k)) return TKD_ERR_BAD_ARG;
    if (a->topk_k && (glu || a->epilogue == TKD_EPI_OUT32 || a->epilogue == TKD_EPI_RESIDUAL)) return TKD_ERR_BAD_ARG;
    if ((a->epilogue == TKD_EPI_OUT32) != (a->out_dtype == TKD_DT_F32)) return TKD_ERR_BAD_ARG;
    if (a->out_dtype != TKD_DT_F32 && a->out_dtype != TKD_DT_BF16) return TKD_ERR_BAD_ARG;
    if (a->nranks < 0 || a->nranks > TKD_MAX_RANKS || (a->nranks > 1 && (a->rank < 0 || a->rank >= a->nranks)))
        return TKD_ERR_BAD_ARG;

    TkdParams& p = L->p;
    memset(&p, 0, sizeof(p));
    p.fmt = a->fmt;
    p.M = a->m;
    p.K = (int)a->k;
    p.nseg = a->nblocks;
    p.epi = a->epilogue;
    p.act = a->act;
    p.mul16 = 16, p.mul128 = 128;
    const int mt = a->m <= 8 ? 1 : (a->m <= 16 ? 2 : 4);
    const int sab = tkd_sab(a->fmt);
    const int chunk_k = tkd_chunk_k(a->fmt);
    // k per slice: a function of K and the format only (a column's sum must not depend on anything else). 1024 (less
    // for a short K) divides the items well among the CTAs; but every slice a panel is cut into is another M x 128 sums
    // through the scratch buffer for the CTA that adds the panel up, and another hand-over: a long K is cut into four
    // slices, at most 4096 each (config 3, K 14336, one row: 18.8 us with 1024, 16.4 with 1792, 15.6 with 3584).
    int ks_k = a->k >= 4096 ? 1024 : (a->k >= 2048 ? 512 : 256);
    {
        int part = (int)((a->k / 4 + chunk_k - 1) / chunk_k) * chunk_k;
        if (part > 4096) part = 4096;
        if (part > ks_k) ks_k = part;
    }
    p.ks = a->ks ? a->ks : (ks_k < chunk_k ? chunk_k : ks_k);
    if (p.ks < chunk_k || p.ks % chunk_k || p.ks > 4096) return TKD_ERR_BAD_ARG;
    p.nslices = (p.K + p.ks - 1) / p.ks;
    p.panel_bytes = tkd_panel_bytes(a->fmt, a->k);

    int panels = 0;
    L->weight_bytes = 0;
    for (int s = 0; s < a->nblocks; ++s) {
        const TkdBlock& b = a->block[s];
        if (b.n < 1 || b.out_col0 < 0 || b.n > (1 << 28)) return TKD_ERR_BAD_ARG;
        if (glu && a->epilogue == TKD_EPI_GLU_IL && b.n % 64) return TKD_ERR_BAD_ARG;
        const int64_t npad = tkd_padded_cols(b.n);
        TkdSegDev& d = p.seg[s];
        d.w = static_cast<const uint8_t*>(b.w);
        d.w2 = static_cast<const uint8_t*>(b.w_up);
        d.emax = b.emax;
        d.emax2 = b.emax_up;
        d.n_valid = (int)b.n;
        d.out_col0 = (int)b.out_col0;
        d.panel0 = panels;
        const bool two = a->epilogue == TKD_EPI_GLU2;
        panels += (int)(two ? npad / 64 : npad / TKD_PANEL_COLS);  // a (gate, up) panel: 64 columns of each weight
        L->weight_bytes += (two ? 2 : 1) * tkd_stream_bytes(a->fmt, a->k, npad);
    }
    p.total_panels = panels;
    p.total_items = (int64_t)panels * p.nslices;

    // shared-memory map: barriers, the hand-over buffers of the streaming warps, the GLU exchange buffer, the ring
    const int mp = mt == 1 ? 8 : (mt == 2 ? 24 : 40);
    p.stage_bytes = 8 * tkd_subsa(a->fmt) * sab;
    p.off_pbuf = TKD_SMEM_HEAD;
    if (a->m > 8) {
        // 9 to 32 rows, the tensor-memory kernel: the running sums [128][40] floats, then (from the next 1024-byte
        // boundary of the window, hence the slack) TKD_TC_SLOTS slots of two x tiles (4 KB each), then the ring. (The kernel
        // addresses x by 32-bit element offsets.)
        if (a->ldx > (1 << 26)) return TKD_ERR_BAD_ARG;
        p.tc = 1;
        p.off_tbuf = TKD_SMEM_HEAD;
        p.off_xt = p.off_tbuf + TKD_PANEL_COLS * 40 * 4;
        p.off_ring = (int)align_up(p.off_xt + 1024 + TKD_TC_SLOTS * 2 * 4096, 128);
    } else {
        // (one to eight rows: two hand-over buffers; all of x in shared memory, K rounded up to a chunk, if that leaves
        // the ring at least four stages; rows 64 bytes further apart than their length, so that the eight rows a warp
        // reads together fall on different banks)
        p.off_tbuf = p.off_pbuf + 2 * 2 * TKD_PANEL_COLS * mp * 4;
        p.off_xt = (int)align_up(p.off_tbuf + TKD_PANEL_COLS * mp * 4, 128);
        int64_t xt_bytes = 0;
        const int64_t x_row = (a->k + chunk_k - 1) / chunk_k * chunk_k * 2 + (a->m > 1 ? 64 : 0);
        if (p.off_xt + a->m * x_row + 4 * (int64_t)p.stage_bytes + 256 <= kMaxSmem) {
            p.x_smem = 1;
            p.x_stride = (int)x_row;
            xt_bytes = a->m * x_row;
        }
        p.off_ring = (int)align_up(p.off_xt + xt_bytes, 128);
    }
    p.nstages = (kMaxSmem - p.off_ring) / p.stage_bytes;
    if (p.nstages > TKD_MAX_STAGES) p.nstages = TKD_MAX_STAGES;
    if (p.nstages < 2) return TKD_ERR_UNSUPPORTED;
    L->smem = (size_t)p.off_ring + (size_t)p.nstages * p.stage_bytes;

    if (sms <= 0) sms = sm_count();
    if (sms <= 0) sms = 148;
    if (a->max_ctas > 0 && a->max_ctas < sms) sms = a->max_ctas;
    L->grid = (int)(p.total_items < sms ? p.total_items : sms);
    p.small = (p.total_items + 1) * (int64_t)(L->grid + 1) < (1ll << 32);

    // top-k
    p.topk_k = a->topk_k;
    int units = 0;
    if (a->topk_k) {
        if (a->topk_rows < 1 || a->topk_rows > 16 || a->topk_k < 1 || a->topk_rows * a->topk_k > 64) return TKD_ERR_BAD_ARG;
        if (a->topk_rows > a->m) return TKD_ERR_BAD_ARG;
        if (a->topk_unit < TKD_PANEL_COLS || a->topk_unit % TKD_PANEL_COLS || a->topk_unit > 2048) return TKD_ERR_BAD_ARG;
        p.topk_rows = a->topk_rows;
        p.topk_unit = a->topk_unit;
        p.topk_slot0 = a->topk_slot0;
        p.write_y = a->topk_write_y;
        p.topk_base = a->topk_base;
        p.topk_n = a->topk_n;
        units = (panels * TKD_PANEL_COLS + a->topk_unit - 1) / a->topk_unit;
    }
    // workspace map. The counters live in a fixed region at the start, the same for every call: they must stay zero
    // between calls, so no call's slice sums or outputs may ever be laid over another call's counters.
    if (panels > kMaxPanels || units > kMaxUnits) return TKD_ERR_UNSUPPORTED;
    L->off_counters = 0;
    L->off_units = (int64_t)kMaxPanels * 4;
    L->off_misc = (int64_t)(kMaxPanels + kMaxUnits) * 4;
    L->off_scratch = kCounterBytes;
    const int64_t scratch = p.nslices > 1 ? (int64_t)panels * p.nslices * 2 * p.M * TKD_PANEL_COLS * 4 : 0;
    L->off_ytmp = align_up(L->off_scratch + scratch, 256);
    p.ld_ytmp = (int64_t)panels * TKD_PANEL_COLS;
    const int64_t ytmp = a->topk_k && !a->topk_write_y ? (int64_t)a->topk_rows * p.ld_ytmp * 2 : 0;
    L->ws_bytes = align_up(L->off_ytmp + ytmp, 256);
    return TKD_OK;
}

}  // namespace

extern "C" {

int tkd_version(void) { return 3; }

int tkd_layout_version(void) { return TKD_LAYOUT_VERSION; }

int tkd_struct_bytes(int which) {
    return which == 0 ? (int)sizeof(TkdMatmul) : which == 1 ? (int)sizeof(TkdPlan) : which == 2 ? (int)sizeof(TkdBlock) : which == 3 ? (int)sizeof(TkdMoe) : 0;
}

const char* tkd_error_string(int code) {
    switch (code) {
        case TKD_OK: return "ok";
        case TKD_ERR_BAD_ARG: return "bad argument";
        case TKD_ERR_UNSUPPORTED: return "unsupported";
        case TKD_ERR_TIMEOUT: return "a kernel's bounded wait gave up";
        case TKD_ERR_WORKSPACE: return "workspace missing or too small";
        case TKD_ERR_WIDE: return "exponent spread inside a column group too wide for the stream";
        case TKD_ERR_FIXED_SCRATCH: return "the call needs more scratch than tkd_matmul_noalloc's built-in array holds";
        default: return code > TKD_ERR_CUDA ? cudaGetErrorString((cudaError_t)(code - TKD_ERR_CUDA)) : "unknown";
    }
}

int64_t tkd_padded_cols(int64_t n) { return (n + 127) / 128 * 128; }

int64_t tkd_packed_bytes(int fmt, int64_t k, int64_t n) {
    return fmt_ok(fmt) ? tkd_stream_bytes(fmt, k, tkd_padded_cols(n)) : -1;
}

int tkd_quantise(int fmt, const float* src, int orient, int64_t k, int64_t n, const float* col_div, uint8_t* exps,
                 void* codes, void* stream) {
    if (!fmt_ok(fmt) || fmt == TKD_INT4 || !src || !codes || k < 1 || n < 1 || (fmt != TKD_BF16 && !exps) ||
        (orient != 0 && orient != 1))
        return TKD_ERR_BAD_ARG;
    return launch_err(tkd_launch_quantise(fmt, src, orient, k, n, tkd_padded_cols(n), col_div, exps, codes,
                                          static_cast<cudaStream_t>(stream)));
}

int tkd_pack(int fmt, int64_t k, int64_t n, const uint8_t* exps, const void* codes, void* packed, uint8_t* emax,
             int32_t* info, void* stream) {
    if (!fmt_ok(fmt) || !codes || !packed || k < 1 || n < 1) return TKD_ERR_BAD_ARG;
    if (has_emax(fmt) && (!exps || !emax || !info)) return TKD_ERR_BAD_ARG;
    if (fmt == TKD_INT4 && !exps) return TKD_ERR_BAD_ARG;  // (the group scales)
    return launch_err(tkd_launch_permute(fmt, k, tkd_padded_cols(n), exps, codes, emax, info, packed,
                                         static_cast<cudaStream_t>(stream)));
}

int tkd_dequantise_bf16(int fmt, int64_t k, int64_t n, const uint8_t* exps, const void* codes, void* out_bf16, void* stream) {
    if ((fmt != TKD_BFP8 && fmt != TKD_BFP4) || !exps || !codes || !out_bf16 || k < 1 || n < 1) return TKD_ERR_BAD_ARG;
    return launch_err(tkd_launch_dequantise_bf16(fmt, k, tkd_padded_cols(n), exps, codes, out_bf16,
                                                 static_cast<cudaStream_t>(stream)));
}

int tkd_unpack(int fmt, int64_t k, int64_t n, const void* packed, const uint8_t* emax, float* out, void* stream) {
    if (!fmt_ok(fmt) || !packed || !out || k < 1 || n < 1 || (has_emax(fmt) && !emax)) return TKD_ERR_BAD_ARG;
    return launch_err(
        tkd_launch_unpack(fmt, k, tkd_padded_cols(n), packed, emax, out, static_cast<cudaStream_t>(stream)));
}

int tkd_matmul_plan(const TkdMatmul* a, TkdPlan* plan) {
    Layout L;
    if (!plan) return TKD_ERR_BAD_ARG;
    // (no device needed: without one the plan is made for 148 SMs)
    int sms = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        (void)cudaGetLastError();
        sms = 148;
    }
    const int rc = make_layout(a, &L, sms);
    if (rc) return rc;
    plan->ks = L.p.ks;
    plan->nslices = L.p.nslices;
    plan->panels = L.p.total_panels;
    plan->grid = L.grid;
    plan->stages = L.p.nstages;
    plan->stream_warps = TKD_STREAM_WARPS;
    plan->chunk_k = tkd_chunk_k(L.p.fmt);
    plan->smem_bytes = (int32_t)L.smem;
    plan->items = L.p.total_items;
    plan->weight_bytes = L.weight_bytes;
    return TKD_OK;
}

int tkd_matmul_workspace(const TkdMatmul* a, uint64_t* bytes) {
    Layout L;
    if (!bytes) return TKD_ERR_BAD_ARG;
    int sms = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        (void)cudaGetLastError();
        sms = 148;
    }
    const int rc = make_layout(a, &L, sms);
    if (rc) return rc;
    *bytes = (uint64_t)L.ws_bytes;
    return TKD_OK;
}

static int run_matmul(const TkdMatmul* a, void* workspace, uint64_t workspace_bytes, void* stream) {
    Layout L;
    const int rc = make_layout(a, &L, 0);
    if (rc) return rc;
    TkdParams& p = L.p;
    if (!a->x || !a->out || a->ldx < a->k || a->ldx % 8 || (reinterpret_cast<uintptr_t>(a->x) & 15)) return TKD_ERR_BAD_ARG;
    for (int s = 0; s < a->nblocks; ++s) {
        const TkdBlock& b = a->block[s];
        if (!b.w || (reinterpret_cast<uintptr_t>(b.w) & 15)) return TKD_ERR_BAD_ARG;
        if (has_emax(a->fmt) && !b.emax) return TKD_ERR_BAD_ARG;
        if (a->epilogue == TKD_EPI_GLU2) {
            if (!b.w_up || (reinterpret_cast<uintptr_t>(b.w_up) & 15) || (has_emax(a->fmt) && !b.emax_up))
                return TKD_ERR_BAD_ARG;
        }
        const int64_t width = a->epilogue == TKD_EPI_GLU_IL ? b.n / 2 : b.n;
        if (b.out_col0 + width > a->ldo) return TKD_ERR_BAD_ARG;
    }
    if (a->scale_dtype != TKD_DT_NONE) {
        if (!a->scale || (a->epilogue == TKD_EPI_GLU2 && !a->scale_up)) return TKD_ERR_BAD_ARG;
        if (a->scale_dtype != TKD_DT_BF16 && a->scale_dtype != TKD_DT_F32) return TKD_ERR_BAD_ARG;
    }
    if (a->epilogue == TKD_EPI_RESIDUAL && (!a->residual || a->residual_dtype != TKD_DT_BF16)) return TKD_ERR_BAD_ARG;
    if (a->epilogue == TKD_EPI_OUT32 && a->residual && a->residual_dtype != TKD_DT_F32) return TKD_ERR_BAD_ARG;
    if (a->epilogue != TKD_EPI_RESIDUAL && a->epilogue != TKD_EPI_OUT32 && a->residual) return TKD_ERR_BAD_ARG;
    if (a->topk_k && !a->records) return TKD_ERR_BAD_ARG;
    if (!workspace || workspace_bytes < (uint64_t)L.ws_bytes) return TKD_ERR_WORKSPACE;
    if (workspace && (reinterpret_cast<uintptr_t>(workspace) & 255)) return TKD_ERR_BAD_ARG;

    p.x = static_cast<const uint16_t*>(a->x);
    p.ldx = a->ldx;
    p.scale = a->scale;
    p.scale2 = a->scale_up;
    p.scale_dt = a->scale_dtype;
    p.res = a->residual;
    p.res_dt = a->residual ? a->residual_dtype : TKD_DT_NONE;
    p.ldr = a->ldr;
    p.out = a->out;
    p.out_dt = a->out_dtype;
    p.ldo = a->ldo;
    p.records = static_cast<uint32_t*>(a->records);
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    p.counters = reinterpret_cast<int*>(ws + L.off_counters);
    p.unit_counters = reinterpret_cast<int*>(ws + L.off_units);
    p.scratch = reinterpret_cast<float*>(ws + L.off_scratch);
    p.ytmp = reinterpret_cast<uint16_t*>(ws + L.off_ytmp);
    p.status = a->status;
    p.no_pdl = a->weights_fresh != 0;
    if (a->hadamard) {
        if (a->fmt != TKD_INT4 || a->k % 1024 || !p.x_smem) return TKD_ERR_UNSUPPORTED;
        if (reinterpret_cast<uintptr_t>(a->hadamard) & 15) return TKD_ERR_BAD_ARG;
        p.had = a->hadamard;
    }
    if (a->nranks > 1) {
        if (!a->flags) return TKD_ERR_BAD_ARG;
        p.npeers = a->nranks - 1;
        p.rank = a->rank;
        for (int q = 0; q < p.npeers; ++q) {
            if (!a->peer_flags[q]) return TKD_ERR_BAD_ARG;
            p.peer_out[q] = a->peer_out[q];
            p.peer_records[q] = static_cast<uint32_t*>(a->peer_records[q]);
            p.peer_flags[q] = a->peer_flags[q];
        }
        p.flags = a->flags;
        p.grid_counter = reinterpret_cast<int*>(ws + L.off_misc);
        p.exchange_wait = a->exchange_wait;
    }
    return launch_err(tkd_launch_stream(p, L.grid, L.smem, static_cast<cudaStream_t>(stream)));
}

int tkd_matmul(const TkdMatmul* a, void* stream) {
    if (!a) return TKD_ERR_BAD_ARG;
    return run_matmul(a, a->workspace, a->workspace_bytes, stream);
}

int tkd_matmul_host(const TkdMatmul* a, const void* x_host, void* out_host, void* stream) {
    if (!a || !x_host || !out_host || !a->x || !a->out) return TKD_ERR_BAD_ARG;
    if (a->ldx != a->k) return TKD_ERR_BAD_ARG;  // the staging copy of x is one contiguous block
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(const_cast<void*>(a->x), x_host, (size_t)a->m * a->k * 2, cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return cuda_err(e);
    const int rc = run_matmul(a, a->workspace, a->workspace_bytes, stream);
    if (rc) return rc;
    const size_t esz = a->out_dtype == TKD_DT_F32 ? 4 : 2;
    e = cudaMemcpyAsync(out_host, a->out, (size_t)a->m * a->ldo * esz, cudaMemcpyDeviceToHost, st);
    return cuda_err(e);
}

// ---- tkd_matmul for callers that must not allocate ----------------------------------------------------------------
// The same launch as tkd_matmul, with the kernel's workspace (its panel and unit counters, the slice sums of panels
// spread over several CTAs, the bf16 outputs of a top-k call that writes no y) taken from an array that is part of
// the library's device image instead of from the caller. Every GPU that loads libtkd holds these
// TKD_NOALLOC_SCRATCH_BYTES until the process exits.
//
// tkd_noalloc_scratch below is the HOST-side handle of that array: passing it to a kernel would hand the GPU a host
// address. The array's address on a device comes from cudaGetSymbolAddress, asked once per device with that device
// current, and that address is what the kernel gets.
static __device__ __align__(256) unsigned char tkd_noalloc_scratch[TKD_NOALLOC_SCRATCH_BYTES];

// The array's address on the current device, resolved on first use (a thread that loses the race to publish it has
// resolved the same address). first: set when this call was the one that resolved it.
static int noalloc_address(void** out, bool* first) {
    static std::atomic<void*> dev_ptr[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_err(e);
    if (dev < 0 || dev >= 64) return TKD_ERR_UNSUPPORTED;
    void* ptr = dev_ptr[dev].load(std::memory_order_acquire);
    if (first) *first = false;
    if (!ptr) {
        e = cudaGetSymbolAddress(&ptr, tkd_noalloc_scratch);
        if (e != cudaSuccess) return cuda_err(e);
        void* expected = nullptr;
        if (dev_ptr[dev].compare_exchange_strong(expected, ptr, std::memory_order_acq_rel) && first) *first = true;
    }
    *out = ptr;
    return TKD_OK;
}

int tkd_matmul_noalloc(const TkdMatmul* a, void* stream) {
    Layout L;
    const int rc = make_layout(a, &L, 0);
    if (rc) return rc;
    if ((uint64_t)L.ws_bytes > (uint64_t)TKD_NOALLOC_SCRATCH_BYTES) return TKD_ERR_FIXED_SCRATCH;
    void* ptr = nullptr;
    bool first = false;
    const int ra = noalloc_address(&ptr, &first);
    if (ra) return ra;
    if (first) {
        // first call on this device: the array's counters start from zero
        const cudaError_t e = cudaMemsetAsync(ptr, 0, (size_t)kCounterBytes, static_cast<cudaStream_t>(stream));
        if (e != cudaSuccess) return cuda_err(e);
    }
    return run_matmul(a, ptr, TKD_NOALLOC_SCRATCH_BYTES, stream);
}

int tkd_matmul_noalloc_reset(void* stream) {
    void* ptr = nullptr;
    const int ra = noalloc_address(&ptr, nullptr);
    if (ra) return ra;
    return cuda_err(cudaMemsetAsync(ptr, 0, (size_t)kCounterBytes, static_cast<cudaStream_t>(stream)));
}

int tkd_noalloc_scratch_address(void** ptr) {
    if (!ptr) return TKD_ERR_BAD_ARG;
    return noalloc_address(ptr, nullptr);
}

int tkd_hadamard(const void* x, int64_t ldx, const uint32_t* signs, int rows, int k, void* out, int64_t ldo, void* stream) {
    if (!x || !signs || !out || rows < 1 || rows > 65535 || k < 1024 || k % 1024 || ldx < k || ldo < k || (ldx | ldo) % 4)
        return TKD_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(signs)) & 7)
        return TKD_ERR_BAD_ARG;
    return launch_err(tkd_launch_hadamard(x, ldx, signs, rows, k, out, ldo, static_cast<cudaStream_t>(stream)));
}

int tkd_topk_merge(const uint32_t* records, int nrecords, int rows, int k, int top, uint32_t* out, void* stream) {
    if (!records || !out || nrecords < 1 || rows < 1 || rows > 16 || k < 1 || rows * k > 64 || top < 1 || top > 1024)
        return TKD_ERR_BAD_ARG;
    if ((int64_t)nrecords * k > (1 << 24)) return TKD_ERR_BAD_ARG;
    return launch_err(tkd_launch_topk_merge(records, nrecords, rows, k, top, out, static_cast<cudaStream_t>(stream)));
}

int tkd_head_pick(const uint32_t* records, int nrecords, int rows, int k, int top, uint32_t vocab, const void* x,
                  int64_t ldx, int dim, const void* head_rows, int64_t ld_head, int round_bf16, uint32_t* out,
                  uint32_t* ids_out, void* stream) {
    if (!records || !out || !x || !head_rows || nrecords < 1 || rows < 1 || rows > 32 || k < 1 || top < 1 || top > 32)
        return TKD_ERR_BAD_ARG;
    if (dim < 8 || dim % 8 || ldx < dim || ldx % 8 || ld_head < dim || ld_head % 8 || vocab < 1) return TKD_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(head_rows)) & 15) return TKD_ERR_BAD_ARG;
    if ((int64_t)nrecords * k > (1 << 24)) return TKD_ERR_BAD_ARG;
    return launch_err(tkd_launch_head_pick(records, nrecords, rows, k, top, vocab, static_cast<const uint16_t*>(x), ldx, dim,
                                           static_cast<const uint16_t*>(head_rows), ld_head, round_bf16, out, ids_out,
                                           static_cast<cudaStream_t>(stream)));
}

int tkd_head_pick_records(const uint32_t* records, int nrecords, int rows, int k, uint32_t vocab, const uint32_t* token_map,
                          uint32_t* out, uint32_t* ids_out, void* stream) {
    if (!records || !out || nrecords < 1 || rows < 1 || rows > 32 || k < 1 || vocab < 1) return TKD_ERR_BAD_ARG;
    if ((int64_t)nrecords * k > (1 << 24)) return TKD_ERR_BAD_ARG;
    return launch_err(tkd_launch_head_pick_records(records, nrecords, rows, k, vocab, token_map, out, ids_out,
                                                   static_cast<cudaStream_t>(stream)));
}

// ---- exchange between GPUs -------------------------------------------------------------------------------------------

int tkd_exchange_wait(uint32_t* flags, int nranks, int32_t* status, void* stream) {
    if (!flags || nranks < 1 || nranks > TKD_MAX_RANKS) return TKD_ERR_BAD_ARG;
    return launch_err(tkd_launch_exchange_wait(flags, nranks, status, static_cast<cudaStream_t>(stream)));
}

int tkd_exchange_publish(uint32_t* flags, uint32_t* const* peer_flags, int nranks, int rank, int lag_wait, int32_t* status,
                         void* stream) {
    if (!flags || !peer_flags || nranks < 2 || nranks > TKD_MAX_RANKS || rank < 0 || rank >= nranks) return TKD_ERR_BAD_ARG;
    TkdPeerFlags pf = {};
    for (int q = 0; q < nranks - 1; ++q) {
        if (!peer_flags[q]) return TKD_ERR_BAD_ARG;
        pf.p[q] = peer_flags[q];
    }
    return launch_err(tkd_launch_exchange_publish(flags, pf, nranks, rank, lag_wait, status, static_cast<cudaStream_t>(stream)));
}

int tkd_peer_alloc(uint64_t bytes, void** ptr, void* handle) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is 64 bytes");
    if (!bytes || !ptr || !handle) return TKD_ERR_BAD_ARG;
    void* d = nullptr;
    cudaError_t e = cudaMalloc(&d, (size_t)bytes);
    if (e != cudaSuccess) return cuda_err(e);
    e = cudaMemset(d, 0, (size_t)bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, d);
    if (e != cudaSuccess) {
        (void)cudaFree(d);
        return cuda_err(e);
    }
    memcpy(handle, &h, sizeof(h));
    *ptr = d;
    return TKD_OK;
}

int tkd_peer_free(void* ptr) { return ptr ? cuda_err(cudaFree(ptr)) : TKD_ERR_BAD_ARG; }

int tkd_peer_open(const void* handle, void** ptr) {
    if (!handle || !ptr) return TKD_ERR_BAD_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    return cuda_err(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
}

int tkd_peer_close(void* ptr) { return ptr ? cuda_err(cudaIpcCloseMemHandle(ptr)) : TKD_ERR_BAD_ARG; }

}  // extern "C"
