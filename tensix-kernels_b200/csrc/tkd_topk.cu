// tkd_topk.cu: the best `top` candidates of every row out of a set of top-k records (include/tkd.h: tkd_topk_merge).
//
// One CTA per row. A candidate is (key, index); the order is key descending, index ascending among equal keys, which
// is total (indices are distinct), so every GPU merging the same records gets the same answer. Packed as
// key << 32 | ~index the order is that of 64-bit integers. The candidates (records * k of them, 600 for the
// 151936-column LM head) are held by the threads in a strided fashion; `top` rounds each pick the largest candidate
// below the one picked before: a maximum over the thread's own, a warp shuffle reduction, one exchange through shared
// memory.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tkd_internal.h"

namespace {

constexpr int kThreads = 256;
constexpr int kOwn = 4;  // candidates a thread keeps in registers; more are re-read from memory every round

__global__ void __launch_bounds__(kThreads) tkd_topk_merge_kernel(const uint32_t* __restrict__ records, int nrec, int rows,
                                                                  int k, int top, uint32_t* __restrict__ out) {
    __shared__ unsigned long long red[kThreads / 32];
    // (launched as a programmatic dependent of the kernel before it, normally the stream kernel that writes the
    // records: let the kernel after this one start its CTAs, then wait for the records to be complete)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n = nrec * k;
    auto cand = [&](int c) -> unsigned long long {
        const int rec = c / k, q = c - rec * k;
        const uint32_t* page = records + (size_t)rec * 2 * rows * k;
        const uint32_t key = __ldg(page + r * k + q), idx = __ldg(page + (rows + r) * k + q);
        return key ? ((unsigned long long)key << 32) | (uint32_t)~idx : 0ull;  // (0: an empty slot)
    };
    unsigned long long own[kOwn];
#pragma unroll
    for (int j = 0; j < kOwn; ++j) own[j] = tid + j * kThreads < n ? cand(tid + j * kThreads) : 0ull;
    unsigned long long bound = ~0ull;
    for (int t = 0; t < top; ++t) {
        unsigned long long best = 0;
#pragma unroll
        for (int j = 0; j < kOwn; ++j)
            if (own[j] < bound && own[j] > best) best = own[j];
        for (int c = tid + kOwn * kThreads; c < n; c += kThreads) {
            const unsigned long long v = cand(c);
            if (v < bound && v > best) best = v;
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xFFFFFFFFu, best, o);
            best = other > best ? other : best;
        }
        if (lane == 0) red[warp] = best;
        __syncthreads();
        best = red[0];
#pragma unroll
        for (int w = 1; w < kThreads / 32; ++w) best = red[w] > best ? red[w] : best;
        __syncthreads();
        if (tid == 0) {
            out[r * top + t] = (uint32_t)(best >> 32);
            out[(rows + r) * top + t] = best ? ~(uint32_t)best : 0xFFFFFFFFu;
        }
        bound = best;  // (0: nothing left; the remaining slots come out empty)
    }
}

// The same for up to kWarpMax candidates a row (the LM head's 600): one warp, the candidates in registers (32 a lane,
// fetched with all their loads in flight), and per round two warp-wide reductions in hardware (redux.sync) instead of
// ten shuffles: the largest key, then among the lanes holding it the largest ~index.
constexpr int kWarpMax = 1024;
__global__ void __launch_bounds__(32) tkd_topk_merge_warp_kernel(const uint32_t* __restrict__ records, int nrec, int rows,
                                                                 int k, int top, uint32_t* __restrict__ out) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int r = blockIdx.x, lane = threadIdx.x;
    const int n = nrec * k;
    unsigned long long own[kWarpMax / 32];
#pragma unroll
    for (int j = 0; j < kWarpMax / 32; ++j) {
        const int c = lane + 32 * j;
        own[j] = 0ull;
        if (c < n) {
            const int rec = c / k, q = c - rec * k;
            const uint32_t* page = records + (size_t)rec * 2 * rows * k;
            const uint32_t key = __ldg(page + r * k + q), idx = __ldg(page + (rows + r) * k + q);
            own[j] = key ? ((unsigned long long)key << 32) | (uint32_t)~idx : 0ull;
        }
    }
    unsigned long long bound = ~0ull;
    for (int t = 0; t < top; ++t) {
        unsigned long long mine = 0;
#pragma unroll
        for (int j = 0; j < kWarpMax / 32; ++j)
            if (own[j] < bound && own[j] > mine) mine = own[j];
        const uint32_t key = __reduce_max_sync(0xFFFFFFFFu, (uint32_t)(mine >> 32));
        const uint32_t low = __reduce_max_sync(0xFFFFFFFFu, key && (uint32_t)(mine >> 32) == key ? (uint32_t)mine : 0u);
        const unsigned long long best = key ? ((unsigned long long)key << 32) | low : 0ull;
        if (lane == 0) {
            out[r * top + t] = key;
            out[(rows + r) * top + t] = best ? ~low : 0xFFFFFFFFu;
        }
        bound = best;  // (0: nothing left; the remaining slots come out empty)
    }
}

}  // namespace

int tkd_launch_topk_merge(const uint32_t* records, int nrec, int rows, int k, int top, uint32_t* out, cudaStream_t st) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)rows);
    cfg.blockDim = dim3(kThreads);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (nrec * k <= kWarpMax) {
        cfg.blockDim = dim3(32);
        return (int)cudaLaunchKernelEx(&cfg, tkd_topk_merge_warp_kernel, records, nrec, rows, k, top, out);
    }
    return (int)cudaLaunchKernelEx(&cfg, tkd_topk_merge_kernel, records, nrec, rows, k, top, out);
}

// ---- the LM head's rescore and pick (include/tkd.h: tkd_head_pick, tkd_head_pick_records) --------------------------
namespace {

// a float's bits as an unsigned key in the float order: NaN above everything, -0 equal to +0 (torch's compare)
__device__ __forceinline__ uint32_t order32(uint32_t b) {
    if ((b & 0x7FFFFFFFu) == 0) b = 0;
    if ((b & 0x7F800000u) == 0x7F800000u && (b & 0x007FFFFFu)) return 0xFFFFFFFFu;
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
// a record key's rank for the records-only pick: a NaN of either sign above every key, -0 equal to +0 (key != 0)
__device__ __forceinline__ uint32_t rank16(uint32_t kk) {
    const uint32_t mag = (kk >= 0x8000u ? kk : ~kk) & 0x7FFFu;
    if ((mag & 0x7F80u) == 0x7F80u && (mag & 0x007Fu)) return 0x10000u;
    return kk == 0x7FFFu ? 0x8000u : kk;
}

// One CTA per row r of the step.
//   1. The best `top` slots of row r over the records in order (record by record, slot by slot), by key (RECORDS: by
//      rank16, and top is 1); an equal key keeps the earlier slot; a slot with key 0 or an id at or past `vocab` is empty.
//   2. (not RECORDS) Their exact logits: bf16 x row times the candidates' bf16 head rows, float32 sums (a warp per
//      candidate: every lane sums its 8-element pieces in order, then a shuffle tree), rounded to bf16 with `round`.
//   3. The pick: the largest logit (order32), the lowest id among equals. Row r of out (32 words):
//      [token, the first candidate by the device's own logit, count, 0 ...]; count is the candidates held (RECORDS: all
//      valid slots). No valid slot: [0, 0xFFFFFFFF, 0].
template <bool RECORDS>
__global__ void __launch_bounds__(kThreads) tkd_head_pick_kernel(const uint32_t* __restrict__ records, int nrec, int rows,
                                                                 int k, int top, uint32_t vocab,
                                                                 const uint16_t* __restrict__ x, int64_t ldx, int dim,
                                                                 const uint16_t* __restrict__ head, int64_t ld_head,
                                                                 int round, const uint32_t* __restrict__ tmap,
                                                                 uint32_t* __restrict__ out, uint32_t* __restrict__ ids_out) {
    __shared__ unsigned long long red[kThreads / 32];
    __shared__ uint32_t cid[32], clogit[32];
    __shared__ int held, nvalid[kThreads / 32];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n = nrec * k;
    auto slot = [&](int c, uint32_t& id) -> uint32_t {
        const int rec = c / k, q = c - rec * k;
        const uint32_t* page = records + (size_t)rec * 2 * rows * k;
        const uint32_t key = __ldg(page + r * k + q) & 0xFFFFu;
        id = __ldg(page + (rows + r) * k + q);
        return key && id < vocab ? key : 0u;
    };
    // packed (rank, ~position): the 64-bit order is "larger rank first, earlier slot first"
    auto packed = [&](int c) -> unsigned long long {
        uint32_t id;
        const uint32_t key = slot(c, id);
        return key ? ((unsigned long long)(RECORDS ? rank16(key) : key) << 32) | (uint32_t)~(uint32_t)c : 0ull;
    };
    int mine = 0;
    for (int c = tid; c < n; c += kThreads) mine += packed(c) != 0;
#pragma unroll
    for (int o = 16; o; o >>= 1) mine += __shfl_xor_sync(0xFFFFFFFFu, mine, o);
    if (lane == 0) nvalid[warp] = mine;
    if (tid == 0) held = 0;
    unsigned long long bound = ~0ull;
    for (int t = 0; t < top; ++t) {
        unsigned long long best = 0;
        for (int c = tid; c < n; c += kThreads) {
            const unsigned long long v = packed(c);
            if (v < bound && v > best) best = v;
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xFFFFFFFFu, best, o);
            best = other > best ? other : best;
        }
        if (lane == 0) red[warp] = best;
        __syncthreads();
        best = red[0];
#pragma unroll
        for (int w = 1; w < kThreads / 32; ++w) best = red[w] > best ? red[w] : best;
        if (tid == 0 && best) {
            uint32_t id;
            (void)slot((int)~(uint32_t)best, id);
            cid[t] = id;
            held = t + 1;
        }
        __syncthreads();
        bound = best;
        if (!best) break;
    }
    __syncthreads();
    const int nc = held;
    if constexpr (!RECORDS) {
        const uint16_t* xr = x + (size_t)r * ldx;
        for (int c = warp; c < nc; c += kThreads / 32) {
            const uint16_t* wr = head + (size_t)cid[c] * ld_head;
            float acc = 0.f;
            for (int d = lane * 8; d < dim; d += 256) {
                const uint4 wv = __ldg(reinterpret_cast<const uint4*>(wr + d));
                const uint4 xv = __ldg(reinterpret_cast<const uint4*>(xr + d));
                const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w}, xx[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    acc = fmaf(__uint_as_float(ww[e] << 16), __uint_as_float(xx[e] << 16), acc);
                    acc = fmaf(__uint_as_float(ww[e] & 0xFFFF0000u), __uint_as_float(xx[e] & 0xFFFF0000u), acc);
                }
            }
#pragma unroll
            for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
            if (lane == 0) {
                uint32_t bits = __float_as_uint(acc);
                if (round) bits = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(acc)) << 16;
                clogit[c] = order32(bits);
            }
        }
        __syncthreads();
    }
    if (tid == 0) {
        uint32_t best = 0xFFFFFFFFu, best_key = 0, count = (uint32_t)nc;
        bool any = false;
        if constexpr (RECORDS) {
            count = 0;
            for (int w = 0; w < kThreads / 32; ++w) count += (uint32_t)nvalid[w];
            if (nc) best = cid[0], any = true;
        } else {
            for (int c = 0; c < nc; ++c) {
                const uint32_t kk = clogit[c], id = cid[c];
                if (!any || kk > best_key || (kk == best_key && id < best)) best_key = kk, best = id, any = true;
            }
        }
        uint32_t tok = any ? best : 0u;
        if (RECORDS && any && tmap) tok = __ldg(tmap + best);
        uint32_t* o = out + (size_t)r * 32;
        o[0] = tok;
        o[1] = nc ? cid[0] : 0xFFFFFFFFu;
        o[2] = count;
        for (int w = 3; w < 32; ++w) o[w] = 0;
        if (ids_out && r == 0) ids_out[0] = tok;
    }
}

template <bool RECORDS>
int launch_pick(const uint32_t* records, int nrec, int rows, int k, int top, uint32_t vocab, const uint16_t* x, int64_t ldx,
                int dim, const uint16_t* head, int64_t ld_head, int round, const uint32_t* tmap, uint32_t* out,
                uint32_t* ids_out, cudaStream_t st) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)rows);
    cfg.blockDim = dim3(kThreads);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, tkd_head_pick_kernel<RECORDS>, records, nrec, rows, k, top, vocab, x, ldx, dim, head,
                                   ld_head, round, tmap, out, ids_out);
}

}  // namespace

int tkd_launch_head_pick(const uint32_t* records, int nrec, int rows, int k, int top, uint32_t vocab, const uint16_t* x,
                         int64_t ldx, int dim, const uint16_t* head, int64_t ld_head, int round, uint32_t* out,
                         uint32_t* ids_out, cudaStream_t st) {
    return launch_pick<false>(records, nrec, rows, k, top, vocab, x, ldx, dim, head, ld_head, round, nullptr, out, ids_out, st);
}

int tkd_launch_head_pick_records(const uint32_t* records, int nrec, int rows, int k, uint32_t vocab, const uint32_t* tmap,
                                 uint32_t* out, uint32_t* ids_out, cudaStream_t st) {
    return launch_pick<true>(records, nrec, rows, k, 1, vocab, nullptr, 0, 0, nullptr, 0, 0, tmap, out, ids_out, st);
}
