// tkd_topk.cu: the best `top` candidates of every row out of a set of top-k records (include/tkd.h: tkd_topk_merge).
//
// One CTA per row. A candidate is (key, index); the order is key descending, index ascending among equal keys, which
// is total (indices are distinct), so every GPU merging the same records gets the same answer. Packed as
// key << 32 | ~index the order is that of 64-bit integers. The candidates (records * k of them, 600 for the
// 151936-column LM head) are held by the threads in a strided fashion; `top` rounds each pick the largest candidate
// below the one picked before: a maximum over the thread's own, a warp shuffle reduction, one exchange through shared
// memory.
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
    cfg.numAttrs = tkd_pdl_enabled() ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, tkd_topk_merge_kernel, records, nrec, rows, k, top, out);
}
