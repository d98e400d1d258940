// tkd_stream.cu: the weight-streaming decode matmul for sm_100a.
//
// y[m, n] = sum_k x[m, k] * w[k, n] with its fused output stage, M <= 32 activation rows, the weight a packed HBM
// stream (tkd_layout.h). It takes the place of the reference's three Tensix kernels (dense_reader/kernels/
// dense_reader.cpp: the DRAM loads; dense_compute.cpp: matmul_block accumulation and the output stages;
// dense_writer.cpp: output writes and the running top-k) and of the work split linear.plan makes for them
// (dense_reader/linear.py:187-382).
//
// One persistent CTA per SM, three kinds of warps, coupled by mbarriers only:
//   warp 0        producer: 1-D bulk copies (TMA, no multicast) of the weight stream and of the activation slice into
//                 a ring of shared-memory stages;
//   warps 1-8     streaming warps: warp w multiplies 16 output columns (one group of the stream) over the k slice of
//                 the current item with mma.sync m16n8k16, the weights as A. Block-float codes go in as bf16
//                 subnormals (sign << 15 | magnitude) and the shared exponent is folded into the activations
//                 (x * 2^e' is exact), so a register of two weights costs one rotate and one AND;
//   warps 9-12    output warps (one thread per column of the 128-column panel): add the slice sums in ascending slice
//                 order, run the output stage (exponent factor, scales, SwiGLU/GeGLU, residual, rounding), write y,
//                 and keep the top-k records.
// A work item is (panel of 128 columns, k slice of ks). Items are numbered panel-major and cut into equal contiguous
// runs, one per CTA. Every slice sum starts from zero and the slices of a column are always added in ascending order
// with plain fp32 adds, in registers when one CTA holds all of a panel's slices and through a scratch buffer
// otherwise (the CTA that delivers a panel's last slices adds them up): a column's result depends on K, the format
// and M's bucket only, never on N, on the number of CTAs or on the other weights of a block list.
//
// Every wait is bounded: a wait that gives up records TKD_ERR_TIMEOUT in the status word, and every role then falls
// through to the end of the kernel.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tkd_internal.h"
#include "tkd_layout.h"

namespace {

constexpr uint32_t kSpinLimit = 1u << 22;  // try_wait rounds before a wait gives up (each suspends for a while)
constexpr int kStatusTimeout = 3;          // TKD_ERR_TIMEOUT of include/tkd.h

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: false (and the status word set) when the phase never completes.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status) {
    for (uint32_t i = 0; i < kSpinLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    if (status) atomicExch(status, kStatusTimeout);
    return false;
}
// global -> shared bulk copy (TMA, 1-D, this CTA only), completion counted in bytes on an mbarrier
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ uint32_t rotr32(uint32_t v, int s) { return __funnelshift_r(v, v, s); }
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void bar_output_warps() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float v) { return __bfloat16_as_ushort(__float2bfloat16_rn(v)); }

// dense_ops.h:44-59 of the reference: silu, and gelu_tanh as x * sigmoid(2 u), u = sqrt(2 / pi) (x + 0.044715 x^3)
__device__ __forceinline__ float act_gate(float g, int act) {
    const float u = act ? g * (1.5957691216f + 0.0713548162f * (g * g)) : g;
    return g / (1.f + __expf(-u));
}

struct ItemInfo {
    int panel, slice, k0, kv, seg, pl;
};
__device__ __forceinline__ ItemInfo item_info(const TkdParams& p, int64_t it) {
    ItemInfo I;
    I.panel = (int)(it / p.nslices);
    I.slice = (int)(it - (int64_t)I.panel * p.nslices);
    I.k0 = I.slice * p.ks;
    I.kv = min(p.ks, p.K - I.k0);
    I.seg = 0;
#pragma unroll
    for (int s = 1; s < 4; ++s)
        if (s < p.nseg && I.panel >= p.seg[s].panel0) I.seg = s;
    I.pl = I.panel - p.seg[I.seg].panel0;
    return I;
}
// The group of 16 columns streaming warp w of a panel works on: its run's base, or null when the panel has none.
__device__ __forceinline__ const uint8_t* warp_run(const TkdParams& p, const ItemInfo& I, int w) {
    const TkdSegDev& s = p.seg[I.seg];
    if (p.epi == TKD_EPI_GLU2) {
        const int g = I.pl * 4 + (w & 3);
        if (g >= s.groups) return nullptr;
        return (w < 4 ? s.w : s.w2) + (int64_t)g * p.run_bytes;
    }
    const int g = I.pl * 8 + w;
    return g < s.groups ? s.w + (int64_t)g * p.run_bytes : nullptr;
}

template <int FMT>
struct Fmt;
template <>
struct Fmt<TKD_BFP8> {
    static constexpr int KSA = 32, SAB = 544;
};
template <>
struct Fmt<TKD_BFP4> {
    static constexpr int KSA = 64, SAB = 576;
};
template <>
struct Fmt<TKD_BF16> {
    static constexpr int KSA = 32, SAB = 1024;
};

// One chunk (nsa super-atoms of one group) times the activation slice rows in shared memory.
// xrow[tile]: this lane's row of x (row 8 tile + lane / 4) at the slice's first k, or null beyond M.
template <int FMT, int MT>
__device__ __forceinline__ void chunk_mma(float (&acc)[MT][4], const uint8_t* sub, int nsa, int kk0, int kv,
                                          const uint8_t* const (&xrow)[MT], int lane) {
    const int t = lane & 3;
    for (int sa = 0; sa < nsa; ++sa) {
        const uint8_t* b = sub + sa * Fmt<FMT>::SAB;
        const int kk = kk0 + sa * Fmt<FMT>::KSA;
        if constexpr (FMT == TKD_BFP4) {
            const uint4 ev = *reinterpret_cast<const uint4*>(b + t * 16);
            const uint4 cv = *reinterpret_cast<const uint4*>(b + 64 + lane * 16);
            const uint32_t ew[4] = {ev.x, ev.y, ev.z, ev.w}, cw[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
            for (int qq = 0; qq < 2; ++qq) {
                if (kk + 32 * qq >= kv) break;  // a K that ends in the middle of a super-atom
                uint4 xv[MT];
#pragma unroll
                for (int m = 0; m < MT; ++m)
                    xv[m] = xrow[m] ? *reinterpret_cast<const uint4*>(xrow[m] + (kk + 32 * qq + 8 * t) * 2)
                                    : make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int jj = 0; jj < 2; ++jj) {
                    const uint32_t w = cw[2 * qq + jj], e = ew[2 * qq + jj];
                    const uint32_t a0 = w & 0x80078007u, a1 = rotr32(w, 4) & 0x80078007u;
                    const uint32_t a2 = rotr32(w, 8) & 0x80078007u, a3 = rotr32(w, 12) & 0x80078007u;
                    const uint32_t s0 = e & 0x7F807F80u, s1 = rotr32(e, 8) & 0x7F807F80u;
#pragma unroll
                    for (int m = 0; m < MT; ++m)
                        mma_bf16(acc[m], a0, a1, a2, a3, mul_bf16x2(jj ? xv[m].z : xv[m].x, s0),
                                 mul_bf16x2(jj ? xv[m].w : xv[m].y, s1));
                }
            }
        } else if constexpr (FMT == TKD_BFP8) {
            const uint2 ev = *reinterpret_cast<const uint2*>(b + t * 8);
            const uint4 cv = *reinterpret_cast<const uint4*>(b + 32 + lane * 16);
            uint4 xv[MT];
#pragma unroll
            for (int m = 0; m < MT; ++m)
                xv[m] = xrow[m] ? *reinterpret_cast<const uint4*>(xrow[m] + (kk + 8 * t) * 2) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
                const uint32_t w0 = jj ? cv.z : cv.x, w1 = jj ? cv.w : cv.y, e = jj ? ev.y : ev.x;
                const uint32_t a0 = w0 & 0x807F807Fu, a1 = rotr32(w0, 8) & 0x807F807Fu;
                const uint32_t a2 = w1 & 0x807F807Fu, a3 = rotr32(w1, 8) & 0x807F807Fu;
                const uint32_t s0 = e & 0x7F807F80u, s1 = rotr32(e, 8) & 0x7F807F80u;
#pragma unroll
                for (int m = 0; m < MT; ++m)
                    mma_bf16(acc[m], a0, a1, a2, a3, mul_bf16x2(jj ? xv[m].z : xv[m].x, s0),
                             mul_bf16x2(jj ? xv[m].w : xv[m].y, s1));
            }
        } else {
            uint4 xv[MT];
#pragma unroll
            for (int m = 0; m < MT; ++m)
                xv[m] = xrow[m] ? *reinterpret_cast<const uint4*>(xrow[m] + (kk + 8 * t) * 2) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
                const uint4 a = *reinterpret_cast<const uint4*>(b + jj * 512 + lane * 16);
#pragma unroll
                for (int m = 0; m < MT; ++m)
                    mma_bf16(acc[m], a.x, a.y, a.z, a.w, jj ? xv[m].z : xv[m].x, jj ? xv[m].w : xv[m].y);
            }
        }
    }
}

// bf16 output as the top-k records order it: a monotone 16-bit key, 0 below every value (dense_writer.cpp:215).
__device__ __forceinline__ uint32_t topk_key(uint16_t b) {
    return (uint32_t)(b ^ (0x8000u | (0x7FFFu & (0u - (uint32_t)(b >> 15))))) & 0xFFFFu;
}

template <int FMT, int MT>
__global__ void __launch_bounds__(TKD_THREADS, 1) tkd_stream_kernel(const TkdParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int MP = MT == 1 ? 8 : (MT == 2 ? 24 : 40);  // floats per column in the partial buffers
    constexpr int MR = 8 * MT;                             // rows the accumulators cover
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + TKD_MAX_STAGES);
    const uint32_t xempty0 = smem_u32(bars + 2 * TKD_MAX_STAGES);
    const uint32_t pfull0 = smem_u32(bars + 2 * TKD_MAX_STAGES + TKD_MAX_XSLOTS), pempty0 = pfull0 + 16;
    volatile int* sflag = reinterpret_cast<volatile int*>(smem + TKD_SMEM_HEAD - 16);
    uint8_t* xbuf = smem + p.off_x;
    float* pbuf = reinterpret_cast<float*>(smem + p.off_pbuf);
    float* tbuf = reinterpret_cast<float*>(smem + p.off_tbuf);
    uint8_t* ring = smem + p.off_ring;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < p.nstages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 8);
        }
        for (int s = 0; s < p.xslots; ++s) mbar_init(xempty0 + 8 * s, 8);
        for (int s = 0; s < 2; ++s) {
            mbar_init(pfull0 + 8 * s, 8);
            mbar_init(pempty0 + 8 * s, 4);
        }
        sflag[0] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const int64_t T = p.total_items;
    const int64_t i0 = T * blockIdx.x / gridDim.x, i1 = T * (blockIdx.x + 1) / gridDim.x;
    const int nst = p.nstages, xsl = p.xslots;
    const int M = p.M;

    if (warp == 0) {
        // ---------------------------------------------------------------- producer
        uint32_t st = 0, xi = 0;
        bool ok = true;
        for (int64_t it = i0; it < i1 && ok; ++it, ++xi) {
            const ItemInfo I = item_info(p, it);
            const uint8_t* run = lane < 8 ? warp_run(p, I, lane) : nullptr;
            const int nvalid = __popc(__ballot_sync(0xFFFFFFFFu, run != nullptr));
            const uint32_t xs = xi % xsl;
            if (lane == 0) ok = mbar_wait(xempty0 + 8 * xs, ((xi / xsl) & 1) ^ 1, p.status);
            ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
            if (!ok) break;
            const int nsa_total = (I.kv + Fmt<FMT>::KSA - 1) / Fmt<FMT>::KSA;
            const int sa0 = I.k0 / Fmt<FMT>::KSA;
            const int nch = (nsa_total + p.subsa - 1) / p.subsa;
            for (int ch = 0; ch < nch; ++ch, ++st) {
                const uint32_t s = st % nst;
                if (lane == 0) ok = mbar_wait(empty0 + 8 * s, ((st / nst) & 1) ^ 1, p.status);
                ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
                if (!ok) break;
                const int nsa = min(p.subsa, nsa_total - ch * p.subsa);
                const uint32_t wbytes = (uint32_t)nsa * Fmt<FMT>::SAB;
                const uint32_t xbytes = ch == 0 ? (uint32_t)I.kv * 2u : 0u;
                if (lane == 0) mbar_expect_tx(full0 + 8 * s, nvalid * wbytes + M * xbytes);
                __syncwarp();
                if (run)
                    bulk_g2s(smem_u32(ring + (size_t)s * p.stage_bytes + lane * p.sub_bytes),
                             run + (int64_t)(sa0 + ch * p.subsa) * Fmt<FMT>::SAB, wbytes, full0 + 8 * s);
                if (ch == 0 && lane >= 8)
                    for (int m = lane - 8; m < M; m += 24)
                        bulk_g2s(smem_u32(xbuf + ((size_t)xs * M + m) * p.rs), p.x + (int64_t)m * p.ldx + I.k0, xbytes,
                                 full0 + 8 * s);
            }
        }
        // (every stage issued above is waited for by the streaming warps before they leave; after a timeout the copies
        // still in flight are given a bounded wait here so that none lands after the CTA has gone)
        if (!ok && lane == 0) {
            for (uint32_t back = 1; back <= (uint32_t)nst && back <= st; ++back) {
                const uint32_t q = st - back;
                for (uint32_t i = 0; i < (1u << 16); ++i)
                    if (mbar_try_wait(full0 + 8 * (q % nst), (q / nst) & 1)) break;
            }
        }
    } else if (warp <= 8) {
        // ---------------------------------------------------------------- streaming warps
        const int cw = warp - 1;
        const int g = lane >> 2, t = lane & 3;
        uint32_t st = 0, xi = 0, pi = 0;
        bool ok = true;
        for (int64_t it = i0; it < i1 && ok; ++it, ++xi, ++pi) {
            const ItemInfo I = item_info(p, it);
            const bool valid = warp_run(p, I, cw) != nullptr;
            const uint32_t xs = xi % xsl;
            const uint8_t* xrow[MT];
#pragma unroll
            for (int m = 0; m < MT; ++m)
                xrow[m] = 8 * m + g < M ? xbuf + ((size_t)xs * M + 8 * m + g) * p.rs : nullptr;
            float acc[MT][4];
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;
            const int nsa_total = (I.kv + Fmt<FMT>::KSA - 1) / Fmt<FMT>::KSA;
            const int nch = (nsa_total + p.subsa - 1) / p.subsa;
            for (int ch = 0; ch < nch; ++ch, ++st) {
                const uint32_t s = st % nst;
                ok = mbar_wait(full0 + 8 * s, (st / nst) & 1, p.status);
                if (!ok) break;
                if (valid)
                    chunk_mma<FMT, MT>(acc, ring + (size_t)s * p.stage_bytes + cw * p.sub_bytes,
                                       min(p.subsa, nsa_total - ch * p.subsa), ch * p.subsa * Fmt<FMT>::KSA, I.kv, xrow,
                                       lane);
                __syncwarp();
                if (lane == 0) mbar_arrive(empty0 + 8 * s);
            }
            if (!ok) break;
            if (lane == 0) mbar_arrive(xempty0 + 8 * xs);
            const uint32_t pb = pi & 1;
            ok = mbar_wait(pempty0 + 8 * pb, ((pi >> 1) & 1) ^ 1, p.status);
            if (!ok) break;
            float* pc = pbuf + ((size_t)pb * TKD_PANEL_COLS + cw * 16 + g) * MP + 2 * t;
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                *reinterpret_cast<float2*>(pc + 8 * m) = make_float2(acc[m][0], acc[m][1]);
                *reinterpret_cast<float2*>(pc + 8 * MP + 8 * m) = make_float2(acc[m][2], acc[m][3]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(pfull0 + 8 * pb);
        }
    } else {
        // ---------------------------------------------------------------- output warps
        const int et = tid - 9 * 32;  // the panel column this thread owns
        uint32_t pi = 0;
        int given = 0;                // slices of the current split panel this CTA has put into scratch
        float tot[MR];
        bool ok = true;
        for (int64_t it = i0; it < i1 && ok; ++it, ++pi) {
            const ItemInfo I = item_info(p, it);
            const TkdSegDev& sg = p.seg[I.seg];
            const uint32_t pb = pi & 1;
            ok = mbar_wait(pfull0 + 8 * pb, (pi >> 1) & 1, p.status);
            if (!ok) break;
            float part[MR];
            const float* pc = pbuf + ((size_t)pb * TKD_PANEL_COLS + et) * MP;
#pragma unroll
            for (int m = 0; m < MR; m += 4) {
                const float4 v = *reinterpret_cast<const float4*>(pc + m);
                part[m] = v.x, part[m + 1] = v.y, part[m + 2] = v.z, part[m + 3] = v.w;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(pempty0 + 8 * pb);

            const int64_t pfirst = (int64_t)I.panel * p.nslices;
            const bool whole = pfirst >= i0 && pfirst + p.nslices <= i1;
            const bool last_here = I.slice == p.nslices - 1 || it == i1 - 1;
            bool finish = false;
            if (whole) {
#pragma unroll
                for (int m = 0; m < MR; ++m) tot[m] = I.slice == 0 ? part[m] : tot[m] + part[m];
                finish = I.slice == p.nslices - 1;
            } else {
                float* sc = p.scratch + (((size_t)I.panel * p.nslices + I.slice) * M) * TKD_PANEL_COLS + et;
#pragma unroll
                for (int m = 0; m < MR; ++m)
                    if (m < M) __stcg(sc + (size_t)m * TKD_PANEL_COLS, part[m]);
                ++given;
                if (last_here) {
                    __threadfence();
                    bar_output_warps();
                    if (et == 0) {
                        const int old = atomicAdd(p.counters + I.panel, given);
                        const int last = old + given == p.nslices;
                        if (last) p.counters[I.panel] = 0;  // ready for the next call
                        sflag[0] = last;
                    }
                    bar_output_warps();
                    finish = sflag[0] != 0;
                    given = 0;
                    if (finish) {
                        __threadfence();
                        const float* s0 = p.scratch + ((size_t)I.panel * p.nslices * M) * TKD_PANEL_COLS + et;
#pragma unroll
                        for (int m = 0; m < MR; ++m) tot[m] = 0.f;
                        for (int s = 0; s < p.nslices; ++s)
#pragma unroll
                            for (int m = 0; m < MR; ++m)
                                if (m < M) {
                                    const float v = __ldcg(s0 + ((size_t)s * M + m) * TKD_PANEL_COLS);
                                    tot[m] = s == 0 ? v : tot[m] + v;
                                }
                    }
                    bar_output_warps();  // sflag may be written again only after everyone has read it
                }
            }
            if (!finish) continue;

            // ------------------------------------------------------------ the output stage of one panel
            const bool glu2 = p.epi == TKD_EPI_GLU2;
            // this thread's column within its weight, and the block-float factor of its group
            const int n = glu2 ? I.pl * 64 + (et & 63) : I.pl * TKD_PANEL_COLS + et;
            const uint8_t* em = glu2 && et >= 64 ? sg.emax2 : sg.emax;
            if constexpr (FMT != TKD_BF16) {
                const int ngroup = n >> 4;
                const int e = ngroup < sg.groups ? (int)em[ngroup] + 64 - (FMT == TKD_BFP8 ? 133 : 129) : 0;
#pragma unroll
                for (int m = 0; m < MR; ++m) tot[m] = scalbnf(tot[m], e);
            }
            const bool in_w = n < sg.n_valid;
            if (p.scale_dt != TKD_DT_NONE && in_w) {
                const void* sp = glu2 && et >= 64 ? p.scale2 : p.scale;
                const float sc = p.scale_dt == TKD_DT_BF16 ? bf16_bits_to_f32(static_cast<const uint16_t*>(sp)[n])
                                                           : static_cast<const float*>(sp)[n];
#pragma unroll
                for (int m = 0; m < MR; ++m) tot[m] *= sc;
            }
            uint16_t* y16 = static_cast<uint16_t*>(p.out);
            int ocol = -1;  // the output column this thread writes, if any
            if (p.epi == TKD_EPI_GLU_IL || glu2) {
                float* tc = tbuf + (size_t)et * MP;
#pragma unroll
                for (int m = 0; m < MR; m += 4)
                    *reinterpret_cast<float4*>(tc + m) = make_float4(tot[m], tot[m + 1], tot[m + 2], tot[m + 3]);
                bar_output_warps();
                if (et < 64) {
                    // interleaved: 32 gate columns, then their 32 up columns; two weights: gate 0-63, up 64-127
                    const int gc = glu2 ? et : 64 * (et >> 5) + (et & 31), uc = glu2 ? et + 64 : gc + 32;
                    const int nw = glu2 ? n : I.pl * TKD_PANEL_COLS + uc;  // the pair's last column in the weight
                    if (nw < sg.n_valid) ocol = sg.out_col0 + I.pl * 64 + et;
                    const float* gp = tbuf + (size_t)gc * MP;
                    const float* up = tbuf + (size_t)uc * MP;
#pragma unroll
                    for (int m = 0; m < MR; ++m) tot[m] = act_gate(gp[m], p.act) * up[m];
                }
                bar_output_warps();  // tbuf is free again
            } else if (in_w) {
                ocol = sg.out_col0 + n;
            }
            const bool store = ocol >= 0 && (p.topk_k == 0 || p.write_y);
            if (ocol >= 0) {
                if (p.epi == TKD_EPI_OUT32) {
                    float* y32 = static_cast<float*>(p.out);
#pragma unroll
                    for (int m = 0; m < MR; ++m)
                        if (m < M) {
                            float v = tot[m];
                            if (p.res_dt == TKD_DT_F32) v += static_cast<const float*>(p.res)[(size_t)m * p.ldr + ocol];
                            y32[(size_t)m * p.ldo + ocol] = v;
                        }
                } else {
#pragma unroll
                    for (int m = 0; m < MR; ++m)
                        if (m < M) {
                            float v = tot[m];
                            if (p.epi == TKD_EPI_RESIDUAL)
                                v += bf16_bits_to_f32(static_cast<const uint16_t*>(p.res)[(size_t)m * p.ldr + ocol]);
                            const uint16_t b = f32_to_bf16_bits(v);
                            if (store) y16[(size_t)m * p.ldo + ocol] = b;
                            if (p.topk_k && !p.write_y && m < p.topk_rows) p.ytmp[(size_t)m * p.ld_ytmp + n] = b;
                        }
                }
            }
            if (p.topk_k == 0) continue;

            // ------------------------------------------------------------ top-k records: one per unit of columns,
            // made by the CTA that completes the unit's last panel, from the bf16 outputs themselves
            const int upanels = p.topk_unit / TKD_PANEL_COLS;
            const int unit = I.pl / upanels;
            const int in_unit = min(upanels, p.total_panels - unit * upanels);
            __threadfence();
            bar_output_warps();
            if (et == 0) {
                const int old = atomicAdd(p.unit_counters + unit, 1);
                const int last = old + 1 == in_unit;
                if (last) p.unit_counters[unit] = 0;
                sflag[0] = last;
            }
            bar_output_warps();
            const bool scan = sflag[0] != 0;
            bar_output_warps();
            if (!scan) continue;
            __threadfence();
            const uint16_t* ysrc = p.write_y ? y16 + sg.out_col0 : p.ytmp;
            const int64_t ldy = p.write_y ? p.ldo : p.ld_ytmp;
            const int c0 = unit * p.topk_unit;  // the unit's first column (call-relative)
            uint32_t* red = reinterpret_cast<uint32_t*>(tbuf);
            uint32_t* rec = p.records + (size_t)(p.topk_slot0 + unit) * 2 * p.topk_rows * p.topk_k;
            for (int r = 0; r < p.topk_rows; ++r) {
                // candidates: (key << 16 | 0xFFFF - position in unit) orders by key descending, then column ascending;
                // this thread's 16 (a unit holds at most 2048 columns) are loaded once
                uint32_t cand[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int c = et + j * TKD_PANEL_COLS, col = c0 + c;
                    uint32_t key = 0;
                    if (c < p.topk_unit && col < p.topk_n && col < sg.n_valid)
                        key = topk_key(__ldcg(ysrc + (size_t)r * ldy + col));
                    cand[j] = key ? (key << 16) | (0xFFFFu - (uint32_t)c) : 0u;
                }
                uint32_t bound = 0xFFFFFFFFu;
                for (int q = 0; q < p.topk_k; ++q) {
                    uint32_t best = 0;
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (cand[j] < bound && cand[j] > best) best = cand[j];
#pragma unroll
                    for (int o = 16; o; o >>= 1) best = max(best, __shfl_xor_sync(0xFFFFFFFFu, best, o));
                    if (lane == 0) red[warp - 9] = best;
                    bar_output_warps();
                    best = max(max(red[0], red[1]), max(red[2], red[3]));
                    bar_output_warps();
                    bound = best;  // (0: nothing left, the remaining slots stay empty)
                    if (et == 0) {
                        rec[r * p.topk_k + q] = best >> 16;
                        rec[(p.topk_rows + r) * p.topk_k + q] =
                            best ? p.topk_base + (uint32_t)c0 + (0xFFFFu - (best & 0xFFFFu)) : 0xFFFFFFFFu;
                    }
                }
            }
        }
    }
}

template <int FMT, int MT>
int launch_one(const TkdParams& p, int grid, size_t smem, cudaStream_t st) {
    auto kern = tkd_stream_kernel<FMT, MT>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    kern<<<grid, TKD_THREADS, smem, st>>>(p);
    return (int)cudaGetLastError();
}

template <int FMT>
int launch_fmt(const TkdParams& p, int grid, size_t smem, cudaStream_t st) {
    if (p.M <= 8) return launch_one<FMT, 1>(p, grid, smem, st);
    if (p.M <= 16) return launch_one<FMT, 2>(p, grid, smem, st);
    return launch_one<FMT, 4>(p, grid, smem, st);
}

}  // namespace

int tkd_launch_stream(const TkdParams& p, int grid, size_t smem, cudaStream_t st) {
    switch (p.fmt) {
        case TKD_BFP8: return launch_fmt<TKD_BFP8>(p, grid, smem, st);
        case TKD_BFP4: return launch_fmt<TKD_BFP4>(p, grid, smem, st);
        default: return launch_fmt<TKD_BF16>(p, grid, smem, st);
    }
}
