// tkd_stream_kernel.cuh: the weight-streaming decode matmul for sm_100a (the kernel template; tkd_stream_bfp8.cu,
// tkd_stream_bfp4.cu and tkd_stream_bf16.cu each compile one format's instantiations of it).
//
// y[m, n] = sum_k x[m, k] * w[k, n] with its fused output stage, M <= 8 activation rows (9 to 32 rows:
// tkd_stream_tc.cuh, which shares this file's helpers), the weight a packed HBM stream (tkd_layout.h). It takes the place of the reference's three Tensix kernels (dense_reader/kernels/
// dense_reader.cpp: the DRAM loads; dense_compute.cpp: matmul_block accumulation and the output stages;
// dense_writer.cpp: output writes and the running top-k) and of the work split linear.plan makes for them
// (dense_reader/linear.py:187-382).
//
// One persistent CTA per SM, three kinds of warps, coupled by mbarriers only:
//   warp 0        producer (one lane): one 1-D bulk copy (TMA) per stage of the shared-memory ring; a
//                 stage is one chunk of one panel (128 columns x 256 or 512 k), contiguous in the stream. (A bulk copy costs
//                 the issuing SM about 140 cycles whatever its size, so stages are single copies of 17-35 KB.)
//   warps 1-16    streaming warps: warp (group g, half h) multiplies the 16 columns of group g by every other
//                 super-atom of the chunk with mma.sync m16n8k16, the weights as A. Block-float codes go in as bf16
//                 subnormals (sign << 15 | magnitude) and the shared exponent is folded into the activations
//                 (x * 2^e' is exact), so a register of two weights costs one rotate and one AND. The one row of a
//                 decode call lies in shared memory whole; two to eight rows come straight from global memory through
//                 L1 (16 bytes a lane per 32 k), loaded before the stage is waited for.
//   warps 17-20   output warps (one thread per column of the panel): finish the K sum, run the output stage (exponent
//                 factor, scales, SwiGLU/GeGLU, residual, rounding), write y, and keep the top-k records.
//
// A work item is (panel, k slice of ks). Items are numbered panel-major and cut into equal contiguous runs, one per
// CTA. The sum of a column is defined once and for all as T0 + T1, T_h = the sum over slices, in ascending order, of
// streaming warp h's slice sum (itself acc_even + acc_odd, each started from zero per slice), all plain fp32 adds. A
// streaming warp adds up its own slices in registers as long as its CTA holds the panel from slice 0 on; what a CTA
// holds of a panel otherwise goes through a scratch buffer slice by slice, and the CTA that delivers last adds them
// up in the same order. So a column's result depends on K, the format, ks and M's bucket only, never on N, on the
// number of CTAs or on the other weights of a block list.
//
// Every wait is bounded: a wait that gives up records TKD_ERR_TIMEOUT in the status word, and every role then falls
// through to the end of the kernel.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#include "tkd_internal.h"
#include "tkd_layout.h"



namespace {

constexpr uint32_t kWaitRounds = 1u << 12;   // try_wait rounds before a wait gives up ...
constexpr uint32_t kWaitHintNs = 1000000u;   // ... each suspended for up to this long (woken at once on completion)
constexpr int kStatusTimeout = 3;            // TKD_ERR_TIMEOUT of include/tkd.h
#ifndef TKD_PARK_NS
#define TKD_PARK_NS 100
#endif

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
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(kWaitHintNs)
        : "memory");
    return ok != 0;
}
// Bounded wait: false (and the status word set) when the phase never completes.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status) {
    for (uint32_t i = 0; i < kWaitRounds; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    if (status) atomicExch(status, kStatusTimeout);
    return false;
}
// The same for the roles that spend most of the kernel waiting (the producer lane, the output warps): between tries the
// warp sleeps, so that its polling does not take issue slots and integer-pipe cycles from the streaming warps.
__device__ __forceinline__ bool mbar_wait_parked(uint32_t bar, uint32_t parity, int* status) {
#ifdef TKD_NO_PARKED_SLEEP
    return mbar_wait(bar, parity, status);
#else
    for (uint32_t i = 0; i < (kWaitRounds << 2); ++i) {  // (a failing try_wait has itself waited microseconds)
        if (mbar_try_wait(bar, parity)) return true;
        __nanosleep(TKD_PARK_NS);
    }
    if (status) atomicExch(status, kStatusTimeout);
    return false;
#endif
}
// global -> shared bulk copy (TMA, 1-D, this CTA only), completion counted in bytes on an mbarrier
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
// rotr(w, s) & mask: a funnel shift and an AND. (The rotate as a 32 x 32 -> 64 multiply by 2^(32 - s), to move it
// off the integer pipe this loop is bound by, measured 18 % slower on B200.)
template <int S>
__device__ __forceinline__ uint32_t rot_and(uint32_t w, uint32_t mask) {
    return __funnelshift_r(w, w, S) & mask;
}
// w << s as w * 2^s with the factor in a register the compiler cannot see through (a kernel parameter): an integer
// multiply runs on the FMA pipe, a shift on the integer pipe, and the integer pipe is what the bfloat4_b decode fills.
template <int S>
__device__ __forceinline__ uint32_t shl_fma(uint32_t w, uint32_t pow2) {
#ifdef TKD_PLAIN_SHIFTS
    return w << S;
#else
    uint32_t d;
    asm("mul.lo.u32 %0, %1, %2;" : "=r"(d) : "r"(w), "r"(pow2));
    return d;
#endif
}
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
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Spin (bounded: about a second) until flags[r] has reached `seq` (compared modulo 2^32) for every r < nranks; false
// when it gave up.
__device__ __noinline__ bool flags_wait(const uint32_t* flags, int nranks, uint32_t seq) {
    for (int r = 0; r < nranks; ++r) {
        int rounds = 0;
        while ((int32_t)(ld_acquire_sys(flags + r) - seq) < 0) {
            if (++rounds > (1 << 20)) return false;  // (about a microsecond a round)
            __nanosleep(rounds < 64 ? 20 : 200);
        }
    }
    return true;
}
__device__ __forceinline__ int atom_add_acq_rel(int* p, int v) {
    int old;
    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}
__device__ __forceinline__ void bar_output_warps() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float v) { return __bfloat16_as_ushort(__float2bfloat16_rn(v)); }

// dense_ops.h:44-59 of the reference: silu, and gelu_tanh as x * sigmoid(2 u), u = sqrt(2 / pi) (x + 0.044715 x^3)
__device__ __forceinline__ float act_gate(float g, int act) {
    const float u = act ? g * (1.5957691216f + 0.0713548162f * (g * g)) : g;
    return g / (1.f + __expf(-u));
}

// Quotients of item counts: 32-bit arithmetic when the launch's numbers allow it (p.small): a 64-bit division is a long
// subroutine on the GPU, and these sit on every CTA's way to its first copy and on the way to a panel's completion.
__device__ __forceinline__ int64_t idiv(const TkdParams& p, int64_t num, int64_t den) {
    return p.small ? (int64_t)((uint32_t)num / (uint32_t)den) : num / den;
}

// Where a role stands in its CTA's run of items.
struct Cursor {
    int panel, slice, seg, pl;
};
__device__ __forceinline__ void cursor_init(Cursor& c, const TkdParams& p, int64_t it) {
    c.panel = (int)idiv(p, it, p.nslices);
    c.slice = (int)(it - (int64_t)c.panel * p.nslices);
    c.seg = 0;
#pragma unroll
    for (int s = 1; s < 4; ++s)
        if (s < p.nseg && c.panel >= p.seg[s].panel0) c.seg = s;
    c.pl = c.panel - p.seg[c.seg].panel0;
}
__device__ __forceinline__ void cursor_next(Cursor& c, const TkdParams& p) {
    if (++c.slice == p.nslices) {
        c.slice = 0;
        ++c.panel;
        if (c.seg + 1 < p.nseg && c.panel >= p.seg[c.seg + 1].panel0) ++c.seg;
        c.pl = c.panel - p.seg[c.seg].panel0;
    }
}
// What a CTA does with an item's slice sums (the same answer in every role).
struct Flow {
    bool start;    // the running sum starts over with this slice
    bool split;    // the panel's slices are spread over several CTAs: sums go to the scratch buffer
    bool store;    // split: the running sum is written to the scratch slot of (panel, slice) after this slice
    bool deliver;  // the streaming warps signal the output warps after this slice (whole: with their sums)
    int count;     // split and deliver: slices of the panel this CTA has contributed
};
__device__ __forceinline__ Flow flow_of(const Cursor& c, const TkdParams& p, int64_t it, int64_t i0, int64_t i1) {
    Flow f;
    const int64_t pfirst = (int64_t)c.panel * p.nslices;
    const bool nonprefix = pfirst < i0;  // the run begins inside this panel, past its slice 0
    const bool last_here = c.slice == p.nslices - 1 || it == i1 - 1;
    f.start = nonprefix || c.slice == 0;
    f.split = nonprefix || pfirst + p.nslices > i1;
    f.store = f.split && (nonprefix || last_here);
    f.deliver = last_here;
    f.count = nonprefix ? c.slice - (int)(i0 - pfirst) + 1 : c.slice + 1;
    return f;
}

template <int FMT>
struct Fmt;
template <>
struct Fmt<TKD_BFP8> {
    static constexpr int KSA = 32, SAB = 544, SUBSA = 8, XB = 1;
};
template <>
struct Fmt<TKD_BFP4> {
    static constexpr int KSA = 64, SAB = 576, SUBSA = 8, XB = 2;
};
template <>
struct Fmt<TKD_INT4> {  // (bfloat4_b's geometry: tkd_layout.h)
    static constexpr int KSA = 64, SAB = 576, SUBSA = 8, XB = 2;
};
template <>
struct Fmt<TKD_BF16> {
    static constexpr int KSA = 32, SAB = 1024, SUBSA = 4, XB = 1;
};

// The two mmas of one k32 block of one group of a block-float weight: cw / ew are this lane's code and exponent
// words of the block (bfloat4_b: 2 and 2; bfloat8_b: 4 and 2).
template <int FMT, int MT, int NA>
__device__ __forceinline__ void block_mma(float (&acc)[NA][MT][4], const uint32_t (&cw)[4], const uint32_t (&ew)[2],
                                          const uint4 (&xv)[MT], const uint2 sh) {
#pragma unroll
    for (int jj = 0; jj < 2; ++jj) {
        uint32_t a0, a1, a2, a3;
        uint32_t s0, s1;
        if constexpr (FMT == TKD_BFP4) {
            // (five integer-pipe operations and three multiplies for the 8 codes and 4 exponents of a word each)
            const uint32_t w = cw[jj], t = __funnelshift_r(w, w, 8);
            a0 = w & TKD_MASK_BFP4, a1 = shl_fma<4>(w, sh.x) & TKD_MASK_BFP4;
            a2 = t & TKD_MASK_BFP4, a3 = shl_fma<4>(t, sh.x) & TKD_MASK_BFP4;
            s0 = (ew[jj] & TKD_EMASK_BFP4) | TKD_EBASE_BFP4;
            s1 = (shl_fma<7>(ew[jj], sh.y) & TKD_EMASK_BFP4) | TKD_EBASE_BFP4;
        } else {
            const uint32_t w0 = cw[2 * jj], w1 = cw[2 * jj + 1];
            a0 = w0 & TKD_MASK_BFP8, a1 = rot_and<8>(w0, TKD_MASK_BFP8);
            a2 = w1 & TKD_MASK_BFP8, a3 = rot_and<8>(w1, TKD_MASK_BFP8);
            s0 = ew[jj] & 0x7F807F80u, s1 = rot_and<8>(ew[jj], 0x7F807F80u);
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const uint32_t x0 = jj ? xv[m].z : xv[m].x, x1 = jj ? xv[m].w : xv[m].y;
            mma_bf16(acc[jj % NA][m], a0, a1, a2, a3, mul_bf16x2(x0, s0), mul_bf16x2(x1, s1));
        }
    }
}

__device__ __forceinline__ uint4 ldg_x(const uint16_t* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}

// What a stage of the ring holds for the streaming warps besides the weights: a 16-byte header the producer writes.
// .x: flags; .y: the scratch slot (panel * slices + slice) of the stage's item; .z: first k of the next stage.
enum : uint32_t {
    ST_FIRST = 1,     // first chunk of its item: the slice sums start from zero
    ST_LAST = 2,      // last chunk of its item: the flags below apply
    ST_START = 4,     // the running sum starts over with this slice
    ST_STORE = 8,     // the running sum goes to the scratch slot
    ST_DELIVER = 16,  // the output warps are signalled
    ST_SPLIT = 32,    // ... without the sums (they are in the scratch buffer)
    ST_END = 64,      // last stage of this CTA's run
};

// One streaming warp's share of one chunk: super-atoms h, h + 2, ... of one group. code_a / exp_a: shared-memory
// addresses of this lane's code and exponent words of super-atom h; xb[m]: this lane's row of x at k = 8 t + h * KSA;
// kc: the chunk's first k. FULL: the chunk has all its super-atoms and ends within K (then xpre holds the activations,
// loaded before the stage was waited for, when PRE).
// XSM: a one-row call keeps all of x in shared memory (zero-filled up to a whole chunk): xt_a is the address of this
// lane's 16 bytes of the chunk's first block.
template <int FMT, int MT, int NA, bool FULL, bool PRE, bool XSM = false>
__device__ __forceinline__ void chunk_mma(float (&acc)[NA][MT][4], uint32_t code_a, uint32_t exp_a,
                                          const uint4 (&xpre)[Fmt<FMT>::SUBSA / 2 * Fmt<FMT>::XB][MT],
                                          const uint16_t* const (&xb)[MT], int kc, int K, int h, int nsa, const uint2 sh,
                                          uint32_t xt_a = 0) {
    using F = Fmt<FMT>;
    constexpr int NPW = F::SUBSA / 2;  // super-atoms a warp takes of a chunk
#pragma unroll
    for (int i = 0; i < NPW; ++i) {
        if (!FULL && h + 2 * i >= nsa) break;
        uint32_t cw[F::XB][4], ew[F::XB][2];
        if constexpr (FMT == TKD_BFP4) {
            const uint4 ev = lds128(exp_a + 2 * i * F::SAB), cv = lds128(code_a + 2 * i * F::SAB);
            cw[0][0] = cv.x, cw[0][1] = cv.y, cw[1][0] = cv.z, cw[1][1] = cv.w;
            cw[0][2] = cw[0][3] = cw[1][2] = cw[1][3] = 0;
            ew[0][0] = ev.x, ew[0][1] = ev.y, ew[1][0] = ev.z, ew[1][1] = ev.w;
        } else if constexpr (FMT == TKD_INT4) {
            // (exp_a: this lane's two scale words of the super-atom, one per k32 block: columns g and g + 8)
            const uint2 sv = lds64(exp_a + 2 * i * F::SAB);
            const uint4 cv = lds128(code_a + 2 * i * F::SAB);
            cw[0][0] = cv.x, cw[0][1] = cv.y, cw[1][0] = cv.z, cw[1][1] = cv.w;
            cw[0][2] = cw[0][3] = cw[1][2] = cw[1][3] = 0;
            ew[0][0] = sv.x, ew[1][0] = sv.y, ew[0][1] = ew[1][1] = 0;
        } else if constexpr (FMT == TKD_BFP8) {
            const uint2 ev = lds64(exp_a + 2 * i * F::SAB);
            const uint4 cv = lds128(code_a + 2 * i * F::SAB);
            cw[0][0] = cv.x, cw[0][1] = cv.y, cw[0][2] = cv.z, cw[0][3] = cv.w;
            ew[0][0] = ev.x, ew[0][1] = ev.y;
        }
#pragma unroll
        for (int q = 0; q < F::XB; ++q) {
            const int k = kc + 2 * i * F::KSA + 32 * q;  // (+ h * KSA, which xb carries)
            if (!FULL && k + h * F::KSA >= K) break;     // a K that ends inside a super-atom
            uint4 xv[MT];
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                if constexpr (XSM)  // (the one row of x, whole, in shared memory: xt_a is this lane's address at k = kc)
                    xv[m] = lds128(xt_a + (2 * i * F::KSA + 32 * q) * 2);
                else if constexpr (FULL && PRE)
                    xv[m] = xpre[i * F::XB + q][m];
                else
                    xv[m] = ldg_x(xb[m] + k);
            }
            if constexpr (FMT == TKD_BF16) {
#pragma unroll
                for (int jj = 0; jj < 2; ++jj) {
                    const uint4 a = lds128(code_a + 2 * i * F::SAB + jj * 512);
#pragma unroll
                    for (int m = 0; m < MT; ++m)
                        mma_bf16(acc[jj % NA][m], a.x, a.y, a.z, a.w, jj ? xv[m].z : xv[m].x, jj ? xv[m].w : xv[m].y);
                }
            } else if constexpr (FMT == TKD_INT4) {
                // The k32 block's codes (bf16 subnormals q * 2^-129) times the activations times 2^64, summed from zero;
                // then the block's scale (s * 2^65, a pair of bf16 in ew[q][0]: column g low, g + 8 high) takes the sum
                // into the running one. The running sums alternate between the two accumulator sets by q.
                const float s_lo = __uint_as_float(ew[q][0] << 16), s_hi = __uint_as_float(ew[q][0] & 0xFFFF0000u);
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    float tmp[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int jj = 0; jj < 2; ++jj) {
                        const uint32_t w = cw[q][jj], t8 = __funnelshift_r(w, w, 8);
                        const uint32_t a0 = w & TKD_MASK_BFP4, a1 = shl_fma<4>(w, sh.x) & TKD_MASK_BFP4;
                        const uint32_t a2 = t8 & TKD_MASK_BFP4, a3 = shl_fma<4>(t8, sh.x) & TKD_MASK_BFP4;
                        const uint32_t x0 = jj ? xv[m].z : xv[m].x, x1 = jj ? xv[m].w : xv[m].y;
                        mma_bf16(tmp, a0, a1, a2, a3, mul_bf16x2(x0, 0x5F805F80u), mul_bf16x2(x1, 0x5F805F80u));
                    }
                    float(&a)[4] = acc[q % NA][m];
                    a[0] = fmaf(tmp[0], s_lo, a[0]), a[1] = fmaf(tmp[1], s_lo, a[1]);
                    a[2] = fmaf(tmp[2], s_hi, a[2]), a[3] = fmaf(tmp[3], s_hi, a[3]);
                }
            } else {
                block_mma<FMT, MT, NA>(acc, cw[q], ew[q], xv, sh);
            }
        }
    }
}

// bf16 output as the top-k records order it: a monotone 16-bit key, 0 below every value (dense_writer.cpp:215).
__device__ __forceinline__ uint32_t topk_key(uint16_t b) {
    return (uint32_t)(b ^ (0x8000u | (0x7FFFu & (0u - (uint32_t)(b >> 15))))) & 0xFFFFu;
}

// The top-k records of the unit of columns that panel c.pl belongs to, made by the CTA whose output warps complete the
// unit's last panel, from the bf16 outputs themselves (all four output warps call this after a panel's output stage).
__device__ __forceinline__ void topk_records(const TkdParams& p, const Cursor& c, const TkdSegDev& sg, int et, int ow, int lane,
                                             float* tbuf, volatile int* sflag, uint16_t* y16, int topk_k, int npeers) {
                // ------------------------------------------------------------ top-k records: one per unit of columns,
                // made by the CTA that completes the unit's last panel, from the bf16 outputs themselves
                const int upanels = p.topk_unit / TKD_PANEL_COLS;
                const int unit = c.pl / upanels;
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
                if (!scan) return;
                __threadfence();
                const uint16_t* ysrc = p.write_y ? y16 + sg.out_col0 : p.ytmp;
                const int64_t ldy = p.write_y ? p.ldo : p.ld_ytmp;
                const int col0 = unit * p.topk_unit;  // the unit's first column (call-relative)
                uint32_t* red = reinterpret_cast<uint32_t*>(tbuf);
                const size_t rec_at = (size_t)(p.topk_slot0 + unit) * 2 * p.topk_rows * topk_k;
                uint32_t* rec = p.records + rec_at;
                for (int r = 0; r < p.topk_rows; ++r) {
                    // candidates: (key << 16 | 0xFFFF - position in unit) orders by key descending, then column ascending;
                    // this thread's 16 (a unit holds at most 2048 columns) are loaded once
                    uint32_t cand[16];
    #pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int cc = et + j * TKD_PANEL_COLS, col = col0 + cc;
                        uint32_t key = 0;
                        if (cc < p.topk_unit && col < p.topk_n && col < sg.n_valid)
                            key = topk_key(__ldcg(ysrc + (size_t)r * ldy + col));
                        cand[j] = key ? (key << 16) | (0xFFFFu - (uint32_t)cc) : 0u;
                    }
                    uint32_t bound = 0xFFFFFFFFu;
                    for (int q = 0; q < topk_k; ++q) {
                        uint32_t best = 0;
    #pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (cand[j] < bound && cand[j] > best) best = cand[j];
    #pragma unroll
                        for (int o = 16; o; o >>= 1) best = max(best, __shfl_xor_sync(0xFFFFFFFFu, best, o));
                        if (lane == 0) red[ow] = best;
                        bar_output_warps();
                        best = max(max(red[0], red[1]), max(red[2], red[3]));
                        bar_output_warps();
                        bound = best;  // (0: nothing left, the remaining slots stay empty)
                        if (et == 0) {
                            const uint32_t key = best >> 16;
                            const uint32_t idx = best ? p.topk_base + (uint32_t)col0 + (0xFFFFu - (best & 0xFFFFu)) : 0xFFFFFFFFu;
                            const int at_k = r * topk_k + q, at_i = (p.topk_rows + r) * topk_k + q;
                            rec[at_k] = key;
                            rec[at_i] = idx;
    #pragma unroll 1
                            for (int pq = 0; pq < npeers; ++pq)
                                if (p.peer_records[pq]) {
                                    p.peer_records[pq][rec_at + at_k] = key;
                                    p.peer_records[pq][rec_at + at_i] = idx;
                                }
                        }
                    }
                }
}

// The end of an exchanged call, run by every output warp after its last panel.
__device__ __forceinline__ void exchange_done(const TkdParams& p, int lane, int npeers, volatile int* sflag) {
    // Exchange: every output warp orders its stores GPU-wide (a cheap fence) and counts itself in, first within its
    // CTA (a shared-memory counter, sflag[1]); the CTA's last warp counts the CTA in on the call's one global counter
    // (148 atomics on one address instead of 592: they arrive together at the kernel's end and serialise). The CTA
    // that counts last orders everything system-wide with the call's ONE system fence (system fences serialise
    // across the GPU: one per warp cost this kernel a third of its run), numbers the call and writes that number to
    // this rank's word on every rank. (No CTA barrier: the warps may have left the loop at different points.)
    // exchange_wait 3: none of this; the caller announces the call once the kernel has completed.
    if (p.exchange_wait == 3) return;
    __syncwarp();
    if (lane == 0) {
        __threadfence();
        if (atomicAdd_block(const_cast<int*>(sflag) + 1, 1) != 3) return;
        __threadfence();
        const int old = atomicAdd(p.grid_counter, 1);
        if (old + 1 == (int)gridDim.x) {
            *p.grid_counter = 0;
            const uint32_t seq = p.flags[TKD_FLAG_SEQ] + 1;
            p.flags[TKD_FLAG_SEQ] = seq;
            __threadfence_system();
            for (int q = 0; q < npeers; ++q) st_relaxed_sys(p.peer_flags[q] + p.rank, seq);
            st_relaxed_sys(p.flags + p.rank, seq);
            // (2: the call before this one, whose exchange has had this call's whole run to arrive)
            if (p.exchange_wait && !flags_wait(p.flags, npeers + 1, p.exchange_wait == 2 ? seq - 1 : seq)) {
                if (p.status) atomicExch(p.status, TKD_ERR_TIMEOUT);
            }
        }
    }
}

// The kernel for 1 to 8 rows (9 to 32 run tkd_stream_tc_kernel). Sixteen streaming warps: a warp per column group and half
// of each chunk's super-atoms.
// ONE: the call has one row (the decode case): the row count is a constant 1 and everything that serves more rows falls
// away at compile time. (The length of this kernel's code matters beyond the parts that run: adding two more instances
// of the output stage for 2 and 4 rows made the one-row call 1.5 us slower.)
// PLAIN: no top-k records and no exchange with other GPUs (the plain matmuls of a decode step): that code falls away too.
// KWHOLE: K is a whole number of chunks, so the code for a last, shorter chunk falls away as well.
// XSM: all of x lies in shared memory (always so for ONE; two to eight rows: if it fits beside four stages of the ring).
constexpr int kStreamWarps = 16;
template <int FMT, bool ONE, bool PLAIN, bool KWHOLE, bool XSM>
__global__ void __launch_bounds__((1 + kStreamWarps + 4) * 32, 1) tkd_stream_kernel(const __grid_constant__ TkdParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    using F = Fmt<FMT>;
    constexpr int SW = kStreamWarps;
    constexpr int MT = 1;   // m16n8 tiles of rows (8 rows each)
    constexpr int MP = 8;   // floats per column in the hand-over buffers
    constexpr int MR = 8;   // rows the accumulators cover
    constexpr int NA = 2;   // accumulator sets a streaming warp alternates between
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + TKD_MAX_STAGES);
    const uint32_t pfull0 = smem_u32(bars + 2 * TKD_MAX_STAGES), pempty0 = pfull0 + 16, xbar = pfull0 + 32;
    // NH: halves of a chunk's super-atoms a streaming warp takes; NPB: hand-over buffers between the streaming and the
    // output warps
    constexpr int NH = 1;
    constexpr int NPB = 2;
    volatile int* sflag = reinterpret_cast<volatile int*>(smem + TKD_SMEM_HEAD - 16);
    uint4* hdr = reinterpret_cast<uint4*>(smem + 512);  // one header per stage of the ring
    float* pbuf = reinterpret_cast<float*>(smem + p.off_pbuf);  // [2 buffers][2 halves][128 columns][MP]
    float* tbuf = reinterpret_cast<float*>(smem + p.off_tbuf);  // [128 columns][MP]
    uint8_t* ring = smem + p.off_ring;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // let the kernel after this one in the stream start its CTAs as SMs become free
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (tid == 0) {
        for (int s = 0; s < p.nstages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, SW);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(pfull0 + 8 * s, SW);
            mbar_init(pempty0 + 8 * s, 4);
        }
        mbar_init(xbar, 1);
        sflag[0] = sflag[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const int64_t T = p.total_items;
    const int64_t i0 = idiv(p, T * blockIdx.x, gridDim.x), i1 = idiv(p, T * (blockIdx.x + 1), gridDim.x);
    const int nst = p.nstages;
    const int M = ONE ? 1 : p.M, K = p.K;
    const int topk_k = PLAIN ? 0 : p.topk_k, npeers = PLAIN ? 0 : p.npeers;
    const bool glu2 = p.epi == TKD_EPI_GLU2;
    constexpr int CK = F::SUBSA * F::KSA;
    const int nsa_total = (K + F::KSA - 1) / F::KSA;
    if (i0 >= i1) return;
    // Order of a CTA's items: if its run ends inside a panel that it holds from slice 0 on, those slices come first.
    // Their sum is one of several the panel is added up from by whichever CTA delivers last; done first, that exchange
    // overlaps the rest of the run instead of sitting at the kernel's end.
    const int64_t lastp0 = idiv(p, i1 - 1, p.nslices) * p.nslices;
    const int64_t tail0 = lastp0 > i0 && lastp0 + p.nslices > i1 ? lastp0 : i1;
    const int64_t lead = i1 - tail0;

    if (warp == 0) {
        // ---------------------------------------------------------------- producer
        if (lane != 0) return;
        Cursor c, cn;  // this item, and the one after it
        uint32_t st = 0;
        bool ok = true;
        const int64_t nitems = i1 - i0;
        auto item_at = [&](int64_t j) { return j < lead ? tail0 + j : i0 + (j - lead); };
        cursor_init(cn, p, item_at(0));
        for (int64_t j = 0; j < nitems && ok; ++j) {
            const int64_t it = item_at(j);
            c = cn;
            if (j + 1 < nitems) {
                if (j + 1 == lead)
                    cursor_init(cn, p, item_at(j + 1));
                else
                    cursor_next(cn, p);
            }
            const Flow f = flow_of(c, p, it, i0, i1);
            const TkdSegDev& sg = p.seg[c.seg];
            const int k0 = c.slice * p.ks, kv = min(p.ks, K - k0);
            const int c0 = k0 / CK, nch = (kv + CK - 1) / CK;
            // a panel of a (gate, up) pair is half a panel of each weight: 4 groups of the gate's, 4 of the up's
            const uint8_t* src = sg.w + (int64_t)(glu2 ? c.pl >> 1 : c.pl) * p.panel_bytes;
            const uint8_t* src2 = glu2 ? sg.w2 + (int64_t)(c.pl >> 1) * p.panel_bytes : nullptr;
            for (int ch = 0; ch < nch; ++ch, ++st) {
                const uint32_t s = st % nst;
                ok = mbar_wait_parked(empty0 + 8 * s, ((st / nst) & 1) ^ 1, p.status);
                if (!ok) break;
                const int nsa = min(F::SUBSA, nsa_total - (c0 + ch) * F::SUBSA);
                const uint32_t gbytes = (uint32_t)nsa * F::SAB;  // one group's share of the chunk
                const int64_t coff = (int64_t)(c0 + ch) * (F::SUBSA * F::SAB * 8);
                const uint32_t dst = smem_u32(ring + (size_t)s * p.stage_bytes);
                // the stage's header, ordered before the streaming warps' reads by the arrival below
                const bool last = ch == nch - 1;
                uint32_t fl = (ch == 0 ? ST_FIRST : 0u) | (last && j == nitems - 1 ? ST_END : 0u);
                if (last)
                    fl |= ST_LAST | (f.start ? ST_START : 0u) | (f.store ? ST_STORE : 0u) |
                          (f.deliver ? ST_DELIVER : 0u) | (f.split ? ST_SPLIT : 0u);
                const int knext = last ? cn.slice * p.ks : (c0 + ch + 1) * CK;
                hdr[s] = make_uint4(fl, (uint32_t)(c.panel * p.nslices + c.slice), (uint32_t)knext, 0u);
                mbar_expect_tx(full0 + 8 * s, 8 * gbytes);
                if (glu2) {
                    const int64_t hoff = coff + (int64_t)(c.pl & 1) * 4 * gbytes;
                    bulk_g2s(dst, src + hoff, 4 * gbytes, full0 + 8 * s);
                    bulk_g2s(dst + 4 * gbytes, src2 + hoff, 4 * gbytes, full0 + 8 * s);
                } else {
                    bulk_g2s(dst, src + coff, 8 * gbytes, full0 + 8 * s);
                }
            }
        }
        // (every stage issued above is waited for by the streaming warps before they leave; after a timeout the copies
        // still in flight are given a bounded wait here so that none lands after the CTA has gone)
        if (!ok) {
            for (uint32_t back = 1; back <= (uint32_t)nst && back <= st; ++back) {
                const uint32_t q = st - back;
                for (uint32_t i = 0; i < 64; ++i)
                    if (mbar_try_wait(full0 + 8 * (q % nst), (q / nst) & 1)) break;
            }
        }
    } else if (warp <= SW) {
        // ---------------------------------------------------------------- streaming warps
        // One flat loop over the stages of the ring; everything about items comes with the stage's header.
        const int cw = warp - 1;
        if constexpr (XSM && !KWHOLE) {
            // the rows of x in shared memory end in zeros up to a whole chunk: written here, before the wait below, by
            // whichever lanes, and seen by all after the barrier
            const int pieces = (K + CK - 1) / CK * (CK / 8);  // 16-byte pieces of a row
            const uint32_t xz = smem_u32(smem + p.off_xt);
            for (int r = 0; r < (ONE ? 1 : p.M); ++r)
                for (int e = K / 8 + cw * 32 + lane; e < pieces; e += SW * 32)
                    asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(xz + r * p.x_stride + e * 16), "r"(0u) : "memory");
            asm volatile("bar.sync 2, %0;" ::"n"(SW * 32) : "memory");
        }
        const uint32_t xt0 = smem_u32(smem + p.off_xt);
        // (x, the scratch buffer and the outputs may belong to the kernel before this one: wait for it to complete)
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if constexpr (XSM) {
            // the first thing after that wait: the weights are in the ring already, everything waits for x
            if (cw == 0 && lane == 0) {
                mbar_expect_tx(xbar, (uint32_t)(M * K * 2));
                for (int r = 0; r < M; ++r)
                    bulk_g2s(xt0 + (ONE ? 0 : r * p.x_stride), p.x + (int64_t)r * p.ldx, (uint32_t)(K * 2), xbar);
            }
        }
        const int g8 = cw & 7, h0 = cw >> 3;
        const int g = lane >> 2, t = lane & 3;
        constexpr int NX = F::SUBSA / 2 * F::XB;
        // XSM: the call's rows of x are copied into shared memory once (K rounded up to a chunk, the rest zeros) and
        // every block's 16 bytes a lane come from there. (Through L1 they missed one time in seven with most of the
        // SM's memory given to the ring, each miss a trip to L2 behind the weight stream's traffic, and the stage waits
        // for its slowest warp.)
        static_assert(XSM || !ONE, "the one-row instantiations keep x in shared memory");
        // PRE: x too large for that: the chunk's activations are loaded (through L1) before the stage is waited for
        constexpr bool PRE = !XSM;
        constexpr int EXPB = FMT == TKD_BFP4 || FMT == TKD_INT4 ? 64 : (FMT == TKD_BFP8 ? 32 : 0);
        const uint16_t* xb[NH][MT];
#pragma unroll
        // (a lane whose row lies beyond M reads row M - 1 instead: a B column only feeds its own output column, and
        // the columns beyond M are never read, so those lanes need no predicate and no zero fill)
        for (int hh = 0; hh < NH; ++hh)
#pragma unroll
            for (int m = 0; m < MT; ++m)
                xb[hh][m] = p.x + (int64_t)min(8 * m + g, M - 1) * p.ldx + 8 * t + (h0 + hh) * F::KSA;
        const uint32_t ring_a = smem_u32(ring), hdr_a = smem_u32(hdr);
        const uint32_t code_off = g8 * (F::SUBSA * F::SAB) + h0 * F::SAB + EXPB + lane * 16;
        // (this lane's exponent words of a super-atom; TKD_INT4: its pair of scale words, by its row of the fragment)
        const uint32_t exp_lane = FMT == TKD_INT4 ? g * 8 : t * (EXPB / 4);
        const uint32_t exp_off = g8 * (F::SUBSA * F::SAB) + h0 * F::SAB + exp_lane;
        uint32_t slot = 0, phase = 0, pi = 0;  // ring position and its parity; deliveries so far
        const int64_t first_it = lead > 0 ? tail0 : i0;
        int kc = (int)(first_it - idiv(p, first_it, p.nslices) * p.nslices) * p.ks;
        float acc[NH][NA][MT][4], tot[NH][MT][4];
        const uint2 sh = make_uint2(p.mul16, p.mul128);
        // (a lane's row of x: row g, or the last row for the lanes beyond M, as in xb)
        const uint32_t xs_lane = xt0 + (ONE ? 0 : min(g, M - 1) * p.x_stride) + (8 * t + h0 * F::KSA) * 2;
        bool x_here = true;
        if constexpr (XSM) {
            // The call's rows of x into shared memory, one bulk copy a row (K is a multiple of 32 and the rows are 16-byte
            // aligned: include/tkd.h), issued by one lane as soon as x may be read; every streaming warp waits for their
            // bytes on one barrier. (512 lanes loading and storing their pieces and a barrier among them took 2.0 us of a
            // 13 us launch, all of it before the first chunk.)
            x_here = mbar_wait(xbar, 0, p.status);  // (the copies were issued right after the wait for the kernel before)
            if constexpr (FMT == TKD_INT4) {
                // The ternary projections' block Hadamard (ternary_matmul/t2.py:409-495, hadamard=), on this CTA's copy of
                // x: x' = H_1024 (s * x), unnormalised. A warp takes a (row, block of 1024) at a time, a lane 32
                // consecutive inputs in registers: five butterfly stages inside the lane, five across lanes by shuffles,
                // in the order and with the operands of tkd_hadamard_kernel (stage h pairs i and i + h: a + c, a - c),
                // so both give the same bits; then bf16 again, in place.
                if (p.had && x_here) {
                    const int nblk = K >> 10;
                    for (int task = cw; task < M * nblk; task += SW) {
                        const int r = task / nblk, b = task - r * nblk;
                        const uint32_t xa = xt0 + (ONE ? 0 : r * p.x_stride) + b * 2048 + lane * 64;
                        const uint4* sg = reinterpret_cast<const uint4*>(p.had + ((b << 10) + lane * 32) / 2);
                        float v[32];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const uint4 raw = lds128(xa + 16 * q), sw = __ldg(sg + q);
                            const uint32_t w[4] = {raw.x ^ (sw.x & 0x80008000u), raw.y ^ (sw.y & 0x80008000u),
                                                   raw.z ^ (sw.z & 0x80008000u), raw.w ^ (sw.w & 0x80008000u)};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                v[8 * q + 2 * j] = __uint_as_float(w[j] << 16);
                                v[8 * q + 2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
                            }
                        }
#pragma unroll
                        for (int h = 1; h < 32; h <<= 1)
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (!(i & h)) {
                                    const float a = v[i], c = v[i + h];
                                    v[i] = a + c, v[i + h] = a - c;
                                }
#pragma unroll
                        for (int s = 0; s < 5; ++s) {
                            const bool upper = (lane >> s) & 1;
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                const float o = __shfl_xor_sync(0xFFFFFFFFu, v[i], 1 << s);
                                v[i] = upper ? o - v[i] : v[i] + o;  // (lower: a + c; upper: a - c with a the partner's)
                            }
                        }
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            uint32_t o[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                o[j] = (uint32_t)f32_to_bf16_bits(v[8 * q + 2 * j]) |
                                       ((uint32_t)f32_to_bf16_bits(v[8 * q + 2 * j + 1]) << 16);
                            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(xa + 16 * q), "r"(o[0]), "r"(o[1]), "r"(o[2]),
                                         "r"(o[3])
                                         : "memory");
                        }
                    }
                    asm volatile("bar.sync 2, %0;" ::"n"(SW * 32) : "memory");
                }
            }
        }
        while (x_here) {
            const bool full = KWHOLE || kc + CK <= K;
            uint4 xpre[NX][MT];
            if (PRE && full) {
#pragma unroll
                for (int i = 0; i < F::SUBSA / 2; ++i)
#pragma unroll
                    for (int q = 0; q < F::XB; ++q)
#pragma unroll
                        for (int m = 0; m < MT; ++m) xpre[i * F::XB + q][m] = ldg_x(xb[0][m] + kc + 2 * i * F::KSA + 32 * q);
            }
            if (!mbar_wait(full0 + 8 * slot, phase, p.status)) break;
            const uint4 hd = lds128(hdr_a + 16 * slot);
            const uint32_t fl = hd.x;
            if (fl & ST_FIRST) {
#pragma unroll
                for (int hh = 0; hh < NH; ++hh)
#pragma unroll
                    for (int j = 0; j < NA; ++j)
#pragma unroll
                        for (int m = 0; m < MT; ++m)
                            acc[hh][j][m][0] = acc[hh][j][m][1] = acc[hh][j][m][2] = acc[hh][j][m][3] = 0.f;
            }
            const uint32_t sbase = ring_a + slot * p.stage_bytes;
#pragma unroll
            for (int hh = 0; hh < NH; ++hh) {
                const int h = h0 + hh;
                if (full) {
                    chunk_mma<FMT, MT, NA, true, PRE, XSM>(acc[hh], sbase + code_off + hh * F::SAB, sbase + exp_off + hh * F::SAB,
                                                           xpre, xb[hh], kc, K, h, F::SUBSA, sh, xs_lane + kc * 2);
                } else {
                    // the last chunk of K: fewer super-atoms, the groups closer together
                    const int nsa = nsa_total - kc / CK * F::SUBSA;
                    const uint32_t gb = sbase + g8 * nsa * F::SAB + h * F::SAB;
                    chunk_mma<FMT, MT, NA, false, PRE, XSM>(acc[hh], gb + EXPB + lane * 16, gb + exp_lane, xpre, xb[hh], kc,
                                                            K, h, nsa, sh, xs_lane + kc * 2);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * slot);
            if (++slot == (uint32_t)nst) slot = 0, phase ^= 1;
            kc = (int)hd.z;
            if (!(fl & ST_LAST)) continue;
            // ---- the item's slice is done
#pragma unroll
            for (int hh = 0; hh < NH; ++hh)
#pragma unroll
                for (int m = 0; m < MT; ++m)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float part = NA == 2 ? acc[hh][0][m][e] + acc[hh][NA - 1][m][e] : acc[hh][0][m][e];
                        tot[hh][m][e] = fl & ST_START ? part : tot[hh][m][e] + part;
                    }
            if (fl & ST_STORE) {
                // straight into the scratch slot of (panel, slice): [half][row][128 columns]
#pragma unroll
                for (int hh = 0; hh < NH; ++hh) {
                    float* sc = p.scratch + ((size_t)hd.y * 2 + h0 + hh) * M * TKD_PANEL_COLS + g8 * 16 + g;
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        const int r0 = 8 * m + 2 * t;
                        if (r0 < M) {
                            __stcg(sc + (size_t)r0 * TKD_PANEL_COLS, tot[hh][m][0]);
                            __stcg(sc + (size_t)r0 * TKD_PANEL_COLS + 8, tot[hh][m][2]);
                        }
                        if (r0 + 1 < M) {
                            __stcg(sc + (size_t)(r0 + 1) * TKD_PANEL_COLS, tot[hh][m][1]);
                            __stcg(sc + (size_t)(r0 + 1) * TKD_PANEL_COLS + 8, tot[hh][m][3]);
                        }
                    }
                }
            }
            if (fl & ST_DELIVER) {
                const uint32_t pb = NPB == 2 ? pi & 1 : 0;
                if (!mbar_wait(pempty0 + 8 * pb, ((NPB == 2 ? pi >> 1 : pi) & 1) ^ 1, p.status)) break;
                if (!(fl & ST_SPLIT)) {
#pragma unroll
                    for (int hh = 0; hh < NH; ++hh) {
                        float* pc = pbuf + ((size_t)(pb * 2 + h0 + hh) * TKD_PANEL_COLS + g8 * 16 + g) * MP + 2 * t;
#pragma unroll
                        for (int m = 0; m < MT; ++m) {
                            *reinterpret_cast<float2*>(pc + 8 * m) = make_float2(tot[hh][m][0], tot[hh][m][1]);
                            *reinterpret_cast<float2*>(pc + 8 * MP + 8 * m) = make_float2(tot[hh][m][2], tot[hh][m][3]);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(pfull0 + 8 * pb);
                ++pi;
            }
            if (fl & ST_END) break;
        }
    } else {
        // ---------------------------------------------------------------- output warps
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const int et = tid - (1 + SW) * 32;  // the panel column this thread owns
        const int ow = warp - (1 + SW);
        Cursor c;
        uint32_t pi = 0;
        float tot[MR];
        bool ok = true;
        for (int64_t j = 0; j < i1 - i0 && ok; ++j) {
            const int64_t it = j < lead ? tail0 + j : i0 + (j - lead);
            if (j == 0 || j == lead)
                cursor_init(c, p, it);
            else
                cursor_next(c, p);
            const Flow f = flow_of(c, p, it, i0, i1);
            if (!f.deliver) continue;
            const TkdSegDev& sg = p.seg[c.seg];
            const uint32_t pb = NPB == 2 ? pi & 1 : 0;
            // this thread's column within its weight; its group's exponent byte and its scale are asked for now, so
            // that their latency passes while the streaming warps are still at work
            const int n = glu2 ? c.pl * 64 + (et & 63) : c.pl * TKD_PANEL_COLS + et;
            const bool in_w = n < sg.n_valid;
            int ebyte = 0;
            float sc = 1.f;
            if constexpr (FMT == TKD_BFP8 || FMT == TKD_BFP4) ebyte = (glu2 && et >= 64 ? sg.emax2 : sg.emax)[n >> 4];
            if (p.scale_dt != TKD_DT_NONE && in_w) {
                const void* sp = glu2 && et >= 64 ? p.scale2 : p.scale;
                sc = p.scale_dt == TKD_DT_BF16 ? bf16_bits_to_f32(static_cast<const uint16_t*>(sp)[n])
                                               : static_cast<const float*>(sp)[n];
            }
            ok = mbar_wait_parked(pfull0 + 8 * pb, (NPB == 2 ? pi >> 1 : pi) & 1, p.status);
            if (!ok) break;
            bool finish = !f.split;
            if (!f.split) {
                // the two halves' sums cover the whole panel
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const float* pc = pbuf + ((size_t)(pb * 2 + hh) * TKD_PANEL_COLS + et) * MP;
#pragma unroll
                    for (int m = 0; m < MR; m += 4) {
                        const float4 v = *reinterpret_cast<const float4*>(pc + m);
                        const float part[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) tot[m + e] = hh == 0 ? part[e] : tot[m + e] + part[e];
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(pempty0 + 8 * pb);
            ++pi;
            if (f.split) {
                // the streaming warps have put this CTA's slices of the panel into the scratch buffer (their arrival
                // on the hand-over barrier orders those stores before this point): count them in, and if they were
                // the last the panel waited for, add all of its slices up
                if (et == 0) {
                    // (one release-acquire atomic: the slice sums stored before it, by the streaming warps whose
                    // arrival this thread waited for, are visible to whichever CTA sees the count complete, and that CTA
                    // sees all the others')
                    const int old = atom_add_acq_rel(p.counters + c.panel, f.count);
                    const int last = old + f.count == p.nslices;
                    if (last) p.counters[c.panel] = 0;  // ready for the next call
                    sflag[0] = last;
                }
                bar_output_warps();
                finish = sflag[0] != 0;
                if (finish) {
                    // the panel's first slices came as one sum from the CTA that holds its slice 0: up to where?
                    const int64_t pfirst = (int64_t)c.panel * p.nslices;
                    const int64_t owner = idiv(p, (pfirst + 1) * gridDim.x - 1, T);
                    const int64_t oend = idiv(p, T * (owner + 1), gridDim.x);
                    const int pe = (int)min((int64_t)p.nslices, oend - pfirst);
                    const float* s0 = p.scratch + pfirst * 2 * M * TKD_PANEL_COLS + et;
                    // term (s, hh, m) of the sums; the adds run in slice order, the loads many at a time
                    auto term = [&](int s, int hh, int m) {
                        return __ldcg(s0 + ((size_t)(s * 2 + hh) * M + m) * TKD_PANEL_COLS);
                    };
                    if (M == 1) {
                        float t0 = term(pe - 1, 0, 0), t1 = term(pe - 1, 1, 0);
                        for (int s = pe; s < p.nslices; s += 8) {
                            float v0[8], v1[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                if (s + j < p.nslices) v0[j] = term(s + j, 0, 0), v1[j] = term(s + j, 1, 0);
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                if (s + j < p.nslices) t0 += v0[j], t1 += v1[j];
                        }
                        tot[0] = t0 + t1;
                    } else {
#pragma unroll 1
                        for (int hh = 0; hh < 2; ++hh) {
                            {
                                float th[MR];
#pragma unroll
                                for (int m = 0; m < MR; ++m)
                                    if (m < M) th[m] = term(pe - 1, hh, m);
#pragma unroll 1
                                for (int s = pe; s < p.nslices; ++s) {
                                    float v[MR];
#pragma unroll
                                    for (int m = 0; m < MR; ++m)
                                        if (m < M) v[m] = term(s, hh, m);
#pragma unroll
                                    for (int m = 0; m < MR; ++m)
                                        if (m < M) th[m] += v[m];
                                }
#pragma unroll
                                for (int m = 0; m < MR; ++m) tot[m] = hh == 0 ? th[m] : tot[m] + th[m];
                            }
                        }
                    }
                }
                bar_output_warps();  // sflag may be written again only after everyone has read it
            }
            if (!finish) continue;

            // ------------------------------------------------------------ the output stage of one panel
            // (a generic lambda over the rows it covers: a one-row call runs the one-row instance, an eighth of the code of
            // the eight-row one; this code runs once or twice a CTA, straight from the instruction cache's misses, so
            // its length is its cost)
            uint16_t* y16 = static_cast<uint16_t*>(p.out);
            auto output_stage = [&](auto rows_const) {
                constexpr int R = decltype(rows_const)::value;
                // the block-float factor of this thread's group
                if constexpr (FMT == TKD_BFP8 || FMT == TKD_BFP4) {
                    // 2^e in two factors, each a normal float (e is within -69 .. 191)
                    const int e = tkd_out_exp(FMT, ebyte);
                    const int e1 = e / 2, e2 = e - e1;
                    const float f1 = __uint_as_float((uint32_t)(e1 + 127) << 23), f2 = __uint_as_float((uint32_t)(e2 + 127) << 23);
    #pragma unroll
                    for (int m = 0; m < R; ++m) tot[m] = tot[m] * f1 * f2;
                }
                if (p.scale_dt != TKD_DT_NONE && in_w) {
    #pragma unroll
                    for (int m = 0; m < R; ++m) tot[m] *= sc;
                }
                int ocol = -1;  // the output column this thread writes, if any
                if (p.epi == TKD_EPI_GLU_IL || glu2) {
                    float* tc = tbuf + (size_t)et * MP;
    #pragma unroll
                    for (int m = 0; m < R; ++m) tc[m] = tot[m];
                    bar_output_warps();
                    if (et < 64) {
                        // interleaved: 32 gate columns, then their 32 up columns; two weights: gate 0-63, up 64-127
                        const int gc = glu2 ? et : 64 * (et >> 5) + (et & 31), uc = glu2 ? et + 64 : gc + 32;
                        const int nw = glu2 ? n : c.pl * TKD_PANEL_COLS + uc;  // the pair's last column in the weight
                        if (nw < sg.n_valid) ocol = sg.out_col0 + c.pl * 64 + et;
                        const float* gp = tbuf + (size_t)gc * MP;
                        const float* up = tbuf + (size_t)uc * MP;
    #pragma unroll
                        for (int m = 0; m < R; ++m) tot[m] = act_gate(gp[m], p.act) * up[m];
                    }
                    bar_output_warps();  // tbuf is free again
                } else if (in_w) {
                    ocol = sg.out_col0 + n;
                }
                const bool store = ocol >= 0 && (topk_k == 0 || p.write_y);
                if (ocol >= 0) {
                    // (the residual is read for every row before anything is stored: the output may be the residual's own
                    // memory, and loads placed after stores to what may be the same address would wait for each other row
                    // by row)
                    if (p.epi == TKD_EPI_OUT32) {
                        if (p.res_dt == TKD_DT_F32) {
    #pragma unroll
                            for (int m = 0; m < R; ++m)
                                if (m < M) tot[m] += static_cast<const float*>(p.res)[(size_t)m * p.ldr + ocol];
                        }
                        float* y32 = static_cast<float*>(p.out);
    #pragma unroll
                        for (int m = 0; m < R; ++m)
                            if (m < M) {
                                y32[(size_t)m * p.ldo + ocol] = tot[m];
    #pragma unroll 1
                                for (int q = 0; q < npeers; ++q)
                                    if (p.peer_out[q]) static_cast<float*>(p.peer_out[q])[(size_t)m * p.ldo + ocol] = tot[m];
                            }
                    } else {
                        if (p.epi == TKD_EPI_RESIDUAL) {
    #pragma unroll
                            for (int m = 0; m < R; ++m)
                                if (m < M)
                                    tot[m] += bf16_bits_to_f32(static_cast<const uint16_t*>(p.res)[(size_t)m * p.ldr + ocol]);
                        }
    #pragma unroll
                        for (int m = 0; m < R; ++m)
                            if (m < M) {
                                const uint16_t b = f32_to_bf16_bits(tot[m]);
                                if (store) {
                                    y16[(size_t)m * p.ldo + ocol] = b;
    #pragma unroll 1
                                    for (int q = 0; q < npeers; ++q)
                                        if (p.peer_out[q]) static_cast<uint16_t*>(p.peer_out[q])[(size_t)m * p.ldo + ocol] = b;
                                }
                                if (topk_k && !p.write_y && m < p.topk_rows) p.ytmp[(size_t)m * p.ld_ytmp + n] = b;
                            }
                    }
                }
            };
            if (M == 1) {
                output_stage(std::integral_constant<int, 1>{});
            } else {
                output_stage(std::integral_constant<int, MR>{});
            }
            if (topk_k == 0) continue;

            topk_records(p, c, sg, et, ow, lane, tbuf, sflag, y16, topk_k, npeers);
        
        }
        if (npeers) exchange_done(p, lane, npeers, sflag);
    }
}

template <int FMT, bool ONE, bool PLAIN, bool KWHOLE, bool XSM>
int launch_one(const TkdParams& p, int grid, size_t smem, cudaStream_t st) {
    auto kern = tkd_stream_kernel<FMT, ONE, PLAIN, KWHOLE, XSM>;
    // (once per device and instantiation: allow the largest dynamic shared memory a CTA can have)
    static bool allowed[64] = {false};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64 || !allowed[dev]) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return (int)e;
        if (dev >= 0 && dev < 64) allowed[dev] = true;
    }
    // Programmatic dependent launch: a CTA of this launch may start on an SM as soon as the kernel before it in the
    // stream has left that SM (every CTA of the stream kernel lets its dependents go at once, see the kernel). Its
    // producer then fills the ring with weights, which no earlier kernel writes, while the rest of the earlier kernel
    // drains; everything else waits for the earlier kernel's completion (griddepcontrol.wait).
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((1 + kStreamWarps + 4) * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = p.no_pdl ? 0 : 1;
    return (int)cudaLaunchKernelEx(&cfg, kern, p);
}

template <int FMT, bool KWHOLE>
int launch_rows(const TkdParams& p, int grid, size_t smem, cudaStream_t st) {
    // (p.x_smem: x fits beside the ring in shared memory, which the one-row instantiations rely on)
    if (p.M == 1 && p.x_smem && !p.topk_k && !p.npeers) return launch_one<FMT, true, true, KWHOLE, true>(p, grid, smem, st);
    if (p.M == 1 && p.x_smem) return launch_one<FMT, true, false, KWHOLE, true>(p, grid, smem, st);
    // (9 to 32 rows run tkd_stream_tc_kernel: the caller never gets here with them)
    if (p.x_smem) return launch_one<FMT, false, false, KWHOLE, true>(p, grid, smem, st);
    return launch_one<FMT, false, false, KWHOLE, false>(p, grid, smem, st);
}

template <int FMT>
int launch_fmt(const TkdParams& p, int grid, size_t smem, cudaStream_t st) {
    // (a K of whole chunks, the usual case, runs the instantiation without the code for a last, shorter chunk)
    return p.K % (Fmt<FMT>::SUBSA * Fmt<FMT>::KSA) == 0 ? launch_rows<FMT, true>(p, grid, smem, st)
                                                       : launch_rows<FMT, false>(p, grid, smem, st);
}

}  // namespace
