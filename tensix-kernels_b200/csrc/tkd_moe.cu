// tkd_moe.cu: the mixture-of-experts layer's two matmuls over the chosen experts only, for sm_100a. They take the
// place of the reference's gate_up / down and gate_up_rows / down_rows (moe/moe8.py:710-911, 928-1136; kernels
// moe_gu_reader.cpp, moe_gu_compute.cpp, moe_gu_writer.cpp, moe_dn_reader.cpp, moe_dn_compute.cpp, moe_dn_writer.cpp
// and kernels/moe8_rows.h for the union of the rows' experts).
//
// Every expert's weight is a bfloat4_b stream of tkd_layout.h (tkd_pack), all experts back to back, so the kernel
// finds a chosen expert by its id alone: the ids are read on the device and nothing goes to the host. What a call reads
// is small (k experts of a few MB) and scattered, so instead of the persistent ring of tkd_stream_kernel.cuh this is
// a plain grid: a CTA owns (32 columns of one slot's expert, all of its K), its 4 warps are 2 groups of 16 columns x 2
// runs of super-atoms, and a lane loads its own 16 bytes of codes and 16 bytes of exponents of a super-atom straight
// from global memory into the mma.sync A fragment's registers (the stream is laid out lane by lane, so a warp's load
// is one contiguous 512 bytes), four super-atoms at a time. The decode is the stream kernel's (block_mma), and like it
// the kernel is bound by instruction issue, not by HBM: units this small (384 and 512 CTAs of 128 threads for a layer
// of 8 experts of 2048 x 1536) are what spreads that work evenly over the SMs.
//   gate_up: a unit is 16 columns of a gate tile and the same 16 of its up tile: the CTA finishes 16 outputs,
//            h = routing weight * act(x G + b) * (x U + b), rounded to bf16 once.
//   down:    a CTA writes its slot's partial sums of 32 columns of y to the workspace; the CTA that arrives last at
//            the unit's counter adds the slots up in slot order and writes y (no CTA waits for another).
// R rows (by_union): every CTA builds the set of distinct experts of the R x k ids (a bitmap), slot q is its q-th
// member, the rows are the columns of the mma's B operand (8 a tile), and a CTA keeps the rows' activations in shared
// memory for several units.
#include "tkd_stream_kernel.cuh"

namespace {

constexpr int kMoeGroups = 2;  // groups of 16 columns a CTA covers at a time (gate_up: 16 gate columns and their 16 up columns)
// warps along K per group. One row: 2 (4 warps a CTA, four CTAs an SM; with 4 a warp had too few super-atoms to spread its
// set-up over: the layer of the benchmark 16.9 us, 16.35 with down at 2, 16.8 with gate_up at 2; down at 1: 17.6). By
// union, where the rows' activations leave room for one or two CTAs an SM: 8 (16 warps).
constexpr int kMoeSplitOne = 2, kMoeSplitRows = 8;
__host__ __device__ constexpr int moe_split(bool rows, bool down) { return rows ? kMoeSplitRows : kMoeSplitOne; }
constexpr int kMoeBatch = 4;  // super-atoms whose loads are issued before the first is used (8: spills, slower)
constexpr int kMoeCols = kMoeGroups * 16;

struct MoeParams {
    const uint8_t* w;
    const uint8_t* emax;
    int64_t wbytes;
    int E, K, N, npad, R;
    int RB;  // rows a pass: what fits in shared memory (the weights are read again, from L2, for the next rows)
    const uint16_t* x;
    int64_t ldx;
    const void* ids;
    int ids32, k;
    int64_t ld_ids;
    const uint16_t* rw;
    int64_t ld_w;
    int slots, act;
    const uint16_t* bias;
    uint16_t* out;
    int64_t ldo;
    float* part;    // down: [slot][row][npad] partial sums
    int* counters;  // down: one per block of 64 columns; back to zero when the call ends
    uint32_t mul16, mul128;
};

__device__ __forceinline__ uint4 ldg_stream(const uint8_t* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t moe_id(const MoeParams& p, int64_t i) {
    return p.ids32 ? static_cast<const uint32_t*>(p.ids)[i] : static_cast<const uint16_t*>(p.ids)[i];
}
// a column sum in the stream's units -> its value (tkd_layout.h: 2^tkd_out_exp, in two factors that are normal floats)
__device__ __forceinline__ float moe_scale(float v, int ebyte) {
    const int e = tkd_out_exp(TKD_BFP4, ebyte), e1 = e / 2, e2 = e - e1;
    return v * __uint_as_float((uint32_t)(e1 + 127) << 23) * __uint_as_float((uint32_t)(e2 + 127) << 23);
}
// moe8.py:83-85, 607-616: silu, gelu_tanh, or gpt-oss's clamped SwiGLU min(g, 7) * sigmoid(1.702 min(g, 7)) * (clamp(u, -7, 7) + 1)
__device__ __forceinline__ float moe_glu(float gt, float u, int act) {
    if (act == 2) {
        const float gc = fminf(gt, 7.f);
        return gc / (1.f + __expf(-1.702f * gc)) * (fminf(fmaxf(u, -7.f), 7.f) + 1.f);
    }
    return act_gate(gt, act) * u;
}

// FMT: the experts' stream format (bfloat4_b, or bf16 for a pack held exactly). MT: tiles of 8 rows. ROWS: by_union. DOWN:
// the down matmul.
template <int FMT, int MT, bool ROWS, bool DOWN>
__global__ void __launch_bounds__(kMoeGroups * moe_split(ROWS, DOWN) * 32, ROWS ? (MT == 1 ? 2 : 1) : 4)
    tkd_moe_kernel(const MoeParams p) {
    constexpr int kMoeSplit = moe_split(ROWS, DOWN), kMoeThreads = kMoeGroups * kMoeSplit * 32;
    using F = Fmt<FMT>;  // (k and bytes of a super-atom, super-atoms of a group in a chunk)
    extern __shared__ __align__(16) uint8_t moe_dsm[];
    __shared__ uint32_t bm[32];  // ROWS: a bit per expert some row chose
    __shared__ float wrow[32];   // ROWS: row r's routing weight for this CTA's expert (0: not chosen)
    __shared__ int s_e, s_count, s_last;
    constexpr int RP = 8 * MT + (ROWS ? 1 : 0);  // floats a column of the sums (odd for several rows: no bank conflicts)
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int gi = warp & (kMoeGroups - 1), ksp = warp / kMoeGroups;
    const int q = blockIdx.y;
    const int R = p.R;
    const int Kpad = (p.K + 63) & ~63;
    // bytes from a row of the activations in shared memory to the next (several rows: 16 banks on, so that the 8 rows a
    // quarter-warp's lanes read lie in different banks)
    const int xstride = Kpad * 2 + (ROWS ? 64 : 16);
    uint8_t* xs = moe_dsm;
    float* red = reinterpret_cast<float*>(moe_dsm + (((size_t)p.RB * xstride + 15) & ~(size_t)15));  // [ksp][column][RP]

    // (launched as a programmatic dependent: nothing the kernels before wrote is read above this line, and the kernel
    // after may bring its CTAs in while this one runs: it waits at the same place)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // ---- this CTA's expert
    int e = -1, count = p.slots;
    if constexpr (!ROWS) {
        const uint32_t id = moe_id(p, q);
        if (id < (uint32_t)p.E) e = (int)id;
    } else {
        if (tid < 32) bm[tid] = 0;
        __syncthreads();
        for (int i = tid; i < R * p.k; i += kMoeThreads) {
            const int r = i / p.k;
            const uint32_t id = moe_id(p, r * p.ld_ids + (i - r * p.k));
            if (id < (uint32_t)p.E) atomicOr(&bm[id >> 5], 1u << (id & 31));
        }
        __syncthreads();
        if (warp == 0) {
            const uint32_t word = bm[lane];
            const int c = __popc(word);
            int incl = c;  // set bits up to and including this lane's word
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int v = __shfl_up_sync(0xFFFFFFFFu, incl, d);
                if (lane >= d) incl += v;
            }
            const int total = __shfl_sync(0xFFFFFFFFu, incl, 31);
            if (lane == 0) s_count = total, s_e = -1;
            __syncwarp();
            if (q >= incl - c && q < incl) {  // the slot's expert is the (q - before)-th set bit of this word
                uint32_t wv = word;
                for (int j = incl - c; j < q; ++j) wv &= wv - 1;
                s_e = lane * 32 + __ffs(wv) - 1;
            }
        }
        __syncthreads();
        e = s_e, count = s_count;
        if constexpr (!DOWN) {
            if (tid < 32) {
                float wv = 0.f;
                if (tid < R && e >= 0)
                    for (int s = 0; s < p.k; ++s)
                        if (moe_id(p, tid * p.ld_ids + s) == (uint32_t)e) wv = bf16_bits_to_f32(p.rw[tid * p.ld_w + s]);
                wrow[tid] = wv;
            }
        }
    }

    float w1 = 0.f;  // one row: the slot's routing weight
    if constexpr (!ROWS && !DOWN)
        if (e >= 0) w1 = bf16_bits_to_f32(p.rw[q]);
    // units of 32 weight columns; this CTA takes every gridDim.x-th. gate_up: unit u is half hf = u & 1 of the tile pair
    // j = u >> 1: columns hf * 16 .. + 15 of gate tile j (warps gi 0) and of up tile j (gi 1), 16 outputs.
    const int nunits = (DOWN ? p.npad : p.N) / kMoeCols;
    // (its nmine units, begun at a different one in every slot: the slots' CTAs reach a unit's counter at different times,
    // and the one that adds a unit's slots up, the last to arrive, is a different one from unit to unit. With every CTA
    // going through the units in the same order the last stayed last: 908 us against 407 for 32 rows of 8 experts.)
    const int nmine = (nunits - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x, urot = ROWS ? q : 0;
    const uint8_t* wb = p.w + (int64_t)max(e, 0) * p.wbytes;
    const uint8_t* emx = FMT == TKD_BFP4 ? p.emax + (int64_t)max(e, 0) * (p.npad / 16) : nullptr;
    const int nsa = (p.K + F::KSA - 1) / F::KSA, per = (nsa + kMoeSplit - 1) / kMoeSplit;
    const int sa0 = ksp * per, sa1 = min(nsa, sa0 + per);
    const uint2 sh = make_uint2(p.mul16, p.mul128);
    // The first unit's super-atoms of this warp are asked into L2 at once (one instruction per run inside a chunk), so
    // that the loads behind the first batch, which wait for registers, find them there: one trip to HBM, not two.
    if (e >= 0 && lane == 0 && nmine > 0) {
        const int u = blockIdx.x + urot % nmine * gridDim.x, group = DOWN ? u * kMoeGroups + gi : (u >> 1) * 4 + 2 * gi + (u & 1);
        for (int sa = sa0; sa < sa1;) {
            const int end = min(sa1, (sa | (F::SUBSA - 1)) + 1);
            const uint8_t* s = wb + tkd_sa_offset(FMT, p.K, group, sa);
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(s), "r"((end - sa) * F::SAB) : "memory");
            sa = end;
        }
    }
    for (int r0 = 0; r0 < R; r0 += p.RB) {
        const int Rb = min(p.RB, R - r0);
        const bool last_rows = r0 + p.RB >= R;
        // ---- the activations: gate_up: the rows of x; down: the rows' inputs of slot q. Zeros past K up to a super-atom.
        if (e >= 0) {
            const uint16_t* xsrc = p.x + (int64_t)r0 * p.ldx + (DOWN ? (int64_t)q * p.K : 0);
            const int vec = Kpad / 8;
            for (int i = tid; i < Rb * vec; i += kMoeThreads) {
                const int r = ROWS ? i / vec : 0, c = i - r * vec;
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (c * 8 < p.K) v = __ldg(reinterpret_cast<const uint4*>(xsrc + (int64_t)r * p.ldx) + c);
                *reinterpret_cast<uint4*>(xs + (size_t)r * xstride + (size_t)c * 16) = v;
            }
        }
        __syncthreads();
        uint32_t xa[MT];  // (a lane past the last row reads the last row: its column of the result is never used)
#pragma unroll
        for (int m = 0; m < MT; ++m) xa[m] = smem_u32(xs) + (uint32_t)min(8 * m + g, Rb - 1) * xstride + 16 * t;
        for (int it = 0; it < nmine; ++it) {
            const int u = blockIdx.x + (it + urot) % nmine * gridDim.x;
            const int group = DOWN ? u * kMoeGroups + gi : (u >> 1) * 4 + 2 * gi + (u & 1);
            if (e >= 0) {
                // ---- the group's sums over this warp's run of super-atoms
                float acc[2][MT][4];
#pragma unroll
                for (int a = 0; a < 2; ++a)
#pragma unroll
                    for (int m = 0; m < MT; ++m) acc[a][m][0] = acc[a][m][1] = acc[a][m][2] = acc[a][m][3] = 0.f;
                // (the super-atoms of a group lie back to back inside a chunk of 8: the layout is asked at its starts only)
                const uint8_t* s = wb;
                for (int sa = sa0; sa < sa1; sa += kMoeBatch) {
                    uint4 cv[kMoeBatch], ev[kMoeBatch];
#pragma unroll
                    for (int b = 0; b < kMoeBatch; ++b)
                        if (sa + b < sa1) {
                            s = (b == 0 && sa == sa0) || ((sa + b) & (F::SUBSA - 1)) == 0 ? wb + tkd_sa_offset(FMT, p.K, group, sa + b)
                                                                                          : s + F::SAB;
                            if constexpr (FMT == TKD_BFP4) {
                                ev[b] = ldg_stream(s + t * 16);
                                cv[b] = ldg_stream(s + 64 + lane * 16);
                            } else {  // (bf16: the A fragments of the super-atom's two mmas as they are)
                                cv[b] = ldg_stream(s + lane * 16);
                                ev[b] = ldg_stream(s + 512 + lane * 16);
                            }
                        }
#pragma unroll
                    for (int b = 0; b < kMoeBatch; ++b)
                        if (sa + b < sa1) {
                            if constexpr (FMT == TKD_BFP4) {
#pragma unroll
                                for (int qq = 0; qq < 2; ++qq) {
                                    const uint32_t cw[4] = {qq ? cv[b].z : cv[b].x, qq ? cv[b].w : cv[b].y, 0u, 0u};
                                    const uint32_t ew[2] = {qq ? ev[b].z : ev[b].x, qq ? ev[b].w : ev[b].y};
                                    uint4 xv[MT];
#pragma unroll
                                    for (int m = 0; m < MT; ++m) xv[m] = lds128(xa[m] + (uint32_t)(sa + b) * 128 + 64 * qq);
                                    block_mma<TKD_BFP4, MT, 2>(acc, cw, ew, xv, sh);
                                }
                            } else {
#pragma unroll
                                for (int m = 0; m < MT; ++m) {
                                    const uint4 xv = lds128(xa[m] + (uint32_t)(sa + b) * 64);
                                    mma_bf16(acc[0][m], cv[b].x, cv[b].y, cv[b].z, cv[b].w, xv.x, xv.y);
                                    mma_bf16(acc[1][m], ev[b].x, ev[b].y, ev[b].z, ev[b].w, xv.z, xv.w);
                                }
                            }
                        }
                }
                // D fragment: (column g, rows 2t and 2t + 1), (column g + 8, the same rows)
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    float* d0 = red + ((size_t)(ksp * kMoeCols + gi * 16 + g) * RP) + 8 * m + 2 * t;
                    d0[0] = acc[0][m][0] + acc[1][m][0], d0[1] = acc[0][m][1] + acc[1][m][1];
                    d0[8 * RP] = acc[0][m][2] + acc[1][m][2], d0[8 * RP + 1] = acc[0][m][3] + acc[1][m][3];
                }
            }
            __syncthreads();

            // column c of the unit (gate_up: 0-15 the gate's, 16-31 the up's), row r: the K sum, in the weight's units
            auto column_sum = [&](int c, int r, int grp) {
                float v = 0.f;
#pragma unroll
                for (int sp = 0; sp < kMoeSplit; ++sp) v += red[(size_t)(sp * kMoeCols + c) * RP + r];
                if constexpr (FMT == TKD_BFP4) v = moe_scale(v, emx[grp]);
                return v;
            };
            if constexpr (!DOWN) {
                const int I = p.N / 2, j = u >> 1, hf = u & 1;
                for (int o = tid; o < 16 * Rb; o += kMoeThreads) {
                    const int c = o & 15, r = o >> 4;
                    float val = 0.f;
                    if (e >= 0) {
                        float gt = column_sum(c, r, j * 4 + hf), up = column_sum(16 + c, r, j * 4 + 2 + hf);
                        if (p.bias) {
                            const uint16_t* b = p.bias + (int64_t)e * p.npad + j * 64 + hf * 16 + c;
                            gt += bf16_bits_to_f32(b[0]), up += bf16_bits_to_f32(b[32]);
                        }
                        val = moe_glu(gt, up, p.act) * (ROWS ? wrow[r0 + r] : w1);
                    }
                    p.out[(int64_t)(r0 + r) * p.ldo + (int64_t)q * I + j * 32 + hf * 16 + c] = f32_to_bf16_bits(val);
                }
                __syncthreads();  // (the next unit overwrites the sums)
            } else {
                if (e >= 0)
                    for (int o = tid; o < kMoeCols * Rb; o += kMoeThreads) {
                        const int c = o & (kMoeCols - 1), r = o / kMoeCols;
                        p.part[((int64_t)q * R + r0 + r) * p.npad + u * kMoeCols + c] = column_sum(c, r, u * kMoeGroups + (c >> 4));
                    }
                if (last_rows) {
                    // this slot's sums of the unit's columns are written: the CTA that arrives last adds the slots up
                    __threadfence();
                    __syncthreads();
                    if (tid == 0) s_last = atomicAdd(&p.counters[u], 1) == p.slots - 1;
                    __syncthreads();
                    if (s_last) {
                        __threadfence();
                        for (int o = tid; o < kMoeCols * R; o += kMoeThreads) {
                            const int c = o & (kMoeCols - 1), r = o / kMoeCols, col = u * kMoeCols + c;
                            if (col >= p.N) continue;
                            float v = 0.f;
                            const float* src = p.part + (int64_t)r * p.npad + col;
                            const int64_t step = (int64_t)R * p.npad;
                            for (int sl = 0; sl < count; sl += 8) {  // (eight loads in flight; added in slot order)
                                float part[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    bool live = sl + j < count;
                                    if constexpr (!ROWS) live = live && moe_id(p, sl + j) < (uint32_t)p.E;
                                    part[j] = live ? __ldcg(src + (sl + j) * step) : 0.f;
                                }
#pragma unroll
                                for (int j = 0; j < 8; ++j) v += part[j];
                            }
                            p.out[(int64_t)r * p.ldo + col] = f32_to_bf16_bits(v);
                        }
                        if (tid == 0) p.counters[u] = 0;
                    }
                }
                __syncthreads();  // (the next unit overwrites the sums, and s_last)
            }
        }
        __syncthreads();  // (the next rows overwrite the activations)
    }
}

// ---- the router's top k and their weights (moe/moe8.py:1139-1253 route, kernels/moe_route.cpp of the reference). One warp a
// row: the keys in float64 in shared memory (the reference's core works in fixed point to the same end: picks that equal
// a float64 host computation's), k rounds of a warp-wide argmax (the larger key, the lower id among equal keys), then the
// picks' weights in float64, rounded to bf16 once.
constexpr int kRouteMaxE = 1024;

struct RouteParams {
    const float* logits;
    int64_t ld;
    int E, k, kind, norm, ng, tg, has_slot, ids32;
    const float* bias;
    double scale;
    uint32_t slot;
    void* ids;
    int64_t ld_ids;
    uint16_t* w;
    int64_t ld_w;
    uint16_t* shared;
    int64_t ld_sh;
};

// (the better of two candidates: key, then the lower index; idx < 0: none)
__device__ __forceinline__ void route_better(double& key, int& idx, double k2, int i2) {
    if (i2 >= 0 && (idx < 0 || k2 > key || (k2 == key && i2 < idx))) key = k2, idx = i2;
}
__device__ __forceinline__ void route_warp_best(double& key, int& idx) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        const double k2 = __shfl_xor_sync(0xFFFFFFFFu, key, d);
        const int i2 = __shfl_xor_sync(0xFFFFFFFFu, idx, d);
        route_better(key, idx, k2, i2);
    }
}
__device__ __forceinline__ uint16_t route_bf16(double v) { return f32_to_bf16_bits((float)v); }

__global__ void __launch_bounds__(32) tkd_moe_route_kernel(const RouteParams p) {
    __shared__ double skey[kRouteMaxE], ssig[kRouteMaxE];
    __shared__ uint32_t taken[kRouteMaxE / 32];
    __shared__ int pick[16];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int row = blockIdx.x, lane = threadIdx.x;
    const float* lg = p.logits + (int64_t)row * p.ld;
    const double ninf = -__longlong_as_double(0x7FF0000000000000LL);
    for (int e = lane; e < p.E; e += 32) {
        const double x = (double)lg[e];
        const double sg = 1.0 / (1.0 + exp(-x));
        ssig[e] = sg;
        // kind 0: softmax, by logit; 1: sigmoid + bias; 2: sigmoid without a bias, by logit (sigmoid is increasing, and in
        // float64 it saturates, which would tie logits that differ)
        skey[e] = p.kind == 1 ? sg + (double)p.bias[e] : x;
    }
    if (lane < kRouteMaxE / 32) taken[lane] = 0;
    __syncwarp();
    if (p.ng > 1) {
        // group-limited routing: a group's score is the sum of its two largest keys; the tg best groups stay (the lower
        // group among equal scores), the others' experts are out
        const int ge = p.E / p.ng;
        double score = ninf;
        if (lane < p.ng) {
            double a = ninf, b = ninf;
            for (int i = 0; i < ge; ++i) {
                const double v = skey[lane * ge + i];
                if (v > a) b = a, a = v;
                else if (v > b) b = v;
            }
            score = a + b;
        }
        uint32_t kept = 0;
        for (int j = 0; j < p.tg; ++j) {
            double key = score;
            int idx = (lane < p.ng && !((kept >> lane) & 1u)) ? lane : -1;
            route_warp_best(key, idx);
            if (idx >= 0) kept |= 1u << idx;
        }
        for (int wd = lane; wd < p.E / 32; wd += 32) {
            uint32_t m = 0;
            for (int b = 0; b < 32; ++b)
                if (!((kept >> ((wd * 32 + b) / ge)) & 1u)) m |= 1u << b;
            taken[wd] = m;
        }
        __syncwarp();
    }
    for (int j = 0; j < p.k; ++j) {
        double key = 0.0;
        int idx = -1;
        for (int e = lane; e < p.E; e += 32)
            if (!((taken[e >> 5] >> (e & 31)) & 1u)) route_better(key, idx, skey[e], e);
        route_warp_best(key, idx);
        if (lane == 0) {
            pick[j] = idx;
            if (idx >= 0) taken[idx >> 5] |= 1u << (idx & 31);
        }
        __syncwarp();
    }
    // the weights: softmax over the picks' logits, or the picks' sigmoids (over their sum unless norm is off), times scale
    const int id = lane < p.k ? pick[lane] : -1;
    double v = 0.0;
    if (p.kind == 0) {
        const double top = skey[max(pick[0], 0)];
        if (id >= 0) v = exp(skey[id] - top);
    } else if (id >= 0) {
        v = ssig[id];
    }
    double sum = v;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, d);
    const double wv = (p.kind == 0 || p.norm ? v / sum : v) * p.scale;
    const int slots = p.k + p.has_slot;
    if (lane < slots) {
        const bool extra = lane == p.k;  // the fixed slot: that id at weight 1
        const uint32_t out_id = extra ? p.slot : (uint32_t)max(id, 0);
        if (p.ids32) static_cast<uint32_t*>(p.ids)[(int64_t)row * p.ld_ids + lane] = out_id;
        else static_cast<uint16_t*>(p.ids)[(int64_t)row * p.ld_ids + lane] = (uint16_t)out_id;
        p.w[(int64_t)row * p.ld_w + lane] = route_bf16(extra ? 1.0 : (id >= 0 ? wv : 0.0));
    }
    if (p.shared && lane == 0) p.shared[(int64_t)row * p.ld_sh] = route_bf16(1.0 / (1.0 + exp(-(double)lg[p.E])));
}


size_t moe_smem(int R, int K, int MT, bool rows, bool down) {
    const int Kpad = (K + 63) & ~63, split = moe_split(rows, down);
    return (((size_t)R * (Kpad * 2 + (rows ? 64 : 16)) + 15) & ~(size_t)15) +
           (size_t)split * kMoeCols * (8 * MT + (rows ? 1 : 0)) * sizeof(float);
}

template <int FMT, int MT, bool ROWS, bool DOWN>
int moe_launch(const MoeParams& p, dim3 grid, size_t smem, cudaStream_t st) {
    auto kern = tkd_moe_kernel<FMT, MT, ROWS, DOWN>;
    if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid, cfg.blockDim = dim3(kMoeGroups * moe_split(ROWS, DOWN) * 32);
    cfg.dynamicSmemBytes = smem, cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, kern, p);
}

template <int FMT, bool DOWN>
int moe_dispatch_fmt(const MoeParams& p, bool rows, dim3 grid, size_t smem, int mt, cudaStream_t st) {
    if (!rows) return moe_launch<FMT, 1, false, DOWN>(p, grid, smem, st);
    switch (mt) {
        case 1: return moe_launch<FMT, 1, true, DOWN>(p, grid, smem, st);
        case 2: return moe_launch<FMT, 2, true, DOWN>(p, grid, smem, st);
        case 3: return moe_launch<FMT, 3, true, DOWN>(p, grid, smem, st);
        default: return moe_launch<FMT, 4, true, DOWN>(p, grid, smem, st);
    }
}
template <bool DOWN>
int moe_dispatch(const MoeParams& p, int fmt, bool rows, dim3 grid, size_t smem, int mt, cudaStream_t st) {
    return fmt == TKD_BF16 ? moe_dispatch_fmt<TKD_BF16, DOWN>(p, rows, grid, smem, mt, st)
                           : moe_dispatch_fmt<TKD_BFP4, DOWN>(p, rows, grid, smem, mt, st);
}

bool moe_args_ok(const TkdMoe* a, bool down) {
    if (!a || !a->w || !a->x || !a->ids || !a->out) return false;
    if (a->fmt != TKD_FMT_BFP4 && a->fmt != TKD_FMT_BF16) return false;
    if (a->fmt == TKD_FMT_BFP4 && !a->emax) return false;
    if (a->experts < 1 || a->k_in < 32 || a->k_in % 32 || a->n < 32 || a->n % 32 || a->k < 1 || a->k > 16) return false;
    if (a->rows < 1 || a->rows > 32 || (!a->by_union && a->rows != 1)) return false;
    if (a->by_union && (a->experts > 1024 || a->slots < 1 || a->ld_ids < a->k)) return false;
    if (!a->by_union && a->slots != a->k) return false;
    if (a->expert_bytes < tkd_packed_bytes(a->fmt, a->k_in, a->n) || a->expert_bytes % 16) return false;
    if (a->ldx % 8 || (reinterpret_cast<uintptr_t>(a->x) | reinterpret_cast<uintptr_t>(a->w)) & 15) return false;
    if (down) {
        if (a->ldx < (int64_t)a->slots * a->k_in || a->ldo < a->n) return false;
    } else {
        if (a->n % 64 || !a->route_w || a->ldx < a->k_in || a->ldo < (int64_t)a->slots * (a->n / 2)) return false;
        if (a->act < 0 || a->act > 2 || (a->by_union && a->ld_w < a->k)) return false;
    }
    return true;
}

MoeParams moe_params(const TkdMoe* a) {
    MoeParams p = {};
    p.w = static_cast<const uint8_t*>(a->w), p.emax = a->emax, p.wbytes = a->expert_bytes;
    p.E = a->experts, p.K = a->k_in, p.N = a->n, p.npad = (int)tkd_padded_cols(a->n), p.R = a->rows;
    p.x = static_cast<const uint16_t*>(a->x), p.ldx = a->ldx;
    p.ids = a->ids, p.ids32 = a->ids32, p.k = a->k, p.ld_ids = a->ld_ids;
    p.rw = static_cast<const uint16_t*>(a->route_w), p.ld_w = a->ld_w;
    p.slots = a->slots, p.act = a->act, p.bias = static_cast<const uint16_t*>(a->bias);
    p.out = static_cast<uint16_t*>(a->out), p.ldo = a->ldo;
    p.mul16 = 16, p.mul128 = 128;
    return p;
}

int moe_smem_limit() {
    static int cached = 0;
    if (!cached) {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) != cudaSuccess) return 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return 0;
        cached = v;
    }
    return cached;
}

int moe_sms() {
    static int cached = 0;
    if (!cached) {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            return 148;
        cached = v;
    }
    return cached;
}
// CTAs per slot. One row: a CTA per unit of 32 columns. By union: a CTA keeps the rows' activations in shared memory
// for several units, and all CTAs of the call are resident at once (one an SM, two up to 8 rows): with a second wave, down's last
// arrivals at every unit's counter, and with them all the adding up of slots, fall to that wave's CTAs.
int moe_grid_x(const TkdMoe* a, int nunits) {
    if (!a->by_union) return nunits;
    const int want = (a->rows <= 8 ? 2 : 1) * moe_sms() / a->slots;  // (up to 8 rows: two CTAs fit an SM)
    return want < 1 ? 1 : (want > nunits ? nunits : want);
}

// How many rows a pass of the kernel takes: all of them if their activations fit in shared memory beside the sums,
// else as many tiles of 8 as fit (then fewer than 8). false: not even one row fits.
bool moe_rows_a_pass(const TkdMoe* a, bool down, int* rb, int* mt, size_t* smem) {
    const int64_t limit = (int64_t)moe_smem_limit() - 2048;
    for (int rows = a->rows; rows >= 1; rows = rows > 8 ? ((rows - 1) & ~7) : rows - 1) {
        const int tiles = a->by_union ? (rows + 7) / 8 : 1;
        const size_t need = moe_smem(rows, a->k_in, tiles, a->by_union != 0, down);
        if ((int64_t)need <= limit) {
            *rb = rows, *mt = tiles, *smem = need;
            return true;
        }
    }
    return false;
}

}  // namespace

extern "C" {

int tkd_moe_workspace(const TkdMoe* a, uint64_t* bytes) {
    if (!a || !bytes || a->slots < 1 || a->rows < 1 || a->n < 1) return TKD_ERR_BAD_ARG;
    const int64_t npad = tkd_padded_cols(a->n);
    // the column blocks' counters (a cache line's worth at least), then the slots' partial sums
    *bytes = (uint64_t)(((npad / kMoeCols) * 4 + 255) & ~(int64_t)255) + (uint64_t)a->slots * a->rows * npad * sizeof(float);
    return TKD_OK;
}

int tkd_moe_gate_up(const TkdMoe* a, void* stream) {
    if (!moe_args_ok(a, false)) return TKD_ERR_BAD_ARG;
    MoeParams p = moe_params(a);
    int mt = 1;
    size_t smem = 0;
    if (!moe_rows_a_pass(a, false, &p.RB, &mt, &smem)) return TKD_ERR_UNSUPPORTED;
    const dim3 grid((unsigned)moe_grid_x(a, a->n / kMoeCols), (unsigned)a->slots);
    const int e = moe_dispatch<false>(p, a->fmt, a->by_union != 0, grid, smem, mt, static_cast<cudaStream_t>(stream));
    return e == 0 ? TKD_OK : TKD_ERR_CUDA + e;
}

int tkd_moe_down(const TkdMoe* a, void* stream) {
    if (!moe_args_ok(a, true)) return TKD_ERR_BAD_ARG;
    uint64_t need = 0;
    tkd_moe_workspace(a, &need);
    if (!a->workspace || a->workspace_bytes < need || (reinterpret_cast<uintptr_t>(a->workspace) & 15)) return TKD_ERR_WORKSPACE;
    MoeParams p = moe_params(a);
    const int64_t npad = tkd_padded_cols(a->n);
    p.counters = static_cast<int*>(a->workspace);
    p.part = reinterpret_cast<float*>(static_cast<uint8_t*>(a->workspace) + (((npad / kMoeCols) * 4 + 255) & ~(int64_t)255));
    int mt = 1;
    size_t smem = 0;
    if (!moe_rows_a_pass(a, true, &p.RB, &mt, &smem)) return TKD_ERR_UNSUPPORTED;
    const dim3 grid((unsigned)moe_grid_x(a, (int)(npad / kMoeCols)), (unsigned)a->slots);
    const int e = moe_dispatch<true>(p, a->fmt, a->by_union != 0, grid, smem, mt, static_cast<cudaStream_t>(stream));
    return e == 0 ? TKD_OK : TKD_ERR_CUDA + e;
}

int tkd_moe_route(const float* logits, int64_t ld, int rows, int experts, int k, int kind, const float* bias, double scale,
                  int norm, int n_group, int topk_group, int has_slot, uint32_t slot, void* ids, int ids32, int64_t ld_ids,
                  void* w, int64_t ld_w, void* shared, int64_t ld_shared, void* stream) {
    if (!logits || !ids || !w || rows < 1 || rows > 32 || experts < 32 || experts % 32 || experts > kRouteMaxE) return TKD_ERR_BAD_ARG;
    if (k < 1 || k > 16 || k > experts || (has_slot && k + 1 > 16) || kind < 0 || kind > 2 || (kind == 1 && !bias)) return TKD_ERR_BAD_ARG;
    if (!(scale > 0.0 && scale < 4.0) || (!norm && kind == 0)) return TKD_ERR_BAD_ARG;
    if (ld < experts + (shared ? 1 : 0) || ld_ids < k + (has_slot ? 1 : 0) || ld_w < k + (has_slot ? 1 : 0)) return TKD_ERR_BAD_ARG;
    if (n_group > 1) {
        if (kind != 1 || n_group > 32 || experts % n_group || experts / n_group < 2 || topk_group < 1 || topk_group > n_group ||
            topk_group * (experts / n_group) < k)
            return TKD_ERR_BAD_ARG;
    }
    RouteParams p = {};
    p.logits = logits, p.ld = ld, p.E = experts, p.k = k, p.kind = kind, p.norm = norm, p.ng = n_group > 1 ? n_group : 1;
    p.tg = topk_group, p.has_slot = has_slot ? 1 : 0, p.ids32 = ids32, p.bias = bias, p.scale = scale, p.slot = slot;
    p.ids = ids, p.ld_ids = ld_ids, p.w = static_cast<uint16_t*>(w), p.ld_w = ld_w;
    p.shared = static_cast<uint16_t*>(shared), p.ld_sh = ld_shared;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)rows), cfg.blockDim = dim3(32), cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = 1;
    const int e = (int)cudaLaunchKernelEx(&cfg, tkd_moe_route_kernel, p);
    return e == 0 ? TKD_OK : TKD_ERR_CUDA + e;
}
}
