// tkd_stream_tc.cuh: the stream kernel for 9 to 32 activation rows, on the fifth-generation tensor cores (tcgen05).
//
// The reference multiplies a tile of up to 32 activation rows by each weight tile it has read (dense_reader/kernels/
// dense_compute.cpp:95-143, matmul_block): more rows cost it no more weight traffic and hardly more time. With
// mma.sync the same holds for the traffic but not for the time: 32 rows of accumulators leave room for two streaming
// warps per scheduler, which wait on their own shared-memory loads and mma chains. Here the weights of a panel are
// decoded into bf16 tiles in shared memory once, whatever the row count, and one thread issues tcgen05.mma on them with
// the accumulators in tensor memory:
//
//   warps 3-18     decode warps, in two groups of eight; a unit of two tiles of 64 k is one group's work (units in turn:
//                  while one group waits for its stores to land, the other decodes). A warp turns its 16 columns' share
//                  of the unit into bf16 (code times 2^e', one multiply per two weights: every block-float value is a
//                  bf16 value) and writes it straight into TENSOR MEMORY with tcgen05.st.16x256b, whose thread layout
//                  is the mma A fragment's the stream is packed for (thread (g, t): rows g and g + 8, two 32-bit
//                  columns): the A operand of the MMAs is read from tensor memory, never from shared memory. (A first
//                  version stored the A tiles in shared memory: 32 KB written and 32 KB read by the tensor core per
//                  17 KB of stream made the shared-memory bandwidth the bound, at 3 TB/s.) A warp owns the
//                  tensor-memory lanes of its 16 columns (its number mod 4 is their quarter). A block of 16 k as the
//                  MMA sees it is this layout's: position 4 t + r holds k = 8 t + 4 jj + r of a block of 32 k; the
//                  activations are laid out to match.
//                  The same warps write the tile of activations a unit is multiplied by (32 rows x 64 k, rows past M
//                  zero, K-major with the 128-byte swizzle, in that order of k) into shared memory: each lane loads
//                  its 16 bytes of the NEXT chunk's tiles into registers while it decodes this chunk (they come from
//                  L2, a microsecond away).
//   warps 19-22    output warps (thread = panel column = tensor-memory lane): read a slice's sums with tcgen05.ld, keep
//                  the running sums in shared memory, and from there on do what tkd_stream_kernel's output warps do
//   warp 1         producer (one lane issues): the same ring of packed-weight chunks as tkd_stream_kernel
//   warps 0, 2     one lane of each issues MMAs: D[128 columns, 32 rows] += A (tensor memory) x (x tile)^T, 4 x (K = 16)
//                  a tile, tcgen05.commit onto the unit's "empty" barrier and, at a slice's end, the accumulators' "full"
//
// A slice's sum is accumulated from zero in tensor memory, in two accumulators of 32 columns (the slice's even units
// in d0, its odd units in d1; the slice's sum is d0 + d1). Two such sets, so that the MMAs of the next slice run while
// the output warps drain this one. A column's sum is the ascending sum of its slices' sums in plain fp32 adds, as in
// tkd_stream_kernel, so it depends on K, the format and ks only. No cluster, no multicast, no
// second CTA: cta_group::1 throughout. Every wait is bounded; the kernel always reaches its end, where the warp that
// allocated the tensor memory frees it.
#pragma once
#include "tkd_stream_kernel.cuh"

namespace {

constexpr int kTcGroups = 2;           // groups of decode warps; a unit is one group's
constexpr int kTcSlots = TKD_TC_SLOTS;  // operand slots, each a unit of two tiles of 64 k
constexpr int kTcXTile = 32 * 128;   // bytes of an x tile in shared memory: 32 rows x 64 k of bf16
constexpr int kTcSlot = 2 * kTcXTile;  // ... of a slot's two x tiles
constexpr int kTcACols = 32;         // tensor-memory columns of an A tile: 128 lanes x 64 k of bf16, two to a column
constexpr int kTcAcc0 = 0, kTcA0 = 128;  // tensor-memory columns: two sets of two accumulators of 32, then the A slots
static_assert(kTcA0 + kTcSlots * 2 * kTcACols <= 512, "the A slots must fit the tensor memory");
// Warps: 0 and 2 the MMA issuers, 1 the producer, 3-18 decode, 19-22 output (23 warps: 736 threads may use 88
// registers each, 768 only 80, two fewer than the kernel needs without spilling). The MMA issuer is the warp with the
// lowest number on purpose: the schedulers favour older warps, and as the last warp of the CTA it got an issue slot
// every twenty cycles beside four decode warps that are always ready (its unit of eight MMAs took 770 ns).
constexpr int kTcWarps = 23, kTcMmaWarp = 0, kTcProducerWarp = 1, kTcDecodeWarp0 = 3, kTcOutputWarp0 = 19, kTcMmaWarps = 2;
// the MMA warp number (0, 1) of a warp, or -1: warps 0 and 2
__device__ __forceinline__ int tc_mma_warp(int warp) { return warp == 0 ? 0 : warp == 2 ? 1 : -1; }
constexpr int kTcMP = 40;            // floats per column in tbuf (32 rows, padded)

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major operand tile in the 128-byte swizzle: rows of 128 bytes (64 bf16),
// groups of 8 rows 1024 bytes apart (the stride offset); the leading offset is not used by this layout. Bits 46-47:
// descriptor version 1 (sm_100); bits 61-63: layout 2 (128-byte swizzle). The tile starts on a 1024-byte boundary;
// the k-th block of 16 k inside it is the same descriptor with the start moved on by 32 k bytes.
__device__ __forceinline__ uint64_t tc_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
// Instruction descriptor, kind::f16: D fp32 (bits 4-5 = 1), A and B bf16 (bits 7-9, 10-12 = 1), both K-major (bits 15,
// 16 = 0), N = 32 (bits 17-22 = N / 8), M = 128 (bits 24-28 = M / 16).
constexpr uint32_t kTcIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((32u >> 3) << 17) | ((128u >> 4) << 24);

// D (tensor memory) (+)= A (tensor memory) x B (shared memory, by descriptor). The descriptor comes as its 32-bit
// halves: the issuing thread's own instructions are its cost (a unit's eight MMAs leave it ~40 cycles each), and
// moving a descriptor on is then one 32-bit add instead of a 64-bit one.
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint32_t a_tmem, uint32_t blo, uint32_t bhi, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "r"(blo), "r"(bhi), "r"(kTcIdesc), "r"(accumulate)
        : "memory");
}
// One lane of a converged warp (the hardware's choice). Code under elect.sync instead of `lane == 0` came out faster
// here: the descriptors and addresses of the MMAs it guards stay warp-uniform.
__device__ __forceinline__ bool tc_elect() {
    uint32_t e;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(e));
    return e != 0;
}
// the barrier gets one arrival once every MMA issued so far by this thread has completed
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

template <int FMT, bool KWHOLE>
__global__ void __launch_bounds__(kTcWarps * 32, 1) tkd_stream_tc_kernel(const __grid_constant__ TkdParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    using F = Fmt<FMT>;
    constexpr int SW = 16, MP = kTcMP;
    constexpr int CK = F::SUBSA * F::KSA;
    // A unit of two tiles is written (and its "full" barrier arrived on) by the warps of one group of decode warps.
    constexpr int NWT = 16 / kTcGroups;  // the warps of a group
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + TKD_MAX_STAGES);
    const uint32_t afull0 = smem_u32(bars + 2 * TKD_MAX_STAGES), aempty0 = afull0 + 8 * kTcSlots;
    const uint32_t accfull0 = aempty0 + 8 * kTcSlots, accempty0 = accfull0 + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + TKD_SMEM_HEAD - 32);
    volatile int* sflag = reinterpret_cast<volatile int*>(smem + TKD_SMEM_HEAD - 16);
    uint4* hdr = reinterpret_cast<uint4*>(smem + 512);
    float* tbuf = reinterpret_cast<float*>(smem + p.off_tbuf);  // [128 columns][MP]: the running sums
    uint8_t* ring = smem + p.off_ring;
    // the operand tiles start on a 1024-byte boundary of the shared-memory window (the swizzle is a function of the address)
    const uint32_t ops0 = (smem_u32(smem + p.off_xt) + 1023u) & ~1023u;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (tid == 0) {
        for (int s = 0; s < p.nstages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, SW);
        }
        for (int s = 0; s < kTcSlots; ++s) {
            mbar_init(afull0 + 8 * s, NWT);
            mbar_init(aempty0 + 8 * s, 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(accfull0 + 8 * s, kTcMmaWarps);
            mbar_init(accempty0 + 8 * s, 4);
        }
        sflag[0] = sflag[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const int64_t T = p.total_items;
    const int64_t i0 = idiv(p, T * blockIdx.x, gridDim.x), i1 = idiv(p, T * (blockIdx.x + 1), gridDim.x);
    const int nst = p.nstages;
    const int M = p.M, K = p.K;
    const int topk_k = p.topk_k, npeers = p.npeers;
    const bool glu2 = p.epi == TKD_EPI_GLU2;
    const int nsa_total = (K + F::KSA - 1) / F::KSA;
    if (i0 >= i1) return;  // (before any tensor memory is held; the grid is never larger than the item count)
    const int64_t lastp0 = idiv(p, i1 - 1, p.nslices) * p.nslices;
    const int64_t tail0 = lastp0 > i0 && lastp0 + p.nslices > i1 ? lastp0 : i1;
    const int64_t lead = i1 - tail0;
    const int64_t nitems = i1 - i0;
    auto item_at = [&](int64_t j) { return j < lead ? tail0 + j : i0 + (j - lead); };

    // tensor memory: all 512 columns (two sets of two accumulators of 32, then the A slots of 64), allocated and freed by
    // the MMA warp
    if (warp == kTcMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem0 = *tmem_slot;

    if (warp == kTcProducerWarp) {
        // ---------------------------------------------------------------- producer (as in tkd_stream_kernel; the whole
        // warp walks the loop and one lane issues: a warp whose other lanes wait at the kernel's final barrier while one
        // lane works runs that lane at a fraction of its speed)
        {
            Cursor c, cn;
            uint32_t st = 0;
            bool ok = true;
            cursor_init(cn, p, item_at(0));
            for (int64_t j = 0; j < nitems && ok; ++j) {
                c = cn;
                if (j + 1 < nitems) {
                    if (j + 1 == lead)
                        cursor_init(cn, p, item_at(j + 1));
                    else
                        cursor_next(cn, p);
                }
                const TkdSegDev& sg = p.seg[c.seg];
                const int k0 = c.slice * p.ks, kv = min(p.ks, K - k0);
                const int c0 = k0 / CK, nch = (kv + CK - 1) / CK;
                const uint8_t* src = sg.w + (int64_t)(glu2 ? c.pl >> 1 : c.pl) * p.panel_bytes;
                const uint8_t* src2 = glu2 ? sg.w2 + (int64_t)(c.pl >> 1) * p.panel_bytes : nullptr;
                for (int ch = 0; ch < nch; ++ch, ++st) {
                    const uint32_t s = st % nst;
                    ok = mbar_wait_parked(empty0 + 8 * s, ((st / nst) & 1) ^ 1, p.status);
                    if (!ok) break;
                    const int nsa = min(F::SUBSA, nsa_total - (c0 + ch) * F::SUBSA);
                    const uint32_t gbytes = (uint32_t)nsa * F::SAB;
                    const int64_t coff = (int64_t)(c0 + ch) * (F::SUBSA * F::SAB * 8);
                    const uint32_t dst = smem_u32(ring + (size_t)s * p.stage_bytes);
                    const bool last = ch == nch - 1, end = last && j == nitems - 1;
                    const int knext = end ? K : (last ? cn.slice * p.ks : (c0 + ch + 1) * CK);  // the next stage's first k
                    if (lane == 0) {
                        hdr[s] = make_uint4(end ? ST_END : 0u, 0u, (uint32_t)knext, (uint32_t)((c0 + ch) * CK));
                        mbar_expect_tx(full0 + 8 * s, 8 * gbytes);
                        if (glu2) {
                            const int64_t hoff = coff + (int64_t)(c.pl & 1) * 4 * gbytes;
                            bulk_g2s(dst, src + hoff, 4 * gbytes, full0 + 8 * s);
                            bulk_g2s(dst + 4 * gbytes, src2 + hoff, 4 * gbytes, full0 + 8 * s);
                        } else {
                            bulk_g2s(dst, src + coff, 8 * gbytes, full0 + 8 * s);
                        }
                    }
                    __syncwarp();
                }
            }
            if (!ok) {
                for (uint32_t back = 1; back <= (uint32_t)nst && back <= st; ++back) {
                    const uint32_t q = st - back;
                    for (uint32_t i = 0; i < 64; ++i)
                        if (mbar_try_wait(full0 + 8 * (q % nst), (q / nst) & 1)) break;
                }
            }
        }
    } else if (warp >= kTcDecodeWarp0 && warp < kTcDecodeWarp0 + SW) {
        // ---------------------------------------------------------------- decode warps
        asm volatile("griddepcontrol.wait;" ::: "memory");  // (x may be the output of the kernel before this one)
        // The warps form G groups, and a unit (by its number in this CTA's sequence, mod G) is one group's work from its
        // slot's "empty" to its "full": while a group waits for its stores to land (tcgen05.wait::st, the proxy fence),
        // the others decode. A slot is always the same group's (kTcSlots is a multiple of G), so the group's warps see
        // every phase of its barriers. A warp may touch the tensor-memory lanes 32 (warp % 4) .. + 31 only: its RG row
        // groups of 16 panel columns are among them.
        constexpr int G = kTcGroups, RG = G / 2, PP = G / 2;
        static_assert(kTcSlots % G == 0 && (G == 2 || G == 4), "a slot belongs to one group");
        static_assert(kTcSlots % kTcMmaWarps == 0 && kTcMmaWarps == 2, "and to one MMA warp");
        const int cw = warp - kTcDecodeWarp0;
        const int qtr = warp & 3, sub4 = cw >> 2;  // (any four warps in a row cover the four quarters)
        const int grp = G == 2 ? sub4 >> 1 : sub4;                  // this warp's group
        const int rg0 = G == 2 ? 2 * qtr + (sub4 & 1) : 2 * qtr;    // its first row group
        const int gl = (G == 2 ? 2 * qtr + (sub4 & 1) : qtr) * 32 + lane;  // this lane's number within the group
        const int t = lane & 3;
        constexpr int EXPB = FMT == TKD_BFP4 ? 64 : (FMT == TKD_BFP8 ? 32 : 0);
        constexpr int UPC = CK / 128;              // units of a whole chunk
        constexpr int MU = (UPC + G - 1) / G;      // ... of them one group's, at most
        constexpr int XT = MU * 2 * PP;            // x pieces a lane holds for a chunk
        const uint2 sh = make_uint2(p.mul16, p.mul128);
        const uint32_t ring_a = smem_u32(ring), hdr_a = smem_u32(hdr);
        // the tensor-memory address of this warp's first 16 lanes (panel columns 16 rg0 .. + 15) at the first A column
        const uint32_t alane = tmem0 + ((uint32_t)(16 * rg0) << 16) + kTcA0;
        uint32_t slot = 0, phase = 0, useq = 0;
        // This lane's pieces of an x tile (PP of the 256: piece = (row, 16 bytes of the row)). A piece's 16 bytes (8 k of
        // one row) go to two places of the row's 128 bytes, 8 bytes each: k 0-3 to the block of 16 k with jj = 0 of its
        // block of 32 k, k 4-7 to the one with jj = 1, both at position 4 t (t = the piece's number within the block of
        // 32 k); then the swizzle (16-byte piece ^ row).
        uint32_t xrow[PP];  // (an element offset into x: x is at most 32 rows)
        uint32_t xdst0[PP], xdst1[PP];
        int xk[PP];         // the piece's first k within its tile (past K for a row past M: such a piece stays zero)
#pragma unroll
        for (int pp = 0; pp < PP; ++pp) {
            const int xe = gl + pp * (512 / G), xr_ = xe >> 3, xc_ = xe & 7;
            xrow[pp] = (uint32_t)(min(xr_, M - 1) * p.ldx + 8 * xc_);
            xk[pp] = xr_ < M ? 8 * xc_ : (1 << 30);
            const uint32_t xo0 = 64 * (xc_ >> 2) + 8 * (xc_ & 3), xo1 = xo0 + 32;
            xdst0[pp] = xr_ * 128 + ((((xo0 >> 4) ^ (xr_ & 7)) << 4) | (xo0 & 15));
            xdst1[pp] = xr_ * 128 + ((((xo1 >> 4) ^ (xr_ & 7)) << 4) | (xo1 & 15));
        }
        // the pieces of the group's units u0, u0 + G, .. of the chunk that starts at k0
        auto load_x = [&](uint4 (&v)[XT], int k0, int u0) {
#pragma unroll
            for (int i = 0; i < MU; ++i)
#pragma unroll
                for (int sub = 0; sub < 2; ++sub)
#pragma unroll
                    for (int pp = 0; pp < PP; ++pp) {
                        const int u = u0 + G * i, k = k0 + 64 * (2 * u + sub);  // the tile's first k
                        v[(2 * i + sub) * PP + pp] =
                            u < UPC && k + xk[pp] < K ? ldg_x(p.x + xrow[pp] + k) : make_uint4(0u, 0u, 0u, 0u);
                    }
        };
        uint4 xcur[XT], xnext[XT];
        {
            const int64_t first_it = lead > 0 ? tail0 : i0;
            load_x(xcur, (int)(first_it - idiv(p, first_it, p.nslices) * p.nslices) * p.ks, grp);
        }
        // One store a tile's share: rows g (registers 4 b, 4 b + 1) and g + 8 (4 b + 2, 4 b + 3) of the warp's 16 lanes,
        // 32-bit columns 2 t and 2 t + 1 of block b of 8 columns (16 k); two or four blocks an instruction.
        auto st_a2 = [&](uint32_t taddr, const uint32_t (&r)[8]) {
            asm volatile("tcgen05.st.sync.aligned.16x256b.x2.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
                         "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                         : "memory");
        };
        auto st_a4 = [&](uint32_t taddr, const uint32_t (&r)[16]) {
            asm volatile(
                "tcgen05.st.sync.aligned.16x256b.x4.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, "
                "%15, %16};" ::"r"(taddr),
                "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
                "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
                : "memory");
        };
        // super-atom `sab` (a shared-memory address) of one row group, decoded and stored at tensor-memory column tb:
        // 16 columns of A (32 k; bfloat4_b: 32 columns, 64 k)
        auto decode_sa = [&](uint32_t sab, uint32_t tb) {
            if constexpr (FMT == TKD_BF16) {
                const uint4 a = lds128(sab + lane * 16), b = lds128(sab + 512 + lane * 16);
                const uint32_t r[8] = {a.x, a.z, a.y, a.w, b.x, b.z, b.y, b.w};
                st_a2(tb, r);
            } else {
                uint32_t cwd[4], ewd[4];
                if constexpr (FMT == TKD_BFP8) {
                    const uint2 ev = lds64(sab + t * 8);
                    const uint4 cv = lds128(sab + EXPB + lane * 16);
                    cwd[0] = cv.x, cwd[1] = cv.y, cwd[2] = cv.z, cwd[3] = cv.w;
                    ewd[0] = ev.x, ewd[1] = ev.y, ewd[2] = ewd[3] = 0;
                } else {
                    const uint4 ev = lds128(sab + t * 16), cv = lds128(sab + EXPB + lane * 16);
                    cwd[0] = cv.x, cwd[1] = cv.y, cwd[2] = cv.z, cwd[3] = cv.w;
                    ewd[0] = ev.x, ewd[1] = ev.y, ewd[2] = ev.z, ewd[3] = ev.w;
                }
                uint32_t r[8 * F::XB];
#pragma unroll
                for (int q = 0; q < F::XB; ++q) {
#pragma unroll
                    for (int jj = 0; jj < 2; ++jj) {
                        uint32_t a0, a1, a2, a3, s0, s1;
                        if constexpr (FMT == TKD_BFP4) {
                            const uint32_t w = cwd[2 * q + jj], tt = __funnelshift_r(w, w, 8), ew = ewd[2 * q + jj];
                            a0 = w & TKD_MASK_BFP4, a1 = shl_fma<4>(w, sh.x) & TKD_MASK_BFP4;
                            a2 = tt & TKD_MASK_BFP4, a3 = shl_fma<4>(tt, sh.x) & TKD_MASK_BFP4;
                            s0 = (ew & TKD_EMASK_BFP4) | TKD_EBASE_BFP4;
                            s1 = (shl_fma<7>(ew, sh.y) & TKD_EMASK_BFP4) | TKD_EBASE_BFP4;
                        } else {
                            const uint32_t w0 = cwd[2 * jj], w1 = cwd[2 * jj + 1], ew = ewd[jj];
                            a0 = w0 & TKD_MASK_BFP8, a1 = rot_and<8>(w0, TKD_MASK_BFP8);
                            a2 = w1 & TKD_MASK_BFP8, a3 = rot_and<8>(w1, TKD_MASK_BFP8);
                            s0 = ew & 0x7F807F80u, s1 = rot_and<8>(ew, 0x7F807F80u);
                        }
                        // (the code times 2^e': the weight itself, in units the output stage knows)
                        const int b = 4 * (2 * q + jj);  // block 2 q + jj of the super-atom: columns 16 q + 8 jj
                        r[b] = mul_bf16x2(a0, s0), r[b + 1] = mul_bf16x2(a2, s1);
                        r[b + 2] = mul_bf16x2(a1, s0), r[b + 3] = mul_bf16x2(a3, s1);
                    }
                }
                if constexpr (FMT == TKD_BFP4)
                    st_a4(tb, r);
                else
                    st_a2(tb, r);
            }
        };
        while (true) {
            if (!mbar_wait(full0 + 8 * slot, phase, p.status)) break;
            const uint4 hd = lds128(hdr_a + 16 * slot);
            const int kc = (int)hd.w;
            const bool at_end = (hd.x & ST_END) != 0;
            const int nsa = KWHOLE ? F::SUBSA : min(F::SUBSA, nsa_total - kc / CK * F::SUBSA);
            const int ntiles = (nsa * F::KSA + 63) / 64;
            const int nunits = (ntiles + 1) >> 1;
            const int u0 = (int)((uint32_t)grp - useq) & (G - 1);  // the group's first unit of this chunk
            load_x(xnext, (int)hd.z, (int)((uint32_t)grp - (useq + nunits)) & (G - 1));  // (used a whole chunk from now)
            const uint32_t gb = ring_a + slot * p.stage_bytes + rg0 * nsa * F::SAB;
            bool ok = true;
            // The group's units of the chunk (unrolled: the x pieces are indexed at compile time): the slot is waited
            // for, both tiles decoded and stored, then one proxy fence and one arrival.
#pragma unroll
            for (int i = 0; i < MU; ++i) {
                const int u = u0 + G * i;
                if (u >= nunits) break;
                const uint32_t us = useq + u, ps = us % kTcSlots;
                ok = mbar_wait(aempty0 + 8 * ps, ((us / kTcSlots) & 1) ^ 1, p.status);
                if (!ok) break;
                const uint32_t sb = ops0 + ps * kTcSlot, ta = alane + ps * 2 * kTcACols;
#pragma unroll
                for (int sub = 0; sub < 2; ++sub) {
                    const int ti = 2 * u + sub;  // the tile of the chunk
                    if (ti >= ntiles) break;
#pragma unroll
                    for (int r = 0; r < RG; ++r) {
                        const uint32_t tr = ta + ((uint32_t)(16 * r) << 16) + sub * kTcACols;
                        const uint32_t gr = gb + r * nsa * F::SAB;
                        if constexpr (FMT == TKD_BFP4) {
                            decode_sa(gr + ti * F::SAB, tr);  // (a super-atom is a whole tile)
                        } else {
                            decode_sa(gr + 2 * ti * F::SAB, tr);
                            if (2 * ti + 1 < nsa) decode_sa(gr + (2 * ti + 1) * F::SAB, tr + 16);
                        }
                    }
#pragma unroll
                    for (int pp = 0; pp < PP; ++pp) {
                        const uint4 v = xcur[(2 * i + sub) * PP + pp];
                        const uint32_t xb = sb + sub * kTcXTile;
                        asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(xb + xdst0[pp]), "r"(v.x), "r"(v.y) : "memory");
                        asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(xb + xdst1[pp]), "r"(v.z), "r"(v.w) : "memory");
                    }
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");  // this warp's tensor-memory stores are done
                tc_fence_before();
                fence_proxy_async();  // this lane's shared-memory stores, for the tensor core's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(afull0 + 8 * ps);
            }
            if (!ok) break;
#pragma unroll
            for (int i = 0; i < XT; ++i) xcur[i] = xnext[i];
            useq += nunits;
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * slot);
            if (++slot == (uint32_t)nst) slot = 0, phase ^= 1;
            if (at_end) break;
        }
    } else if (tc_mma_warp(warp) >= 0) {
        // ---------------------------------------------------------------- the MMA issuers (a warp walks the loop, one
        // lane issues). Issuing a unit's eight MMAs costs a warp ~450 ns beside the decode warps (60 cycles an MMA on an
        // idle SM, about 115 here) and its loop as much again, more than the decode of a unit takes: two warps share the
        // units by their number in the CTA's sequence (even: the first warp; odd: the second), so that a slot's
        // barriers are always the same warp's and it sees every phase of them (a parity wait tells phase n from n + 2
        // only then). The accumulator is chosen by the unit's number within its SLICE (even: d0, odd: d1), so that a
        // slice's sums do not depend on where in the sequence it starts; the two warps are on opposite parities at
        // any time, hence on different accumulators.
        {
            const int mw = tc_mma_warp(warp);
            int slice = 0;    // the item's slice of its panel: all this role needs to know of it
            uint32_t us = 0;  // units before this slice
            bool ok = true;
            // the descriptor of slot 0's first x tile as 32-bit halves (a slot further on is kTcSlot / 16 more in the low
            // half, a tile kTcXTile / 16, a block of 16 k 2 more); the A operand: tensor-memory columns, 8 a block
            const uint64_t bd0 = tc_desc(ops0);
            const uint32_t dhi = (uint32_t)(bd0 >> 32), blo0 = (uint32_t)bd0, alo0 = tmem0 + kTcA0;
            for (int64_t j = 0; j < nitems && ok; ++j) {
                if (j == 0 || j == lead) {
                    const int64_t it = item_at(j);
                    slice = (int)(it - idiv(p, it, p.nslices) * p.nslices);
                } else if (++slice == p.nslices) {
                    slice = 0;
                }
                const int kv = min(p.ks, K - slice * p.ks);
                const int nu = (kv + 127) >> 7;  // units of the slice (a chunk is a whole number of units but for K's end)
                const uint32_t buf = (uint32_t)j & 1;
                // the accumulators must have been read out (the slice two before this one)
                ok = mbar_wait(accempty0 + 8 * buf, (((uint32_t)j >> 1) & 1) ^ 1, p.status);
                if (!ok) break;
                tc_fence_after();
                const uint32_t dbase = tmem0 + kTcAcc0 + buf * 64;
                for (int ui = (int)(((uint32_t)mw - us) & 1u); ui < nu; ui += 2) {
                    const uint32_t g = us + ui, ps = g % kTcSlots;
                    ok = mbar_wait(afull0 + 8 * ps, (g / kTcSlots) & 1, p.status);
                    if (!ok) break;
                    tc_fence_after();  // (the decode warps' tensor-memory stores, completed before they arrived)
                    if (tc_elect()) {
                        const uint32_t d = dbase + (ui & 1) * 32, acc = ui >= 2;
                        uint32_t al = alo0 + ps * 2 * kTcACols, bl = blo0 + ps * (kTcSlot >> 4);
                        // (the unit's blocks of 16 k, eight if it is whole: two tiles of four)
                        const int kleft = kv - 128 * ui;
                        const int nb = kleft >= 128 ? 8 : (kleft + 15) >> 4;
#pragma unroll
                        for (int b = 0; b < 8; ++b) {
                            if (b >= nb) break;
                            if (b == 4) al += kTcACols - 32, bl += (kTcXTile >> 4) - 8;
                            tc_mma(d, al + 8 * b, bl + 2 * b, dhi, b ? 1u : acc);
                        }
                        tc_commit(aempty0 + 8 * ps);
                    }
                    __syncwarp();
                }
                us += nu;
                // (a warp without a unit in this slice commits all the same: the barrier counts both)
                if (ok && lane == 0) tc_commit(accfull0 + 8 * buf);
                __syncwarp();
            }
        }
    } else if (warp >= kTcOutputWarp0) {
        // ---------------------------------------------------------------- output warps
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const int ow = warp & 3;          // the quarter of the tensor memory's lanes this warp may read
        const int et = ow * 32 + lane;    // the panel column (= A row = tensor-memory lane) this thread owns
        Cursor c;
        bool ok = true;
        float* const trow = tbuf + (size_t)et * MP;
        uint16_t* y16 = static_cast<uint16_t*>(p.out);
        for (int64_t j = 0; j < nitems && ok; ++j) {
            const int64_t it = item_at(j);
            if (j == 0 || j == lead)
                cursor_init(c, p, it);
            else
                cursor_next(c, p);
            const Flow f = flow_of(c, p, it, i0, i1);
            const TkdSegDev& sg = p.seg[c.seg];
            const int n = glu2 ? c.pl * 64 + (et & 63) : c.pl * TKD_PANEL_COLS + et;
            const bool in_w = n < sg.n_valid;
            int ebyte = 0;
            float sc = 1.f;
            if (f.deliver) {
                if constexpr (FMT != TKD_BF16) ebyte = (glu2 && et >= 64 ? sg.emax2 : sg.emax)[n >> 4];
                if (p.scale_dt != TKD_DT_NONE && in_w) {
                    const void* sp = glu2 && et >= 64 ? p.scale2 : p.scale;
                    sc = p.scale_dt == TKD_DT_BF16 ? bf16_bits_to_f32(static_cast<const uint16_t*>(sp)[n])
                                                   : static_cast<const float*>(sp)[n];
                }
            }
            if (f.deliver && p.res && topk_k == 0) {
                // the panel's residual on its way to L2 while the slice is still being multiplied: row et & 31, line et >> 5
                // of the row's 128 (GLU: 64) columns
                const int rr = et & 31, ln = et >> 5, rsz_ = p.res_dt == TKD_DT_F32 ? 4 : 2;
                const int ncol = (p.epi == TKD_EPI_GLU_IL || glu2) ? 64 : TKD_PANEL_COLS;
                const int nout_valid = p.epi == TKD_EPI_GLU_IL ? sg.n_valid / 2 : sg.n_valid;  // (only elements that exist)
                if (rr < M && ln * 128 < ncol * rsz_ && c.pl * ncol + ln * (128 / rsz_) < nout_valid) {
                    const char* rp = static_cast<const char*>(p.res) +
                                     ((size_t)rr * p.ldr + sg.out_col0 + (size_t)c.pl * ncol) * rsz_ + ln * 128;
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(rp));
                }
            }
            const uint32_t buf = (uint32_t)j & 1;
            ok = mbar_wait(accfull0 + 8 * buf, ((uint32_t)j >> 1) & 1, p.status);
            if (!ok) break;
            tc_fence_after();
            {
                // the slice's sum d0 + d1 (d1 only if the slice has a second unit), sixteen rows at a time: both
                // accumulators' loads are in flight together, and rows past M are not read at all
                const int kv = min(p.ks, K - c.slice * p.ks);
                const bool two = kv > 128;
                const uint32_t ta = tmem0 + ((uint32_t)(ow * 32) << 16) + kTcAcc0 + buf * 64;
                auto ld16 = [&](uint32_t addr, uint32_t (&r)[16]) {
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                        : "r"(addr)
                        : "memory");
                };
#pragma unroll 1
                for (int hf = 0; hf < (M > 16 ? 2 : 1); ++hf) {
                    uint32_t r0[16], r1[16];
                    ld16(ta + 16 * hf, r0);
                    if (two)
                        ld16(ta + 32 + 16 * hf, r1);
                    else {
#pragma unroll
                        for (int m = 0; m < 16; ++m) r1[m] = 0u;
                    }
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    // the running sums of this thread's column: they start over with the slice, or the slice is added
#pragma unroll
                    for (int m = 0; m < 16; m += 4) {
                        float4 q;
                        q.x = two ? __uint_as_float(r0[m]) + __uint_as_float(r1[m]) : __uint_as_float(r0[m]);
                        q.y = two ? __uint_as_float(r0[m + 1]) + __uint_as_float(r1[m + 1]) : __uint_as_float(r0[m + 1]);
                        q.z = two ? __uint_as_float(r0[m + 2]) + __uint_as_float(r1[m + 2]) : __uint_as_float(r0[m + 2]);
                        q.w = two ? __uint_as_float(r0[m + 3]) + __uint_as_float(r1[m + 3]) : __uint_as_float(r0[m + 3]);
                        if (!f.start) {
                            const float4 o = *reinterpret_cast<const float4*>(trow + 16 * hf + m);
                            q = make_float4(o.x + q.x, o.y + q.y, o.z + q.z, o.w + q.w);
                        }
                        *reinterpret_cast<float4*>(trow + 16 * hf + m) = q;
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(accempty0 + 8 * buf);
            }
            if (f.store) {
                // the running sums into the scratch slot of (panel, slice): [row][128 columns] (the first half of a slot
                // as tkd_stream_kernel lays it out; there is no second half here)
                float* scr = p.scratch + (size_t)(c.panel * p.nslices + c.slice) * 2 * M * TKD_PANEL_COLS + et;
#pragma unroll 1
                for (int m = 0; m < M; ++m) __stcg(scr + (size_t)m * TKD_PANEL_COLS, trow[m]);
            }
            if (!f.deliver) continue;
            bool finish = !f.split;
            if (f.split) {
                // count this CTA's slices of the panel in; if they were the last the panel waited for, add all of its
                // slices up (bar.sync orders the 128 threads' scratch stores before thread 0's release)
                bar_output_warps();
                if (et == 0) {
                    const int old = atom_add_acq_rel(p.counters + c.panel, f.count);
                    const int last = old + f.count == p.nslices;
                    if (last) p.counters[c.panel] = 0;
                    sflag[0] = last;
                }
                bar_output_warps();
                finish = sflag[0] != 0;
                if (finish) {
                    const int64_t pfirst = (int64_t)c.panel * p.nslices;
                    const int64_t owner = idiv(p, (pfirst + 1) * gridDim.x - 1, T);
                    const int64_t oend = idiv(p, T * (owner + 1), gridDim.x);
                    const int pe = (int)min((int64_t)p.nslices, oend - pfirst);
                    const float* s0 = p.scratch + pfirst * 2 * M * TKD_PANEL_COLS + et;
                    auto term = [&](int s, int m) { return __ldcg(s0 + ((size_t)(s * 2) * M + m) * TKD_PANEL_COLS); };
                    const int ns = p.nslices - pe + 1;  // sums to add: the owner's, then one per later slice
                    if (j == nitems - 1 && (size_t)ns * M * 512 <= (size_t)nst * p.stage_bytes) {
                        // The CTA's last item: the ring is idle, and the sums (M x 512 bytes a slice, contiguous) are copied
                        // into it 16 bytes at a time, all copies in flight together (one trip to L2 instead of one per 32
                        // loads a thread), then added up in slice order from shared memory.
                        const uint32_t ring_a = smem_u32(ring);
                        const int per = M * 32;  // 16-byte pieces of a slice's sums
                        for (int si = 0; si < ns; ++si) {
                            const float* src = p.scratch + ((pfirst + pe - 1 + si) * 2 * M) * TKD_PANEL_COLS;
                            const uint32_t dst = ring_a + si * per * 16;
                            for (int q = et; q < per; q += 128)
                                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + q * 16), "l"(src + q * 4)
                                             : "memory");
                        }
                        asm volatile("cp.async.wait_all;" ::: "memory");
                        bar_output_warps();
                        const float* rs = reinterpret_cast<const float*>(ring) + et;
#pragma unroll 1
                        for (int rb = 0; rb < M; rb += 8) {  // (eight rows' loads at a time; a row past M re-reads the last)
                            float th[8];
#pragma unroll
                            for (int m = 0; m < 8; ++m) th[m] = rs[(size_t)min(rb + m, M - 1) * TKD_PANEL_COLS];
#pragma unroll 1
                            for (int si = 1; si < ns; ++si) {
                                float v[8];
#pragma unroll
                                for (int m = 0; m < 8; ++m) v[m] = rs[((size_t)si * M + min(rb + m, M - 1)) * TKD_PANEL_COLS];
#pragma unroll
                                for (int m = 0; m < 8; ++m) th[m] += v[m];
                            }
                            *reinterpret_cast<float4*>(trow + rb) = make_float4(th[0], th[1], th[2], th[3]);
                            *reinterpret_cast<float4*>(trow + rb + 4) = make_float4(th[4], th[5], th[6], th[7]);
                        }
                    } else
#pragma unroll 1
                    for (int rb = 0; rb < M; rb += 8) {
                        float th[8];
#pragma unroll 1
                        for (int s = pe - 1; s < p.nslices; s += 4) {
                            float v[4][8];
#pragma unroll
                            for (int q = 0; q < 4; ++q)
#pragma unroll
                                for (int m = 0; m < 8; ++m) v[q][m] = term(min(s + q, p.nslices - 1), min(rb + m, M - 1));
#pragma unroll
                            for (int q = 0; q < 4; ++q)
#pragma unroll
                                for (int m = 0; m < 8; ++m) {
                                    if (s + q >= p.nslices) continue;
                                    th[m] = s + q == pe - 1 ? v[q][m] : th[m] + v[q][m];
                                }
                        }
                        *reinterpret_cast<float4*>(trow + rb) = make_float4(th[0], th[1], th[2], th[3]);
                        *reinterpret_cast<float4*>(trow + rb + 4) = make_float4(th[4], th[5], th[6], th[7]);
                    }
                }
                bar_output_warps();  // sflag may be written again only after everyone has read it
            }
            if (!finish) continue;

            // ------------------------------------------------------------ the output stage of one panel, from the sums
            // in tbuf, eight rows at a time in a rolled loop (the same stage as tkd_stream_kernel's for 9 rows and more)
            {
                float colf = 1.f, colg = 1.f;
                if constexpr (FMT != TKD_BF16) {
                    const int e = tkd_out_exp(FMT, ebyte);
                    const int e1 = e / 2, e2 = e - e1;
                    colf = __uint_as_float((uint32_t)(e1 + 127) << 23), colg = __uint_as_float((uint32_t)(e2 + 127) << 23);
                }
                const float cols = p.scale_dt != TKD_DT_NONE && in_w ? sc : 1.f;
                const bool glu = p.epi == TKD_EPI_GLU_IL || glu2;
                if (topk_k == 0) {
                    // No records: the panel leaves through a transposition in shared memory. Every thread scales its own
                    // column in place; then a lane is a ROW and a warp takes every fourth group of 8 output columns:
                    // 8 sums of the row (consecutive lanes, consecutive words: no bank conflict), the epilogue, one
                    // 16-byte store (two for fp32 output). A fifth of the instructions of a store per element, and the
                    // peers get 16-byte stores too.
                    const int mr = M > 16 ? 32 : 16;
#pragma unroll 1
                    for (int m = 0; m < mr; m += 4) {
                        float4 v = *reinterpret_cast<float4*>(trow + m);
                        v.x = v.x * colf * colg * cols, v.y = v.y * colf * colg * cols;
                        v.z = v.z * colf * colg * cols, v.w = v.w * colf * colg * cols;
                        *reinterpret_cast<float4*>(trow + m) = v;
                    }
                    bar_output_warps();
                    const int nout = glu ? 64 : TKD_PANEL_COLS;        // output columns of the panel
                    const int oc0 = sg.out_col0 + c.pl * nout;         // the first of them
                    // how many of them exist (GLU, interleaved: output o needs column 64 (o >> 5) + (o & 31) + 32)
                    int nv;
                    if (!glu || glu2)
                        nv = min(nout, sg.n_valid - c.pl * nout);
                    else {
                        const int left = sg.n_valid - c.pl * TKD_PANEL_COLS;  // columns of this panel that exist (a multiple of 64)
                        nv = left >= 128 ? 64 : (left >= 64 ? 32 : 0);
                    }
                    const bool f32out = p.epi == TKD_EPI_OUT32;
                    const int esz = f32out ? 4 : 2;
                    const bool vec = ((reinterpret_cast<uintptr_t>(p.out) | (uintptr_t)(p.ldo * esz) | (uintptr_t)(oc0 * esz)) & 15) == 0;
                    const int r = lane;
                    // the residual of this lane's groups, asked for with 16-byte loads two groups ahead (four round trips to
                    // L2 one after the other were most of this stage)
                    const bool res32 = f32out && p.res_dt == TKD_DT_F32, res16 = p.epi == TKD_EPI_RESIDUAL;
                    const int rsz = res32 ? 4 : 2;
                    const bool rvec = vec && (res32 || res16) &&
                                      ((reinterpret_cast<uintptr_t>(p.res) | (uintptr_t)(p.ldr * rsz) | (uintptr_t)(oc0 * rsz)) & 15) == 0;
                    // one group of 8 output columns of this lane's row (have: its residual came in q0, q1)
                    auto group = [&](int cc, bool have, uint4 q0, uint4 q1) {
                            float v[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const int o = 8 * cc + i;
                                if (glu) {
                                    const int gc = glu2 ? o : 64 * (o >> 5) + (o & 31), uc = glu2 ? o + 64 : gc + 32;
                                    v[i] = act_gate(tbuf[(size_t)gc * MP + r], p.act) * tbuf[(size_t)uc * MP + r];
                                } else {
                                    v[i] = tbuf[(size_t)o * MP + r];
                                }
                            }
                            const int here = min(8, nv - 8 * cc);  // columns of this group that exist
                            const size_t at = (size_t)r * p.ldo + oc0 + 8 * cc;
                            if (have && here == 8) {
                                if (res32) {
                                    v[0] += __uint_as_float(q0.x), v[1] += __uint_as_float(q0.y);
                                    v[2] += __uint_as_float(q0.z), v[3] += __uint_as_float(q0.w);
                                    v[4] += __uint_as_float(q1.x), v[5] += __uint_as_float(q1.y);
                                    v[6] += __uint_as_float(q1.z), v[7] += __uint_as_float(q1.w);
                                } else {
                                    v[0] += __uint_as_float(q0.x << 16), v[1] += __uint_as_float(q0.x & 0xFFFF0000u);
                                    v[2] += __uint_as_float(q0.y << 16), v[3] += __uint_as_float(q0.y & 0xFFFF0000u);
                                    v[4] += __uint_as_float(q0.z << 16), v[5] += __uint_as_float(q0.z & 0xFFFF0000u);
                                    v[6] += __uint_as_float(q0.w << 16), v[7] += __uint_as_float(q0.w & 0xFFFF0000u);
                                }
                            } else if (res32) {
                                const float* rp = static_cast<const float*>(p.res) + (size_t)r * p.ldr + oc0 + 8 * cc;
#pragma unroll
                                for (int i = 0; i < 8; ++i)
                                    if (i < here) v[i] += rp[i];
                            } else if (res16) {
                                const uint16_t* rp = static_cast<const uint16_t*>(p.res) + (size_t)r * p.ldr + oc0 + 8 * cc;
#pragma unroll
                                for (int i = 0; i < 8; ++i)
                                    if (i < here) v[i] += bf16_bits_to_f32(rp[i]);
                            }
                            if (f32out) {
                                if (vec && here == 8) {
                                    const float4 lo = make_float4(v[0], v[1], v[2], v[3]), hi = make_float4(v[4], v[5], v[6], v[7]);
                                    float4* op = reinterpret_cast<float4*>(static_cast<float*>(p.out) + at);
                                    op[0] = lo, op[1] = hi;
                                    for (int q = 0; q < npeers; ++q)
                                        if (p.peer_out[q]) {
                                            float4* pp = reinterpret_cast<float4*>(static_cast<float*>(p.peer_out[q]) + at);
                                            pp[0] = lo, pp[1] = hi;
                                        }
                                } else {
#pragma unroll
                                    for (int i = 0; i < 8; ++i) {
                                        if (i >= here) break;
                                        static_cast<float*>(p.out)[at + i] = v[i];
                                        for (int q = 0; q < npeers; ++q)
                                            if (p.peer_out[q]) static_cast<float*>(p.peer_out[q])[at + i] = v[i];
                                    }
                                }
                            } else {
                                uint16_t b[8];
#pragma unroll
                                for (int i = 0; i < 8; ++i) b[i] = f32_to_bf16_bits(v[i]);
                                if (vec && here == 8) {
                                    const uint4 w = make_uint4(b[0] | ((uint32_t)b[1] << 16), b[2] | ((uint32_t)b[3] << 16),
                                                               b[4] | ((uint32_t)b[5] << 16), b[6] | ((uint32_t)b[7] << 16));
                                    *reinterpret_cast<uint4*>(y16 + at) = w;
                                    for (int q = 0; q < npeers; ++q)
                                        if (p.peer_out[q]) *reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.peer_out[q]) + at) = w;
                                } else {
#pragma unroll
                                    for (int i = 0; i < 8; ++i) {
                                        if (i >= here) break;
                                        y16[at + i] = b[i];
                                        for (int q = 0; q < npeers; ++q)
                                            if (p.peer_out[q]) static_cast<uint16_t*>(p.peer_out[q])[at + i] = b[i];
                                    }
                                }
                            }
                    };
                    if (r < M && !(res32 || res16)) {
#pragma unroll 1
                        for (int cc = ow; 8 * cc < nv; cc += 4) group(cc, false, make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u));
                    } else if (r < M) {
#pragma unroll 1
                        for (int half = 0; half < 2; ++half) {  // (two of a warp's four groups at a time)
                            uint4 rq[2][2];
#pragma unroll
                            for (int i = 0; i < 2; ++i) {
                                const int cc = ow + 4 * (2 * half + i);
                                rq[i][0] = rq[i][1] = make_uint4(0u, 0u, 0u, 0u);
                                if (rvec && 8 * cc + 8 <= nv) {
                                    const size_t ra = (size_t)r * p.ldr + oc0 + 8 * cc;
                                    if (res32) {
                                        const uint4* rp = reinterpret_cast<const uint4*>(static_cast<const float*>(p.res) + ra);
                                        rq[i][0] = rp[0], rq[i][1] = rp[1];
                                    } else {
                                        rq[i][0] = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.res) + ra);
                                    }
                                }
                            }
#pragma unroll
                            for (int gi = 0; gi < 2; ++gi) {
                                const int cc = ow + 4 * (2 * half + gi);
                                if (8 * cc < nv) group(cc, rvec, rq[gi][0], rq[gi][1]);
                            }
                        }
                    }
                    bar_output_warps();  // tbuf is free again
                    continue;
                }
                // With records: a store per element, eight rows at a time in a rolled loop (the same stage as
                // tkd_stream_kernel's for 9 rows and more).
                int ocol = -1;
                const float *gp = trow, *up = trow;
                if (glu) {
#pragma unroll 1
                    for (int m = 0; m < (M > 16 ? 32 : 16); m += 4) {
                        float4 v = *reinterpret_cast<float4*>(trow + m);
                        v.x = v.x * colf * colg * cols, v.y = v.y * colf * colg * cols;
                        v.z = v.z * colf * colg * cols, v.w = v.w * colf * colg * cols;
                        *reinterpret_cast<float4*>(trow + m) = v;
                    }
                    bar_output_warps();
                    if (et < 64) {
                        const int gc = glu2 ? et : 64 * (et >> 5) + (et & 31), uc = glu2 ? et + 64 : gc + 32;
                        const int nw = glu2 ? n : c.pl * TKD_PANEL_COLS + uc;
                        if (nw < sg.n_valid) ocol = sg.out_col0 + c.pl * 64 + et;
                        gp = tbuf + (size_t)gc * MP, up = tbuf + (size_t)uc * MP;
                    }
                } else if (in_w) {
                    ocol = sg.out_col0 + n;
                }
                const bool store = ocol >= 0 && (topk_k == 0 || p.write_y);
                if (ocol >= 0) {
#pragma unroll 1
                    for (int r0 = 0; r0 < M; r0 += 8) {
                        float v[8];
#pragma unroll
                        for (int m = 0; m < 8; ++m)
                            v[m] = glu ? act_gate(gp[r0 + m], p.act) * up[r0 + m] : trow[r0 + m] * colf * colg * cols;
                        if (p.epi == TKD_EPI_OUT32 && p.res_dt == TKD_DT_F32) {
#pragma unroll
                            for (int m = 0; m < 8; ++m)
                                if (r0 + m < M) v[m] += static_cast<const float*>(p.res)[(size_t)(r0 + m) * p.ldr + ocol];
                        } else if (p.epi == TKD_EPI_RESIDUAL) {
#pragma unroll
                            for (int m = 0; m < 8; ++m)
                                if (r0 + m < M)
                                    v[m] += bf16_bits_to_f32(static_cast<const uint16_t*>(p.res)[(size_t)(r0 + m) * p.ldr + ocol]);
                        }
#pragma unroll
                        for (int m = 0; m < 8; ++m) {
                            if (r0 + m >= M) break;
                            const size_t at = (size_t)(r0 + m) * p.ldo + ocol;
                            if (p.epi == TKD_EPI_OUT32) {
                                static_cast<float*>(p.out)[at] = v[m];
                                for (int q = 0; q < npeers; ++q)
                                    if (p.peer_out[q]) static_cast<float*>(p.peer_out[q])[at] = v[m];
                            } else {
                                const uint16_t b = f32_to_bf16_bits(v[m]);
                                if (store) {
                                    y16[at] = b;
                                    for (int q = 0; q < npeers; ++q)
                                        if (p.peer_out[q]) static_cast<uint16_t*>(p.peer_out[q])[at] = b;
                                }
                                if (topk_k && !p.write_y && r0 + m < p.topk_rows) p.ytmp[(size_t)(r0 + m) * p.ld_ytmp + n] = b;
                            }
                        }
                    }
                }
                if (glu) bar_output_warps();  // tbuf is free again
            }
            if (topk_k == 0) continue;
            topk_records(p, c, sg, et, ow, lane, tbuf, sflag, y16, topk_k, npeers);
        }
        if (npeers) exchange_done(p, lane, npeers, sflag);
    }
    // ---- the end: everyone is here (a role whose wait gave up falls through to this point too), and the tensor memory
    // goes back
    tc_fence_before();
    __syncthreads();
    if (warp == kTcMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem0), "r"(512u) : "memory");
    }
}

template <int FMT, bool KWHOLE>
int launch_tc(const TkdParams& p, int grid, size_t smem, cudaStream_t st) {
    auto kern = tkd_stream_tc_kernel<FMT, KWHOLE>;
    static bool allowed[64] = {false};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64 || !allowed[dev]) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return (int)e;
        if (dev >= 0 && dev < 64) allowed[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kTcWarps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = p.no_pdl ? 0 : 1;
    return (int)cudaLaunchKernelEx(&cfg, kern, p);
}

template <int FMT>
int launch_fmt_all(const TkdParams& p, int grid, size_t smem, cudaStream_t st) {
    if (p.tc) {
        return p.K % (Fmt<FMT>::SUBSA * Fmt<FMT>::KSA) == 0 ? launch_tc<FMT, true>(p, grid, smem, st)
                                                           : launch_tc<FMT, false>(p, grid, smem, st);
    }
    return launch_fmt<FMT>(p, grid, smem, st);
}

}  // namespace
