// tkd_layout.h: the packed HBM stream of a dense_reader weight, as index arithmetic usable on host and device.
//
// The reference keeps a [K, N] block-float weight as 32 x 32 tiles (64 exponent bytes, then the mantissas; one shared
// exponent per 16 consecutive n at one k; dense_reader/linear.py:49-50, moe/moe8.py:125-154). Here the same numbers
// (sign, magnitude, shared exponent) are laid out for a CTA that streams 128 output columns (a panel: 8 groups of 16)
// through shared memory, one bulk copy per stage, and multiplies each group by mma.sync m16n8k16 with the weights as
// the A operand:
//
//   stream   = panels of 128 columns back to back (N is padded to 128 with zero columns)
//   panel    = chunks of CK k (256 for bfloat8_b, 512 for bfloat4_b, 128 for bfloat16), K ascending; a chunk is what
//              one stage of the ring holds
//   chunk    = its 8 groups back to back, each the chunk's super-atoms, K ascending
//   super-atom (bfloat8_b, 32 k, 544 B)  = 32 B exponent words, then 32 lanes x 16 B of codes
//   super-atom (bfloat4_b, 64 k, 576 B)  = 64 B exponent words, then 32 lanes x 16 B of codes
//   super-atom (bfloat16, 32 k, 1024 B)  = 2 x (32 lanes x 16 B) of A-fragment registers
//
// so bytes per weight stay 1.0625, 0.5625 and 2. Every super-atom size is a multiple of 16 B, and a chunk (or the
// half of it that holds 4 groups) is one contiguous, 16-byte aligned source of a 1-D bulk copy.
//
// Inside a k32 block, lane (g = lane / 4, t = lane % 4) of mma jj (0, 1) owns k = 8 t + 4 jj + r, r = 0..3: the 8
// activations a lane needs for the two mmas are 16 consecutive bytes of a row of x. Fragment registers: a0 = column
// g, r 0-1; a1 = column g + 8, r 0-1; a2 = column g, r 2-3; a3 = column g + 8, r 2-3 (r even in the low half).
//
// A code is kept as a bf16 bit pattern with a zero exponent field: bits 0-7 of a bf16 are linear (the subnormals and
// the first binade: value = bits * 2^-133), so sign << 15 | magnitude << p is +-magnitude * 2^(p - 133). Several
// fragment registers share one 32-bit word, and the shifts that take a word apart are chosen so that as few as
// possible run on the integer pipe, which bounds the bfloat4_b decode (a left shift is a multiply, which the
// FMA pipe takes):
//   bfloat8_b (p = 0, mask 0x807F807F): word = a_even | rotl(a_odd, 8)
//             a_even = w & mask, a_odd = rotr(w, 8) & mask
//   bfloat4_b (p = 4, mask 0x80708070): word = a0 | a1 >> 4 | rotl(a2, 8) | rotl(a3 >> 4, 8)
//             a0 = w & mask, a1 = (w << 4) & mask, t = rotr(w, 8), a2 = t & mask, a3 = (t << 4) & mask
// The exponents are kept biased against the group's largest (emax, one byte per group, a side array), four to a word:
//   bfloat8_b: e' = e - emax + 196 (1 for a row of the group with no non-zero code) as bf16 exponent fields, r 0 at
//             bits 7-14, r 1 at 23-30, r 2 and r 3 the same rotated left by 8; the activation is scaled by 2^(e' - 127)
//   bfloat4_b: f = e - emax + 63 (0 for a row with no non-zero code) in 6 bits, r 0 at bits 7-12, r 1 at 23-28, r 2 at
//             0-5, r 3 at 16-21: (w & 0x1F801F80) | 0x40004000 is the pair of bf16 scales 2^(f + 1) of r 0 and r 1, the
//             same of w << 7 those of r 2 and r 3
// e is recovered exactly for every non-zero code.
//
// TKD_INT4 (the reference's int4 weight with group scales, int4/w4a16.py: symmetric codes q in -7..7, sign-magnitude,
// one bf16 scale per output column and 32 consecutive k, the weight being q * s) shares bfloat4_b's geometry and code
// words: a 3-bit magnitude and a sign are exactly a bfloat4_b code. Where bfloat4_b keeps 64 bytes of exponents, a
// super-atom (64 k x 16 columns) keeps its 32 scales: word 2 g + q (g = 0..7, q = the k32 block) holds the scales of
// columns g (low half) and g + 8 (high half), each as the bf16 of s * 2^65. The kernel multiplies a k32 block of codes
// (bf16 subnormals q * 2^-129) by the activations times 2^64 into a fresh accumulator and adds that, times the stored
// scale, to the running sum: acc += (2^-65 * sum x q) * (s * 2^65).
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define TKD_HD __host__ __device__ __forceinline__
#else
#define TKD_HD inline
#endif

enum { TKD_BFP8 = 0, TKD_BFP4 = 1, TKD_BF16 = 2, TKD_INT4 = 3 };

// Bumped with every change of the stream's bit layout (a packed-weight cache made by another layout is refused).
#define TKD_LAYOUT_VERSION 3

// The exponent bias of the stream: e' = e - emax + bias. A non-zero code whose exponent lies more than TKD_ESPREAD
// below its group's largest marks the weight "wide" (the product of a code and the scaled activation would leave
// fp32's normal range; bfloat4_b's 6-bit field would not hold it either).
#define TKD_ESPREAD 48
TKD_HD int tkd_ebias(int fmt) { return fmt == TKD_BFP4 ? 63 : 196; }
TKD_HD int tkd_emin_ok(int fmt) { return tkd_ebias(fmt) - TKD_ESPREAD; }
// what a row of a group with no non-zero code stores
TKD_HD int tkd_ezero(int fmt) { return fmt == TKD_BFP4 ? 0 : 1; }
// The column sums come out of the kernel in units of 2^tkd_out_exp(fmt, emax of the group):
//   bfloat8_b: code m * 2^-133 times x * 2^(e' - 127) = m x 2^(e - emax - 64) for the true m x 2^(e - 133)
//   bfloat4_b: code m * 2^-129 times x * 2^(f + 1)    = m x 2^(e - emax - 65) for the true m x 2^(e - 129)
TKD_HD int tkd_out_exp(int fmt, int emax) { return fmt == TKD_BFP4 ? emax - 64 : emax + 64 - 133; }

#define TKD_INT4_SCALE_EXP 65
// (the block-float geometry of a format: TKD_INT4 is laid out as bfloat4_b)
TKD_HD int tkd_geo(int fmt) { return fmt == TKD_INT4 ? TKD_BFP4 : fmt; }
TKD_HD int tkd_mant_bits(int fmt) { return fmt == TKD_BFP8 ? 7 : 3; }
TKD_HD int tkd_ksa(int fmt) { return tkd_geo(fmt) == TKD_BFP4 ? 64 : 32; }                          // k per super-atom
TKD_HD int tkd_sab(int fmt) { return fmt == TKD_BFP8 ? 544 : (tkd_geo(fmt) == TKD_BFP4 ? 576 : 1024); }  // bytes per super-atom
TKD_HD int tkd_exp_bytes(int fmt) { return fmt == TKD_BFP8 ? 32 : (tkd_geo(fmt) == TKD_BFP4 ? 64 : 0); }
TKD_HD int tkd_unit_exp(int fmt) { return 126 + tkd_mant_bits(fmt); }  // value = m * 2^(e - unit)
TKD_HD int tkd_chunk_k(int fmt) { return fmt == TKD_BF16 ? 128 : (tkd_geo(fmt) == TKD_BFP4 ? 512 : 256); }  // k per chunk (stage)
TKD_HD int tkd_subsa(int fmt) { return tkd_chunk_k(fmt) / tkd_ksa(fmt); }                  // super-atoms per group and chunk
TKD_HD int64_t tkd_nsa(int fmt, int64_t K) { return (K + tkd_ksa(fmt) - 1) / tkd_ksa(fmt); }
TKD_HD int64_t tkd_run_bytes(int fmt, int64_t K) { return tkd_nsa(fmt, K) * tkd_sab(fmt); }  // one group, all of K
TKD_HD int64_t tkd_panel_bytes(int fmt, int64_t K) { return 8 * tkd_run_bytes(fmt, K); }
TKD_HD int64_t tkd_stream_bytes(int fmt, int64_t K, int64_t npad) { return (npad / 128) * tkd_panel_bytes(fmt, K); }
// super-atoms of chunk c (the last chunk of a panel may be short)
TKD_HD int tkd_chunk_nsa(int fmt, int64_t K, int64_t c) {
    const int64_t left = tkd_nsa(fmt, K) - c * tkd_subsa(fmt);
    return (int)(left < tkd_subsa(fmt) ? left : tkd_subsa(fmt));
}
// byte offset of super-atom `sa` (counted over all of K) of group `group` (counted over the whole weight)
TKD_HD int64_t tkd_sa_offset(int fmt, int64_t K, int64_t group, int64_t sa) {
    const int sub = tkd_subsa(fmt), sab = tkd_sab(fmt);
    const int64_t c = sa / sub;
    return (group >> 3) * tkd_panel_bytes(fmt, K) + c * sub * sab * 8 +
           ((group & 7) * tkd_chunk_nsa(fmt, K, c) + sa % sub) * (int64_t)sab;
}
// ... and back: which (group, sa, byte inside the super-atom) owns byte `off` of the stream
TKD_HD void tkd_sa_owner(int fmt, int64_t K, int64_t off, int64_t* group, int64_t* sa, int* inner) {
    const int sub = tkd_subsa(fmt), sab = tkd_sab(fmt);
    const int64_t pb = tkd_panel_bytes(fmt, K);
    const int64_t panel = off / pb, r = off % pb;
    const int64_t c = r / ((int64_t)sub * sab * 8), r2 = r % ((int64_t)sub * sab * 8);
    const int n = tkd_chunk_nsa(fmt, K, c);
    *group = panel * 8 + r2 / ((int64_t)n * sab);
    *sa = c * sub + (r2 % ((int64_t)n * sab)) / sab;
    *inner = (int)(r2 % sab);
}

TKD_HD uint32_t tkd_rotl(uint32_t v, int s) { return s ? (v << s) | (v >> (32 - s)) : v; }
TKD_HD uint32_t tkd_rotr(uint32_t v, int s) { return s ? (v >> s) | (v << (32 - s)) : v; }

// Where element (k, n) of a weight lives.
struct TkdLoc {
    int64_t code_word;  // byte offset of the 32-bit word holding the code (bf16: of the 16-bit value itself)
    int rot;            // bfloat8_b: the register is rotr(word, rot) & mask; bfloat4_b: which register a0..a3 (see above)
    int half;           // 0: low 16 bits of the register, 1: high
    int64_t exp_word;   // byte offset of the exponent word
    int exp_r;          // 0..3: the exponent's position in that word
};

TKD_HD TkdLoc tkd_locate(int fmt, int64_t K, int64_t k, int64_t n) {
    TkdLoc L;
    const int64_t group = n >> 4;
    const int i = (int)(n & 15);
    const int ksa = tkd_ksa(fmt);
    const int64_t sa = k / ksa;
    const int kk = (int)(k % ksa);
    const int qq = kk >> 5;       // k32 block of the super-atom (bfloat4_b: 0, 1)
    const int kr = kk & 31;
    const int t = kr >> 3, jj = (kr >> 2) & 1, r = kr & 3;
    const int lane = (i & 7) * 4 + t;
    const int ai = (i >> 3) + 2 * (r >> 1);
    const int64_t base = tkd_sa_offset(fmt, K, group, sa);
    L.half = r & 1;
    L.exp_r = r;
    if (fmt == TKD_BF16) {
        L.code_word = base + jj * 512 + lane * 16 + ai * 4 + L.half * 2;
        L.rot = 0;
        L.exp_word = -1;
    } else if (fmt == TKD_BFP8) {
        L.code_word = base + 32 + lane * 16 + (2 * jj + (ai >> 1)) * 4;
        L.rot = 8 * (ai & 1);
        L.exp_word = base + (t * 2 + jj) * 4;
    } else {
        const int j4 = 2 * qq + jj;
        L.code_word = base + 64 + lane * 16 + j4 * 4;
        L.rot = ai;
        L.exp_word = base + (t * 4 + j4) * 4;
        if (fmt == TKD_INT4) {
            // the scale of (column i, k32 block qq): half (i >> 3) of word 2 (i & 7) + qq
            L.exp_word = base + (2 * (i & 7) + qq) * 4;
            L.exp_r = i >> 3;
        }
    }
    return L;
}

#define TKD_MASK_BFP8 0x807F807Fu
#define TKD_MASK_BFP4 0x80708070u
// The fragment register of a word (rot: TkdLoc's), as the kernel takes it out.
TKD_HD uint32_t tkd_reg_from_word(int fmt, uint32_t word, int rot) {
    if (fmt == TKD_BFP8) return tkd_rotr(word, rot) & TKD_MASK_BFP8;
    const uint32_t t = rot & 2 ? tkd_rotr(word, 8) : word;
    return (rot & 1 ? t << 4 : t) & TKD_MASK_BFP4;
}
// A code (sign << mb | magnitude) as the bits it adds to its word.
TKD_HD uint32_t tkd_code_bits(int fmt, uint32_t code, int rot, int half) {
    const int mb = tkd_mant_bits(fmt);
    const uint32_t s = code >> mb, m = code & ((1u << mb) - 1);
    if (fmt == TKD_BFP8) return tkd_rotl(((s << 15) | m) << (16 * half), rot);
    uint32_t v = ((s << 15) | (m << 4)) << (16 * half);
    if (rot & 1) v >>= 4;
    return rot & 2 ? tkd_rotl(v, 8) : v;
}
// ... and back.
TKD_HD uint32_t tkd_code_from_word(int fmt, uint32_t word, int rot, int half) {
    const int mb = tkd_mant_bits(fmt);
    const uint32_t v = (tkd_reg_from_word(fmt, word, rot) >> (16 * half)) & 0xFFFFu;
    return ((v >> 15) << mb) | ((fmt == TKD_BFP8 ? v : v >> 4) & ((1u << mb) - 1));
}
// A biased exponent as the bits it adds to its exponent word.
#define TKD_EMASK_BFP4 0x1F801F80u
#define TKD_EBASE_BFP4 0x40004000u
TKD_HD uint32_t tkd_exp_bits(int fmt, uint32_t e, int r) {
    if (fmt == TKD_BFP8) return tkd_rotl((e << 7) << (16 * (r & 1)), 8 * (r >> 1));
    return (r & 2 ? e : e << 7) << (16 * (r & 1));
}
TKD_HD uint32_t tkd_exp_from_word(int fmt, uint32_t word, int r) {
    if (fmt == TKD_BFP8) return ((tkd_rotr(word, 8 * (r >> 1)) >> (16 * (r & 1))) >> 7) & 0xFFu;
    return (((r & 2 ? word << 7 : word) >> (16 * (r & 1))) >> 7) & 0x3Fu;
}
// The pair of bf16 scales (r 0 and r 1 for pair 0, r 2 and r 3 for pair 1) the kernel multiplies the activations by.
TKD_HD uint32_t tkd_scales_from_word(int fmt, uint32_t word, int pair) {
    if (fmt == TKD_BFP8) return (pair ? tkd_rotr(word, 8) : word) & 0x7F807F80u;
    return ((pair ? word << 7 : word) & TKD_EMASK_BFP4) | TKD_EBASE_BFP4;
}
