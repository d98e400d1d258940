// layout_emul.cpp: a host-side walk through the packed stream exactly as a streaming warp reads it (tkd_layout.h and
// the register decode of tkd_stream.cu), for tests that run without a GPU. Test code only: it is built by
// tests/test_layout_cpu.py with g++ and never linked into the product library.
#include <math.h>
#include <stdint.h>
#include <string.h>

#include <vector>

#include "../tensix-kernels_b200/csrc/tkd_layout.h"

static float bf16f(uint16_t b) { uint32_t u = (uint32_t)b << 16; float f; memcpy(&f, &u, 4); return f; }

extern "C" {

// canonical exps [K][G], codes [K][npad] (uint8, or uint16 bf16 bits) -> stream + emax, by tkd_locate (scatter form)
void emul_pack(int fmt, int64_t K, int64_t npad, const uint8_t* exps, const void* codes_v, uint8_t* emax,
               uint8_t* stream, int* wide) {
    const int64_t G = npad / 16;
    memset(stream, 0, tkd_stream_bytes(fmt, K, npad));
    *wide = 0;
    if (fmt == TKD_BF16) {
        const uint16_t* codes = (const uint16_t*)codes_v;
        for (int64_t k = 0; k < K; ++k)
            for (int64_t n = 0; n < npad; ++n) {
                TkdLoc L = tkd_locate(fmt, K, k, n);
                memcpy(stream + L.code_word, &codes[k * npad + n], 2);
            }
        return;
    }
    const uint8_t* codes = (const uint8_t*)codes_v;
    if (fmt == TKD_INT4) {
        // exps: the bf16 bits of the group scales [ceil(K / 32)][npad]; a scale is stored times 2^TKD_INT4_SCALE_EXP
        const uint16_t* sc = (const uint16_t*)exps;
        for (int64_t kg = 0; kg * 32 < K; ++kg)
            for (int64_t n = 0; n < npad; ++n) {
                TkdLoc L = tkd_locate(fmt, K, kg * 32, n);
                const float v = ldexpf(bf16f(sc[kg * npad + n]), TKD_INT4_SCALE_EXP);
                uint32_t u; memcpy(&u, &v, 4);
                const uint16_t b = (uint16_t)(u >> 16);
                memcpy(stream + L.exp_word + 2 * L.exp_r, &b, 2);
            }
        for (int64_t k = 0; k < K; ++k)
            for (int64_t n = 0; n < npad; ++n) {
                TkdLoc L = tkd_locate(fmt, K, k, n);
                uint32_t w; memcpy(&w, stream + L.code_word, 4);
                w |= tkd_code_bits(fmt, codes[k * npad + n], L.rot, L.half);
                memcpy(stream + L.code_word, &w, 4);
            }
        return;
    }
    std::vector<uint8_t> nz(K * G, 0);
    for (int64_t g = 0; g < G; ++g) {
        int hi = 0, lo = 255;
        for (int64_t k = 0; k < K; ++k) {
            bool any = false;
            for (int i = 0; i < 16; ++i) any |= codes[k * npad + g * 16 + i] != 0;
            nz[k * G + g] = any;
            if (any) { hi = exps[k * G + g] > hi ? exps[k * G + g] : hi; lo = exps[k * G + g] < lo ? exps[k * G + g] : lo; }
        }
        emax[g] = (uint8_t)hi;
        if (lo <= hi && hi - lo > TKD_ESPREAD) *wide = 1;
    }
    // every exponent slot of the stream, padded k included, holds at least the format's "no code" value
    const int64_t kpad = tkd_nsa(fmt, K) * tkd_ksa(fmt);
    for (int64_t k = 0; k < kpad; ++k)
        for (int64_t g = 0; g < G; ++g) {
            TkdLoc L = tkd_locate(fmt, K, k, g * 16);
            int e = tkd_ezero(fmt);
            if (k < K && nz[k * G + g]) {
                e = (int)exps[k * G + g] - (int)emax[g] + tkd_ebias(fmt);
                if (e < tkd_ezero(fmt)) e = tkd_ezero(fmt);
            }
            uint32_t w; memcpy(&w, stream + L.exp_word, 4);
            w |= tkd_exp_bits(fmt, (uint32_t)e, L.exp_r);
            memcpy(stream + L.exp_word, &w, 4);
        }
    for (int64_t k = 0; k < K; ++k)
        for (int64_t n = 0; n < npad; ++n) {
            TkdLoc L = tkd_locate(fmt, K, k, n);
            uint32_t w; memcpy(&w, stream + L.code_word, 4);
            w |= tkd_code_bits(fmt, codes[k * npad + n], L.rot, L.half);
            memcpy(stream + L.code_word, &w, 4);
        }
}

// y [M][npad] = x [M][K] (bf16 bits) times the stream, read lane by lane and mma by mma as the kernel does; products
// and sums in double (the arithmetic under test is the decode, not the rounding of the sums).
void emul_matmul(int fmt, int64_t K, int64_t npad, const uint8_t* stream, const uint8_t* emax, const uint16_t* x,
                 int M, double* y) {
    const int64_t G = npad / 16, nsa = tkd_nsa(fmt, K);
    const int ksa = tkd_ksa(fmt);
    for (int64_t g = 0; g < G; ++g) {
        std::vector<double> acc(16 * M, 0.0);
        for (int64_t sa = 0; sa < nsa; ++sa) {
            const uint8_t* b = stream + tkd_sa_offset(fmt, K, g, sa);
            if (fmt == TKD_INT4) {
                // per k32 block: the codes (bf16 subnormals) times x * 2^64 summed from zero, then the block's stored
                // scale (this lane's word 2 gl + qq: column gl in the low half, gl + 8 in the high) takes the sum over
                for (int lane = 0; lane < 32; ++lane) {
                    const int gl = lane >> 2, t = lane & 3;
                    for (int qq = 0; qq < 2; ++qq) {
                        std::vector<double> tmp(2 * M, 0.0);
                        for (int jj = 0; jj < 2; ++jj) {
                            uint32_t w, a[4];
                            memcpy(&w, b + 64 + lane * 16 + (2 * qq + jj) * 4, 4);
                            const uint32_t t8 = tkd_rotr(w, 8);
                            a[0] = w & TKD_MASK_BFP4, a[1] = (w << 4) & TKD_MASK_BFP4;
                            a[2] = t8 & TKD_MASK_BFP4, a[3] = (t8 << 4) & TKD_MASK_BFP4;
                            for (int r = 0; r < 4; ++r) {
                                const int64_t k = sa * ksa + qq * 32 + 8 * t + 4 * jj + r;
                                if (k >= K) continue;
                                for (int hi = 0; hi < 2; ++hi) {
                                    const double wv = (double)bf16f((uint16_t)(a[hi + 2 * (r >> 1)] >> (16 * (r & 1))));
                                    for (int m = 0; m < M; ++m)
                                        tmp[hi * M + m] += wv * ldexp((double)bf16f(x[m * K + k]), 64);
                                }
                            }
                        }
                        uint32_t sw;
                        memcpy(&sw, b + gl * 8 + qq * 4, 4);
                        for (int hi = 0; hi < 2; ++hi) {
                            const double s = (double)bf16f((uint16_t)(sw >> (16 * hi)));
                            for (int m = 0; m < M; ++m) acc[(gl + 8 * hi) * M + m] += tmp[hi * M + m] * s;
                        }
                    }
                }
                continue;
            }
            for (int lane = 0; lane < 32; ++lane) {
                const int gl = lane >> 2, t = lane & 3;
                for (int j = 0; j < ksa / 16; ++j) {  // the mmas of the super-atom
                    const int qq = j >> 1, jj = j & 1;
                    uint32_t a[4], s0 = 0, s1 = 0;
                    if (fmt == TKD_BFP4) {
                        uint32_t w, e;
                        memcpy(&w, b + 64 + lane * 16 + j * 4, 4);
                        memcpy(&e, b + t * 16 + j * 4, 4);
                        const uint32_t t8 = tkd_rotr(w, 8);  // (the kernel's own five operations)
                        a[0] = w & TKD_MASK_BFP4, a[1] = (w << 4) & TKD_MASK_BFP4;
                        a[2] = t8 & TKD_MASK_BFP4, a[3] = (t8 << 4) & TKD_MASK_BFP4;
                        s0 = (e & TKD_EMASK_BFP4) | TKD_EBASE_BFP4, s1 = ((e << 7) & TKD_EMASK_BFP4) | TKD_EBASE_BFP4;
                    } else if (fmt == TKD_BFP8) {
                        uint32_t w0, w1, e;
                        memcpy(&w0, b + 32 + lane * 16 + (2 * jj) * 4, 4);
                        memcpy(&w1, b + 32 + lane * 16 + (2 * jj + 1) * 4, 4);
                        memcpy(&e, b + t * 8 + jj * 4, 4);
                        a[0] = w0 & 0x807F807Fu, a[1] = tkd_rotr(w0, 8) & 0x807F807Fu;
                        a[2] = w1 & 0x807F807Fu, a[3] = tkd_rotr(w1, 8) & 0x807F807Fu;
                        s0 = e & 0x7F807F80u, s1 = tkd_rotr(e, 8) & 0x7F807F80u;
                    } else {
                        memcpy(a, b + jj * 512 + lane * 16, 16);
                    }
                    const int64_t kb = sa * ksa + qq * 32 + 8 * t + 4 * jj;  // this lane's 4 k of the mma
                    for (int r = 0; r < 4; ++r) {
                        const int64_t k = kb + r;
                        if (k >= K) continue;
                        const uint32_t sreg = r < 2 ? s0 : s1;
                        const double sc = fmt == TKD_BF16 ? 1.0 : (double)bf16f((uint16_t)(sreg >> (16 * (r & 1))));
                        for (int hi = 0; hi < 2; ++hi) {  // columns gl and gl + 8
                            const uint32_t reg = a[hi + 2 * (r >> 1)];
                            const double wv = (double)bf16f((uint16_t)(reg >> (16 * (r & 1))));
                            for (int m = 0; m < M; ++m)
                                acc[(gl + 8 * hi) * M + m] += wv * ((double)bf16f(x[m * K + k]) * sc);
                        }
                    }
                }
            }
        }
        const int e = fmt == TKD_BF16 || fmt == TKD_INT4 ? 0 : tkd_out_exp(fmt, (int)emax[g]);
        for (int i = 0; i < 16; ++i)
            for (int m = 0; m < M; ++m) y[(int64_t)m * npad + g * 16 + i] = ldexp(acc[i * M + m], e);
    }
}

// the stream back to float32 [K][npad], element by element (the unpack kernel's arithmetic)
void emul_unpack(int fmt, int64_t K, int64_t npad, const uint8_t* stream, const uint8_t* emax, float* out) {
    for (int64_t k = 0; k < K; ++k)
        for (int64_t n = 0; n < npad; ++n) {
            TkdLoc L = tkd_locate(fmt, K, k, n);
            float v;
            if (fmt == TKD_BF16) {
                uint16_t b; memcpy(&b, stream + L.code_word, 2);
                v = bf16f(b);
            } else {
                const int mb = tkd_mant_bits(fmt);
                uint32_t w, ew;
                memcpy(&w, stream + L.code_word, 4);
                memcpy(&ew, stream + L.exp_word, 4);
                const uint32_t c = tkd_code_from_word(fmt, w, L.rot, L.half), m = c & ((1u << mb) - 1);
                if (fmt == TKD_INT4) {
                    v = (float)m * ldexpf(bf16f((uint16_t)(ew >> (16 * L.exp_r))), -TKD_INT4_SCALE_EXP);
                } else {
                    const int e = (int)tkd_exp_from_word(fmt, ew, L.exp_r) + (int)emax[n >> 4] - tkd_ebias(fmt);
                    v = m ? ldexpf((float)m, e - tkd_unit_exp(fmt)) : 0.f;
                }
                if ((c >> mb) & 1u) v = -v;
            }
            out[k * npad + n] = v;
        }
}
}
