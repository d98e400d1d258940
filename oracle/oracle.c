/* oracle.c: CPU restatement of the reference's dense_reader arithmetic. TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker the CUDA path is compared with. It is never linked into, imported by or called from the
 * product library; only the tests, the smoke check and the benchmark's CPU-baseline leg use it.
 *
 * What it restates (paths are those of XylolabsInc/tensix-kernels):
 *   - block-float quantiser: moe/moe8.py:117-154 (bfp4_tiles, declared byte-identical to ttnn 0.81.1's host
 *     conversion and pinned by moe/tests/test_moe.py:84-89), generalised from 3 to 7 mantissa bits for bfloat8_b by
 *     the same rule (the quantiser itself lives in the third-party wheel ttnn==0.81.1, call sites
 *     dense_reader/linear.py:155,162). bfloat4_b: pinned against golden vectors made from the reference's own
 *     bfp4_tiles. bfloat8_b: PARITY UNPINNED (no vector for it exists in the reference).
 *   - dequantiser: moe/moe8.py:157-169 (unit exponent 129 for 3 mantissa bits, hence 126 + mantissa bits).
 *   - reference matmul: dense_reader/linear.py:166-169 and dense_reader/tests/test_dense_reader.py:56-58.
 *   - output stages: dense_reader/kernels/dense_compute.cpp:200-356, common/kernels/dense_ops.h:44-85.
 *   - top-k records: dense_reader/kernels/dense_writer.cpp:185-258, decode dense_reader/linear.py:753-768.
 *   - bf16_ceil: dense_reader/linear.py:110-114.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* float32 -> bf16 bits, round to nearest even (NaN kept quiet). */
uint16_t orc_bf16_rne(float f) {
    uint32_t u = f2u(f);
    if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x007FFFFFu)) return (uint16_t)((u >> 16) | 0x0040u);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
float orc_bf16_to_f32(uint16_t b) { return u2f((uint32_t)b << 16); }

/* linear.py:110-114: the smallest bf16 >= s (s > 0). */
float orc_bf16_ceil(float s) {
    float b = orc_bf16_to_f32(orc_bf16_rne(s));
    if (b >= s) return b;
    return u2f(f2u(b) + 0x10000u);
}

/* Quantise w [K][N] (row-major, N a multiple of 16) to the block-float grid with `mb` mantissa bits (3: bfloat4_b,
 * 7: bfloat8_b). One shared exponent per 16 consecutive n at one k (a face row of the reference's 32 x 32 tile).
 * exps [K][N/16]; codes [K][N], each sign << mb | magnitude. moe8.py:134-150. */
void orc_quantise(const float* w, int64_t K, int64_t N, int mb, uint8_t* exps, uint8_t* codes) {
    const int shift = 24 - mb;
    const int64_t G = N / 16;
    const int64_t maxm = (1 << mb) - 1;
    for (int64_t k = 0; k < K; ++k) {
        for (int64_t g = 0; g < G; ++g) {
            const float* p = w + k * N + g * 16;
            uint32_t shared = 0;
            for (int i = 0; i < 16; ++i) {
                uint32_t e = (f2u(p[i]) >> 23) & 0xFF;
                if (e > shared) shared = e;
            }
            exps[k * G + g] = (uint8_t)shared;
            for (int i = 0; i < 16; ++i) {
                uint32_t bits = f2u(p[i]);
                uint32_t e = (bits >> 23) & 0xFF;
                uint32_t sign = bits >> 31;
                int64_t man = (int64_t)((bits & 0x7FFFFFu) | (1u << 23));
                uint32_t diff = shared - e;
                int64_t m = diff > 31 ? 0 : (man >> (diff > 31 ? 31 : diff)); /* truncating shift first */
                int64_t rnd = m & (((int64_t)1 << shift) - 1);
                m >>= shift;
                int64_t guard = m & 1;
                int64_t tie = (int64_t)1 << (shift - 1);
                m += (rnd > tie) || (rnd == tie && guard == 1); /* then nearest, ties to even */
                if (m > maxm) m = maxm;                         /* no exponent bump */
                if (e == 0) m = 0;                              /* zero or denormal */
                uint32_t s = m == 0 ? 0 : sign;
                codes[k * N + g * 16 + i] = (uint8_t)((s << mb) | (uint32_t)m);
            }
        }
    }
}

/* moe8.py:157-169: (-1)^s * m * 2^(shared - (126 + mb)). */
void orc_dequantise(const uint8_t* exps, const uint8_t* codes, int64_t K, int64_t N, int mb, float* out) {
    const int64_t G = N / 16;
    for (int64_t k = 0; k < K; ++k)
        for (int64_t n = 0; n < N; ++n) {
            uint8_t c = codes[k * N + n];
            float mag = (float)(c & ((1 << mb) - 1));
            float v = ldexpf(mag, (int)exps[k * G + n / 16] - (126 + mb));
            out[k * N + n] = (c >> mb) & 1 ? -v : v;
        }
}

/* The reference's tile bytes (moe8.py:125-154): tiles [K/32][N/32][64 + 1024 * (mb + 1) / 8]; per tile 64 exponents
 * (face by face, row by row; faces (r0-15,c0-15), (r0-15,c16-31), (r16-31,c0-15), (r16-31,c16-31)), then the codes in
 * the same order: mb = 3 two per byte, the first in the low nibble; mb = 7 one per byte. */
void orc_tiles(const uint8_t* exps, const uint8_t* codes, int64_t K, int64_t N, int mb, uint8_t* tiles) {
    const int64_t G = N / 16, KT = K / 32, NT = N / 32;
    const int64_t body = mb == 3 ? 512 : 1024, tb = 64 + body;
    for (int64_t kt = 0; kt < KT; ++kt)
        for (int64_t nt = 0; nt < NT; ++nt) {
            uint8_t* t = tiles + (kt * NT + nt) * tb;
            for (int f = 0; f < 4; ++f)
                for (int r = 0; r < 16; ++r) {
                    int64_t k = kt * 32 + (f >> 1) * 16 + r;
                    int64_t n0 = nt * 32 + (f & 1) * 16;
                    t[f * 16 + r] = exps[k * G + n0 / 16];
                    for (int c = 0; c < 16; ++c) {
                        uint8_t code = codes[k * N + n0 + c];
                        int64_t e = f * 256 + r * 16 + c;
                        if (mb == 3) {
                            if (e & 1) t[64 + e / 2] |= (uint8_t)(code << 4);
                            else t[64 + e / 2] = code;
                        } else {
                            t[64 + e] = code;
                        }
                    }
                }
        }
}

/* y[m][n] = sum_k bf16(x)[m][k] * w[k][n], accumulated in double (test_dense_reader.py:56-58) and returned as double.
 * x is given as bf16 bits. */
void orc_matmul_f64(const uint16_t* x, int64_t M, int64_t K, const float* w, int64_t N, double* y) {
    for (int64_t m = 0; m < M; ++m) {
        double* yr = y + m * N;
        for (int64_t n = 0; n < N; ++n) yr[n] = 0.0;
        for (int64_t k = 0; k < K; ++k) {
            double xv = (double)orc_bf16_to_f32(x[m * K + k]);
            if (xv == 0.0) continue;
            const float* wr = w + k * N;
            for (int64_t n = 0; n < N; ++n) yr[n] += xv * (double)wr[n];
        }
    }
}

static double silu(double g) { return g / (1.0 + exp(-g)); }
/* dense_ops.h:44-59: x * sigmoid(1.5957691216 x + 0.0713548162 x^3) == torch gelu(approximate="tanh"). */
static double gelu_tanh(double g) {
    return 0.5 * g * (1.0 + tanh(0.7978845608028654 * (g + 0.044715 * g * g * g)));
}

/* Output stages on the K sums acc [M][N] (double): mode 0 plain (* scale[n] if scale), 1 GLU over an interleaved
 * weight (tile 2j gate, 2j+1 up, 32 columns each; out [M][N/2]), 2 GLU over two sums (acc gate, acc2 up; out [M][N]),
 * 3 residual add (res bf16 bits [M][N]), 4 fp32 as it is (+ res32 if given). act: 0 silu, 1 gelu_tanh. scale2: the up
 * half's scales for mode 2 (scale the gate's); both may be NULL. Result in double; the caller rounds. */
void orc_epilogue(const double* acc, const double* acc2, int64_t M, int64_t N, int mode, int act, const float* scale,
                  const float* scale2, const uint16_t* res, const float* res32, double* out) {
    for (int64_t m = 0; m < M; ++m) {
        if (mode == 1) {
            for (int64_t o = 0; o < N / 2; ++o) {
                int64_t gc = 64 * (o / 32) + o % 32, uc = gc + 32;
                double g = acc[m * N + gc] * (scale ? scale[gc] : 1.0), u = acc[m * N + uc] * (scale ? scale[uc] : 1.0);
                out[m * (N / 2) + o] = (act ? gelu_tanh(g) : silu(g)) * u;
            }
            continue;
        }
        for (int64_t n = 0; n < N; ++n) {
            double v = acc[m * N + n];
            if (mode == 0) v *= scale ? (double)scale[n] : 1.0;
            if (mode == 2) {
                double g = v * (scale ? scale[n] : 1.0), u = acc2[m * N + n] * (scale2 ? scale2[n] : 1.0);
                v = (act ? gelu_tanh(g) : silu(g)) * u;
            }
            if (mode == 3) v += (double)orc_bf16_to_f32(res[m * N + n]);
            if (mode == 4 && res32) v += (double)res32[m * N + n];
            out[m * N + n] = v;
        }
    }
}

/* dense_writer.cpp:215: a bf16 as a monotone uint16 key; 0 is below every value. */
uint32_t orc_key(uint16_t b) { return (uint32_t)(b ^ (0x8000u | (0x7FFFu & (0u - (uint32_t)(b >> 15))))) & 0xFFFFu; }

/* linear.py:762-767: key -> float32 bits' value; key 0 -> -inf. */
float orc_key_value(uint32_t key) {
    if (key == 0) return -INFINITY;
    uint32_t bits = key >= 0x8000u ? (key & 0x7FFFu) : (~key & 0xFFFFu);
    return u2f(bits << 16);
}

/* Canonical top-k of one row of bf16 outputs y[0..n): key descending, index ascending among equal keys; columns whose
 * key is 0 never enter (the reference's `k > floor` with floor 0, dense_writer.cpp:216). keys/idx [k]; empty slots
 * key 0, idx 0xFFFFFFFF. idx = base + column. */
void orc_topk_canonical(const uint16_t* y, int64_t n, int k, uint32_t base, uint32_t* keys, uint32_t* idx) {
    for (int q = 0; q < k; ++q) { keys[q] = 0; idx[q] = 0xFFFFFFFFu; }
    for (int64_t c = 0; c < n; ++c) {
        uint32_t key = orc_key(y[c]);
        if (key == 0) continue;
        int q = k;
        while (q > 0 && keys[q - 1] < key) --q; /* strictly better than what it passes: earlier index stays ahead */
        if (q == k) continue;
        for (int j = k - 1; j > q; --j) { keys[j] = keys[j - 1]; idx[j] = idx[j - 1]; }
        keys[q] = key;
        idx[q] = base + (uint32_t)c;
    }
}

/* The reference writer's own running top-k over columns [c0, c1) in ascending order (dense_writer.cpp:100-109,
 * 185-232): insert iff key > the smallest kept key, replacing the first slot that holds it. Slot order is history
 * dependent; used to list where it differs from the canonical order. */
void orc_topk_scan_ref(const uint16_t* y, int64_t c0, int64_t c1, int64_t n, int k, uint32_t base, uint32_t* keys,
                       uint32_t* idx) {
    int low = 0;
    for (int q = 0; q < k; ++q) { keys[q] = 0; idx[q] = 0xFFFFFFFFu; }
    for (int64_t c = c0; c < c1 && c < n; ++c) {
        uint32_t key = orc_key(y[c]);
        if (key > keys[low]) {
            keys[low] = key;
            idx[low] = base + (uint32_t)c;
            int lo = 0;
            for (int q = 1; q < k; ++q) if (keys[q] < keys[lo]) lo = q;
            low = lo;
        }
    }
}
