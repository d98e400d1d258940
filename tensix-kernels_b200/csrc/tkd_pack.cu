// tkd_pack.cu: the weight packer of the dense_reader path.
//
// Replaces the host conversion the reference reaches through ttnn.from_torch(dtype=bfloat8_b | bfloat4_b | bfloat16)
// in native_weight (dense_reader/linear.py:144-156) and block_float (:159-163): float32 -> block-float numbers
// (one shared 8-bit exponent per 16 consecutive output columns at one k, sign + 7 or 3 magnitude bits), by the rule of
// moe/moe8.py:134-150 (truncating alignment shift, then round to nearest even, clamp without an exponent bump, sign
// dropped for zero), and then the re-layout into the HBM stream of tkd_layout.h. Three passes, each a plain
// HBM-bound kernel:
//   1. tkd_quantise_kernel: float32 -> canonical exps [K, G] and codes [K, Npad] (the same numbers the reference's
//      tiles hold, before any re-layout; what the parity tests compare bit for bit);
//   2. tkd_emax_kernel: per group of 16 columns the largest exponent of a row with a non-zero code (a block a group);
//   3. tkd_permute_kernel: canonical -> stream, one thread per 32-bit word of the stream.
// tkd_unpack_kernel is the inverse (stream -> float32 [K, Npad]), used for the weight's read-back.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tkd_internal.h"
#include "tkd_layout.h"

namespace {

__device__ __forceinline__ float src_at(const float* src, int orient, int64_t K, int64_t N, int64_t k, int64_t n,
                                        const float* col_div) {
    // orient 0: src is [N, K] (a torch [out, in] matrix); 1: src is [K, N]
    float v = orient == 0 ? src[n * K + k] : src[k * N + n];
    if (col_div) v = __fdiv_rn(v, col_div[n]);
    return v;
}

// One thread per (group g, k): 16 values -> one exponent byte and 16 code bytes.
__global__ void tkd_quantise_kernel(const float* __restrict__ src, int orient, int64_t K, int64_t N, int64_t npad,
                                    const float* __restrict__ col_div, int mb, uint8_t* __restrict__ exps,
                                    uint8_t* __restrict__ codes) {
    const int64_t G = npad / 16;
    const int64_t k = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    const int64_t g = blockIdx.y;
    if (k >= K) return;
    uint32_t bits[16];
    uint32_t shared = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int64_t n = g * 16 + i;
        bits[i] = n < N ? __float_as_uint(src_at(src, orient, K, N, k, n, col_div)) : 0u;
        shared = max(shared, (bits[i] >> 23) & 0xFFu);
    }
    const int shift = 24 - mb;
    const uint32_t maxm = (1u << mb) - 1;
    uint32_t out[4] = {0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const uint32_t e = (bits[i] >> 23) & 0xFFu;
        const uint32_t man = (bits[i] & 0x7FFFFFu) | (1u << 23);
        const uint32_t diff = shared - e;
        uint32_t m = diff > 31 ? 0u : (man >> diff);       // truncating alignment
        const uint32_t rnd = m & ((1u << shift) - 1);
        m >>= shift;
        const uint32_t tie = 1u << (shift - 1);
        m += (rnd > tie) || (rnd == tie && (m & 1u));      // nearest, ties to even
        m = min(m, maxm);                                  // no exponent bump
        if (e == 0) m = 0;                                 // zero or denormal
        const uint32_t s = m ? (bits[i] >> 31) : 0u;
        out[i >> 2] |= ((s << mb) | m) << (8 * (i & 3));
    }
    exps[k * G + g] = (uint8_t)shared;
    *reinterpret_cast<uint4*>(codes + k * npad + g * 16) = make_uint4(out[0], out[1], out[2], out[3]);
}

// bfloat16 weights: float32 -> bf16 bits (round to nearest even), canonical [K, Npad] uint16.
__global__ void tkd_tobf16_kernel(const float* __restrict__ src, int orient, int64_t K, int64_t N, int64_t npad,
                                  const float* __restrict__ col_div, uint16_t* __restrict__ codes) {
    const int64_t k = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    const int64_t g = blockIdx.y;
    if (k >= K) return;
    for (int i = 0; i < 16; ++i) {
        const int64_t n = g * 16 + i;
        const float v = n < N ? src_at(src, orient, K, N, k, n, col_div) : 0.f;
        codes[k * npad + n] = __bfloat16_as_ushort(__float2bfloat16_rn(v));
    }
}

__device__ __forceinline__ bool row_nonzero(const uint8_t* codes, int64_t npad, int64_t k, int64_t g) {
    const uint4 c = *reinterpret_cast<const uint4*>(codes + k * npad + g * 16);
    return (c.x | c.y | c.z | c.w) != 0;
}

// One block per group: emax[g] = the largest exponent among its rows that hold a non-zero code (0: none). info[0] is
// OR-ed with 1 when a non-zero row's exponent lies more than TKD_ESPREAD below it (a "wide" weight). The
// block's threads share the rows of K out and reduce (maxima and minima: the order does not matter).
constexpr int kEmaxThreads = 256;
__global__ void __launch_bounds__(kEmaxThreads) tkd_emax_kernel(const uint8_t* __restrict__ exps,
                                                               const uint8_t* __restrict__ codes, int64_t K, int64_t npad,
                                                               uint8_t* __restrict__ emax, int* __restrict__ info) {
    __shared__ int shi[kEmaxThreads / 32], slo[kEmaxThreads / 32];
    const int64_t G = npad / 16, g = blockIdx.x;
    int hi = 0, lo = 255;
    for (int64_t k = threadIdx.x; k < K; k += kEmaxThreads) {
        if (!row_nonzero(codes, npad, k, g)) continue;
        const int e = exps[k * G + g];
        hi = max(hi, e);
        lo = min(lo, e);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        hi = max(hi, __shfl_xor_sync(0xFFFFFFFFu, hi, o));
        lo = min(lo, __shfl_xor_sync(0xFFFFFFFFu, lo, o));
    }
    if ((threadIdx.x & 31) == 0) shi[threadIdx.x >> 5] = hi, slo[threadIdx.x >> 5] = lo;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kEmaxThreads / 32; ++w) hi = max(hi, shi[w]), lo = min(lo, slo[w]);
        emax[g] = (uint8_t)hi;
        if (lo <= hi && hi - lo > TKD_ESPREAD) atomicOr(info, 1);
    }
}

// One thread per 32-bit word of the stream.
__global__ void tkd_permute_kernel(int fmt, int64_t K, int64_t npad, const uint8_t* __restrict__ exps,
                                   const void* __restrict__ codes_v, const uint8_t* __restrict__ emax,
                                   uint32_t* __restrict__ stream) {
    const int64_t words = tkd_stream_bytes(fmt, K, npad) / 4;
    const int64_t wi = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (wi >= words) return;
    const int64_t G = npad / 16;
    const int ksa = tkd_ksa(fmt), eb = tkd_exp_bytes(fmt);
    int64_t g, sa;
    int off;  // byte offset of this word inside its super-atom
    tkd_sa_owner(fmt, K, wi * 4, &g, &sa, &off);
    uint32_t word = 0;
    if (fmt == TKD_BF16) {
        const uint16_t* codes = static_cast<const uint16_t*>(codes_v);
        const int jj = off / 512, lane = (off % 512) / 16, ai = (off % 16) / 4;
        const int t = lane & 3, i = (lane >> 2) + 8 * (ai & 1);
        for (int half = 0; half < 2; ++half) {
            const int64_t k = sa * ksa + 8 * t + 4 * jj + 2 * (ai >> 1) + half;
            const uint32_t v = k < K ? codes[k * npad + g * 16 + i] : 0u;
            word |= v << (16 * half);
        }
    } else if (fmt == TKD_INT4 && off < eb) {
        // the scales of the super-atom's k32 block qq for columns g8 and g8 + 8 (exps: bf16 bits [ceil(K / 32), npad]),
        // each times 2^TKD_INT4_SCALE_EXP (exact: a bf16 keeps its significand; the product is a normal number)
        const uint16_t* sc = reinterpret_cast<const uint16_t*>(exps);
        const int g8 = (off / 4) >> 1, qq = (off / 4) & 1;
        const int64_t kg = sa * 2 + qq;
        for (int half = 0; half < 2; ++half) {
            uint32_t b = 0;
            if (kg * 32 < K) {
                const float v = __uint_as_float((uint32_t)sc[kg * npad + g * 16 + g8 + 8 * half] << 16);
                b = __float_as_uint(v * 0x1p65f) >> 16;
            }
            word |= b << (16 * half);
        }
    } else if (off < eb) {
        const uint8_t* codes = static_cast<const uint8_t*>(codes_v);
        const int per_t = fmt == TKD_BFP4 ? 4 : 2;
        const int t = (off / 4) / per_t, j = (off / 4) % per_t;
        const int qq = fmt == TKD_BFP4 ? j >> 1 : 0, jj = fmt == TKD_BFP4 ? j & 1 : j;
        for (int r = 0; r < 4; ++r) {
            const int64_t k = sa * ksa + qq * 32 + 8 * t + 4 * jj + r;
            int e = tkd_ezero(fmt);
            if (k < K && row_nonzero(codes, npad, k, g))
                e = max(tkd_ezero(fmt), (int)exps[k * G + g] - (int)emax[g] + tkd_ebias(fmt));
            word |= tkd_exp_bits(fmt, (uint32_t)e, r);
        }
    } else {
        const uint8_t* codes = static_cast<const uint8_t*>(codes_v);
        const int co = off - eb;
        const int lane = co / 16, wj = (co % 16) / 4;
        const int t = lane & 3, g8 = lane >> 2;
        if (fmt == TKD_BFP8) {
            const int jj = wj >> 1, apair = wj & 1;  // the word holds a(2 apair) and a(2 apair) + 1
            for (int odd = 0; odd < 2; ++odd)
                for (int half = 0; half < 2; ++half) {
                    const int64_t k = sa * ksa + 8 * t + 4 * jj + 2 * apair + half;
                    const uint32_t c = k < K ? codes[k * npad + g * 16 + g8 + 8 * odd] : 0u;
                    word |= tkd_code_bits(fmt, c, 8 * odd, half);
                }
        } else {
            const int qq = wj >> 1, jj = wj & 1;
            for (int ai = 0; ai < 4; ++ai)
                for (int half = 0; half < 2; ++half) {
                    const int64_t k = sa * ksa + qq * 32 + 8 * t + 4 * jj + 2 * (ai >> 1) + half;
                    const uint32_t c = k < K ? codes[k * npad + g * 16 + g8 + 8 * (ai & 1)] : 0u;
                    word |= tkd_code_bits(fmt, c, ai, half);
                }
        }
    }
    stream[wi] = word;
}

// One thread per element: canonical block-float numbers -> bf16 bits [K, npad]. Every block-float value
// +-m * 2^(e - unit) (m below 2^7, e from 1) is a bf16 value exactly, the subnormal ones included (multiples of 2^-132),
// so the float's low 16 bits are zero and its high 16 are the bf16.
__global__ void tkd_dequantise_bf16_kernel(int fmt, int64_t K, int64_t npad, const uint8_t* __restrict__ exps,
                                           const uint8_t* __restrict__ codes, uint16_t* __restrict__ out) {
    const int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (idx >= K * npad) return;
    const int64_t k = idx / npad, n = idx % npad;
    const int mb = tkd_mant_bits(fmt);
    const uint32_t c = codes[idx], m = c & ((1u << mb) - 1);
    const float v = m ? ldexpf((float)m, (int)exps[k * (npad / 16) + (n >> 4)] - tkd_unit_exp(fmt)) : 0.f;
    out[idx] = (uint16_t)((__float_as_uint(v) >> 16) | (((c >> mb) & 1u) << 15));
}

// One thread per element: stream -> float32 [K, npad].
__global__ void tkd_unpack_kernel(int fmt, int64_t K, int64_t npad, const uint8_t* __restrict__ stream,
                                  const uint8_t* __restrict__ emax, float* __restrict__ out) {
    const int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (idx >= K * npad) return;
    const int64_t k = idx / npad, n = idx % npad;
    const TkdLoc L = tkd_locate(fmt, K, k, n);
    float v;
    if (fmt == TKD_BF16) {
        const uint16_t b = *reinterpret_cast<const uint16_t*>(stream + L.code_word);
        v = __uint_as_float((uint32_t)b << 16);
    } else {
        const int mb = tkd_mant_bits(fmt);
        const uint32_t w = *reinterpret_cast<const uint32_t*>(stream + L.code_word);
        const uint32_t c = tkd_code_from_word(fmt, w, L.rot, L.half);
        const uint32_t m = c & ((1u << mb) - 1);
        const uint32_t ew = *reinterpret_cast<const uint32_t*>(stream + L.exp_word);
        if (fmt == TKD_INT4) {
            // q * s: the stored scale is s * 2^65
            const float s65 = __uint_as_float(((ew >> (16 * L.exp_r)) & 0xFFFFu) << 16);
            v = (float)m * (s65 * 0x1p-65f);
        } else {
            const int e = (int)tkd_exp_from_word(fmt, ew, L.exp_r) + (int)emax[n >> 4] - tkd_ebias(fmt);
            v = m ? ldexpf((float)m, e - tkd_unit_exp(fmt)) : 0.f;
        }
        if ((c >> mb) & 1u) v = -v;
    }
    out[idx] = v;
}

}  // namespace

int tkd_launch_quantise(int fmt, const float* src, int orient, int64_t K, int64_t N, int64_t npad,
                        const float* col_div, uint8_t* exps, void* codes, cudaStream_t st) {
    dim3 grid((unsigned)((K + 127) / 128), (unsigned)(npad / 16));
    if (fmt == TKD_BF16)
        tkd_tobf16_kernel<<<grid, 128, 0, st>>>(src, orient, K, N, npad, col_div, static_cast<uint16_t*>(codes));
    else
        tkd_quantise_kernel<<<grid, 128, 0, st>>>(src, orient, K, N, npad, col_div, tkd_mant_bits(fmt), exps,
                                                  static_cast<uint8_t*>(codes));
    return (int)cudaGetLastError();
}

int tkd_launch_permute(int fmt, int64_t K, int64_t npad, const uint8_t* exps, const void* codes, uint8_t* emax,
                       int* info, void* stream, cudaStream_t st) {
    const int64_t G = npad / 16;
    if (fmt != TKD_BF16 && fmt != TKD_INT4) {
        tkd_emax_kernel<<<(unsigned)G, kEmaxThreads, 0, st>>>(exps, static_cast<const uint8_t*>(codes), K, npad, emax, info);
    }
    const int64_t words = tkd_stream_bytes(fmt, K, npad) / 4;
    tkd_permute_kernel<<<(unsigned)((words + 255) / 256), 256, 0, st>>>(fmt, K, npad, exps, codes, emax,
                                                                       static_cast<uint32_t*>(stream));
    return (int)cudaGetLastError();
}

int tkd_launch_dequantise_bf16(int fmt, int64_t K, int64_t npad, const uint8_t* exps, const void* codes, void* out,
                               cudaStream_t st) {
    const int64_t n = K * npad;
    tkd_dequantise_bf16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(fmt, K, npad, exps, static_cast<const uint8_t*>(codes),
                                                                            static_cast<uint16_t*>(out));
    return (int)cudaGetLastError();
}

int tkd_launch_unpack(int fmt, int64_t K, int64_t npad, const void* stream, const uint8_t* emax, float* out,
                      cudaStream_t st) {
    const int64_t n = K * npad;
    tkd_unpack_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(fmt, K, npad, static_cast<const uint8_t*>(stream),
                                                                  emax, out);
    return (int)cudaGetLastError();
}
