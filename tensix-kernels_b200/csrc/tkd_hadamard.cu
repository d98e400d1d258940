// tkd_hadamard.cu: the block Hadamard rotation the reference's ternary projections put before their matmul
// (ternary_matmul/t2.py:213-217 rotate, :262-340 hadamard; kernels/had_reader.cpp, had_compute.cpp, had_writer.cpp):
// x' = H_1024 (s * x) per block of 1024 inputs, H the Sylvester matrix of +-1 entries, UNNORMALISED (32 times the
// orthonormal transform: the group scales carry the 1/32, as in the reference), s fixed signs per input.
//
// The reference multiplies 32 x 32 tiles by H_32 twice on the matrix engine; here a block is 10 butterfly stages in
// shared memory in fp32 (a fast Walsh-Hadamard transform: 5120 additions instead of 65536 multiply-adds), one CTA per
// (row, block), rounded to bf16 once at the end. A latency-sized kernel: 2 KB in, 2 KB out per block.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tkd_internal.h"

namespace {

constexpr int kBlock = 1024, kThreads = 256;

// signs: the reference's mask words (t2.py:185-202): word q has bit 15 set when input 2 q is negated, bit 31 for 2 q + 1.
__global__ void __launch_bounds__(kThreads) tkd_hadamard_kernel(const uint16_t* __restrict__ x, int64_t ldx,
                                                                const uint32_t* __restrict__ signs, int K,
                                                                uint16_t* __restrict__ out, int64_t ldo) {
    __shared__ float v[kBlock];
    asm volatile("griddepcontrol.wait;" ::: "memory");  // (x may be the output of the kernel before this one)
    const int row = blockIdx.y, b = blockIdx.x, t = threadIdx.x;
    const uint16_t* xr = x + (int64_t)row * ldx + (int64_t)b * kBlock;
    // this thread's inputs 4 t .. 4 t + 3 (8 bytes) and their two sign words
    const uint2 raw = *reinterpret_cast<const uint2*>(xr + 4 * t);
    const uint2 sw = *reinterpret_cast<const uint2*>(signs + (b * kBlock + 4 * t) / 2);
    const uint32_t w0 = raw.x ^ (sw.x & 0x80008000u), w1 = raw.y ^ (sw.y & 0x80008000u);
    v[4 * t] = __uint_as_float(w0 << 16), v[4 * t + 1] = __uint_as_float(w0 & 0xFFFF0000u);
    v[4 * t + 2] = __uint_as_float(w1 << 16), v[4 * t + 3] = __uint_as_float(w1 & 0xFFFF0000u);
    __syncthreads();
    // stage h: pairs (i, i + h) with i's bit h clear; 512 pairs a stage, two a thread
    for (int h = 1; h < kBlock; h <<= 1) {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int p = t + q * kThreads;                    // pair number 0 .. 511
            const int i = ((p & ~(h - 1)) << 1) | (p & (h - 1));  // insert a 0 at bit h
            const float a = v[i], c = v[i + h];
            v[i] = a + c, v[i + h] = a - c;
        }
        __syncthreads();
    }
    uint16_t* o = out + (int64_t)row * ldo + (int64_t)b * kBlock;
    const uint32_t o0 = __bfloat16_as_ushort(__float2bfloat16_rn(v[4 * t])) |
                        ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v[4 * t + 1])) << 16);
    const uint32_t o1 = __bfloat16_as_ushort(__float2bfloat16_rn(v[4 * t + 2])) |
                        ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v[4 * t + 3])) << 16);
    *reinterpret_cast<uint2*>(o + 4 * t) = make_uint2(o0, o1);
}

}  // namespace

int tkd_launch_hadamard(const void* x, int64_t ldx, const uint32_t* signs, int rows, int K, void* out, int64_t ldo,
                        cudaStream_t st) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(K / kBlock), (unsigned)rows);
    cfg.blockDim = dim3(kThreads);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, tkd_hadamard_kernel, static_cast<const uint16_t*>(x), ldx, signs, K,
                                   static_cast<uint16_t*>(out), ldo);
}
