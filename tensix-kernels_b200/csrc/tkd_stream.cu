// tkd_stream.cu: the launch of the stream kernel by weight format, and the small kernel that waits for an exchange.
#include <cuda_runtime.h>
#include <stdint.h>

#include "tkd_internal.h"
#include "tkd_layout.h"

int tkd_launch_stream_bfp8(const TkdParams& p, int grid, size_t smem, cudaStream_t st);
int tkd_launch_stream_bfp4(const TkdParams& p, int grid, size_t smem, cudaStream_t st);
int tkd_launch_stream_bf16(const TkdParams& p, int grid, size_t smem, cudaStream_t st);
int tkd_launch_stream_int4(const TkdParams& p, int grid, size_t smem, cudaStream_t st);

namespace {

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Waits (one warp) until every rank's completed-call count in `flags` has reached this rank's own.
__global__ void tkd_exchange_wait_kernel(uint32_t* flags, int nranks, int* status) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x == 0) {
        const uint32_t seq = ld_acquire_sys(flags + TKD_FLAG_SEQ);
        bool ok = true;
        for (int r = 0; r < nranks && ok; ++r) {
            int rounds = 0;  // (bounded: about a second)
            while ((int32_t)(ld_acquire_sys(flags + r) - seq) < 0) {
                if (++rounds > (1 << 20)) {
                    ok = false;
                    break;
                }
                __nanosleep(rounds < 64 ? 20 : 200);
            }
        }
        if (!ok && status) atomicExch(status, TKD_ERR_TIMEOUT);
        __threadfence_system();
    }
}

// Numbers this rank's exchanged call and tells every rank (one thread). It runs, by stream order, after the stream
// kernel whose peer stores it announces has completed; with lag_wait it then checks (bounded) that every rank's call
// BEFORE this one has been announced here.
__global__ void tkd_exchange_publish_kernel(uint32_t* flags, TkdPeerFlags peers, int nranks, int rank, int lag_wait, int* status) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x != 0) return;
    const uint32_t seq = flags[TKD_FLAG_SEQ] + 1;
    flags[TKD_FLAG_SEQ] = seq;
    __threadfence_system();
    for (int q = 0; q < nranks - 1; ++q)
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(peers.p[q] + rank), "r"(seq) : "memory");
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(flags + rank), "r"(seq) : "memory");
    if (!lag_wait) return;
    for (int r = 0; r < nranks; ++r) {
        int rounds = 0;  // (bounded: about a second)
        while ((int32_t)(ld_acquire_sys(flags + r) - (seq - 1)) < 0) {
            if (++rounds > (1 << 20)) {
                if (status) atomicExch(status, TKD_ERR_TIMEOUT);
                return;
            }
            __nanosleep(rounds < 64 ? 20 : 200);
        }
    }
}

}  // namespace

int tkd_launch_exchange_publish(uint32_t* flags, const TkdPeerFlags& peers, int nranks, int rank, int lag_wait, int* status,
                                cudaStream_t st) {
    tkd_exchange_publish_kernel<<<1, 32, 0, st>>>(flags, peers, nranks, rank, lag_wait, status);
    return (int)cudaGetLastError();
}

int tkd_launch_exchange_wait(uint32_t* flags, int nranks, int* status, cudaStream_t st) {
    tkd_exchange_wait_kernel<<<1, 32, 0, st>>>(flags, nranks, status);
    return (int)cudaGetLastError();
}

int tkd_launch_stream(const TkdParams& p, int grid, size_t smem, cudaStream_t st) {
    switch (p.fmt) {
        case TKD_BFP8: return tkd_launch_stream_bfp8(p, grid, smem, st);
        case TKD_BFP4: return tkd_launch_stream_bfp4(p, grid, smem, st);
        case TKD_INT4: return tkd_launch_stream_int4(p, grid, smem, st);
        default: return tkd_launch_stream_bf16(p, grid, smem, st);
    }
}
