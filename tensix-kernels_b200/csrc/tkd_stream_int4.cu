// tkd_stream_int4.cu: the stream kernel's instantiations for the int4 weight with group scales (one to eight rows: the
// reference's w4a16_linear is a one-token op, int4/w4a16.py; more rows use the weight's dequantised bfloat8_b form).
#include "tkd_stream_kernel.cuh"

int tkd_launch_stream_int4(const TkdParams& p, int grid, size_t smem, cudaStream_t st) {
    return launch_fmt<TKD_INT4>(p, grid, smem, st);
}
