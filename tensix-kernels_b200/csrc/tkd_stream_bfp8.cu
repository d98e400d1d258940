// tkd_stream_bfp8.cu: the stream kernel's instantiations for one weight format (a translation unit per format, so that
// they compile side by side).
#include "tkd_stream_tc.cuh"

int tkd_launch_stream_bfp8(const TkdParams& p, int grid, size_t smem, cudaStream_t st) {
    return launch_fmt_all<TKD_BFP8>(p, grid, smem, st);
}
