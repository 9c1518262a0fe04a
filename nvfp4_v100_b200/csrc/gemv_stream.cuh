// Interface between the GEMV dispatchers (gemv.cu) and the ring-streaming GEMV kernel
// (gemv_stream.cu).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace nvfp4 {

// prologue / epilogue codes: the values of launch_nvfp4_gemv_fused's arguments
enum { GS_PRO_NONE = 0, GS_PRO_RMSNORM = 1 };
enum { GS_EPI_STORE = 0, GS_EPI_RESIDUAL = 1, GS_EPI_SILU_MUL = 2 };

struct StreamArgs {
    const __half* act;
    __half* out;
    const float* norm_w1;     // GS_PRO_RMSNORM: fp32 (1 + weight) [K]
    const __half* residual;   // GS_EPI_RESIDUAL: fp16 [M]
    float eps;
    int M, K;
    int KC;            // weights per ring stage and row (multiple of 256)
    int nst;           // ring stages
    int stage_bytes;   // 9 * KC
    int rb;            // unit in which rows are dealt to the CTAs (4 or 16)
    int ring_off;      // byte offset of the ring in dynamic shared memory
    int probe;         // attribution probes (bit 0: no arithmetic, bit 1: no weight copies)
};

struct StreamPlan {
    int warps, KC, nst, stage_bytes, rb, grid, ring_off, smem;
};

struct StreamConfig {
    int warps = 0, smem_kb = 0, stage_kb = 0, min_stages = 0, ctas_per_sm = 0, rows_per_box = 0,
        enable = 0, probe = 0;
};

StreamConfig& stream_config();

// false when the ring kernel does not take the shape (K % 256 != 0, a prologue it cannot hold,
// too little shared memory for two stages per warp) or is not switched on.
bool plan_stream(int M, int K, int prologue, int epilogue, StreamPlan* out);

// Requirements beyond plan_stream: packed and scales 16-byte aligned, act 16-byte aligned.
cudaError_t launch_stream(const void* packed, const void* scales, const void* act, void* out, int M,
                          int K, int pro, const void* norm_w1, float eps, int epi,
                          const void* residual, const StreamPlan& pl, cudaStream_t st, bool pdl);

}  // namespace nvfp4
