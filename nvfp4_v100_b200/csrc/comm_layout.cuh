// Layout of a rank's communication buffer (see comm.cu), shared by the kernels that use it.
#pragma once

#define NVFP4_COMM_MAX_RANKS 8
#define NVFP4_COMM_FLAGS_OFF 64
#define NVFP4_COMM_DATA_OFF 256
#define NVFP4_COMM_SPIN_LIMIT (1u << 22)
// Tail area (256 bytes after the push area): the greedy-pick exchange and the all-reduce that
// runs inside the consuming GEMV (gemv.cu) keep their words here.
#define NVFP4_TAIL_CAND_OFF 0          // float2 pair[2][8]: (value, index bits) per step parity and rank
#define NVFP4_TAIL_CAND_FLAGS_OFF 128  // u32 flags[8]
#define NVFP4_TAIL_AR_FLAGS_OFF 160    // u32 flags[8] of the in-GEMV all-reduce
#define NVFP4_TAIL_AR_READY_OFF 192    // u32: sequence number of the last all-reduce finished here
#define NVFP4_TAIL_AR_DONE_OFF 196     // u32: CTAs of the running all-reduce that have finished
#define NVFP4_TAIL_BYTES 256

__host__ __device__ inline long long nvfp4_comm_tail_offset(int n) {
    return NVFP4_COMM_DATA_OFF + 2LL * n * 2 + 2LL * 8 * n * 2;
}

