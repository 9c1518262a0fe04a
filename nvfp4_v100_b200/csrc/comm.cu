// One-shot all-reduce + residual add over NVLink peer memory for tensor-parallel decode.
//
// The reference is single-GPU and has no collective.  In tensor-parallel decode every K-split
// layer (o_proj, out_proj, down_proj) ends with a sum of one 5120-element vector over the ranks,
// 128 times per token: a latency problem, not a bandwidth one.  Instead of a library all-reduce
// followed by an add kernel, each rank runs ONE small kernel that
//   1. tells every peer "my partial vector number `seq` is ready" (a release store of `seq` into
//      the peer's flag word, over NVLink),
//   2. waits until every peer has said the same (a BOUNDED spin on its own flag words),
//   3. pulls the peers' vectors with plain peer loads, sums them in rank order in fp32, rounds to
//      fp16, and adds the result to the residual stream h (fp32 add, one rounding).
// The partial vector is written by the GEMV straight into this rank's communication buffer, so
// nothing is copied on the sending side.
//
// Communication buffer (one per rank, cudaMalloc'ed by that rank, opened by the others through
// CUDA IPC):  u32 counter | u32 error | pad | u32 flags[8] at byte 64 | data[2][n] fp16 at byte 256,
// followed by the push area used by the fused GEMV + all-reduce kernel (gemv.cu).
// Vectors alternate between the two data slots (`parity`): a rank can overwrite slot p for call
// s+2 only after it has finished call s+1, which needed every peer's flag for s+1, which a peer
// sends only after it has finished reading call s.
//
// Every wait has an iteration limit; when it runs out the kernel records the fact in the error
// word (readable with nvfp4_comm_status) and carries on, so a missing peer can never hang a GPU.
// Kernels of different ranks wait on one another, so they must run on different GPUs.
#include <cstdio>
#include <cstring>

#include "common.cuh"

#include "comm_layout.cuh"

namespace nvfp4 {

struct CommPeers {
    unsigned char* buf[NVFP4_COMM_MAX_RANKS];  // every rank's communication buffer, as mapped here
};

__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_relaxed_sys_u4(const void* p) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}

// n % 8 == 0.  One CTA; thread i handles elements 8i .. 8i+7 (strided for larger n).
__global__ void __launch_bounds__(1024)
allreduce_residual_kernel(CommPeers peers, int rank, int world, int n, int parity,
                          __half* __restrict__ h) {
    pdl_prologue();
    PDL_FRESH(h);
    __shared__ uint32_t s_seq;
    unsigned char* mine = peers.buf[rank];
    uint32_t* counter = reinterpret_cast<uint32_t*>(mine);
    uint32_t* err = counter + 1;
    const int tid = threadIdx.x;
    if (tid == 0) {
        const uint32_t seq = *counter + 1;
        *counter = seq;
        s_seq = seq;
    }
    __syncthreads();
    const uint32_t seq = s_seq;
    if (tid < world && tid != rank) {
        // the partial vector was written by the previous kernel in this stream; make it visible
        // system-wide before announcing it
        __threadfence_system();
        st_release_sys_u32(reinterpret_cast<uint32_t*>(peers.buf[tid] + NVFP4_COMM_FLAGS_OFF) + rank,
                           seq);
        const uint32_t* flag = reinterpret_cast<const uint32_t*>(mine + NVFP4_COMM_FLAGS_OFF) + tid;
        uint32_t spins = 0;
        // signed distance, so the comparison survives counter wrap-around
        while ((int32_t)(ld_acquire_sys_u32(flag) - seq) < 0) {
            if (++spins > NVFP4_COMM_SPIN_LIMIT) {
                atomicExch(err, 1u + (uint32_t)tid);  // which peer never arrived
                break;
            }
        }
    }
    __syncthreads();
    // A peer that never announced its vector leaves stale bytes in its slot: adding them would
    // corrupt the residual stream silently, so the sum is skipped and h keeps its value (the
    // error word says which peer was missing; the caller checks it).
    if (*reinterpret_cast<volatile uint32_t*>(err) != 0u) return;
    const size_t slot = NVFP4_COMM_DATA_OFF + (size_t)parity * (size_t)n * sizeof(__half);
    for (int i = tid * 8; i < n; i += blockDim.x * 8) {
        // all peers' loads are issued before the first is used: one NVLink round trip, not one
        // per peer
        uint4 v[NVFP4_COMM_MAX_RANKS];
#pragma unroll
        for (int r = 0; r < NVFP4_COMM_MAX_RANKS; r++)
            if (r < world) v[r] = ld_relaxed_sys_u4(peers.buf[r] + slot + (size_t)i * sizeof(__half));
        float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int r = 0; r < NVFP4_COMM_MAX_RANKS; r++) {
            if (r < world) {
                const __half2* p = reinterpret_cast<const __half2*>(&v[r]);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float2 f = __half22float2(p[j]);
                    acc[2 * j] += f.x;
                    acc[2 * j + 1] += f.y;
                }
            }
        }
        uint4 hv = *reinterpret_cast<const uint4*>(h + i);
        __half2* hp = reinterpret_cast<__half2*>(&hv);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float2 f = __half22float2(hp[j]);
            hp[j] = __floats2half2_rn(f.x + round_f16(acc[2 * j]), f.y + round_f16(acc[2 * j + 1]));
        }
        *reinterpret_cast<uint4*>(h + i) = hv;
    }
}

// Tensor-parallel greedy pick without a library collective: every rank finds the maximum of its
// vocabulary slice, stores (value, global index) into slot `rank` of EVERY rank's tail area (peer
// stores over NVLink), announces it with a release store of the step's sequence number, waits
// (bounded) for the others, picks the global maximum (lowest index among equals), appends it to
// the history and advances the step counters, the epoch included.  One CTA.
__global__ void __launch_bounds__(1024)
argmax_exchange_kernel(CommPeers peers, int rank, int world, int n, const __half* __restrict__ logits,
                       int vocab, long long offset, unsigned int* __restrict__ epoch,
                       long long* __restrict__ tok, long long* __restrict__ pos,
                       long long* __restrict__ len, long long* __restrict__ history,
                       long long* __restrict__ hist_count, int hist_cap) {
    pdl_prologue();
    PDL_FRESH(logits); PDL_FRESH(epoch); PDL_FRESH(tok); PDL_FRESH(pos); PDL_FRESH(len); PDL_FRESH(history);
    PDL_FRESH(hist_count);
    __shared__ float s_v[32];
    __shared__ int s_i[32];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = t; i < vocab; i += 1024) {
        const float v = __half2float(logits[i]);
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { s_v[warp] = best; s_i[warp] = bi; }
    __syncthreads();
    if (warp != 0) return;
    best = s_v[lane];
    bi = s_i[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (bi == 0x7fffffff) bi = 0;
    const long long tail = nvfp4_comm_tail_offset(n);
    unsigned char* mine = peers.buf[rank];
    uint32_t* err = reinterpret_cast<uint32_t*>(mine) + 1;
    const uint32_t seq = *epoch + 1u;
    // lane r hands this rank's pair to rank r (its own copy included) and then waits for rank r's
    if (lane < world) {
        unsigned char* dst = peers.buf[lane] + tail;
        float2* pair = reinterpret_cast<float2*>(dst + NVFP4_TAIL_CAND_OFF) + (seq & 1u) * 8u + rank;
        const float2 mine_pair = make_float2(best, __int_as_float((int)(offset + bi)));
        asm volatile("st.relaxed.sys.global.v2.f32 [%0], {%1, %2};\n" ::"l"(pair), "f"(mine_pair.x),
                     "f"(mine_pair.y) : "memory");
        __threadfence_system();
        st_release_sys_u32(reinterpret_cast<uint32_t*>(dst + NVFP4_TAIL_CAND_FLAGS_OFF) + rank, seq);
        const uint32_t* flag =
            reinterpret_cast<const uint32_t*>(mine + tail + NVFP4_TAIL_CAND_FLAGS_OFF) + lane;
        uint32_t spins = 0;
        while ((int32_t)(ld_acquire_sys_u32(flag) - seq) < 0) {
            if (++spins > NVFP4_COMM_SPIN_LIMIT) {
                atomicExch(err, 301u + (uint32_t)lane);
                break;
            }
        }
    }
    __syncwarp();
    if (lane == 0) {
        float gb = -INFINITY;
        long long gi = 0;
        for (int r = 0; r < world; r++) {
            float2 pr;
            const float2* src =
                reinterpret_cast<const float2*>(mine + tail + NVFP4_TAIL_CAND_OFF) + (seq & 1u) * 8u + r;
            asm volatile("ld.relaxed.sys.global.v2.f32 {%0, %1}, [%2];\n"
                         : "=f"(pr.x), "=f"(pr.y) : "l"(src) : "memory");
            const long long i = (long long)__float_as_int(pr.y);
            if (pr.x > gb || (pr.x == gb && i < gi) || r == 0) { gb = pr.x; gi = i; }
        }
        *tok = gi;
        if (history && hist_count) {
            const long long c = *hist_count;
            if (c < hist_cap) history[c] = gi;
            *hist_count = c + 1;
        }
        if (pos) *pos += 1;
        if (len) *len += 1;
        *epoch = seq;
    }
}

}  // namespace nvfp4

extern "C" {

// Bytes a communication buffer for vectors of n fp16 elements needs.
long long nvfp4_comm_buffer_bytes(int n) {
    if (n <= 0 || n % 8 != 0) return -1;
    // header + pull area data[2][n] + push area data[2][8][n] (launch_nvfp4_gemv_allreduce) + tail
    return nvfp4_comm_tail_offset(n) + NVFP4_TAIL_BYTES;
}

// Byte offset of data slot `parity` (0 or 1): where the producing GEMV writes its partial vector.
long long nvfp4_comm_data_offset(int n, int parity) {
    return NVFP4_COMM_DATA_OFF + (long long)(parity & 1) * n * 2;
}

// Zero a freshly allocated buffer (counter, error word, flags, data).  Synchronous.
int nvfp4_comm_init(void* buf, int n) {
    const long long bytes = nvfp4_comm_buffer_bytes(n);
    if (!buf || bytes < 0) return -1;
    if (cudaMemset(buf, 0, (size_t)bytes) != cudaSuccess) return -1;
    return cudaDeviceSynchronize() == cudaSuccess ? 0 : -1;
}

// CUDA IPC: export a cudaMalloc'ed buffer (64-byte handle) / map a peer's buffer here.
int nvfp4_ipc_get_handle(void* dev_ptr, void* handle_out) {
    cudaIpcMemHandle_t hdl;
    if (!dev_ptr || !handle_out) return -1;
    const cudaError_t e = cudaIpcGetMemHandle(&hdl, dev_ptr);
    if (e != cudaSuccess) {
        fprintf(stderr, "nvfp4_ipc_get_handle: %s\n", cudaGetErrorString(e));
        return -1;
    }
    static_assert(sizeof(hdl) == 64, "handle size");
    memcpy(handle_out, &hdl, sizeof(hdl));
    return 0;
}

void* nvfp4_ipc_open_handle(const void* handle) {
    cudaIpcMemHandle_t hdl;
    void* p = nullptr;
    if (!handle) return nullptr;
    memcpy(&hdl, handle, sizeof(hdl));
    const cudaError_t e = cudaIpcOpenMemHandle(&p, hdl, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        fprintf(stderr, "nvfp4_ipc_open_handle: %s\n", cudaGetErrorString(e));
        cudaGetLastError();
        return nullptr;
    }
    return p;
}

int nvfp4_ipc_close_handle(void* p) {
    return (p && cudaIpcCloseMemHandle(p) == cudaSuccess) ? 0 : -1;
}

// Error word of this rank's buffer: 0 = every wait so far was answered; 1 + r = peer r did not
// arrive within the spin limit at some call.  Synchronous (copies 4 bytes to the host).
int nvfp4_comm_status(const void* my_buf) {
    uint32_t v = 0;
    if (!my_buf) return -1;
    if (cudaMemcpy(&v, (const unsigned char*)my_buf + 4, 4, cudaMemcpyDeviceToHost) != cudaSuccess)
        return -1;
    return (int)v;
}

// h[n] (fp16) += f16( sum over ranks of the partial vectors in data slot `parity` ).
// bufs: HOST array of `world` device pointers, entry r = rank r's communication buffer as mapped
// in this process (entry `rank` is this rank's own allocation).  world <= 8, n % 8 == 0.
// Every rank of the group must make the same sequence of calls.  0; -1 bad arguments / launch.
int launch_allreduce_residual(void* h, const void* const* bufs, int rank, int world, int n,
                              int parity, void* stream) {
    if (!h || !bufs || world < 1 || world > NVFP4_COMM_MAX_RANKS || rank < 0 || rank >= world ||
        n <= 0 || n % 8 != 0)
        return -1;
    nvfp4::CommPeers peers;
    for (int r = 0; r < NVFP4_COMM_MAX_RANKS; r++)
        peers.buf[r] = (r < world) ? (unsigned char*)bufs[r] : nullptr;
    for (int r = 0; r < world; r++)
        if (!peers.buf[r]) return -1;
    int threads = (n / 8 + 31) / 32 * 32;
    if (threads > 1024) threads = 1024;
    if (threads < 32) threads = 32;
    return nvfp4::launch_pdl(nvfp4::allreduce_residual_kernel, dim3(1), dim3(threads), 0,
                             (cudaStream_t)stream, peers, rank, world, n, parity & 1, (__half*)h) ==
                   cudaSuccess ? 0 : -1;
}


// Tensor-parallel greedy pick in one launch (see argmax_exchange_kernel): logits fp16 [vocab] is
// this rank's vocabulary slice starting at global index `offset`; epoch is a device u32 that
// counts decode steps on this rank (every rank advances it in step; it also numbers the
// all-reduces that run inside launch_nvfp4_gemv_fused_ar).  No counterpart in the reference.
// 0; -1 bad arguments or launch error.
int launch_argmax_exchange(const void* logits, int vocab, long long offset,
                           const void* const* bufs, int rank, int world, int n, void* epoch,
                           void* tok, void* pos, void* len, void* history, void* hist_count,
                           int hist_cap, void* stream) {
    if (!logits || !bufs || !epoch || !tok || vocab <= 0 || offset < 0 || world < 1 ||
        world > NVFP4_COMM_MAX_RANKS || rank < 0 || rank >= world || n <= 0 || n % 8 != 0)
        return -1;
    nvfp4::CommPeers peers;
    for (int r = 0; r < NVFP4_COMM_MAX_RANKS; r++)
        peers.buf[r] = (r < world) ? (unsigned char*)bufs[r] : nullptr;
    for (int r = 0; r < world; r++)
        if (!peers.buf[r]) return -1;
    return nvfp4::launch_pdl(nvfp4::argmax_exchange_kernel, dim3(1), dim3(1024), 0,
                             (cudaStream_t)stream, peers, rank, world, n, (const __half*)logits,
                             vocab, offset, (unsigned int*)epoch, (long long*)tok, (long long*)pos,
                             (long long*)len, (long long*)history, (long long*)hist_count,
                             hist_cap) == cudaSuccess ? 0 : -1;
}

}  // extern "C"
