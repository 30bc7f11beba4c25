// All-gather over peer memory: every rank pushes its block into slot `rank` of the same buffer on every GPU of the group
// with plain vector stores over NVLink, raises an epoch flag on each of them, and returns once every peer's flag for this
// exchange has arrived. It replaces the small NCCL collectives of the latent-row split (halo rows, GroupNorm sums, K/V
// shards), whose cost is launch and protocol latency, not bandwidth.
//
// The buffers live in one arena per rank, allocated with cudaMalloc and mapped into the other processes through CUDA IPC
// handles (no multicast object, no TMA, no NVLS). Layout of an arena: [0, 4096) control words, then the gather buffers at
// offsets the host hands out identically on every rank. Control words (uint32): [0] exchange counter of this rank,
// [1] ticket of the CTA that finishes last, [2] status (non-zero: a bounded wait gave up), [64 + s] the epoch flag that
// rank s raises here. Every rank issues the same sequence of exchanges, so the exchange counter is the same number on all
// of them; a rank can run at most one exchange ahead of the slowest one, and an exchange never reuses the buffer of the
// previous one, so a buffer is rewritten only a whole step after it was read.
//
// Every wait is bounded; on a time-out the status word is set and the kernel returns.
#include "common.cuh"
#include "katz_b200.h"

namespace katz {

constexpr int PEER_MAX_RANKS = 8;
constexpr int PEER_CTRL_BYTES = 4096;
constexpr unsigned int PEER_WAIT_LIMIT = 1u << 21;      // polls of roughly a microsecond each: a second or two

struct PeerArgs {
    unsigned long long base[PEER_MAX_RANKS];      // arena of every rank as mapped in THIS process
    int rank, world;
};

// The block is `rows` rows of `row16` 16-byte vectors, `pitch16` vectors apart in the source (a column slice of a wider
// tensor is pushed without being made contiguous first); it lands packed.
// wait = 0: push and raise the flags only; whoever consumes the gathered buffer waits for the peers' flags itself (the
// attention kernel does, chunk by chunk, so that the transfer of the remote K/V shards overlaps its work on the local one).
__global__ void __launch_bounds__(256) peer_allgather_kernel(const uint4* __restrict__ src, long long n16, int row16,
                                                             long long pitch16, long long dst_off, PeerArgs a, int wait) {
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    pdl_launch_dependents();
    const long long slot = dst_off + (long long)a.rank * n16 * 16;
    // (row, column) of the source walk along with i: no division per 16-byte vector
    const long long step = (long long)gridDim.x * blockDim.x;
    const long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long step_r = step / row16;
    const int step_c = (int)(step - step_r * row16);
    long long r = i0 / row16;
    int c = (int)(i0 - r * row16);
    for (long long i = i0; i < n16; i += step) {
        const uint4 v = src[r * pitch16 + c];
#pragma unroll 1
        for (int p = 0; p < a.world; ++p) reinterpret_cast<uint4*>(a.base[p] + slot)[i] = v;
        r += step_r;
        c += step_c;
        if (c >= row16) {
            c -= row16;
            ++r;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x != 0) return;
    unsigned int* ctrl = reinterpret_cast<unsigned int*>(a.base[a.rank]);
    if (atomicInc(ctrl + 1, gridDim.x - 1) != gridDim.x - 1) return;      // the ticket wraps to zero by itself
    // last CTA: every store of this rank has been issued and fenced
    __threadfence_system();
    const unsigned int epoch = ctrl[0] + 1;
    ctrl[0] = epoch;
    for (int p = 0; p < a.world; ++p) {
        unsigned int* flag = reinterpret_cast<unsigned int*>(a.base[p]) + 64 + a.rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(epoch) : "memory");
    }
    if (!wait) return;
    for (int s = 0; s < a.world; ++s) {
        const unsigned int* flag = ctrl + 64 + s;
        unsigned int polls = 0;
        for (;;) {
            unsigned int v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
            if ((int)(v - epoch) >= 0) break;
            if (++polls > PEER_WAIT_LIMIT) {
                atomicExch(ctrl + 2, 100u + (unsigned int)s);
                return;
            }
            __nanosleep(64);
        }
    }
}

}  // namespace katz

using namespace katz;

extern "C" int katz_peer_ctrl_bytes(void) { return PEER_CTRL_BYTES; }

extern "C" int katz_peer_arena_alloc(long long bytes, void** ptr) {
    KATZ_CHECK_ARG(ptr, KATZ_EINVAL);
    KATZ_CHECK_ARG(bytes > PEER_CTRL_BYTES, KATZ_ESIZE);
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, (size_t)bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();      // a failed allocation is the caller's to handle: do not leave it for the next launch check
        return (int)e;
    }
    e = cudaMemset(p, 0, PEER_CTRL_BYTES);
    if (e != cudaSuccess) return (int)e;
    *ptr = p;
    return KATZ_OK;
}

extern "C" int katz_peer_arena_free(void* ptr) {
    KATZ_CHECK_ARG(ptr, KATZ_EINVAL);
    cudaError_t e = cudaFree(ptr);
    return e == cudaSuccess ? KATZ_OK : (int)e;
}

extern "C" int katz_peer_ipc_handle_bytes(void) { return (int)sizeof(cudaIpcMemHandle_t); }

extern "C" int katz_peer_ipc_export(void* ptr, void* handle_out) {
    KATZ_CHECK_ARG(ptr && handle_out, KATZ_EINVAL);
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return (int)e;
    }
    memcpy(handle_out, &h, sizeof(h));
    return KATZ_OK;
}

extern "C" int katz_peer_ipc_open(const void* handle, void** ptr) {
    KATZ_CHECK_ARG(handle && ptr, KATZ_EINVAL);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return (int)e;
    }
    *ptr = p;
    return KATZ_OK;
}

extern "C" int katz_peer_ipc_close(void* ptr) {
    KATZ_CHECK_ARG(ptr, KATZ_EINVAL);
    cudaError_t e = cudaIpcCloseMemHandle(ptr);
    return e == cudaSuccess ? KATZ_OK : (int)e;
}

static int peer_allgather_launch(const void* src, long long rows, long long row_bytes, long long src_pitch_bytes,
                                 long long dst_off, const unsigned long long* h_bases, int rank, int world, int wait,
                                 void* stream) {
    KATZ_CHECK_ARG(src && h_bases, KATZ_EINVAL);
    KATZ_CHECK_ARG(world >= 1 && world <= PEER_MAX_RANKS && rank >= 0 && rank < world, KATZ_ESIZE);
    KATZ_CHECK_ARG(rows > 0 && row_bytes > 0 && row_bytes % 16 == 0 && row_bytes < (1ll << 34) && src_pitch_bytes >= row_bytes &&
                       src_pitch_bytes % 16 == 0,
                   KATZ_ESIZE);
    KATZ_CHECK_ARG(dst_off >= PEER_CTRL_BYTES && dst_off % 16 == 0, KATZ_ESIZE);
    KATZ_CHECK_ARG(aligned16(src), KATZ_EALIGN);
    const long long bytes = rows * row_bytes;
    PeerArgs a{};
    for (int p = 0; p < world; ++p) {
        KATZ_CHECK_ARG(h_bases[p] != 0 && (h_bases[p] & 255) == 0, KATZ_EALIGN);
        a.base[p] = h_bases[p];
    }
    a.rank = rank;
    a.world = world;
    const long long n16 = bytes / 16;
    long long ctas = (n16 + 1023) / 1024;      // four vectors per thread
    if (ctas > 64) ctas = 64;
    if (ctas < 1) ctas = 1;
    launch_k(peer_allgather_kernel, dim3((unsigned)ctas), dim3(256), 0, (cudaStream_t)stream, (const uint4*)src, n16,
             (int)(row_bytes / 16), src_pitch_bytes / 16, dst_off, a, wait);
    KATZ_LAUNCH_RET();
}

extern "C" int katz_peer_allgather(const void* src, long long rows, long long row_bytes, long long src_pitch_bytes,
                                   long long dst_off, const unsigned long long* h_bases, int rank, int world, void* stream) {
    return peer_allgather_launch(src, rows, row_bytes, src_pitch_bytes, dst_off, h_bases, rank, world, 1, stream);
}

extern "C" int katz_peer_push(const void* src, long long rows, long long row_bytes, long long src_pitch_bytes, long long dst_off,
                              const unsigned long long* h_bases, int rank, int world, void* stream) {
    return peer_allgather_launch(src, rows, row_bytes, src_pitch_bytes, dst_off, h_bases, rank, world, 0, stream);
}

// Back to zero (after a warm-up in which the ranks were not yet in step, say). Synchronous.
extern "C" int katz_peer_clear_status(void* arena) {
    KATZ_CHECK_ARG(arena, KATZ_EINVAL);
    cudaError_t e = cudaMemset(reinterpret_cast<unsigned int*>(arena) + 2, 0, sizeof(unsigned int));
    return e == cudaSuccess ? 0 : (int)e;
}

extern "C" int katz_peer_status(const void* arena) {
    KATZ_CHECK_ARG(arena, KATZ_EINVAL);
    unsigned int v = 0;
    cudaError_t e = cudaMemcpy(&v, reinterpret_cast<const unsigned int*>(arena) + 2, sizeof(v), cudaMemcpyDeviceToHost);
    return e == cudaSuccess ? (int)v : -1;
}
