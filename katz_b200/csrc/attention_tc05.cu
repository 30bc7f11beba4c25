// Flash-style attention on the tcgen05 tensor path: head_dim 64, fp16 in/out, fp32 softmax, no mask, non-causal.
// Replaces F.scaled_dot_product_attention as called by AttnProcessor2_0
// (diffusers/models/attention_processor.py:1276): softmax(Q K^T / sqrt(64)) V per (batch, head).
//
// One CTA owns 128 query rows of one (batch, head) and walks the keys in tiles of 128. The softmax is bound by the
// special-function unit (one exp2 per score) and by the softmax warps' own instruction stream, and a single CTA leaves
// both idle while its four softmax warps wait for TMEM loads, barriers and the row maximum; so the CTA is sized for TWO
// per SM (80 KB of shared memory, 256 TMEM columns, 168 registers) and the hardware interleaves the two:
//   * warp 0, one elected thread: TMA loads of Q (once) and of the K and V tiles into 2-stage rings (128-byte swizzle;
//     Q/K/V are read in place from the [B, S, ld] projection outputs, head h = columns [64h, 64h+64));
//   * warp 1, one elected thread: S = Q K^T (tcgen05.mma, 128x128x64, K-major operands) into a TMEM accumulator that
//     the softmax frees as soon as the scores sit in registers, then O += P V (128x64x128; V is the MN-major operand
//     in shared memory, P is the A operand read from TENSOR MEMORY: it never crosses shared memory, whose bandwidth the
//     two MMAs' K, V and Q reads and the TMA fills already use) into a second accumulator;
//   * warps 2-5: softmax. A thread owns one query row (= one TMEM lane), so row maxima and sums need no shuffles. It
//     reads S with tcgen05.ld, keeps a running reference maximum that is only raised when the tile maximum exceeds it
//     by more than 2^8 (so the O accumulator is rescaled rarely: tcgen05.ld / scale / tcgen05.st), writes
//     P = exp2(S*scale - m) as fp16 pairs into its lane of the P columns of tensor memory (tcgen05.st) for the second
//     MMA, and at the end normalises O.
// S[j+1] = Q K[j+1]^T is issued before the softmax of tile j has finished, so the two MMAs and the softmax overlap.
// Every mbarrier wait is bounded; a time-out records a status word (shared with the GEMM kernels) and the CTA unwinds.
//
// Wave tail (katz_attention_split_f16): an SM holds two CTAs, so a launch fills 2 x SMs slots at a time and the query
// tiles beyond a whole number of rounds (640 tiles on 296 slots: 48) run as a last round that costs as much as a full
// one. With scratch memory, long tiles (16 key tiles or more) are cut along the KEY axis into `parts` short CTAs, dispatched first;
// each writes its unnormalised O (fp32), its reference maximum and its row sum to scratch, and the last part of a tile
// to arrive (a ticket, no waiting) adds the parts in index order, so the result does not depend on which one that was.
#include "tc05.cuh"
#include "katz_b200.h"

namespace katz {

using namespace tc05;

constexpr int FA_BM = 128, FA_BN = 128, FA_D = 64, FA_ST = 3;
constexpr int FA_CTAS_PER_SM = 2;
constexpr int FA_THREADS = 192;
constexpr int FA_TILE = 128 * 128;                     // bytes of a 128-row x 64-half tile (Q; one 64-key sub-tile of P)
constexpr int FA_KV_TILE = FA_BN * 128;                // bytes of a key or value tile
constexpr int FA_TMEM_COLS = 256;                      // S at columns 0..127, O at 128..191, P (fp16 pairs) at 192..255
constexpr int FA_SMEM = FA_TILE + 2 * FA_ST * FA_KV_TILE + 256;     // Q, K ring, V ring, barriers
static_assert(FA_CTAS_PER_SM * (FA_SMEM + 1024) <= 228 * 1024, "the CTAs of one SM must fit its shared memory");
static_assert(FA_CTAS_PER_SM * FA_TMEM_COLS <= 512, "and its tensor memory");
constexpr float FA_RESCALE_THRESHOLD = 8.0f;           // log2 units
constexpr uint32_t FA_PEER_WAIT_LIMIT = 1u << 19;      // polls of about two microseconds: a second or so

int* tc05_status_device_ptr();   // defined next to the status word (gemm_tc05.cu)

struct FaParams {
    __half* O;
    int Sq, Sk, ldo;
    long long bso;
    float scale_log2e;
    int kv_chunk_rows;
    int* status;
    // work decoding: blockIdx.x -> (query tile, key-tile range). Query tiles are numbered x fastest, then head, then batch.
    int tiles_x, H;
    int n_full;                 // query tiles [0, n_full) are whole CTAs
    int n_small, parts;         // query tiles [n_full, n_full + n_small / parts) are cut into `parts` CTAs each
    int* counters;              // one ticket per cut query tile, zero between launches
    float2* part_ml;            // [cut tile][part][row]: (reference maximum in log2 units, row sum)
    float4* part_o;             // [cut tile][part][16 column quads][128 rows]: unnormalised O
    // K/V chunks that peers push into this GPU's memory (latent-row split): the control words of this rank's peer arena
    // ([0]: number of the exchange that delivered them, [64 + r]: the last exchange whose block from rank r has landed),
    // this rank's own chunk, and the number of chunks. NULL: every chunk is there when the kernel starts.
    const unsigned int* peer_ctrl;
    int self_chunk, n_chunks;
};

__device__ __forceinline__ void tma_load_4d_fa(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar) {
    tma_load_4d(dst, map, c0, c1, c2, c3, bar);
}
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
        "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: the A operand (here P, fp16, two consecutive keys per 32-bit column, lane = row) is read
// from tensor memory, so it never crosses shared memory.
__device__ __forceinline__ void umma_f16_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// kind::f16 instruction descriptor with an MN-major B operand (bit 16)
__host__ __device__ constexpr uint32_t idesc_f16_bmn(int M, int N) { return idesc_f16(M, N) | (1u << 16); }

__global__ void __launch_bounds__(FA_THREADS, FA_CTAS_PER_SM) attention_tc05_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                                       const __grid_constant__ CUtensorMap tmK,
                                                                       const __grid_constant__ CUtensorMap tmV, const FaParams p) {
    // the 128-byte swizzle wants 1024-byte aligned tiles; there is no room for alignment slack when two CTAs share an
    // SM, so the alignment is requested from the compiler and checked
    extern __shared__ __align__(1024) unsigned char smem[];
    if ((smem_u32(smem) & 1023u) != 0) {
        if (threadIdx.x == 0) atomicExch(p.status, 10);
        return;
    }
    const uint32_t sQ = smem_u32(smem);
    const uint32_t sK0 = sQ + FA_TILE, sV0 = sK0 + FA_ST * FA_KV_TILE;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + FA_TILE + 2 * FA_ST * FA_KV_TILE);
    // barrier map
    const uint32_t b0 = smem_u32(bars);
    const uint32_t q_full = b0, k_full = b0 + 8, k_empty = k_full + 8 * FA_ST, v_full = k_empty + 8 * FA_ST,
                   v_empty = v_full + 8 * FA_ST, s_full = v_empty + 8 * FA_ST, s_free = s_full + 8, p_full = s_free + 8,
                   p_free = p_full + 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 1 + 4 * FA_ST + 4);
    volatile int* ticket_slot = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int NT_ALL = (p.Sk + FA_BN - 1) / FA_BN;
    // the short CTAs come first in the grid: they are dispatched first and the whole-tile CTAs fill in behind them
    int qt, j0 = 0, j1 = NT_ALL, part = 0, cut = -1;
    if ((int)blockIdx.x < p.n_small) {
        cut = (int)blockIdx.x / p.parts;
        part = (int)blockIdx.x - cut * p.parts;
        qt = p.n_full + cut;
        j0 = (int)((long long)part * NT_ALL / p.parts);
        j1 = (int)((long long)(part + 1) * NT_ALL / p.parts);
    } else {
        qt = (int)blockIdx.x - p.n_small;
    }
    const int qx = qt % p.tiles_x, hb = qt / p.tiles_x;
    const int q0 = qx * FA_BM, h = hb % p.H, b = hb / p.H;
    const int NT = j1 - j0;      // key tiles of this CTA: j0 .. j1-1

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        mbar_init(q_full, 1);
        for (int s = 0; s < FA_ST; ++s) {
            mbar_init(k_full + 8 * s, 1);
            mbar_init(k_empty + 8 * s, 1);
            mbar_init(v_full + 8 * s, 1);
            mbar_init(v_empty + 8 * s, 1);
        }
        mbar_init(s_full, 1);
        mbar_init(s_free, 4);
        mbar_init(p_full, 4);
        mbar_init(p_free, 1);
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), FA_TMEM_COLS);
        tmem_relinquish();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // Everything above (barriers, TMEM, descriptor prefetch) may overlap the previous kernel's tail: the producer and the
    // softmax warps call pdl_wait() themselves before their first global-memory access (the MMA thread touches none).
    const uint32_t tS0 = tmem_base, tO = tmem_base + FA_BN, tP = tO + FA_D;      // S | O | P

    if (warp == 0) {
        // ------------------------------------------------------------------------------------ TMA producer
        if (elect_one()) {
            bool ok = true;
            pdl_wait();
            pdl_launch_dependents();
            mbar_expect_tx(q_full, FA_TILE);
            tma_load_4d_fa(sQ, &tmQ, h * FA_D, q0, b, 0, q_full);
            // Peer mode: the chunks are walked starting with this rank's own shard, and the first tile of every other chunk
            // waits (bounded) for that rank's flag: its K/V cross NVLink while the tiles before it are being worked on.
            unsigned int epoch = 0;
            int landed = p.self_chunk;
            if (p.peer_ctrl) epoch = *reinterpret_cast<const volatile unsigned int*>(p.peer_ctrl);
            for (int j = 0; j < NT && ok; ++j) {
                const int s = j % FA_ST;
                const uint32_t ph = (j / FA_ST) & 1;
                const int key0 = (j0 + j) * FA_BN;
                int chunk = key0 / p.kv_chunk_rows;
                const int row = key0 - chunk * p.kv_chunk_rows;
                if (p.peer_ctrl) {
                    chunk += p.self_chunk;
                    if (chunk >= p.n_chunks) chunk -= p.n_chunks;
                    if (chunk != landed) {
                        const unsigned int* flag = p.peer_ctrl + 64 + chunk;
                        bool there = false;
                        for (uint32_t polls = 0; polls < FA_PEER_WAIT_LIMIT; ++polls) {
                            unsigned int v;
                            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
                            if ((int)(v - epoch) >= 0) {
                                there = true;
                                break;
                            }
                            __nanosleep(64);
                        }
                        // a chunk that never came: the status word voids the result, and the loads go ahead on whatever the
                        // buffer holds, so that the other roles finish at once instead of running out their own waits
                        if (!there) atomicExch(p.status, 14);
                        asm volatile("fence.proxy.async;" ::: "memory");      // the TMA loads below read what the peer wrote
                        landed = chunk;
                    }
                }
                if (!mbar_wait(k_empty + 8 * s, ph ^ 1)) { ok = false; break; }
                mbar_expect_tx(k_full + 8 * s, FA_KV_TILE);
                tma_load_4d_fa(sK0 + s * FA_KV_TILE, &tmK, h * FA_D, row, b, chunk, k_full + 8 * s);
                if (!mbar_wait(v_empty + 8 * s, ph ^ 1)) { ok = false; break; }
                mbar_expect_tx(v_full + 8 * s, FA_KV_TILE);
                tma_load_4d_fa(sV0 + s * FA_KV_TILE, &tmV, h * FA_D, row, b, chunk, v_full + 8 * s);
            }
            if (!ok) atomicCAS(p.status, 0, 11);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            constexpr uint32_t idesc_qk = idesc_f16(FA_BM, FA_BN);
            constexpr uint32_t idesc_pv = idesc_f16_bmn(FA_BM, FA_D);
            pdl_wait();      // the bounded waits below must not count polls while the producer still waits for the dependency
            bool ok = mbar_wait(q_full, 0);
            auto issue_qk = [&](int j) -> bool {
                const int s = j % FA_ST;
                if (!mbar_wait(k_full + 8 * s, (j / FA_ST) & 1)) return false;
                if (!mbar_wait(s_free, (j & 1) ^ 1)) return false;       // the softmax holds tile j-1's scores in registers
                fence_after_sync();
                const uint64_t ad = smem_desc_sw128(sQ), bd = smem_desc_sw128(sK0 + s * FA_KV_TILE);
#pragma unroll
                for (int k = 0; k < FA_D / 16; ++k) umma_f16(tS0, ad + 2 * k, bd + 2 * k, idesc_qk, k != 0);
                umma_commit(s_full);
                umma_commit(k_empty + 8 * s);
                return true;
            };
            if (ok) ok = issue_qk(0);
            for (int j = 0; j < NT && ok; ++j) {
                if (j + 1 < NT) {
                    ok = issue_qk(j + 1);
                    if (!ok) break;
                }
                const int s = j % FA_ST;
                if (!mbar_wait(p_full, j & 1)) { ok = false; break; }
                if (!mbar_wait(v_full + 8 * s, (j / FA_ST) & 1)) { ok = false; break; }
                fence_after_sync();
                const uint32_t va = sV0 + s * FA_KV_TILE;
#pragma unroll
                for (int k = 0; k < FA_BN / 16; ++k) {
                    // A = P from tensor memory: 16 keys per step = 8 columns of fp16 pairs.
                    // B = V (MN-major): 16 key rows per step = two 8-row swizzle groups = 2048 B.
                    const uint64_t bd = smem_desc_sw128(va + k * 2048);
                    umma_f16_ta(tO, tP + 8 * k, bd, idesc_pv, (j | k) != 0);
                }
                umma_commit(v_empty + 8 * s);
                umma_commit(p_free);
            }
            if (!ok) atomicExch(p.status, 12);
        }
    } else {
        // ------------------------------------------------------------------------------------ softmax, one row per thread
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const uint32_t lane_base = (uint32_t)(q * 32) << 16;
        float m_used = -INFINITY, l_sum = 0.f;
        bool ok = true;
        pdl_wait();      // O is written at the end; nothing of this kernel may reach global memory before the previous one is done
        for (int j = 0; j < NT; ++j) {
            ok = mbar_wait(s_full, j & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            fence_after_sync();
            const uint32_t tS = tS0 + lane_base;
            const int kbase = (j0 + j) * FA_BN;
            const bool tail = kbase + FA_BN > p.Sk;
            // the whole S row (128 fp32) comes into registers with ONE wait: four TMEM loads in flight together
            uint32_t r[FA_BN];
#pragma unroll
            for (int c = 0; c < FA_BN; c += 32) tmem_ld_32x32(tS + c, r + c);
            tmem_ld_wait();
            // S is in registers: the accumulator buffer can take the next Q K^T already
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(s_free);
            if (tail) {
#pragma unroll
                for (int e = 0; e < FA_BN; ++e)
                    if (kbase + e >= p.Sk) r[e] = __float_as_uint(-INFINITY);
            }
            // row maximum with four independent chains
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int e = 0; e < FA_BN; e += 4) {
#pragma unroll
                for (int u = 0; u < 4; ++u) mx4[u] = fmaxf(mx4[u], __uint_as_float(r[e + u]));
            }
            float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            mx *= p.scale_log2e;                             // the scale is positive: max commutes with it
            // raise the reference maximum only when it is far too low; O and l are rescaled then
            const bool raise = mx > m_used + FA_RESCALE_THRESHOLD;
            const float m_new = raise ? mx : m_used;
            const float corr = (raise && j > 0) ? exp2f(m_used - m_new) : 1.0f;
            if (j > 0 && __any_sync(0xffffffffu, raise)) {
                // O is about to be rescaled: O += P V of tile j-1 must have landed. That MMA signals p_free; this thread
                // last observed that barrier one phase back (at tile j-1, for tile j-2), so the parity wait is
                // unambiguous. The same wait below (P free for writing) then passes at once.
                ok = mbar_wait(p_free, (j - 1) & 1);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                fence_after_sync();
#pragma unroll 1
                for (int c = 0; c < FA_D; c += 32) {
                    uint32_t r[32];
                    tmem_ld_32x32(tO + lane_base + c, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * corr);
                    tmem_st_32x32(tO + lane_base + c, r);
                }
                tmem_st_wait();
                fence_before_sync();
            }
            l_sum *= corr;
            m_used = m_new;
            // P free? (the P V MMA of tile j-1 has finished reading it; it was issued while this tile's scores were loaded)
            ok = mbar_wait(p_free, (j & 1) ^ 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            // P = exp2(S*scale - m) (masked keys hold -inf -> 0), row sum on four chains, fp16 pairs into this row's lane of the
            // P columns of tensor memory (keys 2c, 2c+1 in column c)
            float ls4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < FA_BN; c += 32) {
                uint32_t pk[16];
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    const float p0 = ex2_approx(fmaf(__uint_as_float(r[c + e]), p.scale_log2e, -m_used));
                    const float p1 = ex2_approx(fmaf(__uint_as_float(r[c + e + 1]), p.scale_log2e, -m_used));
                    ls4[(e >> 1) & 3] += p0 + p1;
                    pk[e >> 1] = pack_half2(p0, p1);
                }
                tmem_st_32x16(tP + lane_base + (c >> 1), pk);
            }
            l_sum += (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
            // P has landed in tensor memory; then signal
            tmem_st_wait();
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
        }
        if (ok) {
            ok = mbar_wait(p_free, (NT - 1) & 1);     // the last O += P V has landed
            ok = __all_sync(0xffffffffu, ok);
        }
        if (!ok && lane == 0) atomicExch(p.status, 13);
        const int qrow = q0 + row;
        __half* op = p.O + (size_t)b * p.bso + (size_t)qrow * p.ldo + h * FA_D;
        if (cut < 0) {
            if (ok) {
                fence_after_sync();
                const float inv = 1.0f / l_sum;
#pragma unroll 1
                for (int c = 0; c < FA_D; c += 32) {
                    uint32_t r[32];
                    tmem_ld_32x32(tO + lane_base + c, r);
                    tmem_ld_wait();
                    if (qrow < p.Sq) {
#pragma unroll
                        for (int k4 = 0; k4 < 4; ++k4) {
                            uint4 o;
                            o.x = pack_half2(__uint_as_float(r[8 * k4]) * inv, __uint_as_float(r[8 * k4 + 1]) * inv);
                            o.y = pack_half2(__uint_as_float(r[8 * k4 + 2]) * inv, __uint_as_float(r[8 * k4 + 3]) * inv);
                            o.z = pack_half2(__uint_as_float(r[8 * k4 + 4]) * inv, __uint_as_float(r[8 * k4 + 5]) * inv);
                            o.w = pack_half2(__uint_as_float(r[8 * k4 + 6]) * inv, __uint_as_float(r[8 * k4 + 7]) * inv);
                            *reinterpret_cast<uint4*>(op + c + 8 * k4) = o;
                        }
                    }
                }
            }
        } else {
            // One part of a cut query tile: leave (m, l, unnormalised O) in scratch, take a ticket, and if every other part
            // has arrived, add them up in index order. A part that timed out still takes its ticket (the status word
            // already says the result is void), so the counter returns to zero whatever happened.
            const size_t slot = (size_t)cut * p.parts;
            if (ok) {
                fence_after_sync();
                float4* so = p.part_o + (slot + part) * (16 * FA_BM);
#pragma unroll 1
                for (int c = 0; c < FA_D; c += 32) {
                    uint32_t r[32];
                    tmem_ld_32x32(tO + lane_base + c, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int k4 = 0; k4 < 8; ++k4)      // quad-major: the 32 rows of a warp write 512 contiguous bytes
                        so[(c / 4 + k4) * FA_BM + row] = make_float4(__uint_as_float(r[4 * k4]), __uint_as_float(r[4 * k4 + 1]),
                                                                    __uint_as_float(r[4 * k4 + 2]), __uint_as_float(r[4 * k4 + 3]));
                }
                p.part_ml[(slot + part) * FA_BM + row] = make_float2(m_used, l_sum);
            }
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");      // the four softmax warps
            if (threadIdx.x == 64) *ticket_slot = atomicAdd(p.counters + cut, 1);
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (*ticket_slot == p.parts - 1) {
                __threadfence();
                if (threadIdx.x == 64) p.counters[cut] = 0;      // every part has its ticket: ready for the next launch
                float M = -INFINITY;
                for (int pp = 0; pp < p.parts; ++pp) M = fmaxf(M, __ldcg(p.part_ml + (slot + pp) * FA_BM + row).x);
                float L = 0.f;
                for (int pp = 0; pp < p.parts; ++pp) {
                    const float2 ml = __ldcg(p.part_ml + (slot + pp) * FA_BM + row);
                    L = fmaf(exp2f(ml.x - M), ml.y, L);
                }
                const float inv = 1.0f / L;
#pragma unroll 1
                for (int c4 = 0; c4 < 16; c4 += 4) {
                    float4 acc[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int pp = 0; pp < p.parts; ++pp) {
                        const float w = exp2f(__ldcg(p.part_ml + (slot + pp) * FA_BM + row).x - M);
                        const float4* so = p.part_o + (slot + pp) * (16 * FA_BM);
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const float4 v = __ldcg(so + (c4 + u) * FA_BM + row);
                            acc[u].x = fmaf(w, v.x, acc[u].x);
                            acc[u].y = fmaf(w, v.y, acc[u].y);
                            acc[u].z = fmaf(w, v.z, acc[u].z);
                            acc[u].w = fmaf(w, v.w, acc[u].w);
                        }
                    }
                    if (qrow < p.Sq) {
#pragma unroll
                        for (int u = 0; u < 4; u += 2) {
                            uint4 o;
                            o.x = pack_half2(acc[u].x * inv, acc[u].y * inv);
                            o.y = pack_half2(acc[u].z * inv, acc[u].w * inv);
                            o.z = pack_half2(acc[u + 1].x * inv, acc[u + 1].y * inv);
                            o.w = pack_half2(acc[u + 1].z * inv, acc[u + 1].w * inv);
                            *reinterpret_cast<uint4*>(op + 4 * (c4 + u)) = o;
                        }
                    }
                }
            }
        }
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        fence_after_sync();
        tmem_dealloc(tmem_base, FA_TMEM_COLS);
    }
}

// ---- host side ---------------------------------------------------------------------------------------------------
typedef CUresult (*FaEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static FaEncodeFn fa_encode_fn() {
    static FaEncodeFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* f = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<FaEncodeFn>(f);
    }
    return fn;
}

// [chunks][B][rows][cols] view of a token-major buffer: box = 64 columns x 128 rows
static int fa_encode(CUtensorMap* map, const void* base, int cols, long long rows, int B, int chunks, long long ld,
                     long long bs, long long chunk_stride, int box_rows) {
    FaEncodeFn enc = fa_encode_fn();
    if (!enc) return KATZ_ENOTREADY;
    cuuint64_t dims[4] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)B, (cuuint64_t)chunks};
    cuuint64_t strides[3] = {(cuuint64_t)ld * 2, (cuuint64_t)bs * 2, (cuuint64_t)chunk_stride * 2};
    cuuint32_t box[4] = {(cuuint32_t)FA_D, (cuuint32_t)box_rows, 1, 1};
    cuuint32_t es[4] = {1, 1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), dims, strides, box, es,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : KATZ_EINVAL;
}

}  // namespace katz

using namespace katz;

// Slots of one dispatch round: two CTAs per SM.
static int fa_slots() {
    static int n = 0;
    if (!n) {
        int dev = 0, sms = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
        n = FA_CTAS_PER_SM * sms;
    }
    return n;
}
constexpr long long FA_COUNTER_BYTES = 4096;                                   // tickets of up to 1024 cut query tiles
constexpr long long FA_PART_BYTES = FA_BM * FA_D * 4 + FA_BM * 8;              // one part: O (fp32) + (m, l) per row

// Which query tiles are cut and into how many parts. Only the tiles beyond a whole number of dispatch rounds are cut
// (all of them when there is less than one round), into as many parts as fit the slots of one round. A part costs
// about as much as two or three key tiles beyond its own (its set-up, its partial result, its share of the final sum),
// so it must be at least four key tiles long, and query tiles of fewer than sixteen key tiles are never cut: measured at 8
// key tiles (2 x 20 heads x 1024 tokens), every cut was slower than the second round it replaced.
static void fa_plan(int n_q, int key_tiles, long long scratch_bytes, int* n_full, int* cut_tiles, int* parts) {
    *n_full = n_q;
    *cut_tiles = 0;
    *parts = 1;
    const int slots = fa_slots();
    const int rest = n_q % slots;
    if (rest == 0 || key_tiles < 16 || rest > 1024) return;
    int pt = slots / rest;
    if (pt > key_tiles / 4) pt = key_tiles / 4;
    if (pt > 16) pt = 16;
    if (pt < 2) return;
    if (FA_COUNTER_BYTES + (long long)rest * pt * FA_PART_BYTES > scratch_bytes) return;
    *n_full = n_q - rest;
    *cut_tiles = rest;
    *parts = pt;
}

static int attention_launch(const void* Q, const void* K, const void* V, void* O, int B, int H, int Sq, int Sk, int head_dim,
                            int ldq, int ldk, int ldv, int ldo, long long bsq, long long bsk, long long bsv, long long bso,
                            float scale, int kv_chunk_rows, long long kv_chunk_stride, void* scratch, long long scratch_bytes,
                            const void* peer_ctrl, int self_chunk, void* stream) {

    KATZ_CHECK_ARG(Q && K && V && O, KATZ_EINVAL);
    KATZ_CHECK_ARG(head_dim == 64, KATZ_ESIZE);
    KATZ_CHECK_ARG(B > 0 && H > 0 && Sq > 0 && Sk > 0 && B <= 65535 && H <= 65535, KATZ_ESIZE);
    KATZ_CHECK_ARG(ldq % 8 == 0 && ldk % 8 == 0 && ldv % 8 == 0 && ldo % 8 == 0, KATZ_EALIGN);
    KATZ_CHECK_ARG(bsq % 8 == 0 && bsk % 8 == 0 && bsv % 8 == 0 && bso % 8 == 0, KATZ_EALIGN);
    KATZ_CHECK_ARG(aligned16(Q) && aligned16(K) && aligned16(V) && aligned16(O), KATZ_EALIGN);
    KATZ_CHECK_ARG(ldq >= H * 64 && ldk >= H * 64 && ldv >= H * 64, KATZ_ESIZE);
    int chunks = 1;
    long long rows = Sk, cstride = 0;
    if (kv_chunk_rows > 0 && kv_chunk_rows < Sk) {
        KATZ_CHECK_ARG(kv_chunk_rows % FA_BN == 0 && Sk % kv_chunk_rows == 0 && kv_chunk_stride % 8 == 0 && kv_chunk_stride > 0,
                       KATZ_ESIZE);
        chunks = Sk / kv_chunk_rows;
        rows = kv_chunk_rows;
        cstride = kv_chunk_stride;
    } else {
        kv_chunk_rows = ((Sk + FA_BN - 1) / FA_BN) * FA_BN;
    }
    // strides of size-1 dimensions still have to be valid (non-zero multiples of 16 bytes)
    const long long bsq_e = B > 1 ? bsq : (long long)Sq * ldq, bsk_e = B > 1 ? bsk : rows * ldk, bsv_e = B > 1 ? bsv : rows * ldv;
    KATZ_CHECK_ARG(bsq_e > 0 && bsk_e > 0 && bsv_e > 0, KATZ_ESIZE);
    CUtensorMap tq, tk, tv;
    int rc = fa_encode(&tq, Q, H * 64, Sq, B, 1, ldq, bsq_e, bsq_e * B, FA_BM);
    if (rc) return rc;
    rc = fa_encode(&tk, K, H * 64, rows, B, chunks, ldk, bsk_e, chunks > 1 ? cstride : bsk_e * B, FA_BN);
    if (rc) return rc;
    rc = fa_encode(&tv, V, H * 64, rows, B, chunks, ldv, bsv_e, chunks > 1 ? cstride : bsv_e * B, FA_BN);
    if (rc) return rc;
    FaParams p{};
    p.O = (__half*)O; p.Sq = Sq; p.Sk = Sk; p.ldo = ldo; p.bso = bso;
    p.scale_log2e = scale * 1.44269504088896340736f;
    p.kv_chunk_rows = kv_chunk_rows;
    p.status = tc05_status_device_ptr();
    if (!p.status) return KATZ_ENOTREADY;
    static bool attr_dev[KATZ_MAX_DEVICES] = {false};
    bool& attr = attr_dev[current_device_index()];
    if (!attr) {
        cudaError_t e = cudaFuncSetAttribute(attention_tc05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FA_SMEM);
        if (e != cudaSuccess) return (int)e;
        // all of the SM's L1/shared storage as shared memory: two CTAs of this kernel per SM
        e = cudaFuncSetAttribute(attention_tc05_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return (int)e;
        attr = true;
    }
    p.tiles_x = (Sq + FA_BM - 1) / FA_BM;
    p.H = H;
    if (peer_ctrl) {
        KATZ_CHECK_ARG(chunks > 1 && self_chunk >= 0 && self_chunk < chunks && chunks <= 8 && ((uintptr_t)peer_ctrl & 3) == 0, KATZ_EINVAL);
        p.peer_ctrl = (const unsigned int*)peer_ctrl;
        p.self_chunk = self_chunk;
        p.n_chunks = chunks;
    }
    const long long n_q = (long long)p.tiles_x * H * B;
    KATZ_CHECK_ARG(n_q < (1ll << 30), KATZ_ESIZE);
    int cut_tiles = 0;
    fa_plan((int)n_q, (Sk + FA_BN - 1) / FA_BN, scratch ? scratch_bytes : 0, &p.n_full, &cut_tiles, &p.parts);
    p.n_small = cut_tiles * p.parts;
    if (cut_tiles) {
        unsigned char* sc = (unsigned char*)scratch;
        p.counters = (int*)sc;
        p.part_ml = (float2*)(sc + FA_COUNTER_BYTES);
        p.part_o = (float4*)(sc + FA_COUNTER_BYTES + (long long)cut_tiles * p.parts * FA_BM * 8);
    }
    dim3 grid((unsigned)(p.n_small + p.n_full));
    launch_k(attention_tc05_kernel, grid, FA_THREADS, FA_SMEM, (cudaStream_t)stream, tq, tk, tv, p);
    KATZ_LAUNCH_RET();
}

extern "C" long long katz_attention_split_scratch_bytes(void) {
    // parts x cut tiles never exceeds one dispatch round
    return FA_COUNTER_BYTES + (long long)fa_slots() * FA_PART_BYTES;
}

extern "C" int katz_attention_split_f16(const void* Q, const void* K, const void* V, void* O, int B, int H, int Sq, int Sk,
                                        int head_dim, int ldq, int ldk, int ldv, int ldo, long long bsq, long long bsk,
                                        long long bsv, long long bso, float scale, int kv_chunk_rows,
                                        long long kv_chunk_stride, void* scratch, long long scratch_bytes, void* stream) {
    KATZ_CHECK_ARG(scratch && aligned16(scratch) && scratch_bytes >= FA_COUNTER_BYTES, KATZ_EINVAL);
    return attention_launch(Q, K, V, O, B, H, Sq, Sk, head_dim, ldq, ldk, ldv, ldo, bsq, bsk, bsv, bso, scale, kv_chunk_rows,
                            kv_chunk_stride, scratch, scratch_bytes, nullptr, 0, stream);
}

extern "C" int katz_attention_peer_f16(const void* Q, const void* K, const void* V, void* O, int B, int H, int Sq, int Sk,
                                       int head_dim, int ldq, int ldk, int ldv, int ldo, long long bsq, long long bsk,
                                       long long bsv, long long bso, float scale, int kv_chunk_rows,
                                       long long kv_chunk_stride, void* scratch, long long scratch_bytes, const void* peer_ctrl,
                                       int self_chunk, void* stream) {
    KATZ_CHECK_ARG(peer_ctrl, KATZ_EINVAL);
    KATZ_CHECK_ARG(!scratch || (aligned16(scratch) && scratch_bytes >= FA_COUNTER_BYTES), KATZ_EINVAL);
    return attention_launch(Q, K, V, O, B, H, Sq, Sk, head_dim, ldq, ldk, ldv, ldo, bsq, bsk, bsv, bso, scale, kv_chunk_rows,
                            kv_chunk_stride, scratch, scratch_bytes, peer_ctrl, self_chunk, stream);
}

extern "C" int katz_attention_f16(const void* Q, const void* K, const void* V, void* O, int B, int H, int Sq, int Sk,
                                  int head_dim, int ldq, int ldk, int ldv, int ldo, long long bsq, long long bsk,
                                  long long bsv, long long bso, float scale, int kv_chunk_rows, long long kv_chunk_stride,
                                  void* stream) {
    return attention_launch(Q, K, V, O, B, H, Sq, Sk, head_dim, ldq, ldk, ldv, ldo, bsq, bsk, bsv, bso, scale, kv_chunk_rows,
                            kv_chunk_stride, nullptr, 0, nullptr, 0, stream);
}
