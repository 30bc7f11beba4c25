// tcgen05 GEMM / implicit-GEMM 3x3 convolution: C[M,N] = A[M,K] * W[N,K]^T with a fused epilogue.
//
// One persistent CTA per SM walks output tiles of 128 x BN (BN = 128, 160 or 256; 160 divides every channel count of
// the SDXL UNet and puts the 2048-token GEMMs on 128 of the 148 SMs in a single wave):
//   * warp 0, one elected thread: TMA tile loads (128-byte swizzle) into a multi-stage shared-memory ring, running
//     ahead across tile boundaries;
//   * warp 1, one elected thread: tcgen05.mma kind::f16 (128 x BN x 16 per instruction), fp32 accumulators in TMEM,
//     two accumulator buffers so tile i+1's main loop overlaps tile i's epilogue;
//   * warps 2-13: epilogue, three warps per TMEM lane quarter taking every third 32-column chunk. tcgen05.ld brings a
//     32-row x 32-column block into registers with one row per thread; bias / per-batch row vector / SiLU / residual /
//     scale are applied there, and the block moves to and from global memory as a 32 x 64-byte TMA box (residual in,
//     result out) staged in swizzled shared memory.
// Linear layers read A through a 2-D tensor map. The 3x3 stride-1 convolution reads the NHWC activation through a 4-D
// tensor map as nine shifted tile loads per channel chunk (out-of-image pixels arrive as zeros): no im2col buffer.
// GEGLU mode loads the two halves of the projection weight into one B tile (rows n..n+BN/2 and F+n..F+n+BN/2), so
// the value and gate columns of an output element sit in the same thread and `h * gelu(g)` is the epilogue.
//
// Every mbarrier wait is bounded (tc05.cuh): on a time-out the CTA records a status word, stops storing, frees its
// TMEM and returns; the host reads the word with katz_tc05_status().
//
// Replaces the cuBLAS / cuDNN calls behind nn.Linear and nn.Conv2d in the reference's UNet
// (diffusers/models/attention_processor.py:1256-1284, attention.py:649, activations.py:145-149, resnet.py:378,408).
#include "tc05.cuh"
#include "katz_b200.h"

namespace katz {

using namespace tc05;

constexpr int TBM = 128, TBK = 64;
constexpr int TC_THREADS = 448;   // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-13: epilogue
constexpr int TMEM_COLS = 512;    // two accumulator buffers at columns 0 and 256
constexpr int BOX_BYTES = 32 * 64;    // epilogue box: 32 rows x 32 fp16 columns, 64-byte swizzle
constexpr int EPI_WARPS = 12;
constexpr int EPI_PER_Q = EPI_WARPS / 4;      // epilogue warps per TMEM lane quarter: they take every EPI_PER_Q-th 32-column chunk
// boxes per epilogue warp: one per chunk it handles in a tile (the warps of a lane quarter share a tile's 32-column chunks),
// so a warp never waits for a TMA store inside a tile
__host__ __device__ constexpr int tc05_boxes_per_warp(int bn_out) { return (bn_out / 32 + EPI_PER_Q - 1) / EPI_PER_Q; }

struct Tc05Params {
    __half* C;
    const __half* bias;
    const __half* rowvec;
    const __half* residual;
    int M, N, K;            // N = output columns (GEGLU: F, the gated width)
    int ldc, ldr, ld_rowvec, rows_per_batch;
    int act;
    float out_scale;
    int m_tiles, n_tiles;
    int geglu_F;            // > 0: GEGLU mode, weight has 2F rows
    int rows_img;           // rows of one image of the output tensor map (M for a linear layer, H*W for a convolution)
    // convolution geometry (stride 1, output size = input size)
    int conv, H, W, TW, TH, tiles_w, tiles_h, cin_chunks, ksize, pad_h, pad_w, stride;   // H, W: OUTPUT size
    int* status;
    // LayerNorm folded into this GEMM (kernel template LN): A holds the RAW rows x, W holds W * diag(gamma); the epilogue
    // turns acc = x W'^T into rstd * acc - rstd * mean * c1 + c2 with c1[n] = sum_k W'[n,k], c2[n] = sum_k W[n,k] beta[k] (+
    // bias). Row statistics come as partial (sum, sum of squares) per 32-column chunk of the producer's output:
    // ln_stats[slot][M] (float2), ln_slots slots covering the K columns of x.
    const float2* ln_stats;
    const float2* ln_c12;       // (c1[n], c2[n]) interleaved: one 16-byte load brings both vectors for two columns
    int ln_slots;
    float ln_eps;
    // this GEMM's own output feeds a folded LayerNorm: per 32-column chunk and row, (sum, sum of squares) of the fp16 values
    // stored, written to stats_out[chunk][M]
    float2* stats_out;
};

__device__ int g_tc05_status = 0;

__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_32x8(uint32_t taddr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}

// Exact-form GELU x * Phi(x) with erf from Abramowitz & Stegun 7.1.26 (|error| <= 1.5e-7 on erf, far below the fp16
// rounding that follows): 1 - erf(z) = (a1 t + ... + a5 t^5) exp(-z^2), t = 1 / (1 + p z), z = |x| / sqrt(2).
// Two values at a time: ten packed instructions, four special-function ones (two reciprocals, two exp2) and four
// scalar ones for the pair, against erff's thirty per value.
__device__ __forceinline__ float rcp_approx(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float2 gelu_erf_fast2(float2 x) {
    const float2 ax = make_float2(fabsf(x.x), fabsf(x.y));
    const float2 den = fma2(ax, make_float2(0.3275911f * 0.70710678f, 0.3275911f * 0.70710678f), make_float2(1.0f, 1.0f));
    // approximate reciprocal and exp2 (one special-function instruction each, about 1 ulp): the rounded forms are short
    // instruction sequences with a slow-path branch, and eight of them per thread and 16-column group were most of
    // this epilogue's time
    const float2 t = make_float2(rcp_approx(den.x), rcp_approx(den.y));
    float2 h = fma2(t, make_float2(0.5f * 1.061405429f, 0.5f * 1.061405429f), make_float2(0.5f * -1.453152027f, 0.5f * -1.453152027f));
    h = fma2(t, h, make_float2(0.5f * 1.421413741f, 0.5f * 1.421413741f));
    h = fma2(t, h, make_float2(0.5f * -0.284496736f, 0.5f * -0.284496736f));
    h = fma2(t, h, make_float2(0.5f * 0.254829592f, 0.5f * 0.254829592f));
    const float2 xx = mul2(mul2(x, x), make_float2(-0.5f * 1.4426950408889634f, -0.5f * 1.4426950408889634f));
    const float2 e = make_float2(ex2_approx(xx.x), ex2_approx(xx.y));
    const float2 r = mul2(x, mul2(mul2(h, t), e));          // x * Phi(-|x|): the sign of x
    // x >= 0: x - r (r >= 0); x < 0: r (r < 0)  ==  max(x, 0) - |r|
    return make_float2(fmaxf(x.x, 0.f) - fabsf(r.x), fmaxf(x.y, 0.f) - fabsf(r.y));
}

__device__ __forceinline__ float rhalf(float v) { return __half2float(__float2half_rn(v)); }

// One thread's 32 accumulator columns of a chunk -> its 64-byte row of the box: + bias, + row vector (AUX), SiLU (ACT),
// + residual (RES, already in the box), * scale, rounded to fp16. The options are compile-time so that the body is
// straight-line code without the conversions and additions of absent terms.
template <bool ACT, bool RES, bool AUX, bool STATS = false>
__device__ __forceinline__ void epilogue_chunk(const uint32_t* r, unsigned char* rowp, uint32_t swz, const uint4* b4,
                                               const uint4* v4, float out_scale, float2* sums = nullptr) {
    float2 s1 = make_float2(0.f, 0.f), s2 = make_float2(0.f, 0.f);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        uint4* cell = reinterpret_cast<uint4*>(rowp + (((uint32_t)k ^ swz) << 4));
        uint4 r4 = make_uint4(0, 0, 0, 0);
        if (RES) r4 = *cell;
        const uint32_t bw[4] = {b4[k].x, b4[k].y, b4[k].z, b4[k].w}, vw[4] = {v4[k].x, v4[k].y, v4[k].z, v4[k].w},
                       rw[4] = {r4.x, r4.y, r4.z, r4.w};
        uint32_t ow[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            // packed fp32 arithmetic: one instruction per pair of columns for each of the additions and the scaling (the
            // epilogue of a single-wave launch is bound by instruction issue: three warps share a scheduler)
            float2 v = add2(make_float2(__uint_as_float(r[k * 8 + 2 * e]), __uint_as_float(r[k * 8 + 2 * e + 1])), unpack_half2(bw[e]));
            if (AUX) v = add2(v, unpack_half2(vw[e]));
            if (ACT) v = make_float2(silu_f(v.x), silu_f(v.y));
            if (RES) v = add2(v, unpack_half2(rw[e]));
            v = mul2(v, make_float2(out_scale, out_scale));
            if (STATS) {
                // row statistics for a LayerNorm folded into the next GEMM, from the fp32 values (their fp16 rounding moves
                // a 1280-term sum by parts in 1e5)
                s1 = add2(s1, v);
                s2 = fma2(v, v, s2);
            }
            ow[e] = pack_half2(v.x, v.y);
        }
        *cell = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
    if (STATS) *sums = make_float2(s1.x + s1.y, s2.x + s2.y);
}

// LayerNorm-folded epilogue of one chunk: out = half(acc * rstd + (c2[n] - rstd * mean * c1[n])). c12 holds (c1, c2) per
// column; it is the same for every row (warp-uniform addresses: broadcast loads that stay in L1).
__device__ __forceinline__ void epilogue_chunk_ln(const uint32_t* r, unsigned char* rowp, uint32_t swz, const float2* c12,
                                                  int ncols, float rstd, float nrm) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        uint32_t ow[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int col = k * 8 + 2 * e;
            const float4 cc = col < ncols ? __ldg(reinterpret_cast<const float4*>(c12 + col)) : make_float4(0.f, 0.f, 0.f, 0.f);
            const float v0 = fmaf(__uint_as_float(r[col]), rstd, fmaf(nrm, cc.x, cc.y));
            const float v1 = fmaf(__uint_as_float(r[col + 1]), rstd, fmaf(nrm, cc.z, cc.w));
            ow[e] = pack_half2(v0, v1);
        }
        *reinterpret_cast<uint4*>(rowp + (((uint32_t)k ^ swz) << 4)) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

// PAIR: two CTAs of a cluster share every tcgen05.mma (cta_group::2, M = 256): each loads its own 128-row A tile and HALF
// of the B tile, the leader issues the instruction for both, each CTA's TMEM receives its own 128 rows and each runs its
// own epilogue. Per k-step a CTA then takes 16 + BN/2 x 128 B from L2 instead of 16 + BN x 128 B; the main loop is bound
// by that delivery, not by the tensor pipe. No load is multicast; only completion signals cross the pair.
template <int BN, int STAGES, bool GEGLU, bool PAIR, bool LN>
__global__ void __launch_bounds__(TC_THREADS, 1) tc05_gemm_kernel(const __grid_constant__ CUtensorMap tmA,
                                                                  const __grid_constant__ CUtensorMap tmB,
                                                                  const __grid_constant__ CUtensorMap tmC,
                                                                  const __grid_constant__ CUtensorMap tmR,
                                                                  const Tc05Params p) {
    constexpr int A_BYTES = TBM * TBK * 2;
    constexpr int B_BYTES = (PAIR ? BN / 2 : BN) * TBK * 2;      // this CTA's part of the B tile
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int BN_OUT = GEGLU ? BN / 2 : BN;      // output columns per tile
    constexpr int NBW = tc05_boxes_per_warp(BN_OUT), EPI_BOXES = EPI_WARPS * NBW;
    extern __shared__ unsigned char smem_raw[];
    // 1024-byte alignment: the swizzle pattern and the UMMA descriptors assume it
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* box_base = smem + STAGES * STAGE_BYTES;                 // 1024-byte aligned (stages are multiples of 1 KB)
    uint64_t* bars = reinterpret_cast<uint64_t*>(box_base + EPI_BOXES * BOX_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4 + EPI_BOXES);
    static_assert(EPI_BOXES <= 48, "barrier area");
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const uint32_t tfull0 = smem_u32(bars + 2 * STAGES), tempty0 = smem_u32(bars + 2 * STAGES + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KT = p.K / TBK;
    // PAIR: a work item is a pair of vertically adjacent tiles; CTA rank r of cluster c takes the r-th tile of items
    // c, c + clusters, ... Without pairs an item is one tile and every CTA is its own "cluster".
    const uint32_t rank = PAIR ? cluster_ctarank() : 0;
    const int item0 = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int item_stride = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    const int total_tiles = (PAIR ? (p.m_tiles + 1) / 2 : p.m_tiles) * p.n_tiles;      // work items

    // barrier set-up spread over the lanes of warp 0 (about forty barriers; one thread took half a microsecond)
    if (warp == 0) {
        constexpr int NBAR = 2 * STAGES + 4 + EPI_BOXES;
        for (int i = lane; i < NBAR; i += 32) {
            // full / empty / accumulator full / residual box: one arrival; accumulator free: one per epilogue warp (of
            // both CTAs of a pair)
            const bool acc_free = i >= 2 * STAGES + 2 && i < 2 * STAGES + 4;
            mbar_init(smem_u32(bars + i), acc_free ? EPI_WARPS * (PAIR ? 2 : 1) : 1);
        }
        fence_barrier_init();
        if (lane == 0) {
            tma_prefetch_desc(&tmA);
            tma_prefetch_desc(&tmB);
            tma_prefetch_desc(&tmC);
            if (p.residual) tma_prefetch_desc(&tmR);
        }
    }
    if (warp == 1) {
        if (PAIR) {
            tmem_alloc_pair(smem_u32(tmem_slot), TMEM_COLS);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
            tmem_relinquish();
        }
    }
    fence_before_sync();
    __syncthreads();
    // The peer's barriers must be initialised before anything signals them. The cluster barrier's round trip (most of a
    // microsecond in a trace) is split: every thread arrives here, and each role waits right before its first access to
    // the peer, after whatever else it has to wait for (the producer: the previous kernel).
    if (PAIR) cluster_arrive_relaxed();      // warp 0 issued fence.mbarrier_init.release.cluster after its initialisations
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // Everything above (barriers, TMEM, descriptor prefetch) and each role's index arithmetic may overlap the previous
    // kernel's tail: the roles call pdl_wait() themselves, before their first global-memory access.

    if (warp == 0) {
        // ------------------------------------------------------------------------------------ TMA producer
        const bool elected = elect_one();
        if (elected) {
            pdl_wait();                 // the kernels this launch depends on are done (overlaps the cluster barrier)
            pdl_launch_dependents();
        }
        if (PAIR) cluster_wait();
        if (elected) {
            bool ok = true;
            uint32_t it = 0, issued = 0;
            for (int tile = item0; tile < total_tiles && ok; tile += item_stride) {
                const int mi = tile / p.n_tiles, nt = tile - mi * p.n_tiles;
                const int mt = PAIR ? 2 * mi + (int)rank : mi;      // past the last tile for the odd one out: loads zeros
                int m0 = mt * TBM, cb = 0, ch0 = 0, cw0 = 0;
                if (p.conv) {
                    const int tpi = p.tiles_w * p.tiles_h;
                    cb = mt / tpi;
                    const int r = mt - cb * tpi;
                    const int ty = r / p.tiles_w;
                    ch0 = ty * p.TH;
                    cw0 = (r - ty * p.tiles_w) * p.TW;
                }
                const int n0 = nt * BN_OUT;
                // the convolution's k-steps walk (tap row, tap column, channel chunk) with counters: two integer divisions
                // per k-step in this one thread took longer than the tensor pipe needs for the k-step
                int cc = 0, kx = 0, ky = 0;
                for (int kt = 0; kt < KT; ++kt, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(empty0 + 8 * s, ph ^ 1)) { ok = false; break; }
                    const uint32_t sa = smem_base + s * STAGE_BYTES;
                    if constexpr (PAIR) {
                        // both CTAs' bytes are counted on the leader's barrier, which the leader arms for both
                        const uint32_t fb = mapa_shared(full0 + 8 * s, 0);
                        if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * STAGE_BYTES);
                        if (p.conv) {
                            tma_load_4d_pair(sa, &tmA, cc * TBK, cw0 * p.stride + kx - p.pad_w, ch0 * p.stride + ky - p.pad_h, cb, fb);
                        } else {
                            tma_load_2d_pair(sa, &tmA, kt * TBK, m0, fb);
                        }
                        // this CTA's half of the B tile: the upper columns, or in GEGLU mode the gate rows of the weight
                        tma_load_2d_pair(sa + A_BYTES, &tmB, kt * TBK,
                                         GEGLU ? (rank ? p.geglu_F + n0 : n0) : n0 + (int)rank * (BN / 2), fb);
                    } else {
                        const uint32_t fb = full0 + 8 * s;
                        mbar_expect_tx(fb, STAGE_BYTES);
                        if (p.conv) {
                            // the tensor map walks the input with the convolution's stride: TW x TH pixels per box
                            tma_load_4d(sa, &tmA, cc * TBK, cw0 * p.stride + kx - p.pad_w, ch0 * p.stride + ky - p.pad_h, cb, fb);
                        } else {
                            tma_load_2d(sa, &tmA, kt * TBK, m0, fb);
                        }
                        if (GEGLU) {
                            tma_load_2d(sa + A_BYTES, &tmB, kt * TBK, n0, fb);
                            tma_load_2d(sa + A_BYTES + B_BYTES / 2, &tmB, kt * TBK, p.geglu_F + n0, fb);
                        } else {
                            tma_load_2d(sa + A_BYTES, &tmB, kt * TBK, n0, fb);
                        }
                    }
                    issued = it + 1;
                    if (++cc == p.cin_chunks) {
                        cc = 0;
                        if (++kx == p.ksize) {
                            kx = 0;
                            ++ky;
                        }
                    }
                }
            }
            if (!ok) {
                atomicExch(p.status, 1);
                // let copies already in flight land before the CTA's shared memory is released (a pair's peer waits in
                // the cluster barrier of the teardown instead: its copies are counted on the leader's barriers)
                if (!PAIR || rank == 0) {
                    const uint32_t first = issued > (uint32_t)STAGES ? issued - STAGES : 0;
                    for (uint32_t j = first; j < issued; ++j) mbar_wait(full0 + 8 * (j % STAGES), (j / STAGES) & 1);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------------------------ MMA issuer
        if (PAIR) cluster_wait();
        if ((!PAIR || rank == 0) && elect_one()) {
            constexpr uint32_t idesc = idesc_f16(PAIR ? 2 * TBM : TBM, BN);
            bool ok = true;
            uint32_t it = 0, t = 0;
            // no global access here, but the bounded waits below count polls: they must not start counting while the
            // kernels this launch depends on (which the producer waits for) may still run for a long time
            pdl_wait();
            for (int tile = item0; tile < total_tiles && ok; tile += item_stride, ++t) {
                const uint32_t buf = t & 1;
                if (!mbar_wait(tempty0 + 8 * buf, ((t >> 1) & 1) ^ 1)) { ok = false; break; }
                fence_after_sync();
                const uint32_t tacc = tmem_base + buf * 256;
                for (int kt = 0; kt < KT; ++kt, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(full0 + 8 * s, ph)) { ok = false; break; }
                    fence_after_sync();
                    const uint32_t sa = smem_base + s * STAGE_BYTES;
                    const uint64_t ad = smem_desc_sw128(sa), bd = smem_desc_sw128(sa + A_BYTES);
#pragma unroll
                    for (int k = 0; k < TBK / 16; ++k) {
                        // +32 bytes per 16-element K step inside the 128-byte swizzle row (encoded >> 4)
                        if (PAIR) umma_f16_pair(tacc, ad + 2 * k, bd + 2 * k, idesc, (kt | k) != 0);
                        else umma_f16(tacc, ad + 2 * k, bd + 2 * k, idesc, (kt | k) != 0);
                    }
                    // stage reusable once these MMAs have read it (in both CTAs of a pair)
                    if (PAIR) umma_commit_pair(empty0 + 8 * s, 3);
                    else umma_commit(empty0 + 8 * s);
                }
                if (ok) {
                    if (PAIR) umma_commit_pair(tfull0 + 8 * buf, 3);
                    else umma_commit(tfull0 + 8 * buf);
                }
            }
            if (!ok) atomicExch(p.status, 2);
        }
    } else {
        // ------------------------------------------------------------------------------------ epilogue
        // Twelve warps: three per TMEM lane quarter, taking every third 32-column chunk of the tile (the epilogue of a
        // single-tile launch is pure latency after the last MMA, and two warps per scheduler hid little of it). Thread = tile row. A
        // chunk of the warp's 32 rows is one 32 x 64-byte box: the residual box arrives by TMA (requested one of the
        // warp's chunks ahead: the first while the tile's main loop is still running), each thread updates its own
        // row of the box in shared memory, and the box leaves by TMA store, which clips rows past M (or past the
        // image) and columns past N. Bias and row-vector values are the same for every row: broadcast loads, requested
        // one chunk ahead. (Per-row global accesses from the threads cost 32 cache lines per instruction and made the
        // epilogue slower than the main loop; so did per-element branches on the launch-uniform options.)
        const int ew = warp - 2;                // epilogue warp 0..7
        const int q = warp & 3;                 // TMEM lane quarter this warp may read
        const int half = ew >> 2;               // which of the quarter's EPI_PER_Q warps: chunks half, half + EPI_PER_Q, ...
        unsigned char* boxes = box_base + ew * NBW * BOX_BYTES;
        const uint32_t rfull0 = smem_u32(bars + 2 * STAGES + 4 + ew * NBW);
        constexpr int NCH = BN_OUT / 32;
        static_assert(BN_OUT % 32 == 0, "output tile width must be a multiple of the 32-column box");
        const bool has_res = p.residual != nullptr;
        const uint32_t swz = (uint32_t)((lane >> 1) & 3);      // 64-byte swizzle: 16-byte chunk index ^ ((row >> 1) & 3)
        bool ok = true;
        uint32_t t = 0, rpar = 0;               // tiles done by the CTA; parity bit per residual box of this warp
        if (ew == EPI_WARPS - 1 && lane == 0 && item0 < total_tiles) {
            // The weights of the CTA's first tile go to L2 now: they are cold in HBM (5 GB of weights stream through a 126 MB
            // L2 every step), and loads that have to come from DRAM kept the tensor pipe waiting after the dependency had
            // resolved. The prefetch needs no dependency (it only warms L2, the point of coherence) and is issued from an
            // epilogue thread, idle until the first tile is done: each request costs its issuer about 40 ns, which the
            // producer thread cannot spare.
            const int pn0 = (item0 % p.n_tiles) * BN_OUT;
            const int kmax = KT < 64 ? KT : 64;
            for (int kt = 0; kt < kmax; ++kt) {
                if constexpr (PAIR) {
                    tma_prefetch_l2_2d(&tmB, kt * TBK, GEGLU ? (rank ? p.geglu_F + pn0 : pn0) : pn0 + (int)rank * (BN / 2));
                } else {
                    tma_prefetch_l2_2d(&tmB, kt * TBK, pn0);
                    if (GEGLU) tma_prefetch_l2_2d(&tmB, kt * TBK, p.geglu_F + pn0);
                }
            }
        }
        pdl_wait();                             // bias, row vector and residual are global reads
        if (PAIR) cluster_wait();
        for (int tile = item0; tile < total_tiles && ok; tile += item_stride, ++t) {
            const uint32_t buf = t & 1;
            const int mi = tile / p.n_tiles, nt = tile - mi * p.n_tiles;
            const int mt = PAIR ? 2 * mi + (int)rank : mi;
            const int n0 = nt * BN_OUT;
            // coordinates of this warp's 32 rows in the output tensor map {N, rows per image, images}
            int y0, z0;
            if (p.conv) {
                const int tpi = p.tiles_w * p.tiles_h;
                z0 = mt / tpi;
                const int r = mt - z0 * tpi;
                const int ty = r / p.tiles_w;
                y0 = ty * p.TH * p.W + (r - ty * p.tiles_w) * p.TW + q * 32;
            } else {
                y0 = mt * TBM + q * 32;
                z0 = 0;
            }
            // warp-uniform: do any of this warp's 32 rows exist? (a pair's odd tile out lies past the last tile)
            const bool rows_in = mt < p.m_tiles && y0 < p.rows_img;
            // global output row of this thread (linear layers and convolutions alike: images are stored one after another)
            const long long grow = (long long)z0 * p.rows_img + y0 + lane;
            const bool row_in = rows_in && (y0 + lane) < p.rows_img;
            float ln_rstd = 1.f, ln_nrm = 0.f;
            if constexpr (LN) {
                // fold this row's partial sums (one float2 per 32-column chunk of x, rows contiguous per chunk): the loads
                // overlap the tile's main loop
                float s1 = 0.f, s2 = 0.f;
                if (row_in) {
                    const float2* sp = p.ln_stats + grow;
                    for (int c0 = 0; c0 < p.ln_slots; c0 += 8) {      // eight loads in flight at a time
                        float2 v[8];
#pragma unroll
                        for (int u = 0; u < 8; ++u)
                            v[u] = c0 + u < p.ln_slots ? __ldg(sp + (size_t)(c0 + u) * p.M) : make_float2(0.f, 0.f);
#pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            s1 += v[u].x;
                            s2 += v[u].y;
                        }
                    }
                }
                const float inv_n = 1.0f / (float)p.K;
                const float mean = s1 * inv_n;
                const float var = fmaxf(fmaf(-mean, mean, s2 * inv_n), 0.f);
                ln_rstd = rsqrtf(var + p.ln_eps);
                ln_nrm = -ln_rstd * mean;
            }
            const __half* bias_p = (p.bias && rows_in) ? p.bias + n0 : nullptr;
            const __half* aux_p = nullptr;             // gate bias (GEGLU) or the image's row vector
            if (!rows_in) {
                // nothing to load
            } else if (GEGLU) {
                if (p.bias) aux_p = p.bias + p.geglu_F + n0;
            } else if (p.rowvec) {
                aux_p = p.rowvec + (size_t)(p.conv ? z0 : (mt * TBM) / p.rows_per_batch) * p.ld_rowvec + n0;
            }
            auto load_vec = [&](const __half* base, int col) {     // 8 columns of a per-column vector, zeros past N
                return (base && n0 + col < p.N) ? __ldg(reinterpret_cast<const uint4*>(base + col)) : make_uint4(0, 0, 0, 0);
            };
            auto request_residual = [&](int c, uint32_t b) {     // lane 0 only: chunk c of this tile into box b
                const uint32_t bar = rfull0 + 8 * b;
                mbar_expect_tx(bar, BOX_BYTES);
                tma_load_3d(smem_u32(boxes + b * BOX_BYTES), &tmR, n0 + c * 32, y0, z0, bar);
            };
            if (lane == 0) {
                // every box of this warp was stored in the previous tile: those stores must have read shared memory before
                // anything (a residual load, a thread of this warp) writes the boxes again. The wait overlaps the main loop.
                bulk_wait_read<0>();
                if (has_res && rows_in) {
#pragma unroll
                    for (int cc = 0; cc < NBW; ++cc) {
                        const int c = EPI_PER_Q * cc + half;
                        if (c < NCH && n0 + c * 32 < p.N) request_residual(c, cc);
                    }
                }
            }
            uint4 nb4[4], nv4[4];               // bias / aux values of the warp's next chunk (GEGLU: of its next 16-column group)
            if (!GEGLU) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    nb4[k] = load_vec(bias_p, half * 32 + k * 8);
                    nv4[k] = load_vec(aux_p, half * 32 + k * 8);
                }
            } else if (!LN) {
                // GEGLU: value and gate bias of the warp's first 16-column group (nb4[0..1], nv4[0..1]); every group below
                // requests the next group's before it starts, so that no group waits for a global load
                nb4[0] = load_vec(bias_p, half * 32);
                nb4[1] = load_vec(bias_p, half * 32 + 8);
                nv4[0] = load_vec(aux_p, half * 32);
                nv4[1] = load_vec(aux_p, half * 32 + 8);
            }
            ok = mbar_wait(tfull0 + 8 * buf, (t >> 1) & 1);
            ok = __all_sync(0xffffffffu, ok);   // tcgen05.ld below is warp-collective: decide as a warp
            if (!ok) {
                if (lane == 0) atomicExch(p.status, 3);
                break;
            }
            fence_after_sync();
            const uint32_t tacc = tmem_base + buf * 256 + ((uint32_t)(q * 32) << 16);
#pragma unroll
            for (int cc = 0; cc < NBW; ++cc) {
                const int c = EPI_PER_Q * cc + half;
                if (!rows_in || c >= NCH || n0 + c * 32 >= p.N) break;      // nothing of this box (or of the rest) exists
                const uint32_t b = cc;
                unsigned char* rowp = boxes + b * BOX_BYTES + lane * 64;
                uint32_t r[GEGLU ? 1 : 32];
                uint4 cb4[4], cv4[4];
                if (!GEGLU) {
                    tmem_ld_32x32(tacc + c * 32, r);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        cb4[k] = nb4[k];
                        cv4[k] = nv4[k];
                    }
                    if (c + EPI_PER_Q < NCH) {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            nb4[k] = load_vec(bias_p, (c + EPI_PER_Q) * 32 + k * 8);
                            nv4[k] = load_vec(aux_p, (c + EPI_PER_Q) * 32 + k * 8);
                        }
                    }
                }
                if (has_res) {
                    ok = mbar_wait(rfull0 + 8 * b, (rpar >> cc) & 1);
                    rpar ^= 1u << cc;
                }
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) {
                    if (!GEGLU) tmem_ld_wait();
                    if (lane == 0) atomicExch(p.status, 4);
                    break;
                }
                if constexpr (GEGLU) {
                    // The gate's erf makes this epilogue instruction-bound: packed fp32 arithmetic (two values per
                    // instruction) and a rolled loop over 16-column groups, which keeps the code inside the instruction
                    // cache (fully unrolled it ran 2.5x slower).
#pragma unroll 1
                    for (int k2 = 0; k2 < 2; ++k2) {
                        const int col = c * 32 + k2 * 16;
                        uint32_t v16[16], g16[16];
                        tmem_ld_32x16(tacc + col, v16);
                        tmem_ld_32x16(tacc + BN / 2 + col, g16);
                        const uint4 bA = nb4[0], bB = nb4[1], gA = nv4[0], gB = nv4[1];
                        if constexpr (!LN) {
                            // the next group of this warp: the other half of this chunk, else the first half of its next chunk
                            const int ncol = k2 == 0 ? col + 16 : (c + EPI_PER_Q) * 32;
                            if (ncol < BN_OUT) {
                                nb4[0] = load_vec(bias_p, ncol);
                                nb4[1] = load_vec(bias_p, ncol + 8);
                                nv4[0] = load_vec(aux_p, ncol);
                                nv4[1] = load_vec(aux_p, ncol + 8);
                            }
                        }
                        const uint32_t bw[8] = {bA.x, bA.y, bA.z, bA.w, bB.x, bB.y, bB.z, bB.w};
                        const uint32_t gw[8] = {gA.x, gA.y, gA.z, gA.w, gB.x, gB.y, gB.z, gB.w};
                        tmem_ld_wait();
                        uint32_t ow[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            // activations.py:146-149 on fp16 tensors: proj output, gelu and product each round to half.
                            // The product of two halfs is exact in fp32, so its rounding is the half2 multiply.
                            float2 vv, gg;
                            if constexpr (LN) {
                                const int nn = n0 + col + 2 * e;
                                const bool in = nn < p.N;
                                const float4 cv = in ? __ldg(reinterpret_cast<const float4*>(p.ln_c12 + nn)) : make_float4(0.f, 0.f, 0.f, 0.f);
                                const float4 cg = in ? __ldg(reinterpret_cast<const float4*>(p.ln_c12 + p.geglu_F + nn)) : make_float4(0.f, 0.f, 0.f, 0.f);
                                const float2 rs = make_float2(ln_rstd, ln_rstd), nm = make_float2(ln_nrm, ln_nrm);
                                vv = fma2(make_float2(__uint_as_float(v16[2 * e]), __uint_as_float(v16[2 * e + 1])), rs,
                                          fma2(nm, make_float2(cv.x, cv.z), make_float2(cv.y, cv.w)));
                                gg = fma2(make_float2(__uint_as_float(g16[2 * e]), __uint_as_float(g16[2 * e + 1])), rs,
                                          fma2(nm, make_float2(cg.x, cg.z), make_float2(cg.y, cg.w)));
                            } else {
                                vv = add2(make_float2(__uint_as_float(v16[2 * e]), __uint_as_float(v16[2 * e + 1])), unpack_half2(bw[e]));
                                gg = add2(make_float2(__uint_as_float(g16[2 * e]), __uint_as_float(g16[2 * e + 1])), unpack_half2(gw[e]));
                            }
                            const __half2 vh = __floats2half2_rn(vv.x, vv.y);
                            const float2 gr = __half22float2(__floats2half2_rn(gg.x, gg.y));
                            const float2 ge = gelu_erf_fast2(gr);
                            const __half2 oh = __hmul2(vh, __floats2half2_rn(ge.x, ge.y));
                            ow[e] = *reinterpret_cast<const uint32_t*>(&oh);
                        }
                        *reinterpret_cast<uint4*>(rowp + (((uint32_t)(2 * k2) ^ swz) << 4)) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                        *reinterpret_cast<uint4*>(rowp + (((uint32_t)(2 * k2 + 1) ^ swz) << 4)) = make_uint4(ow[4], ow[5], ow[6], ow[7]);
                    }
                } else {
                    tmem_ld_wait();
                    // act and residual are uniform over the launch: one branch per chunk picks a straight-line body
                    // (SiLU only follows the tiny embedding GEMMs: it keeps the general body)
                    if constexpr (LN) {
                        const int ncols = p.N - (n0 + c * 32);
                        epilogue_chunk_ln(r, rowp, swz, p.ln_c12 + n0 + c * 32, ncols < 32 ? ncols : 32, ln_rstd, ln_nrm);
                    } else if (p.stats_out != nullptr) {
                        // this output feeds a folded LayerNorm: per row, (sum, sum of squares) of this chunk's 32 values
                        // (columns past N come from zero operands and zero vectors: they add nothing). Launches with a
                        // row vector or an activation do not ask for statistics.
                        float2 sums;
                        if (has_res) epilogue_chunk<false, true, false, true>(r, rowp, swz, cb4, cv4, p.out_scale, &sums);
                        else epilogue_chunk<false, false, false, true>(r, rowp, swz, cb4, cv4, p.out_scale, &sums);
                        if (row_in) p.stats_out[(size_t)((n0 >> 5) + c) * p.M + grow] = sums;
                    } else if (p.act == 1) {
                        if (has_res) epilogue_chunk<true, true, true>(r, rowp, swz, cb4, cv4, p.out_scale);
                        else epilogue_chunk<true, false, true>(r, rowp, swz, cb4, cv4, p.out_scale);
                    } else if (aux_p) {
                        if (has_res) epilogue_chunk<false, true, true>(r, rowp, swz, cb4, cv4, p.out_scale);
                        else epilogue_chunk<false, false, true>(r, rowp, swz, cb4, cv4, p.out_scale);
                    } else {
                        if (has_res) epilogue_chunk<false, true, false>(r, rowp, swz, cb4, cv4, p.out_scale);
                        else epilogue_chunk<false, false, false>(r, rowp, swz, cb4, cv4, p.out_scale);
                    }
                }
                fence_proxy_async();            // this thread's row of the box -> visible to the TMA store
                __syncwarp();
                if (lane == 0) {
                    tma_store_3d(&tmC, n0 + c * 32, y0, z0, smem_u32(boxes + b * BOX_BYTES));
                    bulk_commit();
                }
            }
            if (!ok) break;
            // this warp is done reading the accumulator buffer: tell the MMA thread, which waits for it before the tile
            // after next reuses the buffer. Nobody waits for the arrivals of a CTA's last two tiles, and the release at
            // cluster scope cost a microsecond at the very end of a single-tile launch: those are skipped.
            if (tile + 2 * item_stride < total_tiles) {
                fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    if (PAIR) mbar_arrive_cluster(mapa_shared(tempty0 + 8 * buf, 0));      // the leader's MMA thread waits for both CTAs
                    else mbar_arrive(tempty0 + 8 * buf);
                }
            }
        }
        if (lane == 0) bulk_wait_read<0>();     // every store has read its box (the writes complete with the kernel)
    }
    // ---------------------------------------------------------------------------------------- teardown
    fence_before_sync();
    __syncthreads();
    if (PAIR) {      // neither CTA leaves (or frees TMEM) while the other may still signal it or read its tiles
        cluster_arrive_relaxed();
        cluster_wait();
    }
    if (warp == 1) {
        fence_after_sync();
        if (PAIR) tmem_dealloc_pair(tmem_base, TMEM_COLS);
        else tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---- host side ---------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* f = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(f);
    }
    return fn;
}

static int encode_2d(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                     uint32_t box_inner, uint32_t box_outer) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return KATZ_ENOTREADY;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_stride_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t es[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, es,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : KATZ_EINVAL;
}

// Output / residual tensor as {N columns, rows per image, images} with 32 x 32 boxes (64-byte rows, 64-byte swizzle):
// what an epilogue warp stores per chunk. A linear layer is one image of M rows.
static int encode_out(CUtensorMap* map, const void* base, int N, long long rows_per_image, int images, int ld) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return KATZ_ENOTREADY;
    cuuint64_t dims[3] = {(cuuint64_t)N, (cuuint64_t)rows_per_image, (cuuint64_t)images};
    cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)rows_per_image * ld * 2};
    cuuint32_t box[3] = {32, 32, 1};
    cuuint32_t es[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, es,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : KATZ_EINVAL;
}

// Input of the implicit-GEMM convolution: boxes of TW x TH pixels x 64 channels. With stride 2 the map's traversal stride
// picks every second pixel (the box then spans 2 TW x 2 TH pixels of the tensor and still delivers TW x TH).
static int encode_nhwc(CUtensorMap* map, const void* base, int B, int H, int W, int C, int TW, int TH, int stride) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return KATZ_ENOTREADY;
    cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)C * 2, (cuuint64_t)W * C * 2, (cuuint64_t)H * W * C * 2};
    cuuint32_t box[4] = {(cuuint32_t)TBK, (cuuint32_t)(TW * stride), (cuuint32_t)(TH * stride), 1};
    cuuint32_t es[4] = {1, (cuuint32_t)stride, (cuuint32_t)stride, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), dims, strides, box, es,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : KATZ_EINVAL;
}

static int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
    }
    return n;
}

template <int BN, int STAGES, bool GEGLU, bool PAIR>
static constexpr int tc05_smem() {
    constexpr int boxes = EPI_WARPS * tc05_boxes_per_warp(GEGLU ? BN / 2 : BN);
    return STAGES * (TBM * TBK * 2 + (PAIR ? BN / 2 : BN) * TBK * 2) + boxes * BOX_BYTES + (2 * STAGES + 4 + boxes) * 8 + 16 + 1024;
}

template <int BN, int STAGES, bool GEGLU, bool PAIR, bool LN = false>
static int launch_tc05(const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& c, const CUtensorMap& r,
                       const Tc05Params& p, cudaStream_t st) {
    static bool attr_dev[KATZ_MAX_DEVICES] = {false};
    static int max_ctas_dev[KATZ_MAX_DEVICES] = {0};
    const int dev_index = current_device_index();
    bool& attr = attr_dev[dev_index];
    int& max_ctas = max_ctas_dev[dev_index];
    constexpr int smem = tc05_smem<BN, STAGES, GEGLU, PAIR>();
    static_assert(smem <= 232448, "shared memory budget");
    auto kernel = tc05_gemm_kernel<BN, STAGES, GEGLU, PAIR, LN>;
    if (!attr) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        max_ctas = sm_count();
        if (PAIR) {
            // how many CTA pairs the device can hold at once (a pair sits on two SMs of one TPC)
            cudaLaunchConfig_t cfg{};
            cfg.gridDim = dim3(2 * sm_count());
            cfg.blockDim = dim3(TC_THREADS);
            cfg.dynamicSmemBytes = smem;
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeClusterDimension;
            at[0].val.clusterDim.x = 2;
            at[0].val.clusterDim.y = 1;
            at[0].val.clusterDim.z = 1;
            cfg.attrs = at;
            cfg.numAttrs = 1;
            int clusters = 0;
            e = cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg);
            if (e != cudaSuccess || clusters <= 0) return e != cudaSuccess ? (int)e : KATZ_ENOTREADY;
            max_ctas = 2 * clusters;
        }
        attr = true;
    }
    const int items = (PAIR ? (p.m_tiles + 1) / 2 : p.m_tiles) * p.n_tiles;
    const int per_item = PAIR ? 2 : 1;
    const int grid = items * per_item < max_ctas ? items * per_item : max_ctas;
    launch_k_cluster(kernel, grid, TC_THREADS, smem, st, PAIR ? 2 : 1, a, b, c, r, p);
    KATZ_LAUNCH_RET();
}

static int* status_ptr() {
    static int* ptr_dev[KATZ_MAX_DEVICES] = {nullptr};      // the symbol has one address per device
    int*& ptr = ptr_dev[current_device_index()];
    if (!ptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_tc05_status) == cudaSuccess) ptr = (int*)p;
    }
    return ptr;
}

int* tc05_status_device_ptr() { return status_ptr(); }

// Tile width by wave efficiency: tiles of width bn cost ~bn per wave; pick the width with the least total cost.
static int pick_bn(int m_tiles, int n_out, bool geglu, bool pair) {
    const int sms = sm_count();
    // 96: small M (batch 1, row shards), where wider tiles leave SMs idle. 192: GEGLU on CTA pairs only, for the shapes
    // whose 256-wide tiles end a little over a whole number of waves (2048 x 10240: 4.3 waves of 256, 5.8 of 192)
    const int cand[5] = {256, 192, 160, 128, 96};
    int best = 128;
    double best_cost = 1e30;
    for (int i = 0; i < 5; ++i) {
        const int bn = cand[i];
        if (geglu && (bn == 160 || bn == 96)) continue;      // half of it is not a whole number of 32-column boxes
        if (bn == 192 && !(geglu && pair)) continue;
        const int out_w = geglu ? bn / 2 : bn;
        const long long tiles = (long long)m_tiles * ceil_div(n_out, out_w);
        const long long waves = (tiles + sms - 1) / sms;
        // per-tile time: a k-step of a CTA pair is bound by shared-memory bandwidth, (128 + bn/2) x 128 B in and the same
        // out at 128 B/clk = 256 + bn cycles (2 bn of tcgen05.mma fit under it up to bn = 256), plus the tile's fixed
        // overhead (epilogue drain, barrier round trips). Measured against forced widths on the step's shapes: the model
        // picks the fastest or a width within 1 % of it everywhere.
        // (GEGLU: the epilogue is several times heavier per tile and hides less: 72 fits the measured 128- and 256-wide launches)
        const double cost = (double)waves * (bn + (geglu ? 72.0 : 280.0));
        if (cost < best_cost) {
            best_cost = cost;
            best = bn;
        }
    }
    return best;
}

// A CTA pair per 256 x BN tile where the shape has at least two row tiles. KATZ_TC05_PAIR=0 turns pairs off.
static bool use_pairs(const Tc05Params& p, bool geglu) {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("KATZ_TC05_PAIR");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    (void)geglu;
    return on && p.m_tiles >= 2;
}

template <bool GEGLU, bool LN = false>
static int dispatch(const CUtensorMap& a, const CUtensorMap& b, Tc05Params& p, int bn, bool pair, int rows_per_image, int images,
                    cudaStream_t st) {
    p.status = status_ptr();
    if (!p.status) return KATZ_ENOTREADY;
    CUtensorMap c, r;
    int rc = encode_out(&c, p.C, p.N, rows_per_image, images, p.ldc);
    if (rc) return rc;
    rc = encode_out(&r, p.residual ? p.residual : p.C, p.N, rows_per_image, images, p.residual ? p.ldr : p.ldc);
    if (rc) return rc;
    if (pair) {
        // stage counts: what fits beside the epilogue boxes (8 KB to 64 KB) in 227 KB
        if (bn == 256) return launch_tc05<256, GEGLU ? 5 : 4, GEGLU, true, LN>(a, b, c, r, p, st);
        if constexpr (GEGLU) {
            if (bn == 192) return launch_tc05<192, 7, true, true, LN>(a, b, c, r, p, st);
        }
        if constexpr (!GEGLU) {
            if (bn == 160) return launch_tc05<160, 6, false, true, LN>(a, b, c, r, p, st);
            if (bn == 96) return launch_tc05<96, 8, false, true, LN>(a, b, c, r, p, st);
        }
        return launch_tc05<128, 7, GEGLU, true, LN>(a, b, c, r, p, st);
    }
    if constexpr (!GEGLU) {
        if (bn == 160) return launch_tc05<160, 4, false, false, LN>(a, b, c, r, p, st);
        if (bn == 96) return launch_tc05<96, 6, false, false, LN>(a, b, c, r, p, st);
    }
    if (bn == 256) return launch_tc05<256, 3, GEGLU, false, LN>(a, b, c, r, p, st);
    return launch_tc05<128, GEGLU ? 6 : 5, GEGLU, false, LN>(a, b, c, r, p, st);
}

// W' = W diag(gamma) (fp16), c12[n] = (sum_k W'[n,k], sum_k W[n,k] beta[k] + bias[n]) in fp32: the per-weight constants of a
// LayerNorm folded into the linear layer that consumes it. One warp per output row.
__global__ void __launch_bounds__(256) ln_fold_kernel(const __half* __restrict__ W, const __half* __restrict__ gamma,
                                                      const __half* __restrict__ beta, const __half* __restrict__ bias,
                                                      __half* __restrict__ Wf, float2* __restrict__ c12, int N, int K) {
    pdl_wait();
    // writes weights that later kernels may fetch before their own dependency wait: no early release of dependents
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + warp;
    if (n >= N) return;
    const __half* w = W + (size_t)n * K;
    __half* wf = Wf + (size_t)n * K;
    float s1 = 0.f, s2 = 0.f;
    for (int k = lane * 8; k < K; k += 256) {
        const uint4 wv = *reinterpret_cast<const uint4*>(w + k);
        const uint4 gv = __ldg(reinterpret_cast<const uint4*>(gamma + k));
        const uint4 bv = __ldg(reinterpret_cast<const uint4*>(beta + k));
        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w}, gw[4] = {gv.x, gv.y, gv.z, gv.w}, bw[4] = {bv.x, bv.y, bv.z, bv.w};
        uint32_t ow[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 wf2 = unpack_half2(ww[e]), g2 = unpack_half2(gw[e]), b2 = unpack_half2(bw[e]);
            ow[e] = pack_half2(wf2.x * g2.x, wf2.y * g2.y);
            const float2 o2 = unpack_half2(ow[e]);          // the folded weight as the GEMM will read it
            s1 += o2.x + o2.y;
            s2 = fmaf(wf2.x, b2.x, fmaf(wf2.y, b2.y, s2));
        }
        *reinterpret_cast<uint4*>(wf + k) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
    if (lane == 0) c12[n] = make_float2(s1, s2 + (bias ? __half2float(bias[n]) : 0.f));
}

}  // namespace katz

using namespace katz;

extern "C" int katz_ln_fold_f16(const void* W, const void* gamma, const void* beta, const void* bias, void* Wf, void* c12,
                                int N, int K, void* stream) {
    KATZ_CHECK_ARG(W && gamma && beta && Wf && c12, KATZ_EINVAL);
    KATZ_CHECK_ARG(N > 0 && K > 0 && K % 8 == 0, KATZ_ESIZE);
    KATZ_CHECK_ARG(aligned16(W) && aligned16(gamma) && aligned16(beta) && aligned16(Wf) && ((uintptr_t)c12 & 7) == 0, KATZ_EALIGN);
    launch_k(ln_fold_kernel, ceil_div(N, 8), 256, 0, (cudaStream_t)stream, (const __half*)W, (const __half*)gamma,
             (const __half*)beta, (const __half*)bias, (__half*)Wf, (float2*)c12, N, K);
    KATZ_LAUNCH_RET();
}

extern "C" int katz_tc05_status(void) {
    int v = -1;
    if (cudaMemcpyFromSymbol(&v, g_tc05_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

extern "C" int katz_tc05_clear_status(void) {
    int v = 0;
    return cudaMemcpyToSymbol(g_tc05_status, &v, sizeof(int)) == cudaSuccess ? 0 : KATZ_ENOTREADY;
}

static int linear_common(const void* A, int lda, const void* W, void* C, int ldc, int M, int N_out, int K, const void* bias,
                         const void* rowvec, int ld_rowvec, int rows_per_batch, const void* residual, int ldr, int act,
                         float out_scale, int geglu_F, void* stream, const katz_linear_extras* ex = nullptr) {
    KATZ_CHECK_ARG(A && W && C, KATZ_EINVAL);
    KATZ_CHECK_ARG(M > 0 && N_out > 0 && K > 0, KATZ_ESIZE);
    KATZ_CHECK_ARG(K % TBK == 0 && N_out % 8 == 0, KATZ_ESIZE);
    KATZ_CHECK_ARG(lda % 8 == 0 && ldc % 8 == 0, KATZ_EALIGN);
    KATZ_CHECK_ARG(aligned16(A) && aligned16(W) && aligned16(C), KATZ_EALIGN);
    KATZ_CHECK_ARG(!bias || aligned16(bias), KATZ_EALIGN);
    KATZ_CHECK_ARG(!rowvec || (aligned16(rowvec) && ld_rowvec % 8 == 0), KATZ_EALIGN);
    // a tile's 128 rows must share one row vector
    KATZ_CHECK_ARG(!rowvec || (rows_per_batch > 0 && rows_per_batch % TBM == 0), KATZ_ESIZE);
    KATZ_CHECK_ARG(!residual || (aligned16(residual) && ldr % 8 == 0), KATZ_EALIGN);
    CUtensorMap ta, tb;
    int rc = encode_2d(&ta, A, K, M, (uint64_t)lda * 2, TBK, TBM);
    if (rc) return rc;
    Tc05Params p{};
    p.C = (__half*)C; p.bias = (const __half*)bias; p.rowvec = (const __half*)rowvec; p.residual = (const __half*)residual;
    p.M = M; p.N = N_out; p.K = K; p.ldc = ldc; p.ldr = ldr; p.ld_rowvec = ld_rowvec; p.rows_per_batch = rows_per_batch;
    p.act = act; p.out_scale = out_scale; p.geglu_F = geglu_F;
    p.m_tiles = ceil_div(M, TBM);
    p.rows_img = M;
    KATZ_CHECK_ARG((long long)p.m_tiles * ceil_div(N_out, 64) < (1ll << 30), KATZ_ESIZE);
    const bool geglu = geglu_F > 0;
    const bool pair = use_pairs(p, geglu);
    const int bn = pick_bn(p.m_tiles, N_out, geglu, pair);
    const int out_w = geglu ? bn / 2 : bn;
    p.n_tiles = ceil_div(N_out, out_w);
    const uint64_t w_rows = geglu ? 2ull * geglu_F : (uint64_t)N_out;
    rc = encode_2d(&tb, W, K, w_rows, (uint64_t)K * 2, TBK, (geglu || pair) ? bn / 2 : bn);      // box rows: what one load brings
    if (rc) return rc;
    bool ln = false;
    if (ex) {
        if (ex->stats_out) {
            KATZ_CHECK_ARG(((uintptr_t)ex->stats_out & 7) == 0, KATZ_EALIGN);
            p.stats_out = reinterpret_cast<float2*>(ex->stats_out);
        }
        if (ex->ln_stats) {
            // the folded LayerNorm replaces bias, row vector, activation and residual of this call
            KATZ_CHECK_ARG(ex->ln_c12 && ex->ln_slots > 0 && !bias && !rowvec && !residual && act == 0 && out_scale == 1.0f, KATZ_EINVAL);
            KATZ_CHECK_ARG(((uintptr_t)ex->ln_stats & 7) == 0 && aligned16(ex->ln_c12), KATZ_EALIGN);
            p.ln_stats = reinterpret_cast<const float2*>(ex->ln_stats);
            p.ln_c12 = reinterpret_cast<const float2*>(ex->ln_c12);
            p.ln_slots = ex->ln_slots;
            p.ln_eps = ex->ln_eps;
            ln = true;
        }
    }
    if (ln)
        return geglu ? dispatch<true, true>(ta, tb, p, bn, pair, M, 1, (cudaStream_t)stream)
                     : dispatch<false, true>(ta, tb, p, bn, pair, M, 1, (cudaStream_t)stream);
    return geglu ? dispatch<true>(ta, tb, p, bn, pair, M, 1, (cudaStream_t)stream)
                 : dispatch<false>(ta, tb, p, bn, pair, M, 1, (cudaStream_t)stream);
}

extern "C" int katz_linear_ex_f16(const void* A, int lda, const void* W, void* C, int ldc, int M, int N, int K,
                                  const void* bias, const void* rowvec, int ld_rowvec, int rows_per_batch,
                                  const void* residual, int ldr, int act, float out_scale, const katz_linear_extras* ex,
                                  void* stream) {
    return linear_common(A, lda, W, C, ldc, M, N, K, bias, rowvec, ld_rowvec, rows_per_batch, residual, ldr, act, out_scale, 0,
                         stream, ex);
}

extern "C" int katz_linear_geglu_ex_f16(const void* A, int lda, const void* W, void* C, int ldc, int M, int F, int K,
                                        const void* bias, const katz_linear_extras* ex, void* stream) {
    KATZ_CHECK_ARG(F > 0 && F % 16 == 0, KATZ_ESIZE);
    return linear_common(A, lda, W, C, ldc, M, F, K, bias, nullptr, 0, 0, nullptr, 0, 0, 1.0f, F, stream, ex);
}

extern "C" int katz_linear_f16(const void* A, int lda, const void* W, void* C, int ldc, int M, int N, int K,
                               const void* bias, const void* rowvec, int ld_rowvec, int rows_per_batch,
                               const void* residual, int ldr, int act, float out_scale, void* stream) {
    return linear_common(A, lda, W, C, ldc, M, N, K, bias, rowvec, ld_rowvec, rows_per_batch, residual, ldr, act, out_scale, 0,
                         stream);
}

extern "C" int katz_linear_geglu_f16(const void* A, int lda, const void* W, void* C, int ldc, int M, int F, int K,
                                     const void* bias, void* stream) {
    KATZ_CHECK_ARG(F > 0 && F % 16 == 0, KATZ_ESIZE);
    return linear_common(A, lda, W, C, ldc, M, F, K, bias, nullptr, 0, 0, nullptr, 0, 0, 1.0f, F, stream);
}

extern "C" int katz_conv3x3_nhwc_f16(const void* X, const void* W, void* Y, int B, int Hin, int Win, int Cin, int Cout,
                                     int stride, int pad_h, const void* bias, const void* rowvec, int ld_rowvec,
                                     const void* residual, int act, float out_scale, void* stream) {
    KATZ_CHECK_ARG(X && W && Y, KATZ_EINVAL);
    KATZ_CHECK_ARG(B > 0 && Hin > 0 && Win > 0 && Cin > 0 && Cout > 0, KATZ_ESIZE);
    KATZ_CHECK_ARG((pad_h == 0 || pad_h == 1) && (stride == 1 || stride == 2), KATZ_EINVAL);
    KATZ_CHECK_ARG(Hin + 2 * pad_h >= 3 && (stride == 1 || Win % 2 == 0), KATZ_ESIZE);
    const int H = (Hin + 2 * pad_h - 3) / stride + 1;   // output rows
    const int Wd = (Win + 2 - 3) / stride + 1;          // output columns
    KATZ_CHECK_ARG(H > 0, KATZ_ESIZE);
    KATZ_CHECK_ARG(Cin % TBK == 0 && Cout % 8 == 0, KATZ_ESIZE);
    const int TW = Wd < 128 ? Wd : 128;
    KATZ_CHECK_ARG((TW & (TW - 1)) == 0 && TW >= 8 && Wd % TW == 0, KATZ_ESIZE);
    const int TH = 128 / TW;
    KATZ_CHECK_ARG(aligned16(X) && aligned16(W) && aligned16(Y), KATZ_EALIGN);
    KATZ_CHECK_ARG(!bias || aligned16(bias), KATZ_EALIGN);
    KATZ_CHECK_ARG(!rowvec || (aligned16(rowvec) && ld_rowvec % 8 == 0), KATZ_EALIGN);
    KATZ_CHECK_ARG(!residual || aligned16(residual), KATZ_EALIGN);
    CUtensorMap ta, tb;
    int rc = encode_nhwc(&ta, X, B, Hin, Win, Cin, TW, TH, stride);
    if (rc) return rc;
    Tc05Params p{};
    p.C = (__half*)Y; p.bias = (const __half*)bias; p.rowvec = (const __half*)rowvec; p.residual = (const __half*)residual;
    p.M = B * H * Wd; p.N = Cout; p.K = 9 * Cin; p.ldc = Cout; p.ldr = Cout; p.ld_rowvec = ld_rowvec; p.rows_per_batch = H * Wd;
    p.act = act; p.out_scale = out_scale;
    p.conv = 1; p.H = H; p.W = Wd; p.TW = TW; p.TH = TH; p.tiles_w = Wd / TW; p.tiles_h = ceil_div(H, TH);
    p.cin_chunks = Cin / TBK; p.ksize = 3; p.pad_h = pad_h; p.pad_w = 1; p.stride = stride;
    p.m_tiles = B * p.tiles_w * p.tiles_h;
    p.rows_img = H * Wd;
    const bool pair = use_pairs(p, false);
    const int bn = pick_bn(p.m_tiles, Cout, false, pair);
    p.n_tiles = ceil_div(Cout, bn);
    rc = encode_2d(&tb, W, (uint64_t)9 * Cin, Cout, (uint64_t)9 * Cin * 2, TBK, pair ? bn / 2 : bn);
    if (rc) return rc;
    return dispatch<false>(ta, tb, p, bn, pair, H * Wd, B, (cudaStream_t)stream);
}
