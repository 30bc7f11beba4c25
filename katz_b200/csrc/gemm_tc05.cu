// tcgen05 GEMM / implicit-GEMM 3x3 convolution: C[M,N] = A[M,K] * W[N,K]^T with a fused epilogue.
//
// One persistent CTA per SM walks output tiles of 128 x BN (BN = 128, 160 or 256; 160 divides every channel count of
// the SDXL UNet and puts the 2048-token GEMMs on 128 of the 148 SMs in a single wave):
//   * warp 0, one elected thread: TMA tile loads (128-byte swizzle) into a multi-stage shared-memory ring, running
//     ahead across tile boundaries;
//   * warp 1, one elected thread: tcgen05.mma kind::f16 (128 x BN x 16 per instruction), fp32 accumulators in TMEM,
//     two accumulator buffers so tile i+1's main loop overlaps tile i's epilogue;
//   * warps 2-5: epilogue. tcgen05.ld brings a 32-row x 32-column block per warp into registers with one row per
//     thread, so a thread owns 64 contiguous bytes of an output row: bias / per-batch row vector / SiLU / residual /
//     scale are applied in registers and the row segment leaves as 16-byte stores; residual and row-vector values
//     are requested two chunks ahead, the first two while the tile's main loop is still running.
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
constexpr int TC_THREADS = 192;   // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-5: epilogue
constexpr int TMEM_COLS = 512;    // two accumulator buffers at columns 0 and 256
constexpr int STG_BYTES = 4 * 1024;   // bias slices of the four epilogue warps (bias + gate bias, 256 halfs each)

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
    // convolution geometry (stride 1, output size = input size)
    int conv, H, W, TW, TH, tiles_w, tiles_h, cin_chunks, ksize, pad_h, pad_w;   // H, W: OUTPUT size
    int* status;
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

__device__ __forceinline__ float rhalf(float v) { return __half2float(__float2half_rn(v)); }

template <int BN, int STAGES, bool GEGLU>
__global__ void __launch_bounds__(TC_THREADS, 1) tc05_gemm_kernel(const __grid_constant__ CUtensorMap tmA,
                                                                  const __grid_constant__ CUtensorMap tmB,
                                                                  const Tc05Params p) {
    constexpr int A_BYTES = TBM * TBK * 2;
    constexpr int B_BYTES = BN * TBK * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int BN_OUT = GEGLU ? BN / 2 : BN;      // output columns per tile
    extern __shared__ unsigned char smem_raw[];
    // 1024-byte alignment: the swizzle pattern and the UMMA descriptors assume it
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* staging = smem + STAGES * STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES + STG_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const uint32_t tfull0 = smem_u32(bars + 2 * STAGES), tempty0 = smem_u32(bars + 2 * STAGES + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KT = p.K / TBK;
    const int total_tiles = p.m_tiles * p.n_tiles;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tfull0 + 8 * b, 1);
            mbar_init(tempty0 + 8 * b, 4);    // one arrival per epilogue warp
        }
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------------------------ TMA producer
        if (elect_one()) {
            bool ok = true;
            uint32_t it = 0, issued = 0;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int mt = tile / p.n_tiles, nt = tile - mt * p.n_tiles;
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
                for (int kt = 0; kt < KT; ++kt, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(empty0 + 8 * s, ph ^ 1)) { ok = false; break; }
                    const uint32_t fb = full0 + 8 * s;
                    mbar_expect_tx(fb, STAGE_BYTES);
                    const uint32_t sa = smem_base + s * STAGE_BYTES;
                    if (p.conv) {
                        const int tap = kt / p.cin_chunks;
                        const int cc = kt - tap * p.cin_chunks;
                        const int ky = tap / p.ksize, kx = tap - ky * p.ksize;
                        tma_load_4d(sa, &tmA, cc * TBK, cw0 + kx - p.pad_w, ch0 + ky - p.pad_h, cb, fb);
                    } else {
                        tma_load_2d(sa, &tmA, kt * TBK, m0, fb);
                    }
                    if (GEGLU) {
                        tma_load_2d(sa + A_BYTES, &tmB, kt * TBK, n0, fb);
                        tma_load_2d(sa + A_BYTES + B_BYTES / 2, &tmB, kt * TBK, p.geglu_F + n0, fb);
                    } else {
                        tma_load_2d(sa + A_BYTES, &tmB, kt * TBK, n0, fb);
                    }
                    issued = it + 1;
                }
            }
            if (!ok) {
                atomicExch(p.status, 1);
                // let copies already in flight land before the CTA's shared memory is released
                const uint32_t first = issued > (uint32_t)STAGES ? issued - STAGES : 0;
                for (uint32_t j = first; j < issued; ++j) mbar_wait(full0 + 8 * (j % STAGES), (j / STAGES) & 1);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            constexpr uint32_t idesc = idesc_f16(TBM, BN);
            bool ok = true;
            uint32_t it = 0, t = 0;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++t) {
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
                        umma_f16(tacc, ad + 2 * k, bd + 2 * k, idesc, (kt | k) != 0);
                    }
                    umma_commit(empty0 + 8 * s);   // stage reusable once these MMAs have read it
                }
                if (ok) umma_commit(tfull0 + 8 * buf);
            }
            if (!ok) atomicExch(p.status, 2);
        }
    } else {
        // ------------------------------------------------------------------------------------ epilogue
        // Thread = tile row (the TMEM lane it may read); its 32 accumulator columns of a chunk are 64 contiguous bytes
        // of the output row, so residual, row vector and output move as 16-byte vectors straight from and to global
        // memory. Everything the epilogue reads from global memory is requested before it is needed: the tile's bias
        // goes to shared memory and the first two chunks' residual / row-vector values to registers while the main
        // loop of the tile is still running; later chunks are requested two chunks ahead.
        const int q = warp & 3;                 // TMEM lane quarter this warp may read
        __half* sbias = reinterpret_cast<__half*>(staging) + q * 512;      // [0,256): bias, [256,512): gate bias
        constexpr int NCH = (BN_OUT + 31) / 32;
        bool ok = true;
        uint32_t t = 0;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++t) {
            const uint32_t buf = t & 1;
            const int mt = tile / p.n_tiles, nt = tile - mt * p.n_tiles;
            const int n0 = nt * BN_OUT;
            const int row = q * 32 + lane;
            long long m;
            bool valid;
            int bidx;
            if (p.conv) {
                const int tpi = p.tiles_w * p.tiles_h;
                const int cb = mt / tpi;
                const int r = mt - cb * tpi;
                const int ty = r / p.tiles_w;
                const int th = row / p.TW, tw = row - th * p.TW;
                const int h = ty * p.TH + th;
                valid = h < p.H;
                m = ((long long)cb * p.H + h) * p.W + (r - ty * p.tiles_w) * p.TW + tw;
                bidx = cb;
            } else {
                m = (long long)mt * TBM + row;
                valid = m < p.M;
                bidx = p.rowvec ? (int)(m / p.rows_per_batch) : 0;
            }
            __half* crow = p.C + (size_t)m * p.ldc + n0;
            const __half* rrow = p.residual ? p.residual + (size_t)m * p.ldr + n0 : nullptr;
            const __half* vrow = p.rowvec ? p.rowvec + (size_t)bidx * p.ld_rowvec + n0 : nullptr;
            // bias slice of the tile -> shared memory (zeros past N or without a bias)
            {
                uint4 bv = make_uint4(0, 0, 0, 0), gv = make_uint4(0, 0, 0, 0);
                const int col = n0 + lane * 8;
                if (p.bias && lane * 8 < BN_OUT && col < p.N) {
                    bv = *reinterpret_cast<const uint4*>(p.bias + col);
                    if (GEGLU) gv = *reinterpret_cast<const uint4*>(p.bias + p.geglu_F + col);
                }
                *reinterpret_cast<uint4*>(sbias + lane * 8) = bv;
                if (GEGLU) *reinterpret_cast<uint4*>(sbias + 256 + lane * 8) = gv;
            }
            uint4 pre_res[2][4], pre_rv[2][4];
            auto prefetch = [&](int c, uint4* res, uint4* rv) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int col = c * 32 + k * 8;
                    const bool in = valid && col < BN_OUT && n0 + col < p.N;
                    res[k] = (in && rrow) ? *reinterpret_cast<const uint4*>(rrow + col) : make_uint4(0, 0, 0, 0);
                    rv[k] = (in && vrow) ? *reinterpret_cast<const uint4*>(vrow + col) : make_uint4(0, 0, 0, 0);
                }
            };
            if (!GEGLU) {
                prefetch(0, pre_res[0], pre_rv[0]);
                if (NCH > 1) prefetch(1, pre_res[1], pre_rv[1]);
            }
            __syncwarp();
            ok = mbar_wait(tfull0 + 8 * buf, (t >> 1) & 1);
            ok = __all_sync(0xffffffffu, ok);   // tcgen05.ld below is warp-collective: decide as a warp
            if (!ok) {
                if (lane == 0) atomicExch(p.status, 3);
                break;
            }
            fence_after_sync();
            const uint32_t tacc = tmem_base + buf * 256 + ((uint32_t)(q * 32) << 16);
            if constexpr (GEGLU) {
                // the gate's erf makes this epilogue instruction-bound: a rolled loop over 8-column groups keeps the code
                // small enough for the instruction cache (fully unrolled it ran 2.5x slower)
#pragma unroll 1
                for (int col = 0; col < BN_OUT; col += 8) {
                    uint32_t r[8], g[8];
                    tmem_ld_32x8(tacc + col, r);
                    tmem_ld_32x8(tacc + BN / 2 + col, g);
                    tmem_ld_wait();
                    const uint4 b4 = *reinterpret_cast<const uint4*>(sbias + col);
                    const uint4 g4 = *reinterpret_cast<const uint4*>(sbias + 256 + col);
                    const uint32_t bw[4] = {b4.x, b4.y, b4.z, b4.w}, gw[4] = {g4.x, g4.y, g4.z, g4.w};
                    uint32_t ow[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        // activations.py:146-149 on fp16 tensors: proj output, gelu and product each round to half
                        const float2 bf = unpack_half2(bw[e]), gb = unpack_half2(gw[e]);
                        const float v0 = __uint_as_float(r[2 * e]) + bf.x, v1 = __uint_as_float(r[2 * e + 1]) + bf.y;
                        const float g0 = __uint_as_float(g[2 * e]) + gb.x, g1 = __uint_as_float(g[2 * e + 1]) + gb.y;
                        ow[e] = pack_half2(rhalf(v0) * rhalf(gelu_erf_f(rhalf(g0))) * p.out_scale,
                                           rhalf(v1) * rhalf(gelu_erf_f(rhalf(g1))) * p.out_scale);
                    }
                    if (valid && n0 + col < p.N) *reinterpret_cast<uint4*>(crow + col) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                }
            } else {
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                const bool tail16 = (BN_OUT % 32 != 0) && c == NCH - 1;       // a 16-column last chunk
                uint32_t r[32], g[GEGLU ? 32 : 1];
                if (!tail16) {
                    tmem_ld_32x32(tacc + c * 32, r);
                    if (GEGLU) tmem_ld_32x32(tacc + BN / 2 + c * 32, g);
                } else {
                    tmem_ld_32x16(tacc + c * 32, r);
                    if (GEGLU) tmem_ld_32x16(tacc + BN / 2 + c * 32, g);
                }
                tmem_ld_wait();
                uint4* res = pre_res[c & 1];
                uint4* rv = pre_rv[c & 1];
#pragma unroll
                for (int k = 0; k < (tail16 ? 2 : 4); ++k) {
                    const int col = c * 32 + k * 8;
                    const uint4 b4 = *reinterpret_cast<const uint4*>(sbias + col);
                    const uint32_t bw[4] = {b4.x, b4.y, b4.z, b4.w};
                    const uint32_t rw[4] = {res[k].x, res[k].y, res[k].z, res[k].w};
                    const uint32_t vw[4] = {rv[k].x, rv[k].y, rv[k].z, rv[k].w};
                    uint32_t gw[4] = {0, 0, 0, 0};
                    if (GEGLU) {
                        const uint4 g4 = *reinterpret_cast<const uint4*>(sbias + 256 + col);
                        gw[0] = g4.x; gw[1] = g4.y; gw[2] = g4.z; gw[3] = g4.w;
                    }
                    uint32_t ow[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 bf = unpack_half2(bw[e]);
                        float v0 = __uint_as_float(r[k * 8 + 2 * e]) + bf.x, v1 = __uint_as_float(r[k * 8 + 2 * e + 1]) + bf.y;
                        if (GEGLU) {
                            // activations.py:146-149 on fp16 tensors: proj output, gelu and product each round to half
                            const float2 gb = unpack_half2(gw[e]);
                            const float g0 = __uint_as_float(g[k * 8 + 2 * e]) + gb.x, g1 = __uint_as_float(g[k * 8 + 2 * e + 1]) + gb.y;
                            v0 = rhalf(v0) * rhalf(gelu_erf_f(rhalf(g0)));
                            v1 = rhalf(v1) * rhalf(gelu_erf_f(rhalf(g1)));
                        }
                        if (p.rowvec) {
                            const float2 a = unpack_half2(vw[e]);
                            v0 += a.x; v1 += a.y;
                        }
                        if (p.act == 1) {
                            v0 = silu_f(v0); v1 = silu_f(v1);
                        }
                        if (p.residual) {
                            const float2 a = unpack_half2(rw[e]);
                            v0 += a.x; v1 += a.y;
                        }
                        ow[e] = pack_half2(v0 * p.out_scale, v1 * p.out_scale);
                    }
                    if (valid && n0 + col < p.N) *reinterpret_cast<uint4*>(crow + col) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                }
                if (c + 2 < NCH) prefetch(c + 2, pre_res[c & 1], pre_rv[c & 1]);
            }
            }
            // this warp is done reading the accumulator buffer (and the bias slice)
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty0 + 8 * buf);
        }
    }
    // ---------------------------------------------------------------------------------------- teardown
    fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLS);
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

static int encode_nhwc(CUtensorMap* map, const void* base, int B, int H, int W, int C, int TW, int TH) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return KATZ_ENOTREADY;
    cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)C * 2, (cuuint64_t)W * C * 2, (cuuint64_t)H * W * C * 2};
    cuuint32_t box[4] = {(cuuint32_t)TBK, (cuuint32_t)TW, (cuuint32_t)TH, 1};
    cuuint32_t es[4] = {1, 1, 1, 1};
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

template <int BN, int STAGES, bool GEGLU>
static constexpr int tc05_smem() {
    return STAGES * (TBM * TBK * 2 + BN * TBK * 2) + STG_BYTES + (2 * STAGES + 4) * 8 + 16 + 1024;
}

template <int BN, int STAGES, bool GEGLU>
static int launch_tc05(const CUtensorMap& a, const CUtensorMap& b, const Tc05Params& p, cudaStream_t st) {
    static bool attr = false;
    constexpr int smem = tc05_smem<BN, STAGES, GEGLU>();
    static_assert(smem <= 232448, "shared memory budget");
    if (!attr) {
        cudaError_t e = cudaFuncSetAttribute(tc05_gemm_kernel<BN, STAGES, GEGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        attr = true;
    }
    const int total = p.m_tiles * p.n_tiles;
    const int grid = total < sm_count() ? total : sm_count();
    tc05_gemm_kernel<BN, STAGES, GEGLU><<<grid, TC_THREADS, smem, st>>>(a, b, p);
    KATZ_LAUNCH_RET();
}

static int* status_ptr() {
    static int* ptr = nullptr;
    if (!ptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_tc05_status) == cudaSuccess) ptr = (int*)p;
    }
    return ptr;
}

int* tc05_status_device_ptr() { return status_ptr(); }

// Tile width by wave efficiency: tiles of width bn cost ~bn per wave; pick the width with the least total cost.
static int pick_bn(int m_tiles, int n_out, bool geglu) {
    const int sms = sm_count();
    const int cand[3] = {256, 160, 128};
    int best = 128;
    double best_cost = 1e30;
    for (int i = 0; i < 3; ++i) {
        const int bn = cand[i];
        const int out_w = geglu ? bn / 2 : bn;
        const long long tiles = (long long)m_tiles * ceil_div(n_out, out_w);
        const long long waves = (tiles + sms - 1) / sms;
        // per-tile time ~ MMA time (prop. to bn) + fixed overhead per tile (epilogue drain, barrier round trips)
        const double cost = (double)waves * (bn + 24.0);
        if (cost < best_cost) {
            best_cost = cost;
            best = bn;
        }
    }
    return best;
}

template <bool GEGLU>
static int dispatch(const CUtensorMap& a, const CUtensorMap& b, Tc05Params& p, int bn, cudaStream_t st) {
    p.status = status_ptr();
    if (!p.status) return KATZ_ENOTREADY;
    if (bn == 256) return launch_tc05<256, 4, GEGLU>(a, b, p, st);
    if (bn == 160) return launch_tc05<160, 6, GEGLU>(a, b, p, st);
    return launch_tc05<128, 6, GEGLU>(a, b, p, st);
}

}  // namespace katz

using namespace katz;

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
                         float out_scale, int geglu_F, void* stream) {
    KATZ_CHECK_ARG(A && W && C, KATZ_EINVAL);
    KATZ_CHECK_ARG(M > 0 && N_out > 0 && K > 0, KATZ_ESIZE);
    KATZ_CHECK_ARG(K % TBK == 0 && N_out % 8 == 0, KATZ_ESIZE);
    KATZ_CHECK_ARG(lda % 8 == 0 && ldc % 8 == 0, KATZ_EALIGN);
    KATZ_CHECK_ARG(aligned16(A) && aligned16(W) && aligned16(C), KATZ_EALIGN);
    KATZ_CHECK_ARG(!bias || aligned16(bias), KATZ_EALIGN);
    KATZ_CHECK_ARG(!rowvec || (aligned16(rowvec) && ld_rowvec % 8 == 0 && rows_per_batch > 0), KATZ_EALIGN);
    KATZ_CHECK_ARG(!residual || (aligned16(residual) && ldr % 8 == 0), KATZ_EALIGN);
    CUtensorMap ta, tb;
    int rc = encode_2d(&ta, A, K, M, (uint64_t)lda * 2, TBK, TBM);
    if (rc) return rc;
    Tc05Params p{};
    p.C = (__half*)C; p.bias = (const __half*)bias; p.rowvec = (const __half*)rowvec; p.residual = (const __half*)residual;
    p.M = M; p.N = N_out; p.K = K; p.ldc = ldc; p.ldr = ldr; p.ld_rowvec = ld_rowvec; p.rows_per_batch = rows_per_batch;
    p.act = act; p.out_scale = out_scale; p.geglu_F = geglu_F;
    p.m_tiles = ceil_div(M, TBM);
    KATZ_CHECK_ARG((long long)p.m_tiles * ceil_div(N_out, 64) < (1ll << 30), KATZ_ESIZE);
    const bool geglu = geglu_F > 0;
    const int bn = pick_bn(p.m_tiles, N_out, geglu);
    const int out_w = geglu ? bn / 2 : bn;
    p.n_tiles = ceil_div(N_out, out_w);
    const uint64_t w_rows = geglu ? 2ull * geglu_F : (uint64_t)N_out;
    rc = encode_2d(&tb, W, K, w_rows, (uint64_t)K * 2, TBK, geglu ? bn / 2 : bn);
    if (rc) return rc;
    return geglu ? dispatch<true>(ta, tb, p, bn, (cudaStream_t)stream) : dispatch<false>(ta, tb, p, bn, (cudaStream_t)stream);
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

extern "C" int katz_conv3x3_nhwc_f16(const void* X, const void* W, void* Y, int B, int Hin, int Wd, int Cin, int Cout,
                                     int pad_h, const void* bias, const void* rowvec, int ld_rowvec, const void* residual, int act,
                                     float out_scale, void* stream) {
    KATZ_CHECK_ARG(X && W && Y, KATZ_EINVAL);
    KATZ_CHECK_ARG(B > 0 && Hin > 0 && Wd > 0 && Cin > 0 && Cout > 0, KATZ_ESIZE);
    KATZ_CHECK_ARG(pad_h == 0 || pad_h == 1, KATZ_EINVAL);
    const int H = Hin + 2 * pad_h - 2;   // output rows
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
    int rc = encode_nhwc(&ta, X, B, Hin, Wd, Cin, TW, TH);
    if (rc) return rc;
    Tc05Params p{};
    p.C = (__half*)Y; p.bias = (const __half*)bias; p.rowvec = (const __half*)rowvec; p.residual = (const __half*)residual;
    p.M = B * H * Wd; p.N = Cout; p.K = 9 * Cin; p.ldc = Cout; p.ldr = Cout; p.ld_rowvec = ld_rowvec; p.rows_per_batch = H * Wd;
    p.act = act; p.out_scale = out_scale;
    p.conv = 1; p.H = H; p.W = Wd; p.TW = TW; p.TH = TH; p.tiles_w = Wd / TW; p.tiles_h = ceil_div(H, TH);
    p.cin_chunks = Cin / TBK; p.ksize = 3; p.pad_h = pad_h; p.pad_w = 1;
    p.m_tiles = B * p.tiles_w * p.tiles_h;
    const int bn = pick_bn(p.m_tiles, Cout, false);
    p.n_tiles = ceil_div(Cout, bn);
    rc = encode_2d(&tb, W, (uint64_t)9 * Cin, Cout, (uint64_t)9 * Cin * 2, TBK, bn);
    if (rc) return rc;
    return dispatch<false>(ta, tb, p, bn, (cudaStream_t)stream);
}
