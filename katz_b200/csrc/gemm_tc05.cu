// tcgen05 GEMM / implicit-GEMM 3x3 convolution: C[M,N] = A[M,K] * W[N,K]^T with a fused epilogue.
//
//   * operands: TMA tile loads (128-byte swizzle) into a multi-stage shared-memory ring, one elected thread;
//   * math: tcgen05.mma kind::f16, 128 x BN x 16 per instruction, fp32 accumulator in TMEM, one elected thread;
//   * epilogue: four warps read TMEM with tcgen05.ld, add bias / per-batch row vector / residual, apply SiLU and
//     write fp16 with 16-byte stores.
// Linear layers read A through a 2-D tensor map; the 3x3 stride-1 convolution reads the NHWC activation through a
// 4-D tensor map as nine shifted tile loads per channel chunk (out-of-image pixels arrive as zeros), so no im2col
// buffer exists. One CTA computes one 128 x BN output tile; with BN = 128 two CTAs share an SM so one tile's epilogue
// overlaps the other's main loop.
//
// Every mbarrier wait is bounded (tc05.cuh): on a time-out the CTA records a status word, skips its stores, frees its
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

struct Tc05Params {
    __half* C;
    const __half* bias;
    const __half* rowvec;
    const __half* residual;
    int M, N, K;
    int ldc, ldr, ld_rowvec, rows_per_batch;
    int act;
    float out_scale;
    // convolution geometry (stride 1, output size = input size)
    int conv, H, W, TW, TH, tiles_w, tiles_h, cin_chunks, ksize, pad;
    int* status;
};

__device__ int g_tc05_status = 0;

template <int BN, int STAGES>
__global__ void __launch_bounds__(TC_THREADS) tc05_gemm_kernel(const __grid_constant__ CUtensorMap tmA,
                                                               const __grid_constant__ CUtensorMap tmB, const Tc05Params p) {
    constexpr int A_BYTES = TBM * TBK * 2;
    constexpr int B_BYTES = BN * TBK * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    extern __shared__ unsigned char smem_raw[];
    // 1024-byte alignment: the swizzle pattern and the UMMA descriptors assume it
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES), tfull = smem_u32(bars + 2 * STAGES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BN;
    int m0 = 0, cb = 0, ch0 = 0, cw0 = 0;
    if (p.conv) {
        const int tpi = p.tiles_w * p.tiles_h;
        cb = blockIdx.y / tpi;
        const int r = blockIdx.y - cb * tpi;
        const int ty = r / p.tiles_w;
        ch0 = ty * p.TH;
        cw0 = (r - ty * p.tiles_w) * p.TW;
    } else {
        m0 = blockIdx.y * TBM;
    }
    const int KT = p.K / TBK;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(tfull, 1);
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), BN);
        tmem_relinquish();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    bool ok = true;
    if (warp == 0) {
        // ------------------------------------------------------------------------------------ TMA producer
        if (elect_one()) {
            int issued = 0;
            for (int kt = 0; kt < KT; ++kt) {
                const int s = kt % STAGES;
                const uint32_t ph = (kt / STAGES) & 1;
                if (!mbar_wait(empty0 + 8 * s, ph ^ 1)) { ok = false; break; }
                const uint32_t fb = full0 + 8 * s;
                mbar_expect_tx(fb, STAGE_BYTES);
                const uint32_t sa = smem_base + s * STAGE_BYTES;
                if (p.conv) {
                    const int tap = kt / p.cin_chunks;
                    const int cc = kt - tap * p.cin_chunks;
                    const int ky = tap / p.ksize, kx = tap - ky * p.ksize;
                    tma_load_4d(sa, &tmA, cc * TBK, cw0 + kx - p.pad, ch0 + ky - p.pad, cb, fb);
                } else {
                    tma_load_2d(sa, &tmA, kt * TBK, m0, fb);
                }
                tma_load_2d(sa + A_BYTES, &tmB, kt * TBK, n0, fb);
                issued = kt + 1;
            }
            if (!ok) {
                atomicExch(p.status, 1);
                // let copies already in flight land before the CTA's shared memory is released
                for (int kt = max(0, issued - STAGES); kt < issued; ++kt)
                    mbar_wait(full0 + 8 * (kt % STAGES), (kt / STAGES) & 1);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            constexpr uint32_t idesc = idesc_f16(TBM, BN);
            for (int kt = 0; kt < KT; ++kt) {
                const int s = kt % STAGES;
                const uint32_t ph = (kt / STAGES) & 1;
                if (!mbar_wait(full0 + 8 * s, ph)) { ok = false; break; }
                fence_after_sync();
                const uint32_t sa = smem_base + s * STAGE_BYTES;
                const uint64_t ad = smem_desc_sw128(sa), bd = smem_desc_sw128(sa + A_BYTES);
#pragma unroll
                for (int k = 0; k < TBK / 16; ++k) {
                    // +32 bytes per 16-element K step inside the 128-byte swizzle row (encoded >> 4)
                    umma_f16(tmem_base, ad + 2 * k, bd + 2 * k, idesc, (kt | k) != 0);
                }
                umma_commit(empty0 + 8 * s);   // stage reusable once these MMAs have read it
            }
            if (ok) umma_commit(tfull);
            else atomicExch(p.status, 2);
        }
    } else {
        // ------------------------------------------------------------------------------------ epilogue
        const int q = warp & 3;                 // TMEM lane quarter this warp may read
        const int row = q * 32 + lane;
        ok = mbar_wait(tfull, 0);
        ok = __all_sync(0xffffffffu, ok);   // tcgen05.ld below is warp-collective: decide as a warp
        if (!ok && lane == 0) atomicExch(p.status, 3);
        fence_after_sync();
        long long m;
        bool valid;
        int bidx;
        if (p.conv) {
            const int th = row / p.TW, tw = row - th * p.TW;
            const int h = ch0 + th;
            valid = h < p.H;
            m = ((long long)cb * p.H + h) * p.W + cw0 + tw;
            bidx = cb;
        } else {
            m = m0 + row;
            valid = m < p.M;
            bidx = p.rowvec ? (int)(m / p.rows_per_batch) : 0;
        }
        valid = valid && ok;
#pragma unroll 1
        for (int chunk = 0; chunk < BN / 32; ++chunk) {
            uint32_t r[32];
            if (ok) {
                tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + chunk * 32, r);
                tmem_ld_wait();
            }
            if (!valid) continue;
#pragma unroll
            for (int g8 = 0; g8 < 4; ++g8) {
                const int nb = n0 + chunk * 32 + g8 * 8;
                if (nb >= p.N) break;
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[g8 * 8 + e]);
                if (p.bias) {
                    const uint4 u = *reinterpret_cast<const uint4*>(p.bias + nb);
                    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float2 f = unpack_half2(w[e]);
                        v[2 * e] += f.x;
                        v[2 * e + 1] += f.y;
                    }
                }
                if (p.rowvec) {
                    const uint4 u = *reinterpret_cast<const uint4*>(p.rowvec + (size_t)bidx * p.ld_rowvec + nb);
                    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float2 f = unpack_half2(w[e]);
                        v[2 * e] += f.x;
                        v[2 * e + 1] += f.y;
                    }
                }
                if (p.act == 1) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] = silu_f(v[e]);
                }
                if (p.residual) {
                    const uint4 u = *reinterpret_cast<const uint4*>(p.residual + (size_t)m * p.ldr + nb);
                    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float2 f = unpack_half2(w[e]);
                        v[2 * e] += f.x;
                        v[2 * e + 1] += f.y;
                    }
                }
                uint4 o;
                o.x = pack_half2(v[0] * p.out_scale, v[1] * p.out_scale);
                o.y = pack_half2(v[2] * p.out_scale, v[3] * p.out_scale);
                o.z = pack_half2(v[4] * p.out_scale, v[5] * p.out_scale);
                o.w = pack_half2(v[6] * p.out_scale, v[7] * p.out_scale);
                *reinterpret_cast<uint4*>(p.C + (size_t)m * p.ldc + nb) = o;
            }
        }
    }
    // ---------------------------------------------------------------------------------------- teardown
    fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        fence_after_sync();
        tmem_dealloc(tmem_base, BN);
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

template <int BN, int STAGES>
static constexpr int tc05_smem() {
    return STAGES * (TBM * TBK * 2 + BN * TBK * 2) + (2 * STAGES + 1) * 8 + 16 + 1024;
}

template <int BN, int STAGES>
static int launch_tc05(const CUtensorMap& a, const CUtensorMap& b, const Tc05Params& p, dim3 grid, cudaStream_t st) {
    static bool attr = false;
    constexpr int smem = tc05_smem<BN, STAGES>();
    if (!attr) {
        cudaError_t e = cudaFuncSetAttribute(tc05_gemm_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        attr = true;
    }
    tc05_gemm_kernel<BN, STAGES><<<grid, TC_THREADS, smem, st>>>(a, b, p);
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

static int dispatch(const CUtensorMap& a, const CUtensorMap& b, Tc05Params& p, int m_tiles, cudaStream_t st) {
    p.status = status_ptr();
    if (!p.status) return KATZ_ENOTREADY;
    // Tile width: 256 halves the A-operand re-reads per MMA when the grid still fills the machine; 128 otherwise,
    // with the shallow ring when two CTAs can share an SM.
    const int t256 = ceil_div(p.N, 256) * m_tiles, t128 = ceil_div(p.N, 128) * m_tiles;
    if (m_tiles > 65535) return KATZ_ESIZE;
    if (p.N % 256 == 0 && t256 >= 148) return launch_tc05<256, 4>(a, b, p, dim3(ceil_div(p.N, 256), m_tiles), st);
    if (t128 > 148) return launch_tc05<128, 3>(a, b, p, dim3(ceil_div(p.N, 128), m_tiles), st);
    return launch_tc05<128, 6>(a, b, p, dim3(ceil_div(p.N, 128), m_tiles), st);
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

extern "C" int katz_linear_f16(const void* A, int lda, const void* W, void* C, int ldc, int M, int N, int K,
                               const void* bias, const void* rowvec, int ld_rowvec, int rows_per_batch,
                               const void* residual, int ldr, int act, float out_scale, void* stream) {
    KATZ_CHECK_ARG(A && W && C, KATZ_EINVAL);
    KATZ_CHECK_ARG(M > 0 && N > 0 && K > 0, KATZ_ESIZE);
    KATZ_CHECK_ARG(K % TBK == 0 && N % 8 == 0, KATZ_ESIZE);
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
    p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.ldr = ldr; p.ld_rowvec = ld_rowvec; p.rows_per_batch = rows_per_batch;
    p.act = act; p.out_scale = out_scale;
    const int m_tiles = ceil_div(M, TBM);
    const int t256 = ceil_div(N, 256) * m_tiles;
    const int bn = (N % 256 == 0 && t256 >= 148) ? 256 : 128;
    rc = encode_2d(&tb, W, K, N, (uint64_t)K * 2, TBK, bn);
    if (rc) return rc;
    return dispatch(ta, tb, p, m_tiles, (cudaStream_t)stream);
}

extern "C" int katz_conv3x3_nhwc_f16(const void* X, const void* W, void* Y, int B, int H, int Wd, int Cin, int Cout,
                                     const void* bias, const void* rowvec, int ld_rowvec, const void* residual, int act,
                                     float out_scale, void* stream) {
    KATZ_CHECK_ARG(X && W && Y, KATZ_EINVAL);
    KATZ_CHECK_ARG(B > 0 && H > 0 && Wd > 0 && Cin > 0 && Cout > 0, KATZ_ESIZE);
    KATZ_CHECK_ARG(Cin % TBK == 0 && Cout % 8 == 0, KATZ_ESIZE);
    const int TW = Wd < 128 ? Wd : 128;
    KATZ_CHECK_ARG((TW & (TW - 1)) == 0 && TW >= 8 && Wd % TW == 0, KATZ_ESIZE);
    const int TH = 128 / TW;
    KATZ_CHECK_ARG(aligned16(X) && aligned16(W) && aligned16(Y), KATZ_EALIGN);
    KATZ_CHECK_ARG(!bias || aligned16(bias), KATZ_EALIGN);
    KATZ_CHECK_ARG(!rowvec || (aligned16(rowvec) && ld_rowvec % 8 == 0), KATZ_EALIGN);
    KATZ_CHECK_ARG(!residual || aligned16(residual), KATZ_EALIGN);
    CUtensorMap ta, tb;
    int rc = encode_nhwc(&ta, X, B, H, Wd, Cin, TW, TH);
    if (rc) return rc;
    Tc05Params p{};
    p.C = (__half*)Y; p.bias = (const __half*)bias; p.rowvec = (const __half*)rowvec; p.residual = (const __half*)residual;
    p.M = B * H * Wd; p.N = Cout; p.K = 9 * Cin; p.ldc = Cout; p.ldr = Cout; p.ld_rowvec = ld_rowvec; p.rows_per_batch = H * Wd;
    p.act = act; p.out_scale = out_scale;
    p.conv = 1; p.H = H; p.W = Wd; p.TW = TW; p.TH = TH; p.tiles_w = Wd / TW; p.tiles_h = ceil_div(H, TH);
    p.cin_chunks = Cin / TBK; p.ksize = 3; p.pad = 1;
    const int m_tiles = B * p.tiles_w * p.tiles_h;
    const int t256 = ceil_div(Cout, 256) * m_tiles;
    const int bn = (Cout % 256 == 0 && t256 >= 148) ? 256 : 128;
    rc = encode_2d(&tb, W, (uint64_t)9 * Cin, Cout, (uint64_t)9 * Cin * 2, TBK, bn);
    if (rc) return rc;
    return dispatch(ta, tb, p, m_tiles, (cudaStream_t)stream);
}
