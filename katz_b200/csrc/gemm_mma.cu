// Implicit-GEMM on the legacy mma.sync tensor path: C[M,N] = gather(A)[M,K] * W[N,K]^T (+ epilogue).
//
// This is the general-shape kernel: it takes any stride / padding / kernel size, a fused nearest-2x
// upsample of the input, a channel-concatenated pair of inputs, and ragged M/N/K. The tcgen05 kernels
// (gemm_tc05.cu) cover the large aligned shapes; whatever they decline runs here.
//
// Replaces the library calls the reference makes for nn.Linear
// (diffusers/models/attention_processor.py:1256-1284, attention.py:649, activations.py:145-149) and
// nn.Conv2d (resnet.py:378,408; downsampling.py:147; upsampling.py:180-184).
#include "common.cuh"
#include "katz_b200.h"

namespace katz {

constexpr int BM = 128, BN = 128, BK = 32, STAGES = 4, NTHREADS = 256;
constexpr int STAGE_BYTES = (BM + BN) * BK * 2;
constexpr int IGEMM_SMEM = STAGES * STAGE_BYTES;

struct IgemmParams {
    const __half* A;
    const __half* A2;
    const __half* W;
    __half* C;
    const __half* bias;
    const __half* rowvec;
    const __half* residual;
    int M, N, K;
    int lda, ldc, ldr, ld_rowvec, rows_per_batch;
    // conv geometry (logical input Hin x Win is the post-upsample size)
    int Hin, Win, C1, C2, Hout, Wout, ksize, stride, pad_h, pad_w, upsample;
    int act;
    float out_scale;
};

template <bool CONV>
__global__ void __launch_bounds__(NTHREADS) igemm_kernel(const IgemmParams p) {
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    pdl_launch_dependents();
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int warp_m = warp & 1, warp_n = warp >> 1;
    const int bm = blockIdx.x * BM, bn = blockIdx.y * BN;      // row tiles on x: a 2048 x 2048 image has more than 65535 of them
    const int Cin = p.C1 + p.C2;

    // ---- loader bookkeeping: each thread moves two A chunks and two W chunks of 16 B per stage
    const int lrow = tid >> 2, lchunk = tid & 3;
    int a_b[2], a_oy[2], a_ox[2];
    bool a_ok[2];
    const __half* a_rowptr[2];
    const __half* w_rowptr[2];
    bool w_ok[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        int m = bm + lrow + i * 64;
        a_ok[i] = m < p.M;
        int mm = a_ok[i] ? m : 0;
        if (CONV) {
            int hw = p.Hout * p.Wout;
            a_b[i] = mm / hw;
            int r = mm - a_b[i] * hw;
            a_oy[i] = r / p.Wout;
            a_ox[i] = r - a_oy[i] * p.Wout;
            a_rowptr[i] = nullptr;
        } else {
            a_rowptr[i] = p.A + (size_t)mm * p.lda;
            a_b[i] = a_oy[i] = a_ox[i] = 0;
        }
        int n = bn + lrow + i * 64;
        w_ok[i] = n < p.N;
        w_rowptr[i] = p.W + (size_t)(w_ok[i] ? n : 0) * p.K;
    }
    const int Hs = p.upsample ? (p.Hin >> 1) : p.Hin;
    const int Ws = p.upsample ? (p.Win >> 1) : p.Win;

    auto load_stage = [&](int stage, int kt) {
        unsigned char* sA = smem + stage * STAGE_BYTES;
        unsigned char* sB = sA + BM * BK * 2;
        const int k = kt * BK + lchunk * 8;
        const bool k_ok = k < p.K;
        int ky = 0, kx = 0, c = 0;
        if (CONV && k_ok) {
            int tap = k / Cin;
            c = k - tap * Cin;
            ky = tap / p.ksize;
            kx = tap - ky * p.ksize;
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = lrow + i * 64;
            const uint32_t off = r * 64 + ((lchunk ^ ((r >> 1) & 3)) << 4);
            // A
            {
                const __half* src = p.A;
                int bytes = 0;
                if (k_ok && a_ok[i]) {
                    if (CONV) {
                        int iy = a_oy[i] * p.stride - p.pad_h + ky;
                        int ix = a_ox[i] * p.stride - p.pad_w + kx;
                        if (iy >= 0 && iy < p.Hin && ix >= 0 && ix < p.Win) {
                            if (p.upsample) {
                                iy >>= 1;
                                ix >>= 1;
                            }
                            size_t pix = ((size_t)a_b[i] * Hs + iy) * Ws + ix;
                            src = (c < p.C1) ? p.A + pix * p.C1 + c : p.A2 + pix * p.C2 + (c - p.C1);
                            bytes = 16;
                        }
                    } else {
                        src = a_rowptr[i] + k;
                        bytes = 16;
                    }
                }
                cp_async16(smem_u32(sA + off), src, bytes);
            }
            // W
            {
                const __half* src = p.W;
                int bytes = 0;
                if (k_ok && w_ok[i]) {
                    src = w_rowptr[i] + k;
                    bytes = 16;
                }
                cp_async16(smem_u32(sB + off), src, bytes);
            }
        }
    };

    float acc[4][4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

    const int KT = ceil_div(p.K, BK);
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < KT) load_stage(s, s);
        cp_async_commit();
    }

    for (int kt = 0; kt < KT; ++kt) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        {
            int nk = kt + STAGES - 1;
            if (nk < KT) load_stage(nk % STAGES, nk);
            cp_async_commit();
        }
        const unsigned char* sA = smem + (kt % STAGES) * STAGE_BYTES;
        const unsigned char* sB = sA + BM * BK * 2;
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
            uint32_t af[4][4], bf[4][2];
#pragma unroll
            for (int mf = 0; mf < 4; ++mf) {
                int r = warp_m * 64 + mf * 16 + (lane & 15);
                int ch = ks * 2 + (lane >> 4);
                uint32_t addr = smem_u32(sA + r * 64 + ((ch ^ ((r >> 1) & 3)) << 4));
                ldmatrix_x4(af[mf][0], af[mf][1], af[mf][2], af[mf][3], addr);
            }
#pragma unroll
            for (int np = 0; np < 2; ++np) {
                int r = warp_n * 32 + np * 16 + (lane & 7) + ((lane >> 4) << 3);
                int ch = ks * 2 + ((lane >> 3) & 1);
                uint32_t addr = smem_u32(sB + r * 64 + ((ch ^ ((r >> 1) & 3)) << 4));
                ldmatrix_x4(bf[np * 2][0], bf[np * 2][1], bf[np * 2 + 1][0], bf[np * 2 + 1][1], addr);
            }
#pragma unroll
            for (int mf = 0; mf < 4; ++mf)
#pragma unroll
                for (int nf = 0; nf < 4; ++nf) mma_f16_16816(acc[mf][nf], af[mf], bf[nf]);
        }
    }
    cp_async_wait<0>();

    // ---- epilogue: bias, per-batch row vector, activation, residual, scale
#pragma unroll
    for (int mf = 0; mf < 4; ++mf) {
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
            const int m = bm + warp_m * 64 + mf * 16 + (lane >> 2) + hrow * 8;
            if (m >= p.M) continue;
            const int bidx = p.rowvec ? (m / p.rows_per_batch) : 0;
#pragma unroll
            for (int nf = 0; nf < 4; ++nf) {
                const int n = bn + warp_n * 32 + nf * 8 + (lane & 3) * 2;
                if (n >= p.N) continue;
                float v0 = acc[mf][nf][hrow * 2], v1 = acc[mf][nf][hrow * 2 + 1];
                const bool pair = (n + 1 < p.N);
                if (p.bias) {
                    v0 += __half2float(p.bias[n]);
                    if (pair) v1 += __half2float(p.bias[n + 1]);
                }
                if (p.rowvec) {
                    const __half* rv = p.rowvec + (size_t)bidx * p.ld_rowvec + n;
                    v0 += __half2float(rv[0]);
                    if (pair) v1 += __half2float(rv[1]);
                }
                if (p.act == 1) {
                    v0 = silu_f(v0);
                    v1 = silu_f(v1);
                }
                if (p.residual) {
                    const __half* rp = p.residual + (size_t)m * p.ldr + n;
                    v0 += __half2float(rp[0]);
                    if (pair) v1 += __half2float(rp[1]);
                }
                v0 *= p.out_scale;
                v1 *= p.out_scale;
                __half* cp = p.C + (size_t)m * p.ldc + n;
                if (pair && ((reinterpret_cast<uintptr_t>(cp) & 3) == 0)) {
                    *reinterpret_cast<__half2*>(cp) = __floats2half2_rn(v0, v1);
                } else {
                    cp[0] = __float2half_rn(v0);
                    if (pair) cp[1] = __float2half_rn(v1);
                }
            }
        }
    }
}

static int launch_igemm(const IgemmParams& p, bool conv, cudaStream_t st) {
    static bool attr_dev[KATZ_MAX_DEVICES] = {false};
    bool& attr_set = attr_dev[current_device_index()];
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(igemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, IGEMM_SMEM);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(igemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, IGEMM_SMEM);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    dim3 grid(ceil_div(p.M, BM), ceil_div(p.N, BN));
    if (grid.y > 65535) return KATZ_ESIZE;
    if (conv)
        launch_k(igemm_kernel<true>, grid, NTHREADS, IGEMM_SMEM, st, p);
    else
        launch_k(igemm_kernel<false>, grid, NTHREADS, IGEMM_SMEM, st, p);
    KATZ_LAUNCH_RET();
}

}  // namespace katz

using namespace katz;

extern "C" int katz_linear_f16_mma(const void* A, int lda, const void* W, void* C, int ldc, int M, int N, int K,
                                   const void* bias, const void* rowvec, int ld_rowvec, int rows_per_batch,
                                   const void* residual, int ldr, int act, float out_scale, void* stream) {
    KATZ_CHECK_ARG(A && W && C, KATZ_EINVAL);
    KATZ_CHECK_ARG(M > 0 && N > 0 && K > 0, KATZ_ESIZE);
    KATZ_CHECK_ARG(K % 8 == 0 && lda % 8 == 0, KATZ_EALIGN);
    KATZ_CHECK_ARG(aligned16(A) && aligned16(W), KATZ_EALIGN);
    KATZ_CHECK_ARG(!rowvec || rows_per_batch > 0, KATZ_EINVAL);
    IgemmParams p{};
    p.A = (const __half*)A;
    p.W = (const __half*)W;
    p.C = (__half*)C;
    p.bias = (const __half*)bias;
    p.rowvec = (const __half*)rowvec;
    p.residual = (const __half*)residual;
    p.M = M; p.N = N; p.K = K;
    p.lda = lda; p.ldc = ldc; p.ldr = ldr; p.ld_rowvec = ld_rowvec; p.rows_per_batch = rows_per_batch;
    p.act = act; p.out_scale = out_scale;
    return launch_igemm(p, false, (cudaStream_t)stream);
}

extern "C" int katz_conv2d_nhwc_f16_mma(const void* X, const void* X2, const void* W, void* Y, int B, int Hin, int Win,
                                        int C1, int C2, int Cout, int ksize, int stride, int pad_h, int pad_w, int upsample,
                                        const void* bias, const void* rowvec, int ld_rowvec, const void* residual,
                                        int act, float out_scale, void* stream) {
    KATZ_CHECK_ARG(X && W && Y, KATZ_EINVAL);
    KATZ_CHECK_ARG(B > 0 && Hin > 0 && Win > 0 && C1 > 0 && Cout > 0 && C2 >= 0, KATZ_ESIZE);
    KATZ_CHECK_ARG(C2 == 0 || X2, KATZ_EINVAL);
    KATZ_CHECK_ARG(C1 % 8 == 0 && C2 % 8 == 0, KATZ_EALIGN);
    KATZ_CHECK_ARG(aligned16(X) && aligned16(W) && (!X2 || aligned16(X2)), KATZ_EALIGN);
    KATZ_CHECK_ARG(ksize >= 1 && stride >= 1 && pad_h >= 0 && pad_w >= 0, KATZ_EINVAL);
    KATZ_CHECK_ARG(!upsample || (Hin % 2 == 0 && Win % 2 == 0), KATZ_EINVAL);
    IgemmParams p{};
    p.A = (const __half*)X;
    p.A2 = (const __half*)X2;
    p.W = (const __half*)W;
    p.C = (__half*)Y;
    p.bias = (const __half*)bias;
    p.rowvec = (const __half*)rowvec;
    p.residual = (const __half*)residual;
    p.Hin = Hin; p.Win = Win; p.C1 = C1; p.C2 = C2;
    p.ksize = ksize; p.stride = stride; p.pad_h = pad_h; p.pad_w = pad_w; p.upsample = upsample;
    p.Hout = (Hin + 2 * pad_h - ksize) / stride + 1;
    p.Wout = (Win + 2 * pad_w - ksize) / stride + 1;
    KATZ_CHECK_ARG(p.Hout > 0 && p.Wout > 0, KATZ_ESIZE);
    long long M = (long long)B * p.Hout * p.Wout;
    KATZ_CHECK_ARG(M < (1ll << 31), KATZ_ESIZE);
    p.M = (int)M; p.N = Cout; p.K = ksize * ksize * (C1 + C2);
    p.ldc = Cout; p.ldr = Cout; p.ld_rowvec = ld_rowvec; p.rows_per_batch = p.Hout * p.Wout;
    p.act = act; p.out_scale = out_scale;
    return launch_igemm(p, true, (cudaStream_t)stream);
}
