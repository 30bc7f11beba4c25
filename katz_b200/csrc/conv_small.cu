// Direct 3x3 convolution (padding 1, stride 1 or 2) for NHWC tensors with FEW channels: the layers of the ControlNet
// conditioning embedding (controlnet.py:113-127: 3 -> 16 -> 16 -> 32 -> 32 -> 96 -> 96 -> 256 channels on a 1024 x 1024
// image, SiLU after each) whose input has at most 32 channels, which nn.Conv2d / cuDNN run in the reference. These layers are bound by moving the image, not
// by arithmetic, and an implicit GEMM with 128-wide output tiles spends its time on padding: 16 output channels fill an
// eighth of a tile, and every k-slice re-gathers the input.
//
// Here a CTA owns a tile of TH x 32 output pixels. It brings the input patch of the tile (with its one-pixel border,
// zeros outside the image) and the weights of up to NC (16, 32 or 64) output channels into shared memory ONCE, and its eight warps run
// mma.sync m16n8k16 over (tap, 16-channel chunk): A fragments are ldmatrix reads of 16 neighbouring pixels at the tap's
// offset in the patch, B fragments are ldmatrix reads of the weights. Pixel rows of the patch and weight rows carry 16
// bytes of padding so that the eight rows of an ldmatrix fall into different banks. Bias and SiLU in the epilogue.
#include "common.cuh"
#include "katz_b200.h"

namespace katz {

constexpr int CS_TW = 32;            // output pixels per tile row
constexpr int CS_THREADS = 256;      // eight warps

struct ConvSmallParams {
    const __half* X;
    const __half* W;
    const __half* bias;
    __half* Y;
    int B, Hin, Win, Cin, Cout, Hout, Wout, pad_h, act;
    int n_split;      // output-channel passes spread over grid.z (1: one CTA runs all passes over its patch)
};

// CIN: input channels as held in shared memory (a multiple of 16; 8 real channels are padded with zeros). S: stride.
// TH output rows per CTA: 8 with stride 1 (each warp one row: two blocks of 16 pixels), 4 with stride 2 (each warp one
// block of 16 pixels). NC: output channels per pass over the patch.
template <int CIN, int S, int NC>
__global__ void __launch_bounds__(CS_THREADS) conv3x3_small_kernel(const ConvSmallParams p) {
    constexpr int TH = S == 1 ? 8 : 4;
    constexpr int MB = S == 1 ? 2 : 1;                     // 16-pixel blocks per warp
    constexpr int PH = (TH - 1) * S + 3, PW = (CS_TW - 1) * S + 3;      // patch size in input pixels
    constexpr int PS = CIN * 2 + 16;                       // bytes of a patch pixel (padded)
    constexpr int WS = 9 * CIN * 2 + 16;                   // bytes of a weight row (one output channel, padded)
    constexpr int KC = CIN / 16;                           // 16-channel chunks per tap
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    pdl_launch_dependents();
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* s_patch = smem;
    unsigned char* s_w = smem + ((PH * PW * PS + 127) / 128) * 128;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int ox0 = blockIdx.x * CS_TW, oy0 = blockIdx.y * TH, b = blockIdx.z / p.n_split, pass = blockIdx.z - b * p.n_split;
    const int iy0 = oy0 * S - p.pad_h, ix0 = ox0 * S - 1;
    const int cin_chunks = p.Cin / 8;                      // 16-byte chunks that exist in global memory per pixel

    // ---- input patch -> shared memory (zeros outside the image and in the channel padding)
    constexpr int CH = CIN / 8;                            // 16-byte chunks per patch pixel
    for (int idx = tid; idx < PH * PW * CH; idx += CS_THREADS) {
        const int c = idx % CH, pix = idx / CH;
        const int py = pix / PW, px = pix - py * PW;
        const int iy = iy0 + py, ix = ix0 + px;
        const bool ok = c < cin_chunks && iy >= 0 && iy < p.Hin && ix >= 0 && ix < p.Win;
        const __half* src = ok ? p.X + (((size_t)b * p.Hin + iy) * p.Win + ix) * p.Cin + c * 8 : p.X;
        cp_async16(smem_u32(s_patch + pix * PS + c * 16), src, ok ? 16 : 0);
    }
    cp_async_commit();

    const int my_row = S == 1 ? warp : warp >> 1;          // output row of this warp inside the tile
    const int my_x0 = S == 1 ? 0 : (warp & 1) * 16;        // first output column of its first 16-pixel block

    const int n_first = p.n_split > 1 ? pass * NC : 0, n_end = p.n_split > 1 ? min(p.Cout, n_first + NC) : p.Cout;
    for (int n0 = n_first; n0 < n_end; n0 += NC) {
        const int nc = min(NC, p.Cout - n0);            // output channels of this pass (a multiple of 8)
        __syncthreads();                                   // the previous pass has finished reading s_w
        // ---- weights of this pass: rows n0 .. n0+nc-1, [tap][CIN] with zero padding of missing input channels
        for (int idx = tid; idx < NC * 9 * CH; idx += CS_THREADS) {
            const int c = idx % CH, t = (idx / CH) % 9, n = idx / (9 * CH);
            const bool ok = n < nc && c < cin_chunks;
            const __half* src = ok ? p.W + ((size_t)(n0 + n) * 9 + t) * p.Cin + c * 8 : p.W;
            cp_async16(smem_u32(s_w + n * WS + (t * CIN + c * 8) * 2), src, ok ? 16 : 0);
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();

        float acc[MB][NC / 8][4];
#pragma unroll
        for (int m = 0; m < MB; ++m)
#pragma unroll
            for (int j = 0; j < NC / 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[m][j][e] = 0.f;
        const int nb = nc / 8;                             // 8-channel blocks of this pass

#pragma unroll 1
        for (int t = 0; t < 9; ++t) {
            const int ky = t / 3, kx = t - ky * 3;
#pragma unroll
            for (int kc = 0; kc < KC; ++kc) {
                uint32_t af[MB][4];
#pragma unroll
                for (int m = 0; m < MB; ++m) {
                    // 16 neighbouring output pixels of one row: matrices (pixels 0-7 | 8-15) x (channels 0-7 | 8-15)
                    const int px = (my_x0 + m * 16 + (lane & 15)) * S + kx, py = my_row * S + ky;
                    const uint32_t addr = smem_u32(s_patch + (py * PW + px) * PS + (kc * 16 + (lane >> 4) * 8) * 2);
                    ldmatrix_x4(af[m][0], af[m][1], af[m][2], af[m][3], addr);
                }
#pragma unroll
                for (int j = 0; j < NC / 8; j += 2) {
                    if (j < nb) {
                        uint32_t bf[4];
                        const int n = j * 8 + (lane & 7) + ((lane >> 4) << 3);
                        const uint32_t addr = smem_u32(s_w + n * WS + (t * CIN + kc * 16 + ((lane >> 3) & 1) * 8) * 2);
                        ldmatrix_x4(bf[0], bf[1], bf[2], bf[3], addr);
#pragma unroll
                        for (int m = 0; m < MB; ++m) {
                            mma_f16_16816(acc[m][j], af[m], bf);
                            mma_f16_16816(acc[m][j + 1], af[m], bf + 2);
                        }
                    }
                }
            }
        }

        // ---- epilogue: bias, SiLU, fp16 pairs
        const int oy = oy0 + my_row;
        if (oy < p.Hout) {
#pragma unroll
            for (int m = 0; m < MB; ++m) {
#pragma unroll
                for (int hrow = 0; hrow < 2; ++hrow) {
                    const int ox = ox0 + my_x0 + m * 16 + (lane >> 2) + hrow * 8;
                    if (ox >= p.Wout) continue;
                    __half* yp = p.Y + (((size_t)b * p.Hout + oy) * p.Wout + ox) * p.Cout + n0;
#pragma unroll
                    for (int j = 0; j < NC / 8; ++j) {
                        const int n = j * 8 + (lane & 3) * 2;
                        if (n >= nc) continue;
                        float v0 = acc[m][j][hrow * 2], v1 = acc[m][j][hrow * 2 + 1];
                        if (p.bias) {
                            const float2 bb = __half22float2(*reinterpret_cast<const __half2*>(p.bias + n0 + n));
                            v0 += bb.x;
                            v1 += bb.y;
                        }
                        if (p.act == 1) {
                            v0 = silu_f(v0);
                            v1 = silu_f(v1);
                        }
                        *reinterpret_cast<__half2*>(yp + n) = __floats2half2_rn(v0, v1);
                    }
                }
            }
        }
    }
}

template <int CIN, int S, int NC>
static int launch_conv_small(const ConvSmallParams& p, cudaStream_t st) {
    constexpr int TH = S == 1 ? 8 : 4;
    constexpr int PH = (TH - 1) * S + 3, PW = (CS_TW - 1) * S + 3;
    constexpr int PS = CIN * 2 + 16, WS = 9 * CIN * 2 + 16;
    constexpr int smem = ((PH * PW * PS + 127) / 128) * 128 + NC * WS;
    static_assert(smem <= 227 * 1024, "patch and weights must fit shared memory");
    static bool attr_dev[KATZ_MAX_DEVICES] = {false};
    bool& attr = attr_dev[current_device_index()];
    if (!attr) {
        cudaError_t e = cudaFuncSetAttribute(conv3x3_small_kernel<CIN, S, NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        attr = true;
    }
    // a layer with many output channels on a small image (the UNet's conv_in: 8 -> 320 channels at 128 x 128) has few
    // tiles and many passes: with a patch this cheap to reload, the passes go on the grid as well
    ConvSmallParams q = p;
    const int passes = ceil_div(p.Cout, NC);
    const long long tiles = (long long)ceil_div(p.Wout, CS_TW) * ceil_div(p.Hout, TH) * p.B;
    q.n_split = (CIN <= 16 && passes > 1 && tiles < 592) ? passes : 1;
    dim3 grid(ceil_div(p.Wout, CS_TW), ceil_div(p.Hout, TH), p.B * q.n_split);
    if (grid.y > 65535 || grid.z > 65535) return KATZ_ESIZE;
    launch_k(conv3x3_small_kernel<CIN, S, NC>, grid, CS_THREADS, smem, st, q);
    KATZ_LAUNCH_RET();
}

}  // namespace katz

using namespace katz;

extern "C" int katz_conv3x3_small_nhwc_f16(const void* X, const void* W, void* Y, int B, int Hin, int Win, int Cin, int Cout,
                                           int stride, int pad_h, const void* bias, int act, void* stream) {
    KATZ_CHECK_ARG(X && W && Y, KATZ_EINVAL);
    KATZ_CHECK_ARG(B > 0 && Hin > 0 && Win > 0, KATZ_ESIZE);
    KATZ_CHECK_ARG(Cin == 8 || Cin == 16 || Cin == 32, KATZ_ESIZE);
    KATZ_CHECK_ARG(Cout > 0 && Cout % 8 == 0 && Cout <= 1024, KATZ_ESIZE);
    KATZ_CHECK_ARG((stride == 1 || stride == 2) && (pad_h == 0 || pad_h == 1) && (act == 0 || act == 1), KATZ_EINVAL);
    KATZ_CHECK_ARG(aligned16(X) && aligned16(W) && aligned16(Y) && (!bias || aligned16(bias)), KATZ_EALIGN);
    ConvSmallParams p{};
    p.X = (const __half*)X; p.W = (const __half*)W; p.bias = (const __half*)bias; p.Y = (__half*)Y;
    p.B = B; p.Hin = Hin; p.Win = Win; p.Cin = Cin; p.Cout = Cout; p.pad_h = pad_h; p.act = act;
    p.Hout = (Hin + 2 * pad_h - 3) / stride + 1;
    p.Wout = (Win + 2 - 3) / stride + 1;
    KATZ_CHECK_ARG(p.Hout > 0 && p.Wout > 0, KATZ_ESIZE);
    cudaStream_t st = (cudaStream_t)stream;
    // NC, the output channels per pass, sets the accumulator registers: narrow layers take a narrow NC so that more CTAs
    // share an SM (a CTA's life is mostly the latency of its one patch load)
    const int nc = Cout <= 16 ? 16 : Cout <= 32 ? 32 : 64;
    if (Cin <= 16) {
        if (stride == 1) return nc == 16 ? launch_conv_small<16, 1, 16>(p, st) : nc == 32 ? launch_conv_small<16, 1, 32>(p, st) : launch_conv_small<16, 1, 64>(p, st);
        return nc == 16 ? launch_conv_small<16, 2, 16>(p, st) : nc == 32 ? launch_conv_small<16, 2, 32>(p, st) : launch_conv_small<16, 2, 64>(p, st);
    }
    if (stride == 1) return nc == 16 ? launch_conv_small<32, 1, 16>(p, st) : nc == 32 ? launch_conv_small<32, 1, 32>(p, st) : launch_conv_small<32, 1, 64>(p, st);
    return nc == 16 ? launch_conv_small<32, 2, 16>(p, st) : nc == 32 ? launch_conv_small<32, 2, 32>(p, st) : launch_conv_small<32, 2, 64>(p, st);
}
