// Small streaming kernels of the UNet step: GEGLU gating, residual intake, embeddings, layout moves, Euler/CFG.
#include "common.cuh"
#include "katz_b200.h"

namespace katz {

__device__ __forceinline__ float rh(float v) { return __half2float(__float2half_rn(v)); }

// fast_kernel::fast_gelu_mul_fp16 (fast_kernel/csrc/gelu.cuh:29-42): half arithmetic with one float tanh,
// out = 0.5*x*(1+tanh(0.79788456*(x+0.044715*x^3)))*m, every intermediate rounded to half as the reference does.
__device__ __forceinline__ float fast_gelu_mul_one(float x, float m) {
    const float alpha = rh(0.7978845608028654f), beta = rh(0.044714998453855515f);
    float t = rh(beta * x);
    t = rh(t * x);
    t = rh(t * x);
    t = rh(x + t);
    t = rh(alpha * t);
    float th = rh(tanhf(t));
    float r = rh(0.5f * x);
    r = rh(r * rh(1.0f + th));
    return rh(r * m);
}

__global__ void fast_gelu_mul_kernel(const __half2* __restrict__ x, const __half2* __restrict__ m, __half2* __restrict__ out,
                                     long long npairs) {
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    pdl_launch_dependents();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < npairs; i += (long long)gridDim.x * blockDim.x) {
        float2 xv = __half22float2(x[i]), mv = __half22float2(m[i]);
        out[i] = __floats2half2_rn(fast_gelu_mul_one(xv.x, mv.x), fast_gelu_mul_one(xv.y, mv.y));
    }
}

// The same on 16-byte packs of eight halves (the reference op moves packs of that size, elementwise.cuh:113-124);
// the launcher takes it when the three pointers are 16-byte aligned, and leaves the tail (n % 8) to the pair kernel.
__global__ void fast_gelu_mul_v8_kernel(const uint4* __restrict__ x, const uint4* __restrict__ m, uint4* __restrict__ out,
                                        long long npacks) {
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    pdl_launch_dependents();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < npacks; i += (long long)gridDim.x * blockDim.x) {
        uint4 xv = x[i], mv = m[i], o;
        const __half2* xh = reinterpret_cast<const __half2*>(&xv);
        const __half2* mh = reinterpret_cast<const __half2*>(&mv);
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float2 a = __half22float2(xh[k]), b = __half22float2(mh[k]);
            oh[k] = __floats2half2_rn(fast_gelu_mul_one(a.x, b.x), fast_gelu_mul_one(a.y, b.y));
        }
        out[i] = o;
    }
}

// Unfused GEGLU of the reference torch path (activations.py:146-149): h, g = chunk(proj(x)); h * gelu(g), erf GELU,
// gelu result and product each rounded to half as torch's fp16 ops do.
__global__ void geglu_erf_kernel(const __half* __restrict__ hg, __half* __restrict__ out, long long M, int F, int ld) {
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    pdl_launch_dependents();
    const int FP = F >> 1;
    const long long total = M * FP;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        long long r = i / FP;
        int c = (int)(i - r * FP) * 2;
        const __half* row = hg + r * ld;
        float2 h = __half22float2(*reinterpret_cast<const __half2*>(row + c));
        float2 g = __half22float2(*reinterpret_cast<const __half2*>(row + F + c));
        float o0 = rh(gelu_erf_f(g.x)) * h.x, o1 = rh(gelu_erf_f(g.y)) * h.y;
        *reinterpret_cast<__half2*>(out + r * F + c) = __floats2half2_rn(o0, o1);
    }
}

// dst = dst_in + sum_i scale_i * r_i  (ControlNet intake, unet_2d_condition.py:1281-1292,1418-1439)
struct IntakeArgs {
    const __half* r[8];
    float scale[8];
    int n;
};
__global__ void residual_intake_kernel(const __half2* __restrict__ src, __half2* __restrict__ dst, IntakeArgs a,
                                       long long npairs) {
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    pdl_launch_dependents();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < npairs; i += (long long)gridDim.x * blockDim.x) {
        float2 acc = make_float2(0.f, 0.f);
        for (int k = 0; k < a.n; ++k) {
            float2 v = __half22float2(reinterpret_cast<const __half2*>(a.r[k])[i]);
            acc.x += v.x * a.scale[k];
            acc.y += v.y * a.scale[k];
        }
        // the reference sums the nets in fp16, then adds to the skip tensor in fp16
        float2 s = __half22float2(src[i]);
        dst[i] = __floats2half2_rn(s.x + rh(acc.x), s.y + rh(acc.y));
    }
}

// get_timestep_embedding (embeddings.py:26-66) with flip_sin_to_cos=True, downscale_freq_shift=0, scale=1:
// out[r, 0:half] = cos(t_r * f_i), out[r, half:dim] = sin(t_r * f_i), f_i = exp(-ln(10000) * i / half)
__global__ void timestep_embedding_kernel(const float* __restrict__ t, __half* __restrict__ out, int rows, int dim,
                                          int ld_out) {
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    pdl_launch_dependents();
    const int half_dim = dim >> 1;
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * half_dim) return;
    int r = i / half_dim, j = i - r * half_dim;
    float f = expf(-9.210340371976184f * (float)j / (float)half_dim);
    float a = t[r] * f;
    out[(size_t)r * ld_out + j] = __float2half_rn(cosf(a));
    out[(size_t)r * ld_out + half_dim + j] = __float2half_rn(sinf(a));
}

__global__ void silu_kernel(const __half2* __restrict__ x, __half2* __restrict__ y, long long npairs) {
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    pdl_launch_dependents();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < npairs; i += (long long)gridDim.x * blockDim.x) {
        float2 v = __half22float2(x[i]);
        y[i] = __floats2half2_rn(silu_f(v.x), silu_f(v.y));
    }
}

__global__ void add_kernel(const __half2* __restrict__ a, const __half2* __restrict__ b, __half2* __restrict__ y,
                           long long npairs) {
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    pdl_launch_dependents();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < npairs; i += (long long)gridDim.x * blockDim.x) {
        float2 u = __half22float2(a[i]), v = __half22float2(b[i]);
        y[i] = __floats2half2_rn(u.x + v.x, u.y + v.y);
    }
}

// NCHW (C real channels) -> NHWC with the channel count padded to Cpad (zeros), and back.
__global__ void nchw_to_nhwc_kernel(const __half* __restrict__ x, __half* __restrict__ y, int B, int C, int HW, int Cpad) {
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    pdl_launch_dependents();
    long long total = (long long)B * HW * Cpad;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        int c = (int)(i % Cpad);
        long long p = i / Cpad;
        int hw = (int)(p % HW);
        int b = (int)(p / HW);
        y[i] = c < C ? x[((size_t)b * C + c) * HW + hw] : __float2half(0.f);
    }
}
__global__ void nhwc_to_nchw_kernel(const __half* __restrict__ x, __half* __restrict__ y, int B, int C, int HW, int Cpad) {
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    pdl_launch_dependents();
    long long total = (long long)B * C * HW;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        int hw = (int)(i % HW);
        long long p = i / HW;
        int c = (int)(p % C);
        int b = (int)(p / C);
        y[i] = x[((size_t)b * HW + hw) * Cpad + c];
    }
}

// torch evaluates `tensor / cpu_scalar` and `cpu_scalar * half_tensor` differently on the two devices the reference
// can run on; both are reproduced bit for bit:
//   mode 0 (torch on CUDA, the reference's serving path): division by a host scalar is a multiplication by its fp32
//          reciprocal, and the fp32 sigma multiplies the fp16 prediction at full precision;
//   mode 1 (torch on CPU): true division, and sigma is rounded to fp16 before `sigma * model_output`.
//
// scale_model_input (scheduling_euler_discrete.py:294-295): the fp16 latent divided by sqrt(sigma^2 + 1) (sigma is an
// fp32 scalar, so torch keeps the result in fp16), optionally written twice (batch-2 CFG input).
__global__ void euler_scale_input_kernel(const __half* __restrict__ x, __half* __restrict__ out, long long n, float sigma,
                                         int copies, int mode) {
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    pdl_launch_dependents();
    // sigma**2, + 1, ** 0.5 are three separately rounded fp32 operations in the reference: no fused multiply-add
    const float den = __fsqrt_rn(__fadd_rn(__fmul_rn(sigma, sigma), 1.0f));
    const float inv = __fdiv_rn(1.0f, den);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float xv = __half2float(x[i]);
        __half h = __float2half_rn(mode == 0 ? __fmul_rn(xv, inv) : __fdiv_rn(xv, den));
        for (int c = 0; c < copies; ++c) out[(size_t)c * n + i] = h;
    }
}

// CFG combine (pipeline_controlnet_sd_xl_katz.py:1649-1655) + EulerDiscreteScheduler.step
// (scheduling_euler_discrete.py:498-537) with s_churn = 0, epsilon prediction. eps = u + g*(c-u) in fp16; the step
// upcasts the fp16 latent to fp32: pred_x0 = x - half(sigma*eps); d = (x - pred_x0)/sigma; x' = half(x + d*dt).
__global__ void euler_cfg_step_kernel(__half* __restrict__ x, const __half* __restrict__ eps_uncond,
                                      const __half* __restrict__ eps_cond, long long n, float guidance, float sigma,
                                      float sigma_next, int mode) {
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    pdl_launch_dependents();
    const float dt = __fsub_rn(sigma_next, sigma);
    const float sigma_mul = mode == 0 ? sigma : rh(sigma);
    const float inv_sigma = __fdiv_rn(1.0f, sigma);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float u = __half2float(eps_uncond[i]);
        float e = u;
        if (eps_cond) {
            float c = __half2float(eps_cond[i]);
            e = rh(u + rh(guidance * rh(c - u)));
        }
        float xv = __half2float(x[i]);
        // each torch op rounds on its own: keep the compiler from contracting them into fused multiply-adds
        float pred = __fsub_rn(xv, rh(__fmul_rn(sigma_mul, e)));
        float num = __fsub_rn(xv, pred);
        float d = mode == 0 ? __fmul_rn(num, inv_sigma) : __fdiv_rn(num, sigma);
        x[i] = __float2half_rn(__fadd_rn(xv, __fmul_rn(d, dt)));
    }
}

// y[r, :] = x1[r, :C1] ++ x2[r, :C2], 16-byte chunks (C1, C2 multiples of 8)
// The index type is 32-bit whenever the element count allows: these kernels move 16 bytes per index, and the 64-bit
// divisions that split a flat index cost more instructions than the copy itself.
template <typename I>
__global__ void concat_channels_kernel(const uint4* __restrict__ x1, const uint4* __restrict__ x2, uint4* __restrict__ y,
                                       long long rows, int ch1, int ch2) {
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    pdl_launch_dependents();
    const I ch = (I)(ch1 + ch2);
    const I total = (I)(rows * (ch1 + ch2));
    for (I i = (I)blockIdx.x * (I)blockDim.x + threadIdx.x; i < total; i += (I)gridDim.x * (I)blockDim.x) {
        const I r = i / ch;
        const int c = (int)(i - r * ch);
        y[i] = c < ch1 ? x1[(size_t)r * ch1 + c] : x2[(size_t)r * ch2 + (c - ch1)];
    }
}

// Nearest-neighbour 2x upsample of an NHWC tensor (Upsample2D's F.interpolate, upsampling.py:165-172), 16-byte chunks.
template <typename I>
__global__ void upsample2x_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, int B, int H, int W, int ch) {
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    pdl_launch_dependents();
    const I total = (I)((long long)B * (2 * H) * (2 * W) * ch);
    for (I i = (I)blockIdx.x * (I)blockDim.x + threadIdx.x; i < total; i += (I)gridDim.x * (I)blockDim.x) {
        I p = i / (I)ch;
        const int c = (int)(i - p * (I)ch);
        const I q = p / (I)(2 * W);
        const int ox = (int)(p - q * (I)(2 * W));
        const I b = q / (I)(2 * H);
        const int oy = (int)(q - b * (I)(2 * H));
        y[i] = x[(((size_t)b * H + (oy >> 1)) * W + (ox >> 1)) * ch + c];
    }
}

// y[r, :] = softmax(x[r, :]) over `cols` fp16 logits, fp32 arithmetic: the probabilities of the VAE's one-head attention
// (attention_processor.py:1276 for a head of 512 channels, which the 64-channel flash kernels do not cover; its scores
// come from a GEMM). One CTA per row; a row of up to 256 * 8 * SM_MAXV logits stays in registers between the passes.
constexpr int SM_THREADS = 256, SM_MAXV = 8;
__global__ void __launch_bounds__(SM_THREADS) softmax_rows_kernel(const __half* __restrict__ x, __half* __restrict__ y, int cols,
                                                                  long long ld_x, long long ld_y) {
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    pdl_launch_dependents();
    __shared__ float red[SM_THREADS / 32];
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const uint4* xr = reinterpret_cast<const uint4*>(x + (long long)blockIdx.x * ld_x);
    uint4* yr = reinterpret_cast<uint4*>(y + (long long)blockIdx.x * ld_y);
    const int packs = cols >> 3;
    uint4 v[SM_MAXV];
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < SM_MAXV; ++i) {
        const int p = tid + i * SM_THREADS;
        if (p < packs) {
            v[i] = xr[p];
            const __half2* h = reinterpret_cast<const __half2*>(&v[i]);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float2 f = __half22float2(h[k]);
                m = fmaxf(m, fmaxf(f.x, f.y));
            }
        }
    }
    m = warp_max(m);
    if (lane == 0) red[wid] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int w = 1; w < SM_THREADS / 32; ++w) m = fmaxf(m, red[w]);
    __syncthreads();
    const float L2E = 1.4426950408889634f, ml = m * L2E;
    float e[SM_MAXV][8];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < SM_MAXV; ++i) {
        if (tid + i * SM_THREADS < packs) {
            const __half2* h = reinterpret_cast<const __half2*>(&v[i]);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float2 f = __half22float2(h[k]);
                e[i][2 * k] = ex2_fast(fmaf(f.x, L2E, -ml));
                e[i][2 * k + 1] = ex2_fast(fmaf(f.y, L2E, -ml));
                sum += e[i][2 * k] + e[i][2 * k + 1];
            }
        }
    }
    sum = warp_sum(sum);
    if (lane == 0) red[wid] = sum;
    __syncthreads();
    sum = 0.f;
#pragma unroll
    for (int w = 0; w < SM_THREADS / 32; ++w) sum += red[w];       // fixed order: every thread gets the same bits
    const float inv = 1.0f / sum;
#pragma unroll
    for (int i = 0; i < SM_MAXV; ++i) {
        const int p = tid + i * SM_THREADS;
        if (p < packs) {
            uint4 o;
            __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
            for (int k = 0; k < 4; ++k) oh[k] = __floats2half2_rn(e[i][2 * k] * inv, e[i][2 * k + 1] * inv);
            yr[p] = o;
        }
    }
}

static inline int ew_grid(long long n, int threads) {
    long long g = (n + threads - 1) / threads;
    long long cap = 148ll * 16;
    return (int)(g < cap ? (g > 0 ? g : 1) : cap);
}

}  // namespace katz

using namespace katz;

extern "C" int katz_fast_gelu_mul_f16(const void* x, const void* m, void* out, long long n, void* stream) {
    KATZ_CHECK_ARG(x && m && out, KATZ_EINVAL);
    KATZ_CHECK_ARG(n > 0 && n % 2 == 0, KATZ_ESIZE);
    KATZ_CHECK_ARG(((uintptr_t)x & 3) == 0 && ((uintptr_t)m & 3) == 0 && ((uintptr_t)out & 3) == 0, KATZ_EALIGN);
    long long done = 0;
    if ((((uintptr_t)x | (uintptr_t)m | (uintptr_t)out) & 15) == 0 && n >= 8) {
        done = n & ~7ll;
        launch_k(fast_gelu_mul_v8_kernel, ew_grid(done / 8, 256), 256, 0, (cudaStream_t)stream, (const uint4*)x, (const uint4*)m,
                 (uint4*)out, done / 8);
        if (done == n) KATZ_LAUNCH_RET();
    }
    launch_k(fast_gelu_mul_kernel, ew_grid((n - done) / 2, 256), 256, 0, (cudaStream_t)stream, (const __half2*)((const __half*)x + done),
             (const __half2*)((const __half*)m + done), (__half2*)((__half*)out + done), (n - done) / 2);
    KATZ_LAUNCH_RET();
}

extern "C" int katz_geglu_erf_f16(const void* hg, void* out, long long M, int F, int ld, void* stream) {
    KATZ_CHECK_ARG(hg && out, KATZ_EINVAL);
    KATZ_CHECK_ARG(M > 0 && F > 0 && F % 2 == 0 && ld % 2 == 0 && ld >= 2 * F, KATZ_ESIZE);
    KATZ_CHECK_ARG(((uintptr_t)hg & 3) == 0 && ((uintptr_t)out & 3) == 0, KATZ_EALIGN);
    launch_k(geglu_erf_kernel, ew_grid(M * (F / 2), 256), 256, 0, (cudaStream_t)stream, (const __half*)hg, (__half*)out, M, F, ld);
    KATZ_LAUNCH_RET();
}

extern "C" int katz_residual_intake_f16(const void* src, void* dst, const void* const* residuals, const float* scales,
                                        int n_res, long long n, void* stream) {
    KATZ_CHECK_ARG(src && dst && residuals && scales, KATZ_EINVAL);
    KATZ_CHECK_ARG(n_res >= 1 && n_res <= 8, KATZ_ESIZE);
    KATZ_CHECK_ARG(n > 0 && n % 2 == 0, KATZ_ESIZE);
    IntakeArgs a{};
    a.n = n_res;
    for (int i = 0; i < n_res; ++i) {
        KATZ_CHECK_ARG(residuals[i] && ((uintptr_t)residuals[i] & 3) == 0, KATZ_EALIGN);
        a.r[i] = (const __half*)residuals[i];
        a.scale[i] = scales[i];
    }
    launch_k(residual_intake_kernel, ew_grid(n / 2, 256), 256, 0, (cudaStream_t)stream, (const __half2*)src, (__half2*)dst, a, n / 2);
    KATZ_LAUNCH_RET();
}

extern "C" int katz_timestep_embedding_f16(const float* t, void* out, int rows, int dim, int ld_out, void* stream) {
    KATZ_CHECK_ARG(t && out, KATZ_EINVAL);
    KATZ_CHECK_ARG(rows > 0 && dim > 0 && dim % 2 == 0 && ld_out >= dim, KATZ_ESIZE);
    int n = rows * (dim / 2);
    launch_k(timestep_embedding_kernel, ceil_div(n, 128), 128, 0, (cudaStream_t)stream, t, (__half*)out, rows, dim, ld_out);
    KATZ_LAUNCH_RET();
}

// Row shard [B, h, W, C] -> the input a 3x3 convolution of the shard reads: the neighbours' adjacent rows (zeros at the
// image edge) attached above and / or below, optionally seen through a nearest 2x upsample (then rows [1, 2h+3) of the
// upsampled padded shard, 2W wide: exactly what the 2h output rows read). One pass instead of an allocation, three
// copies, an upsample and a slice copy. `edges` is the all-gather of every rank's first and last row, [P][2][B][W][C].
template <typename I>
__global__ void halo_assemble_kernel(const uint4* __restrict__ x, const uint4* __restrict__ edges, uint4* __restrict__ out,
                                     int B, int h, int W, int ch, int Ho, int Wo, int top, int upsample, int rank, int world,
                                     long long total_) {
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    pdl_launch_dependents();
    const I total = (I)total_;
    for (I i = (I)blockIdx.x * (I)blockDim.x + threadIdx.x; i < total; i += (I)gridDim.x * (I)blockDim.x) {
        I r = i / (I)ch;
        const int c = (int)(i - r * (I)ch);
        const I r2 = r / (I)Wo;
        const int w = (int)(r - r2 * (I)Wo);
        const int b = (int)(r2 / (I)Ho);
        const int j = (int)(r2 - (I)b * (I)Ho);
        const int sr = upsample ? (j + 1) / 2 - 1 : j - top;
        const int sw = upsample ? w >> 1 : w;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (sr >= 0 && sr < h) {
            v = x[(((long long)b * h + sr) * W + sw) * ch + c];
        } else if (edges) {
            const int p = sr < 0 ? rank - 1 : rank + 1, e = sr < 0 ? 1 : 0;      // the neighbour's last / first row
            if (p >= 0 && p < world) v = edges[((((long long)p * 2 + e) * B + b) * W + sw) * ch + c];
        }
        out[i] = v;
    }
}

extern "C" int katz_halo_assemble_f16(const void* x, const void* edges, void* out, int B, int h, int W, int C, int top,
                                      int bottom, int upsample, int rank, int world, void* stream) {
    KATZ_CHECK_ARG(x && out, KATZ_EINVAL);
    KATZ_CHECK_ARG(B > 0 && h > 0 && W > 0 && C > 0 && C % 8 == 0, KATZ_ESIZE);
    KATZ_CHECK_ARG((top == 0 || top == 1) && (bottom == 0 || bottom == 1) && world >= 1 && rank >= 0 && rank < world, KATZ_EINVAL);
    KATZ_CHECK_ARG(!upsample || (top == 1 && bottom == 1), KATZ_EINVAL);
    KATZ_CHECK_ARG(world == 1 || edges, KATZ_EINVAL);
    KATZ_CHECK_ARG(aligned16(x) && aligned16(out) && (!edges || aligned16(edges)), KATZ_EALIGN);
    const int Ho = upsample ? 2 * h + 2 : h + top + bottom, Wo = upsample ? 2 * W : W;
    const long long total = (long long)B * Ho * Wo * (C / 8);
    if (total < (1ll << 31))
        launch_k(halo_assemble_kernel<unsigned int>, ew_grid(total, 256), 256, 0, (cudaStream_t)stream, (const uint4*)x,
                 (const uint4*)edges, (uint4*)out, B, h, W, C / 8, Ho, Wo, top, upsample, rank, world, total);
    else
        launch_k(halo_assemble_kernel<long long>, ew_grid(total, 256), 256, 0, (cudaStream_t)stream, (const uint4*)x,
                 (const uint4*)edges, (uint4*)out, B, h, W, C / 8, Ho, Wo, top, upsample, rank, world, total);
    KATZ_LAUNCH_RET();
}

extern "C" int katz_softmax_rows_f16(const void* x, void* y, int rows, int cols, long long ld_x, long long ld_y, void* stream) {
    KATZ_CHECK_ARG(x && y, KATZ_EINVAL);
    KATZ_CHECK_ARG(rows > 0 && cols > 0 && cols % 8 == 0 && cols <= SM_THREADS * 8 * SM_MAXV, KATZ_ESIZE);
    KATZ_CHECK_ARG(ld_x >= cols && ld_y >= cols && ld_x % 8 == 0 && ld_y % 8 == 0, KATZ_ESIZE);
    KATZ_CHECK_ARG((((uintptr_t)x | (uintptr_t)y) & 15) == 0, KATZ_EALIGN);
    launch_k(softmax_rows_kernel, rows, SM_THREADS, 0, (cudaStream_t)stream, (const __half*)x, (__half*)y, cols, ld_x, ld_y);
    KATZ_LAUNCH_RET();
}

extern "C" int katz_silu_f16(const void* x, void* y, long long n, void* stream) {
    KATZ_CHECK_ARG(x && y, KATZ_EINVAL);
    KATZ_CHECK_ARG(n > 0 && n % 2 == 0, KATZ_ESIZE);
    launch_k(silu_kernel, ew_grid(n / 2, 256), 256, 0, (cudaStream_t)stream, (const __half2*)x, (__half2*)y, n / 2);
    KATZ_LAUNCH_RET();
}

extern "C" int katz_add_f16(const void* a, const void* b, void* y, long long n, void* stream) {
    KATZ_CHECK_ARG(a && b && y, KATZ_EINVAL);
    KATZ_CHECK_ARG(n > 0 && n % 2 == 0, KATZ_ESIZE);
    launch_k(add_kernel, ew_grid(n / 2, 256), 256, 0, (cudaStream_t)stream, (const __half2*)a, (const __half2*)b, (__half2*)y, n / 2);
    KATZ_LAUNCH_RET();
}

extern "C" int katz_concat_channels_f16(const void* x1, const void* x2, void* y, long long rows, int C1, int C2,
                                        void* stream) {
    KATZ_CHECK_ARG(x1 && x2 && y, KATZ_EINVAL);
    KATZ_CHECK_ARG(rows > 0 && C1 > 0 && C2 > 0 && C1 % 8 == 0 && C2 % 8 == 0, KATZ_ESIZE);
    KATZ_CHECK_ARG(aligned16(x1) && aligned16(x2) && aligned16(y), KATZ_EALIGN);
    long long n = rows * ((C1 + C2) / 8);
    if (n < (1ll << 31))
        launch_k(concat_channels_kernel<unsigned int>, ew_grid(n, 256), 256, 0, (cudaStream_t)stream, (const uint4*)x1,
                 (const uint4*)x2, (uint4*)y, rows, C1 / 8, C2 / 8);
    else
        launch_k(concat_channels_kernel<long long>, ew_grid(n, 256), 256, 0, (cudaStream_t)stream, (const uint4*)x1,
                 (const uint4*)x2, (uint4*)y, rows, C1 / 8, C2 / 8);
    KATZ_LAUNCH_RET();
}

extern "C" int katz_upsample_nearest2x_nhwc_f16(const void* x, void* y, int B, int H, int W, int C, void* stream) {
    KATZ_CHECK_ARG(x && y, KATZ_EINVAL);
    KATZ_CHECK_ARG(B > 0 && H > 0 && W > 0 && C > 0 && C % 8 == 0, KATZ_ESIZE);
    KATZ_CHECK_ARG(aligned16(x) && aligned16(y), KATZ_EALIGN);
    long long n = (long long)B * 4 * H * W * (C / 8);
    if (n < (1ll << 31))
        launch_k(upsample2x_kernel<unsigned int>, ew_grid(n, 256), 256, 0, (cudaStream_t)stream, (const uint4*)x, (uint4*)y, B, H, W, C / 8);
    else
        launch_k(upsample2x_kernel<long long>, ew_grid(n, 256), 256, 0, (cudaStream_t)stream, (const uint4*)x, (uint4*)y, B, H, W, C / 8);
    KATZ_LAUNCH_RET();
}

extern "C" int katz_nchw_to_nhwc_f16(const void* x, void* y, int B, int C, int HW, int Cpad, void* stream) {
    KATZ_CHECK_ARG(x && y, KATZ_EINVAL);
    KATZ_CHECK_ARG(B > 0 && C > 0 && HW > 0 && Cpad >= C, KATZ_ESIZE);
    long long n = (long long)B * HW * Cpad;
    launch_k(nchw_to_nhwc_kernel, ew_grid(n, 256), 256, 0, (cudaStream_t)stream, (const __half*)x, (__half*)y, B, C, HW, Cpad);
    KATZ_LAUNCH_RET();
}

extern "C" int katz_nhwc_to_nchw_f16(const void* x, void* y, int B, int C, int HW, int Cpad, void* stream) {
    KATZ_CHECK_ARG(x && y, KATZ_EINVAL);
    KATZ_CHECK_ARG(B > 0 && C > 0 && HW > 0 && Cpad >= C, KATZ_ESIZE);
    long long n = (long long)B * HW * C;
    launch_k(nhwc_to_nchw_kernel, ew_grid(n, 256), 256, 0, (cudaStream_t)stream, (const __half*)x, (__half*)y, B, C, HW, Cpad);
    KATZ_LAUNCH_RET();
}

extern "C" int katz_euler_scale_input(const void* x, void* out, long long n, float sigma, int copies, int mode,
                                      void* stream) {
    KATZ_CHECK_ARG(x && out, KATZ_EINVAL);
    KATZ_CHECK_ARG(n > 0 && copies >= 1, KATZ_ESIZE);
    launch_k(euler_scale_input_kernel, ew_grid(n, 256), 256, 0, (cudaStream_t)stream, (const __half*)x, (__half*)out, n, sigma,
             copies, mode);
    KATZ_LAUNCH_RET();
}

extern "C" int katz_euler_cfg_step(void* x, const void* eps_uncond, const void* eps_cond, long long n, float guidance,
                                   float sigma, float sigma_next, int mode, void* stream) {
    KATZ_CHECK_ARG(x && eps_uncond, KATZ_EINVAL);
    KATZ_CHECK_ARG(n > 0 && sigma != 0.f, KATZ_ESIZE);
    launch_k(euler_cfg_step_kernel, ew_grid(n, 256), 256, 0, (cudaStream_t)stream, (__half*)x, (const __half*)eps_uncond,
                                                                           (const __half*)eps_cond, n, guidance, sigma, sigma_next, mode);
    KATZ_LAUNCH_RET();
}
