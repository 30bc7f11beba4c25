// GroupNorm (+ optional SiLU) and LayerNorm, fp16 in/out, fp32 statistics.
//
// GroupNorm replaces fast_kernel::group_norm_fp16 (fast_kernel/csrc/group_norm.cu:155-274, which lowers to the
// LayerNorm kernels of normalize.cuh:558-834 with one CTA per (batch, group) row: 64 CTAs at SDXL shapes) and
// torch's nn.GroupNorm in Transformer2DModel (transformer_2d.py:173-175). Here the NHWC tensor is cut into row
// slabs so the grid covers every SM: a statistics pass writes one (sum, sum of squares) partial per
// (batch, slab, group) into caller-provided scratch, and the apply pass folds the partials in fp64 and normalises.
//
// LayerNorm replaces nn.LayerNorm(C, eps=1e-5, affine) of BasicTransformerBlock (attention.py:195,225,253).
#include "common.cuh"
#include "katz_b200.h"

namespace katz {

constexpr int GN_THREADS = 256;
constexpr int GN_MAXP = 8;      // channel pairs per thread: C <= 2 * 256 * 8 = 4096
constexpr int GN_MAXG = 64;

__global__ void __launch_bounds__(GN_THREADS) gn_stats_nhwc_kernel(const __half* __restrict__ x, float* __restrict__ partial,
                                                                   int HW, int C, int G, int rows_per_slab) {
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    pdl_launch_dependents();
    // per-thread partials parked in shared memory and summed per group in a FIXED order: the statistics, and with them
    // every GroupNorm output, are bit-reproducible from run to run (no floating-point atomics)
    __shared__ float2 s_part[GN_MAXP][GN_THREADS];
    const int slab = blockIdx.x, b = blockIdx.y, nslab = gridDim.x;
    const int tid = threadIdx.x;
    const int CP = C >> 1, cpg = C / G;
    const int r0 = slab * rows_per_slab;
    const int r1 = min(HW, r0 + rows_per_slab);
    float sum[GN_MAXP], sq[GN_MAXP];
#pragma unroll
    for (int i = 0; i < GN_MAXP; ++i) sum[i] = sq[i] = 0.f;
    const __half2* xb = reinterpret_cast<const __half2*>(x) + (size_t)b * HW * CP;
    for (int r = r0; r < r1; ++r) {
        const __half2* xr = xb + (size_t)r * CP;
#pragma unroll
        for (int i = 0; i < GN_MAXP; ++i) {
            int cp = tid + i * GN_THREADS;
            if (cp < CP) {
                float2 v = __half22float2(xr[cp]);
                sum[i] += v.x + v.y;
                sq[i] += v.x * v.x + v.y * v.y;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < GN_MAXP; ++i) s_part[i][tid] = make_float2(sum[i], sq[i]);
    __syncthreads();
    if (tid < G) {
        const int cp0 = tid * (cpg >> 1), cp1 = cp0 + (cpg >> 1);
        float s = 0.f, q = 0.f;
        for (int cp = cp0; cp < cp1; ++cp) {
            const float2 v = s_part[cp / GN_THREADS][cp % GN_THREADS];
            s += v.x;
            q += v.y;
        }
        float* o = partial + (((size_t)b * nslab + slab) * G + tid) * 2;
        o[0] = s;
        o[1] = q;
    }
}

__global__ void __launch_bounds__(GN_THREADS) gn_apply_nhwc_kernel(const __half* __restrict__ x, __half* __restrict__ y,
                                                                   const float* __restrict__ partial, int nslab_stats,
                                                                   const __half* __restrict__ gamma,
                                                                   const __half* __restrict__ beta, int HW, int C, int G,
                                                                   int rows_per_slab, float eps, int act) {
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    pdl_launch_dependents();
    __shared__ float s_mean[GN_MAXG], s_rstd[GN_MAXG];
    const int slab = blockIdx.x, b = blockIdx.y;
    const int tid = threadIdx.x;
    const int CP = C >> 1, cpg = C / G;
    if (tid < G) {
        double s = 0.0, q = 0.0;
        const float* pp = partial + ((size_t)b * nslab_stats * G + tid) * 2;
        for (int i = 0; i < nslab_stats; ++i) {
            s += (double)pp[(size_t)i * G * 2];
            q += (double)pp[(size_t)i * G * 2 + 1];
        }
        double n = (double)HW * cpg;
        double mean = s / n;
        double var = q / n - mean * mean;
        if (var < 0.0) var = 0.0;
        s_mean[tid] = (float)mean;
        s_rstd[tid] = (float)(1.0 / sqrt(var + (double)eps));
    }
    __syncthreads();
    float sc[GN_MAXP][2], sh[GN_MAXP][2];
#pragma unroll
    for (int i = 0; i < GN_MAXP; ++i) {
        int cp = tid + i * GN_THREADS;
        if (cp < CP) {
            int g = (cp * 2) / cpg;
            float ga0 = gamma ? __half2float(gamma[cp * 2]) : 1.f, ga1 = gamma ? __half2float(gamma[cp * 2 + 1]) : 1.f;
            float be0 = beta ? __half2float(beta[cp * 2]) : 0.f, be1 = beta ? __half2float(beta[cp * 2 + 1]) : 0.f;
            sc[i][0] = s_rstd[g] * ga0;
            sc[i][1] = s_rstd[g] * ga1;
            sh[i][0] = be0 - s_mean[g] * sc[i][0];
            sh[i][1] = be1 - s_mean[g] * sc[i][1];
        }
    }
    const int r0 = slab * rows_per_slab;
    const int r1 = min(HW, r0 + rows_per_slab);
    const __half2* xb = reinterpret_cast<const __half2*>(x) + (size_t)b * HW * CP;
    __half2* yb = reinterpret_cast<__half2*>(y) + (size_t)b * HW * CP;
    for (int r = r0; r < r1; ++r) {
#pragma unroll
        for (int i = 0; i < GN_MAXP; ++i) {
            int cp = tid + i * GN_THREADS;
            if (cp < CP) {
                float2 v = __half22float2(xb[(size_t)r * CP + cp]);
                float a0 = v.x * sc[i][0] + sh[i][0];
                float a1 = v.y * sc[i][1] + sh[i][1];
                if (act == 1) {
                    a0 = silu_f(a0);
                    a1 = silu_f(a1);
                }
                yb[(size_t)r * CP + cp] = __floats2half2_rn(a0, a1);
            }
        }
    }
}

// ---- 16-byte vectorised NHWC kernels (C % 8 == 0). Thread = (row lane, 8-channel chunk): the chunk stays fixed while
// the thread walks rows, so per-channel accumulators (stats) or per-channel scale/shift (apply) live in registers and
// every global access is a full 16-byte load or store with several rows in flight per thread.
// With `mr_out` set the CTA that finishes last for its image (a ticket counter that wraps back to zero, so it needs no
// reset) folds all partials of the image, in a fixed order, into mean and 1/std per group: one fold per image instead of
// one per CTA of the normalising pass.
__global__ void gn_stats_v8_kernel(const __half* __restrict__ x, float* __restrict__ partial, int HW, int C, int G,
                                   int rows_per_slab, int R, float* __restrict__ mr_out, unsigned int* __restrict__ tickets,
                                   double n_total, float eps, double* __restrict__ dsum_out) {
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    pdl_launch_dependents();
    extern __shared__ float s_dyn[];    // [blockDim][16]: 8 channel sums then 8 channel sums of squares
    const int slab = blockIdx.x, b = blockIdx.y, nslab = gridDim.x;
    const int NC = C >> 3, cpg = C / G;
    const int tid = threadIdx.x;
    const int cc = tid % NC, rl = tid / NC;
    const int r0 = slab * rows_per_slab, r1 = min(HW, r0 + rows_per_slab);
    float sm[8], sq[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) sm[e] = sq[e] = 0.f;
    const uint4* xb = reinterpret_cast<const uint4*>(x) + (size_t)b * HW * NC + cc;
    int r = r0 + rl;
    for (; r + 3 * R < r1; r += 4 * R) {
        uint4 u[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) u[k] = xb[(size_t)(r + k * R) * NC];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t w[4] = {u[k].x, u[k].y, u[k].z, u[k].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = unpack_half2(w[e]);
                sm[2 * e] += f.x; sq[2 * e] += f.x * f.x;
                sm[2 * e + 1] += f.y; sq[2 * e + 1] += f.y * f.y;
            }
        }
    }
    for (; r < r1; r += R) {
        const uint4 u = xb[(size_t)r * NC];
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = unpack_half2(w[e]);
            sm[2 * e] += f.x; sq[2 * e] += f.x * f.x;
            sm[2 * e + 1] += f.y; sq[2 * e + 1] += f.y * f.y;
        }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        s_dyn[tid * 16 + e] = sm[e];
        s_dyn[tid * 16 + 8 + e] = sq[e];
    }
    __syncthreads();
    // Up to eight threads per group, each summing a strided subset of the group's (channel, row lane) entries, then a
    // shuffle tree: a fixed summation order, so the statistics are bit-reproducible.
    int lpg = 8;
    while (G * lpg > (int)blockDim.x) lpg >>= 1;
    if ((tid & ~31) < G * lpg) {                  // whole warps take part in the shuffles
        const int g = tid / lpg, sub = tid % lpg;
        float s = 0.f, q = 0.f;
        if (g < G) {
            const int n = cpg * R;
            for (int idx = sub; idx < n; idx += lpg) {
                const int l = idx / cpg, c = g * cpg + (idx - l * cpg);
                const float* e = s_dyn + (l * NC + (c >> 3)) * 16 + (c & 7);
                s += e[0];
                q += e[8];
            }
        }
        for (int o = lpg >> 1; o > 0; o >>= 1) {
            s += __shfl_xor_sync(0xffffffffu, s, o);
            q += __shfl_xor_sync(0xffffffffu, q, o);
        }
        if (g < G && sub == 0) {
            float* o = partial + (((size_t)b * nslab + slab) * G + g) * 2;
            o[0] = s;
            o[1] = q;
            __threadfence();
        }
    }
    if (!mr_out && !dsum_out) return;
    __shared__ int s_last;
    __syncthreads();
    if (tid == 0) s_last = atomicInc(tickets + b, (unsigned int)(nslab - 1)) == (unsigned int)(nslab - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    double* s_part = reinterpret_cast<double*>(s_dyn);      // [parts][G][2]; the per-thread sums above are no longer needed
    int parts = (int)blockDim.x / G;
    if (parts > 16) parts = 16;
    while (parts > 1 && parts * G * 16 > (int)blockDim.x * 64) --parts;
    if (tid < parts * G) {
        const int g = tid % G, part = tid / G;
        double s = 0.0, q = 0.0;
        const float2* pp = reinterpret_cast<const float2*>(partial) + (size_t)b * nslab * G + g;
        for (int i = part; i < nslab; i += parts) {
            const float2 v = __ldcg(pp + (size_t)i * G);
            s += (double)v.x;
            q += (double)v.y;
        }
        s_part[(part * G + g) * 2] = s;
        s_part[(part * G + g) * 2 + 1] = q;
    }
    __syncthreads();
    if (tid < G) {
        double s = 0.0, q = 0.0;
        for (int i = 0; i < parts; ++i) {
            s += s_part[(i * G + tid) * 2];
            q += s_part[(i * G + tid) * 2 + 1];
        }
        if (dsum_out) {
            // a shard of a row-split tensor: hand out the raw sums, the normalising pass adds the shards' sums
            dsum_out[((size_t)b * G + tid) * 2] = s;
            dsum_out[((size_t)b * G + tid) * 2 + 1] = q;
            return;
        }
        const double mean = s / n_total;
        double var = q / n_total - mean * mean;
        if (var < 0.0) var = 0.0;
        mr_out[((size_t)b * G + tid) * 2] = (float)mean;
        mr_out[((size_t)b * G + tid) * 2 + 1] = (float)(1.0 / sqrt(var + (double)eps));
    }
}

__global__ void gn_apply_v8_kernel(const __half* __restrict__ x, __half* __restrict__ y, const float* __restrict__ mr,
                                   const __half* __restrict__ gamma, const __half* __restrict__ beta, int HW,
                                   int C, int G, int rows_per_slab, int R, double n_total, float eps, int act,
                                   const double* __restrict__ dsums, int n_parts) {
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    pdl_launch_dependents();
    extern __shared__ float s_dyn[];    // [C] scale, [C] shift
    __shared__ float s_mean[GN_MAXG], s_rstd[GN_MAXG];
    const int slab = blockIdx.x, b = blockIdx.y;
    const int NC = C >> 3, cpg = C / G;
    const int tid = threadIdx.x;
    if (tid < G && mr) {
        s_mean[tid] = mr[((size_t)b * G + tid) * 2];
        s_rstd[tid] = mr[((size_t)b * G + tid) * 2 + 1];
    } else if (tid < G) {
        // dsums: [n_parts][B][G][2], one part per shard of a row-split tensor, added in part order
        double s = 0.0, q = 0.0;
        for (int i = 0; i < n_parts; ++i) {
            const double* d = dsums + (((size_t)i * gridDim.y + b) * G + tid) * 2;
            s += d[0];
            q += d[1];
        }
        const double mean = s / n_total;
        double var = q / n_total - mean * mean;
        if (var < 0.0) var = 0.0;
        s_mean[tid] = (float)mean;
        s_rstd[tid] = (float)(1.0 / sqrt(var + (double)eps));
    }
    __syncthreads();
    for (int c = tid; c < C; c += blockDim.x) {
        const int g = c / cpg;
        const float ga = gamma ? __half2float(gamma[c]) : 1.f, be = beta ? __half2float(beta[c]) : 0.f;
        const float sc = s_rstd[g] * ga;
        s_dyn[c] = sc;
        s_dyn[C + c] = be - s_mean[g] * sc;
    }
    __syncthreads();
    const int cc = tid % NC, rl = tid / NC;
    float sc[8], sh[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        sc[e] = s_dyn[cc * 8 + e];
        sh[e] = s_dyn[C + cc * 8 + e];
    }
    const int r0 = slab * rows_per_slab, r1 = min(HW, r0 + rows_per_slab);
    const uint4* xb = reinterpret_cast<const uint4*>(x) + (size_t)b * HW * NC + cc;
    uint4* yb = reinterpret_cast<uint4*>(y) + (size_t)b * HW * NC + cc;
    auto norm8 = [&](const uint4& u) -> uint4 {
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = unpack_half2(w[e]);
            float a0 = f.x * sc[2 * e] + sh[2 * e], a1 = f.y * sc[2 * e + 1] + sh[2 * e + 1];
            if (act == 1) {
                a0 = silu_f(a0);
                a1 = silu_f(a1);
            }
            o[e] = pack_half2(a0, a1);
        }
        return make_uint4(o[0], o[1], o[2], o[3]);
    };
    int r = r0 + rl;
    for (; r + 3 * R < r1; r += 4 * R) {
        uint4 u[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) u[k] = xb[(size_t)(r + k * R) * NC];
#pragma unroll
        for (int k = 0; k < 4; ++k) yb[(size_t)(r + k * R) * NC] = norm8(u[k]);
    }
    for (; r < r1; r += R) yb[(size_t)r * NC] = norm8(xb[(size_t)r * NC]);
}

// Folds the per-slab partials of one shard into [B, G, 2] fp64 sums (fixed order): the quantity that is summed across
// ranks when the latent is row-split.
__global__ void gn_fold_kernel(const float* __restrict__ partial, int nslab, int G, double* __restrict__ sums) {
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    pdl_launch_dependents();
    const int b = blockIdx.x, g = threadIdx.x;
    if (g >= G) return;
    double s = 0.0, q = 0.0;
    const float* pp = partial + ((size_t)b * nslab * G + g) * 2;
    for (int i = 0; i < nslab; ++i) {
        s += (double)pp[(size_t)i * G * 2];
        q += (double)pp[(size_t)i * G * 2 + 1];
    }
    sums[((size_t)b * G + g) * 2] = s;
    sums[((size_t)b * G + g) * 2 + 1] = q;
}

// Channels-first variant: each (batch, group) is one contiguous run of (C/G)*HW values.
__global__ void __launch_bounds__(1024) gn_nchw_kernel(const __half* __restrict__ x, __half* __restrict__ y,
                                                       const __half* __restrict__ gamma, const __half* __restrict__ beta,
                                                       int HW, int C, int G, float eps, int act) {
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    pdl_launch_dependents();
    __shared__ double s_a[32], s_b[32];
    __shared__ float s_mean, s_rstd;
    const int g = blockIdx.x, b = blockIdx.y, cpg = C / G;
    const size_t base = ((size_t)b * C + (size_t)g * cpg) * HW;
    const long long n = (long long)cpg * HW;
    double s = 0.0, q = 0.0;
    for (long long i = threadIdx.x; i < n; i += blockDim.x) {
        float v = __half2float(x[base + i]);
        s += v;
        q += (double)v * v;
    }
    for (int o = 16; o > 0; o >>= 1) {
        s += __shfl_xor_sync(0xffffffffu, s, o);
        q += __shfl_xor_sync(0xffffffffu, q, o);
    }
    if ((threadIdx.x & 31) == 0) {
        s_a[threadIdx.x >> 5] = s;
        s_b[threadIdx.x >> 5] = q;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        double ts = 0, tq = 0;
        for (int i = 0; i < (int)(blockDim.x >> 5); ++i) {
            ts += s_a[i];
            tq += s_b[i];
        }
        double mean = ts / (double)n, var = tq / (double)n - mean * mean;
        if (var < 0) var = 0;
        s_mean = (float)mean;
        s_rstd = (float)(1.0 / sqrt(var + (double)eps));
    }
    __syncthreads();
    const float mean = s_mean, rstd = s_rstd;
    for (long long i = threadIdx.x; i < n; i += blockDim.x) {
        int c = g * cpg + (int)(i / HW);
        float ga = gamma ? __half2float(gamma[c]) : 1.f, be = beta ? __half2float(beta[c]) : 0.f;
        float a = (__half2float(x[base + i]) - mean) * rstd * ga + be;
        if (act == 1) a = silu_f(a);
        y[base + i] = __float2half_rn(a);
    }
}

constexpr int LN_MAXCH = 10;  // 16-byte chunks per lane: C <= 32 * 10 * 8 = 2560

template <int MAXCH>
__global__ void __launch_bounds__(256) layer_norm_kernel(const __half* __restrict__ x, __half* __restrict__ y,
                                                         const __half* __restrict__ gamma, const __half* __restrict__ beta,
                                                         int rows, int C, float eps) {
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int nch = C >> 3;
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * C);
    // one warp per row; every global load of the row, of gamma and of beta is requested before anything is consumed
    uint4 xv[MAXCH], gv[MAXCH], bv[MAXCH];
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
        const int ch = lane + i * 32;
        if (ch < nch) xv[i] = xr[ch];
    }
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
        const int ch = lane + i * 32;
        if (ch < nch) {
            gv[i] = __ldg(reinterpret_cast<const uint4*>(gamma) + ch);
            bv[i] = __ldg(reinterpret_cast<const uint4*>(beta) + ch);
        }
    }
    float v[MAXCH][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
        const int ch = lane + i * 32;
        if (ch < nch) {
            const uint32_t w[4] = {xv[i].x, xv[i].y, xv[i].z, xv[i].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = unpack_half2(w[e]);
                v[i][2 * e] = f.x;
                v[i][2 * e + 1] = f.y;
                s += f.x + f.y;
            }
        }
    }
    const float mean = warp_sum(s) / (float)C;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
        const int ch = lane + i * 32;
        if (ch < nch) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float d = v[i][e] - mean;
                q += d * d;
            }
        }
    }
    const float rstd = rsqrtf(warp_sum(q) / (float)C + eps);
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * C);
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
        const int ch = lane + i * 32;
        if (ch < nch) {
            const uint32_t gw[4] = {gv[i].x, gv[i].y, gv[i].z, gv[i].w}, bw[4] = {bv[i].x, bv[i].y, bv[i].z, bv[i].w};
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 gg = unpack_half2(gw[e]), bb = unpack_half2(bw[e]);
                o[e] = pack_half2((v[i][2 * e] - mean) * rstd * gg.x + bb.x, (v[i][2 * e + 1] - mean) * rstd * gg.y + bb.y);
            }
            yr[ch] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
}

// Scratch layout of the NHWC kernels: [0, 1024) one ticket counter per image (zero whenever no call is in flight: the
// counters wrap back by themselves), then mean and 1/std per (image, group), then the per-slab partial sums.
constexpr int GN_MAX_TICKETS = 256;
struct GnScratch {
    unsigned int* tickets;
    float* mr;
    float* partial;
};
static long long gn_partial_offset(int B, int G) { return (1024 + (long long)B * G * 8 + 255) / 256 * 256; }
static GnScratch gn_carve(void* scratch, int B, int G) {
    unsigned char* p = reinterpret_cast<unsigned char*>(scratch);
    return GnScratch{reinterpret_cast<unsigned int*>(p), reinterpret_cast<float*>(p + 1024),
                     reinterpret_cast<float*>(p + gn_partial_offset(B, G))};
}

static int gn_rows_per_slab(int HW, int B) {
    // aim at about 2 CTAs per SM over the whole grid, slabs of at least 8 rows
    int target = (148 * 2 + B - 1) / B;
    int rows = (HW + target - 1) / target;
    if (rows < 8) rows = 8;
    return rows;
}

}  // namespace katz

using namespace katz;

extern "C" long long katz_group_norm_scratch_bytes(int B, int HW, int C, int G) {
    if (B <= 0 || HW <= 0 || G <= 0) return -1;
    int rows = gn_rows_per_slab(HW, B);
    long long nslab = ceil_div(HW, rows);
    return gn_partial_offset(B, G) + (long long)B * nslab * G * 2 * (long long)sizeof(float);
}

extern "C" int katz_group_norm_nhwc_f16(const void* x, void* y, const void* gamma, const void* beta, int B, int HW, int C,
                                        int G, float eps, int act, void* scratch, long long scratch_bytes,
                                        void* stream) {
    KATZ_CHECK_ARG(x && y && scratch, KATZ_EINVAL);
    KATZ_CHECK_ARG(B > 0 && HW > 0 && C > 0 && G > 0 && G <= GN_MAXG, KATZ_ESIZE);
    KATZ_CHECK_ARG(B <= 65535, KATZ_ESIZE);
    KATZ_CHECK_ARG(C % G == 0 && (C / G) % 2 == 0, KATZ_ESIZE);
    KATZ_CHECK_ARG(C <= 2 * GN_THREADS * GN_MAXP, KATZ_ESIZE);
    KATZ_CHECK_ARG(act == 0 || act == 1, KATZ_EINVAL);
    KATZ_CHECK_ARG(((uintptr_t)x & 3) == 0 && ((uintptr_t)y & 3) == 0 && ((uintptr_t)scratch & 3) == 0, KATZ_EALIGN);
    KATZ_CHECK_ARG(scratch_bytes >= katz_group_norm_scratch_bytes(B, HW, C, G), KATZ_ESIZE);
    const int rows = gn_rows_per_slab(HW, B);
    const int nslab = ceil_div(HW, rows);
    dim3 grid(nslab, B);
    cudaStream_t st = (cudaStream_t)stream;
    const int NC = C / 8;
    if (C % 8 == 0 && NC <= 1024 && B <= GN_MAX_TICKETS && aligned16(x) && aligned16(y) && ((uintptr_t)scratch & 255) == 0) {
        const int R = NC >= 512 ? 1 : 512 / NC;
        const int threads = NC * R;
        static bool attr_dev[KATZ_MAX_DEVICES] = {false};
        bool& attr = attr_dev[current_device_index()];
        if (!attr) {
            cudaFuncSetAttribute(gn_stats_v8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 1024 * 64);
            cudaFuncSetAttribute(gn_apply_v8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * 8192 * 4);
            attr = true;
        }
        const GnScratch sc = gn_carve(scratch, B, G);
        const double n_total = (double)HW * (C / G);
        launch_k(gn_stats_v8_kernel, grid, threads, threads * 64, st, (const __half*)x, sc.partial, HW, C, G, rows, R, sc.mr,
                 sc.tickets, n_total, eps, nullptr);
        launch_k(gn_apply_v8_kernel, grid, threads, 2 * C * 4, st, (const __half*)x, (__half*)y, sc.mr, (const __half*)gamma,
                 (const __half*)beta, HW, C, G, rows, R, n_total, eps, act, nullptr, 0);
        KATZ_LAUNCH_RET();
    }
    float* partial = gn_carve(scratch, B, G).partial;      // the ticket counters at the head of the scratch stay untouched
    launch_k(gn_stats_nhwc_kernel, grid, GN_THREADS, 0, st, (const __half*)x, partial, HW, C, G, rows);
    launch_k(gn_apply_nhwc_kernel, grid, GN_THREADS, 0, st, (const __half*)x, (__half*)y, partial, nslab,
                                                      (const __half*)gamma, (const __half*)beta, HW, C, G, rows, eps, act);
    KATZ_LAUNCH_RET();
}

static int gn_v8_setup(int C, int* R, int* threads) {
    const int NC = C / 8;
    if (C % 8 != 0 || NC > 1024) return KATZ_ESIZE;
    *R = NC >= 512 ? 1 : 512 / NC;
    *threads = NC * (*R);
    static bool attr_dev[KATZ_MAX_DEVICES] = {false};
    bool& attr = attr_dev[current_device_index()];
    if (!attr) {
        cudaFuncSetAttribute(gn_stats_v8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 1024 * 64);
        cudaFuncSetAttribute(gn_apply_v8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * 8192 * 4);
        attr = true;
    }
    return 0;
}

extern "C" int katz_group_norm_stats_nhwc_f16(const void* x, double* sums, int B, int HW, int C, int G, void* scratch,
                                              long long scratch_bytes, void* stream) {
    KATZ_CHECK_ARG(x && sums && scratch, KATZ_EINVAL);
    KATZ_CHECK_ARG(B > 0 && B <= 65535 && HW > 0 && C > 0 && G > 0 && G <= GN_MAXG && C % G == 0, KATZ_ESIZE);
    KATZ_CHECK_ARG(aligned16(x) && ((uintptr_t)sums & 7) == 0 && ((uintptr_t)scratch & 7) == 0, KATZ_EALIGN);
    KATZ_CHECK_ARG(scratch_bytes >= katz_group_norm_scratch_bytes(B, HW, C, G), KATZ_ESIZE);
    int R, threads;
    int rc = gn_v8_setup(C, &R, &threads);
    if (rc) return rc;
    const int rows = gn_rows_per_slab(HW, B);
    const int nslab = ceil_div(HW, rows);
    cudaStream_t st = (cudaStream_t)stream;
    const GnScratch sc = gn_carve(scratch, B, G);
    if (B <= GN_MAX_TICKETS) {
        // the CTA that finishes last for an image folds the partials into the fp64 sums: one kernel
        launch_k(gn_stats_v8_kernel, dim3(nslab, B), threads, threads * 64, st, (const __half*)x, sc.partial, HW, C, G, rows, R,
                 nullptr, sc.tickets, 0.0, 0.f, sums);
        KATZ_LAUNCH_RET();
    }
    launch_k(gn_stats_v8_kernel, dim3(nslab, B), threads, threads * 64, st, (const __half*)x, sc.partial, HW, C, G, rows, R, nullptr,
             nullptr, 0.0, 0.f, nullptr);
    launch_k(gn_fold_kernel, B, GN_MAXG, 0, st, sc.partial, nslab, G, sums);
    KATZ_LAUNCH_RET();
}

extern "C" int katz_group_norm_apply_nhwc_f16(const void* x, void* y, const double* sums, int n_parts, const void* gamma,
                                              const void* beta, int B, int HW, int C, int G, double n_total, float eps, int act,
                                              void* stream) {
    KATZ_CHECK_ARG(x && y && sums, KATZ_EINVAL);
    KATZ_CHECK_ARG(n_parts >= 1 && n_parts <= 64, KATZ_ESIZE);
    KATZ_CHECK_ARG(B > 0 && B <= 65535 && HW > 0 && C > 0 && G > 0 && G <= GN_MAXG && C % G == 0 && n_total > 0, KATZ_ESIZE);
    KATZ_CHECK_ARG(act == 0 || act == 1, KATZ_EINVAL);
    KATZ_CHECK_ARG(aligned16(x) && aligned16(y) && ((uintptr_t)sums & 7) == 0, KATZ_EALIGN);
    int R, threads;
    int rc = gn_v8_setup(C, &R, &threads);
    if (rc) return rc;
    const int rows = gn_rows_per_slab(HW, B);
    const int nslab = ceil_div(HW, rows);
    launch_k(gn_apply_v8_kernel, dim3(nslab, B), threads, 2 * C * 4, (cudaStream_t)stream, (const __half*)x, (__half*)y, nullptr,
             (const __half*)gamma, (const __half*)beta, HW, C, G, rows, R, n_total, eps, act, sums, n_parts);
    KATZ_LAUNCH_RET();
}

extern "C" int katz_group_norm_nchw_f16(const void* x, void* y, const void* gamma, const void* beta, int B, int HW, int C,
                                        int G, float eps, int act, void* stream) {
    KATZ_CHECK_ARG(x && y, KATZ_EINVAL);
    KATZ_CHECK_ARG(B > 0 && HW > 0 && C > 0 && G > 0 && C % G == 0, KATZ_ESIZE);
    KATZ_CHECK_ARG(B <= 65535, KATZ_ESIZE);
    KATZ_CHECK_ARG(act == 0 || act == 1, KATZ_EINVAL);
    launch_k(gn_nchw_kernel, dim3(G, B), 1024, 0, (cudaStream_t)stream, (const __half*)x, (__half*)y, (const __half*)gamma,
                                                                  (const __half*)beta, HW, C, G, eps, act);
    KATZ_LAUNCH_RET();
}

extern "C" int katz_layer_norm_f16(const void* x, void* y, const void* gamma, const void* beta, int rows, int C, float eps,
                                   void* stream) {
    KATZ_CHECK_ARG(x && y && gamma && beta, KATZ_EINVAL);
    KATZ_CHECK_ARG(rows > 0 && C > 0, KATZ_ESIZE);
    KATZ_CHECK_ARG(C % 8 == 0 && C <= 32 * LN_MAXCH * 8, KATZ_ESIZE);
    KATZ_CHECK_ARG(aligned16(x) && aligned16(y) && aligned16(gamma) && aligned16(beta), KATZ_EALIGN);
    const int rows_per_cta = 4;       // 4 warps per CTA: 2048 rows spread over more SMs than with 8
    if (C <= 32 * 5 * 8)
        launch_k(layer_norm_kernel<5>, ceil_div(rows, rows_per_cta), rows_per_cta * 32, 0, (cudaStream_t)stream, (const __half*)x,
                 (__half*)y, (const __half*)gamma, (const __half*)beta, rows, C, eps);
    else
        launch_k(layer_norm_kernel<LN_MAXCH>, ceil_div(rows, rows_per_cta), rows_per_cta * 32, 0, (cudaStream_t)stream,
                 (const __half*)x, (__half*)y, (const __half*)gamma, (const __half*)beta, rows, C, eps);
    KATZ_LAUNCH_RET();
}

// ---------------------------------------------------------------------------------------------------------------------
// GroupNorm for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc on the path that runs the step: a serving process whose memory
// is fully handed to another allocator at start-up, a plugin loaded into a runtime that forbids driver allocations
// after initialisation, or code running inside a region where an allocation would synchronise the device. For them
// the per-slab partial sums live in a fixed array in the library's own device image instead of caller-provided
// scratch. Every GPU that loads the library holds these 512 KiB until the process exits.
constexpr long long GN_STATIC_SCRATCH_BYTES = 512 * 1024;
static __device__ __align__(256) float g_gn_static_scratch[GN_STATIC_SCRATCH_BYTES / sizeof(float)];

// In host code the array's name is only a handle; the device address is looked up once per device, with that device
// current, and cached. Returns nullptr and sets *err on failure.
static float* gn_static_scratch_ptr(int* err) {
    constexpr int MAX_DEV = 64;
    static float* ptrs[MAX_DEV] = {nullptr};
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        *err = (int)e;
        return nullptr;
    }
    if (dev < 0 || dev >= MAX_DEV) {
        *err = KATZ_ENOTREADY;
        return nullptr;
    }
    if (!ptrs[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_gn_static_scratch);
        if (e != cudaSuccess || !p) {
            *err = e != cudaSuccess ? (int)e : KATZ_ENOTREADY;
            return nullptr;
        }
        ptrs[dev] = static_cast<float*>(p);
    }
    *err = 0;
    return ptrs[dev];
}

extern "C" long long katz_group_norm_static_scratch_bytes(void) { return GN_STATIC_SCRATCH_BYTES; }

// The ticket counters at the head of the array come back to zero at the end of every call. Two calls that overlapped on
// the GPU, or a launch that was aborted, can leave them elsewhere, and every later call would then fold its statistics
// too early or never: this puts them back to zero, in stream order, without allocating.
extern "C" int katz_group_norm_static_scratch_reset(void* stream) {
    int err = 0;
    float* scratch = gn_static_scratch_ptr(&err);
    if (!scratch) return err;
    cudaError_t e = cudaMemsetAsync(scratch, 0, 1024, (cudaStream_t)stream);
    return e == cudaSuccess ? 0 : (int)e;
}

extern "C" int katz_group_norm_nhwc_f16_noalloc(const void* x, void* y, const void* gamma, const void* beta, int B, int HW,
                                                int C, int G, float eps, int act, void* stream) {
    KATZ_CHECK_ARG(x && y, KATZ_EINVAL);
    KATZ_CHECK_ARG(B > 0 && B <= GN_MAX_TICKETS && HW > 0 && C > 0 && G > 0 && G <= GN_MAXG && C % G == 0, KATZ_ESIZE);
    KATZ_CHECK_ARG(act == 0 || act == 1, KATZ_EINVAL);
    KATZ_CHECK_ARG(aligned16(x) && aligned16(y), KATZ_EALIGN);
    // sizes whose partial sums do not fit the fixed array are refused, never truncated
    KATZ_CHECK_ARG(katz_group_norm_scratch_bytes(B, HW, C, G) <= GN_STATIC_SCRATCH_BYTES, KATZ_ESIZE);
    int R, threads;
    int rc = gn_v8_setup(C, &R, &threads);
    if (rc) return rc;
    int err = 0;
    float* scratch = gn_static_scratch_ptr(&err);
    if (!scratch) return err;
    const int rows = gn_rows_per_slab(HW, B);
    const int nslab = ceil_div(HW, rows);
    cudaStream_t st = (cudaStream_t)stream;
    // the statistics pass overwrites every partial and statistic the apply pass reads, and the ticket counters return to
    // zero by themselves, so nothing left by an earlier call is used
    const GnScratch sc = gn_carve(scratch, B, G);
    const double n_total = (double)HW * (C / G);
    launch_k(gn_stats_v8_kernel, dim3(nslab, B), threads, threads * 64, st, (const __half*)x, sc.partial, HW, C, G, rows, R, sc.mr,
             sc.tickets, n_total, eps, nullptr);
    launch_k(gn_apply_v8_kernel, dim3(nslab, B), threads, 2 * C * 4, st, (const __half*)x, (__half*)y, sc.mr, (const __half*)gamma,
             (const __half*)beta, HW, C, G, rows, R, n_total, eps, act, nullptr, 0);
    KATZ_LAUNCH_RET();
}
