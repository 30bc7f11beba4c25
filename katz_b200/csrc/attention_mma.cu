// Flash-style attention, head_dim 64, fp16 in/out, fp32 softmax and accumulation, no mask, non-causal.
// Replaces F.scaled_dot_product_attention as called by AttnProcessor2_0
// (diffusers/models/attention_processor.py:1276): softmax(Q K^T / sqrt(64)) V per (batch, head).
//
// Q/K/V are read in place from [B, S, ld] token-major buffers (head h lives at columns h*64..h*64+63), so the
// outputs of the q/k/v projections are consumed without a head transpose and the result is written in the
// layout the output projection reads.
#include "common.cuh"
#include "katz_b200.h"

namespace katz {

constexpr int ABM = 64, ABN = 64, AD = 64, ATHREADS = 128;

__device__ __forceinline__ uint32_t swz128(int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }

__global__ void __launch_bounds__(ATHREADS) attention_d64_kernel(const __half* __restrict__ Q, const __half* __restrict__ K,
                                                                 const __half* __restrict__ V, __half* __restrict__ O,
                                                                 int Sq, int Sk, int ldq, int ldk, int ldv, int ldo,
                                                                 long long bsq, long long bsk, long long bsv,
                                                                 long long bso, float scale_log2e, int kv_chunk_rows,
                                                                 long long kv_chunk_stride) {
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    pdl_launch_dependents();
    __shared__ __align__(128) unsigned char sQ[ABM * 128];
    __shared__ __align__(128) unsigned char sK[2][ABN * 128];
    __shared__ __align__(128) unsigned char sV[2][ABN * 128];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int q0 = blockIdx.x * ABM, h = blockIdx.y, b = blockIdx.z;
    const __half* Qb = Q + (size_t)b * bsq + h * AD;
    const __half* Kb = K + (size_t)b * bsk + h * AD;
    const __half* Vb = V + (size_t)b * bsv + h * AD;

    // 64 rows x 8 chunks = 512 chunks of 16 B per tile; 4 per thread
    auto load_tile = [&](unsigned char* dst, const __half* base, int row0, int nrows, int ld) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int idx = tid + i * ATHREADS;
            int r = idx >> 3, c = idx & 7;
            int gr = row0 + r;
            bool ok = gr < nrows;
            const __half* src = base + (size_t)(ok ? gr : 0) * ld + c * 8;
            cp_async16(smem_u32(dst + swz128(r, c)), src, ok ? 16 : 0);
        }
    };

    load_tile(sQ, Qb, q0, Sq, ldq);
    cp_async_commit();
    const int NT = ceil_div(Sk, ABN);
    // K/V may arrive as equal chunks of rows that are not adjacent in memory (one chunk per rank after an all-gather):
    // key row j lives at chunk (j / kv_chunk_rows), row (j % kv_chunk_rows); chunks are multiples of the 64-row tile.
    auto load_kv = [&](int buf, int row0) {
        const int chunk = row0 / kv_chunk_rows;
        const long long shift = (long long)chunk * kv_chunk_stride - (long long)chunk * kv_chunk_rows * ldk;
        const long long shiftv = (long long)chunk * kv_chunk_stride - (long long)chunk * kv_chunk_rows * ldv;
        load_tile(sK[buf], Kb + shift, row0, Sk, ldk);
        load_tile(sV[buf], Vb + shiftv, row0, Sk, ldv);
    };
    load_kv(0, 0);
    cp_async_commit();

    float o[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    uint32_t qf[4][4];

    for (int t = 0; t < NT; ++t) {
        if (t + 1 < NT) {
            load_kv((t + 1) & 1, (t + 1) * ABN);
        }
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        if (t == 0) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                int r = warp * 16 + (lane & 15);
                int ch = ks * 2 + (lane >> 4);
                ldmatrix_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], smem_u32(sQ + swz128(r, ch)));
            }
        }
        const unsigned char* k_s = sK[t & 1];
        const unsigned char* v_s = sV[t & 1];

        // 16-key groups of this tile that hold at least one key (the 77 text tokens fill 4 + 1 of the 8 groups of two tiles):
        // the others are skipped in both MMAs and stay masked
        const int kgroups = min(4, (Sk - t * ABN + 15) >> 4);
        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[i][e] = 0.f;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                if (np >= kgroups) continue;
                uint32_t bfr[4];
                int r = np * 16 + (lane & 7) + ((lane >> 4) << 3);
                int ch = ks * 2 + ((lane >> 3) & 1);
                ldmatrix_x4(bfr[0], bfr[1], bfr[2], bfr[3], smem_u32(k_s + swz128(r, ch)));
                mma_f16_16816(s[np * 2], qf[ks], bfr);
                mma_f16_16816(s[np * 2 + 1], qf[ks], bfr + 2);
            }
        }
        // scale into the log2 domain, mask keys past Sk
        const int kbase = t * ABN;
        const bool tail = kbase + ABN > Sk;
#pragma unroll
        for (int nf = 0; nf < 8; ++nf) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v = s[nf][e] * scale_log2e;
                if (tail) {
                    int key = kbase + nf * 8 + (lane & 3) * 2 + (e & 1);
                    if (key >= Sk) v = -INFINITY;
                }
                s[nf][e] = v;
            }
        }
        // online softmax for the two rows this thread owns (lane/4 and lane/4+8)
#pragma unroll
        for (int hr = 0; hr < 2; ++hr) {
            float mx = -INFINITY;
#pragma unroll
            for (int nf = 0; nf < 8; ++nf) mx = fmaxf(mx, fmaxf(s[nf][hr * 2], s[nf][hr * 2 + 1]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            float m_new = fmaxf(m_run[hr], mx);
            float corr = ex2_fast(m_run[hr] - m_new);
            float rs = 0.f;
#pragma unroll
            for (int nf = 0; nf < 8; ++nf) {
                float p0 = ex2_fast(s[nf][hr * 2] - m_new);
                float p1 = ex2_fast(s[nf][hr * 2 + 1] - m_new);
                s[nf][hr * 2] = p0;
                s[nf][hr * 2 + 1] = p1;
                rs += p0 + p1;
            }
            rs += __shfl_xor_sync(0xffffffffu, rs, 1);
            rs += __shfl_xor_sync(0xffffffffu, rs, 2);
            l_run[hr] = l_run[hr] * corr + rs;
            m_run[hr] = m_new;
#pragma unroll
            for (int df = 0; df < 8; ++df) {
                o[df][hr * 2] *= corr;
                o[df][hr * 2 + 1] *= corr;
            }
        }
        // O += P V
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {  // 16 keys per step
            if (kk >= kgroups) continue;
            uint32_t pf[4];
            pf[0] = pack_half2(s[kk * 2][0], s[kk * 2][1]);
            pf[1] = pack_half2(s[kk * 2][2], s[kk * 2][3]);
            pf[2] = pack_half2(s[kk * 2 + 1][0], s[kk * 2 + 1][1]);
            pf[3] = pack_half2(s[kk * 2 + 1][2], s[kk * 2 + 1][3]);
#pragma unroll
            for (int dp = 0; dp < 4; ++dp) {  // 16 d columns per step
                uint32_t vfr[4];
                int r = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                int ch = dp * 2 + (lane >> 4);
                ldmatrix_x4_trans(vfr[0], vfr[1], vfr[2], vfr[3], smem_u32(v_s + swz128(r, ch)));
                mma_f16_16816(o[dp * 2], pf, vfr);
                mma_f16_16816(o[dp * 2 + 1], pf, vfr + 2);
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();

#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
        int row = q0 + warp * 16 + (lane >> 2) + hr * 8;
        if (row >= Sq) continue;
        float inv = 1.0f / l_run[hr];
        __half* op = O + (size_t)b * bso + (size_t)row * ldo + h * AD + (lane & 3) * 2;
#pragma unroll
        for (int df = 0; df < 8; ++df) {
            *reinterpret_cast<__half2*>(op + df * 8) = __floats2half2_rn(o[df][hr * 2] * inv, o[df][hr * 2 + 1] * inv);
        }
    }
}

}  // namespace katz

using namespace katz;

extern "C" int katz_attention_f16_mma(const void* Q, const void* K, const void* V, void* O, int B, int H, int Sq, int Sk,
                                      int head_dim, int ldq, int ldk, int ldv, int ldo, long long bsq, long long bsk,
                                      long long bsv, long long bso, float scale, int kv_chunk_rows,
                                      long long kv_chunk_stride, void* stream) {
    KATZ_CHECK_ARG(Q && K && V && O, KATZ_EINVAL);
    KATZ_CHECK_ARG(head_dim == 64, KATZ_ESIZE);
    KATZ_CHECK_ARG(B > 0 && H > 0 && Sq > 0 && Sk > 0, KATZ_ESIZE);
    KATZ_CHECK_ARG(B <= 65535 && H <= 65535, KATZ_ESIZE);
    KATZ_CHECK_ARG(ldq % 8 == 0 && ldk % 8 == 0 && ldv % 8 == 0 && ldo % 2 == 0, KATZ_EALIGN);
    KATZ_CHECK_ARG(bsq % 8 == 0 && bsk % 8 == 0 && bsv % 8 == 0 && bso % 2 == 0, KATZ_EALIGN);
    KATZ_CHECK_ARG(aligned16(Q) && aligned16(K) && aligned16(V) && ((uintptr_t)O & 3) == 0, KATZ_EALIGN);
    if (kv_chunk_rows <= 0 || kv_chunk_rows >= Sk) {
        kv_chunk_rows = Sk > 0 ? ((Sk + ABN - 1) / ABN) * ABN : ABN;   // one chunk
        kv_chunk_stride = 0;
    } else {
        KATZ_CHECK_ARG(kv_chunk_rows % ABN == 0 && kv_chunk_stride % 8 == 0, KATZ_ESIZE);
    }
    dim3 grid(ceil_div(Sq, ABM), H, B);
    launch_k(attention_d64_kernel, grid, ATHREADS, 0, (cudaStream_t)stream, (const __half*)Q, (const __half*)K,
             (const __half*)V, (__half*)O, Sq, Sk, ldq, ldk, ldv, ldo, bsq, bsk, bsv, bso, scale * 1.44269504088896340736f,
             kv_chunk_rows, kv_chunk_stride);
    KATZ_LAUNCH_RET();
}
