// Fused LoRA merge over a whole set of linears in ONE launch:
//     W_live = (W0 ? W0 : W_live) + sign * sum_i s_i * (B_i @ A_i)        B_i = up [out, r_i], A_i = down [r_i, in]
//
// Reference: lora_utils.py:21-33 and pipeline_controlnet_sd_xl_katz.py:1736-1747 (a Python loop of 722 small GEMMs
// `W[key] += up @ down * scale` followed by a full load_state_dict copy), restore by load_state_dict of a pristine
// copy (sdxl_unet_server.py:217). With W0 (the pristine weights, resident in HBM) the merge reads W0 and writes
// W_live, so merge is one pass and restore is a plain copy, which is how the reference keeps the restore bit-exact.
// With W0 == nullptr the update is in place (sign = -1 gives the subtractive unmerge of
// diffusers/models/lora.py:427-449, which is not bit-exact in floating point).
//
// The work is bound by streaming W through HBM once. One persistent CTA per SM walks the global tile list with a ring
// of shared-memory stages: while tile i is being updated and written back with 16-byte stores, the 16-byte async
// copies of tiles i+1 (and i+2) — the W tile and the first adapter's B and A tiles — are already in flight. The rank-r
// product runs on tensor cores (mma.sync; fp16 inputs, or 3xTF32 for fp32 inputs) out of swizzled shared memory.
// Further adapters / rank chunks beyond 64 are fetched synchronously into a side buffer.
// Rounding follows the reference: fp16: delta = half(acc); delta = half(delta * s); W = half(W + delta), per adapter
// in order. fp32: W += acc * s.
#include <cstdlib>

#include <cstring>

#include "tc05.cuh"
#include "katz_b200.h"

namespace katz {

constexpr int LM_THREADS = 256;
constexpr int LM_TN = 128;        // tile columns
constexpr int LM_MAXR = 64;       // rank processed per pass; larger ranks loop
constexpr int LM_MAX_LAYERS_SMEM = 896;    // per-layer tile counts cached in shared memory up to this many layers

template <typename T>
struct LmCfg;
template <>
struct LmCfg<__half> {
    static constexpr int TM = 128;
    static constexpr int NST = 3;
    static constexpr int W_BYTES = TM * LM_TN * 2;        // 32 KB, 256 B rows, 16 chunks, swizzled
    static constexpr int B_BYTES = TM * 128;              // [TM][64 halfs], 128 B rows, swizzled
    static constexpr int A_BYTES = LM_MAXR * LM_TN * 2;   // [64][128 halfs], 256 B rows, swizzled
    static constexpr int STAGE = W_BYTES + B_BYTES + A_BYTES;
    static constexpr int SMEM = NST * STAGE + B_BYTES + A_BYTES;
};
template <>
struct LmCfg<float> {
    static constexpr int TM = 64;
    static constexpr int NST = 2;
    static constexpr int BP = 68;    // B tile pitch in floats (bank-conflict-free fragment reads)
    static constexpr int AP = 136;   // A tile pitch in floats
    static constexpr int W_BYTES = TM * LM_TN * 4;        // 32 KB, 512 B rows, 32 chunks, swizzled
    static constexpr int B_BYTES = TM * BP * 4;
    static constexpr int A_BYTES = LM_MAXR * AP * 4;
    static constexpr int STAGE = W_BYTES + B_BYTES + A_BYTES;
    static constexpr int SMEM = NST * STAGE + B_BYTES + A_BYTES;
};

__device__ __forceinline__ int find_layer(const int* __restrict__ tile_start, int n_layers, int tile) {
    int lo = 0, hi = n_layers - 1;
    while (lo < hi) {
        int mid = (lo + hi + 1) >> 1;
        if (tile_start[mid] <= tile) lo = mid; else hi = mid - 1;
    }
    return lo;
}

template <typename T>
struct TileRef {
    const katz_lora_layer* L;
    T* W;
    int row0, col0, out_f, in_f, n_lora, rank0;
    float scale0;
};

template <typename T>
__device__ __forceinline__ TileRef<T> decode_tile(const katz_lora_layer* __restrict__ layers, int li, int layer_start,
                                                  int tile) {
    TileRef<T> t;
    t.L = layers + li;
    t.W = reinterpret_cast<T*>(t.L->W);
    t.out_f = t.L->out_features;
    t.in_f = t.L->in_features;
    t.n_lora = t.L->n_lora;
    t.rank0 = t.L->rank[0];
    t.scale0 = t.L->scale[0];
    const int rel = tile - layer_start;
    const int tiles_n = (t.in_f + LM_TN - 1) / LM_TN;
    const int tm = rel / tiles_n;
    t.row0 = tm * LmCfg<T>::TM;
    t.col0 = (rel - tm * tiles_n) * LM_TN;
    return t;
}

template <typename T>
__device__ __forceinline__ uint32_t w_off(int r, int c) {
    if constexpr (sizeof(T) == 2) return r * 256 + ((c ^ (r & 7)) << 4);
    else return r * 512 + ((c ^ ((r & 3) << 1)) << 4);
}
template <typename T>
__device__ __forceinline__ uint32_t b_off(int r, int c) {
    if constexpr (sizeof(T) == 2) return r * 128 + ((c ^ (r & 7)) << 4);
    else return (r * LmCfg<float>::BP + c * 4) * 4;
}
// TC05: the A tile is the MN-major operand of tcgen05.mma: two blocks of [64 k-rows][64 columns], each row 128 bytes
// with the 128-byte swizzle, 8 KB per block (the layout a TMA SWIZZLE_128B load of the block would produce).
template <typename T, bool TC05 = false>
__device__ __forceinline__ uint32_t a_off(int r, int c) {
    if constexpr (TC05) return (c >> 3) * 8192 + r * 128 + (((c & 7) ^ (r & 7)) << 4);
    else if constexpr (sizeof(T) == 2) return r * 256 + ((c ^ (r & 7)) << 4);
    else return (r * LmCfg<float>::AP + c * 4) * 4;
}

// Adapter tiles for rank chunk [k0, k0+kr) of adapter l: B rows row0.., A cols col0..; ASYNC = cp.async into the ring,
// otherwise plain 16-byte loads and stores into the side buffer.
template <typename T, bool ASYNC, bool TC05 = false>
__device__ __forceinline__ void load_adapter_tiles(const TileRef<T>& t, int l, int k0, unsigned char* sB, unsigned char* sA) {
    constexpr int ES = sizeof(T), EPC = 16 / ES, TM = LmCfg<T>::TM, W_CHUNKS_ROW = LM_TN / EPC;
    const T* Bm = reinterpret_cast<const T*>(t.L->B[l]);
    const T* Am = reinterpret_cast<const T*>(t.L->A[l]);
    const int rank = l == 0 ? t.rank0 : t.L->rank[l];
    const int kr = min(LM_MAXR, rank - k0);
    const int kpad = (kr + 15) & ~15;
    constexpr int BSLOTS = LM_MAXR / EPC;        // 16-byte chunk slots per B row (8 for fp16, 16 for fp32)
    const int bchunks = kpad / EPC;
    for (int idx = threadIdx.x; idx < TM * BSLOTS; idx += LM_THREADS) {
        const int r = idx / BSLOTS, c = idx % BSLOTS;
        if (c >= bchunks) continue;
        const int gr = t.row0 + r;
        const bool ok = gr < t.out_f && (c * EPC) < kr;
        const T* src = ok ? Bm + (size_t)gr * rank + k0 + c * EPC : Bm;
        if (ASYNC) {
            cp_async16(smem_u32(sB + b_off<T>(r, c)), src, ok ? 16 : 0);
        } else {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (ok) v = *reinterpret_cast<const uint4*>(src);
            *reinterpret_cast<uint4*>(sB + b_off<T>(r, c)) = v;
        }
    }
    for (int idx = threadIdx.x; idx < kpad * W_CHUNKS_ROW; idx += LM_THREADS) {
        const int r = idx / W_CHUNKS_ROW, c = idx - r * W_CHUNKS_ROW;
        const int gc = t.col0 + c * EPC;
        const bool ok = r < kr && gc < t.in_f;
        const T* src = ok ? Am + (size_t)(k0 + r) * t.in_f + gc : Am;
        if (ASYNC) {
            cp_async16(smem_u32(sA + a_off<T, TC05>(r, c)), src, ok ? 16 : 0);
        } else {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (ok) v = *reinterpret_cast<const uint4*>(src);
            *reinterpret_cast<uint4*>(sA + a_off<T, TC05>(r, c)) = v;
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(LM_THREADS, 1) lora_merge_kernel(const katz_lora_layer* __restrict__ layers,
                                                                   const int* __restrict__ tile_start, int n_layers,
                                                                   int total_tiles, float sign, int counts_in_smem) {
    // Writes weights, which later kernels may fetch before their own dependency wait: dependents are released only by this
    // kernel's completion (no griddepcontrol.launch_dependents).
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    using Cfg = LmCfg<T>;
    constexpr int TM = Cfg::TM, NST = Cfg::NST;
    constexpr int ES = sizeof(T);
    constexpr int EPC = 16 / ES;                 // elements per 16-byte chunk
    constexpr int W_CHUNKS_ROW = LM_TN / EPC;    // 16 (fp16) / 32 (fp32)
    constexpr int NF = ES == 2 ? 8 : 4;          // n-fragments per warp
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* xB = smem + NST * Cfg::STAGE;           // side buffer for further adapters / rank chunks
    unsigned char* xA = xB + Cfg::B_BYTES;
    // The tile -> layer search runs once per tile on the issue side, over a shared-memory copy of the prefix table; the
    // decoded tile travels to the compute side through a small ring, so the update loop makes no dependent global loads.
    __shared__ unsigned short s_count[LM_MAX_LAYERS_SMEM];
    __shared__ TileRef<T> s_ref[NST];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // counts_in_smem is decided on the host (every layer has < 65536 tiles and the table fits)
    if (counts_in_smem) {
        for (int i = tid; i < n_layers; i += LM_THREADS)
            s_count[i] = (unsigned short)((i + 1 < n_layers ? tile_start[i + 1] : total_tiles) - tile_start[i]);
        __syncthreads();
    }
    int cur_li = 0, cur_start = 0;     // issue-side cursor: tiles are visited in increasing order

    auto issue = [&](int j) {
        const int tile = blockIdx.x + j * gridDim.x;
        if (tile < total_tiles) {
            unsigned char* sW = smem + (j % NST) * Cfg::STAGE;
            if (counts_in_smem) {
                while (tile >= cur_start + (int)s_count[cur_li]) {
                    cur_start += s_count[cur_li];
                    ++cur_li;
                }
            } else {
                cur_li = find_layer(tile_start, n_layers, tile);
                cur_start = tile_start[cur_li];
            }
            const TileRef<T> t = decode_tile<T>(layers, cur_li, cur_start, tile);
            if (tid == 0) s_ref[j % NST] = t;
            const T* Wdst = t.W;
            const T* Wsrc = t.L->W0 ? reinterpret_cast<const T*>(t.L->W0) : Wdst;
            for (int idx = tid; idx < TM * W_CHUNKS_ROW; idx += LM_THREADS) {
                const int r = idx / W_CHUNKS_ROW, c = idx - r * W_CHUNKS_ROW;
                const int gr = t.row0 + r, gc = t.col0 + c * EPC;
                const bool ok = gr < t.out_f && gc < t.in_f;
                const T* src = ok ? Wsrc + (size_t)gr * t.in_f + gc : Wsrc;
                cp_async16(smem_u32(sW + w_off<T>(r, c)), src, ok ? 16 : 0);
            }
            if (t.n_lora > 0) load_adapter_tiles<T, true>(t, 0, 0, sW + Cfg::W_BYTES, sW + Cfg::W_BYTES + Cfg::B_BYTES);
        }
        cp_async_commit();
    };

#pragma unroll
    for (int j = 0; j < NST - 1; ++j) issue(j);

    for (int j = 0;; ++j) {
        const int tile = blockIdx.x + j * gridDim.x;
        if (tile >= total_tiles) break;
        cp_async_wait<NST - 2>();
        __syncthreads();               // stage j landed for everyone; everyone has finished with stage j-1
        issue(j + NST - 1);            // refills the stage that tile j-1 used

        unsigned char* sW = smem + (j % NST) * Cfg::STAGE;
        const TileRef<T> t = s_ref[j % NST];

        for (int l = 0; l < t.n_lora; ++l) {
            const int rank = l == 0 ? t.rank0 : t.L->rank[l];
            const float s = (l == 0 ? t.scale0 : t.L->scale[l]) * sign;
            float acc[2][NF][4];
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int jn = 0; jn < NF; ++jn)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[i][jn][e] = 0.f;

            for (int k0 = 0; k0 < rank; k0 += LM_MAXR) {
                const unsigned char* sB;
                const unsigned char* sA;
                if (l == 0 && k0 == 0) {
                    sB = sW + Cfg::W_BYTES;
                    sA = sB + Cfg::B_BYTES;
                } else {
                    __syncthreads();   // previous users of the side buffer are done
                    load_adapter_tiles<T, false>(t, l, k0, xB, xA);
                    __syncthreads();
                    sB = xB;
                    sA = xA;
                }
                const int kr = min(LM_MAXR, rank - k0);
                const int kpad = (kr + 15) & ~15;
                if constexpr (ES == 2) {
                    const int warp_m = warp & 3, warp_n = warp >> 2;   // 4 x 2 warps, warp tile 32 x 64
                    for (int ks = 0; ks < kpad / 16; ++ks) {
                        uint32_t af[2][4];
#pragma unroll
                        for (int mf = 0; mf < 2; ++mf) {
                            const int r = warp_m * 32 + mf * 16 + (lane & 15);
                            const int ch = ks * 2 + (lane >> 4);
                            ldmatrix_x4(af[mf][0], af[mf][1], af[mf][2], af[mf][3], smem_u32(sB + b_off<T>(r, ch)));
                        }
#pragma unroll
                        for (int np = 0; np < 4; ++np) {
                            uint32_t bf[4];
                            const int r = ks * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                            const int ch = warp_n * 8 + np * 2 + (lane >> 4);
                            ldmatrix_x4_trans(bf[0], bf[1], bf[2], bf[3], smem_u32(sA + a_off<T>(r, ch)));
#pragma unroll
                            for (int mf = 0; mf < 2; ++mf) {
                                mma_f16_16816(acc[mf][np * 2], af[mf], bf);
                                mma_f16_16816(acc[mf][np * 2 + 1], af[mf], bf + 2);
                            }
                        }
                    }
                } else {
                    const int warp_m = warp & 1, warp_n = warp >> 1;   // 2 x 4 warps, warp tile 32 x 32
                    const float* fB = reinterpret_cast<const float*>(sB);
                    const float* fA = reinterpret_cast<const float*>(sA);
                    const int g = lane >> 2, q = lane & 3;
                    for (int ks = 0; ks < kpad / 8; ++ks) {
                        uint32_t ahi[2][4], alo[2][4], bhi[4][2], blo[4][2];
#pragma unroll
                        for (int mf = 0; mf < 2; ++mf) {
                            const int r = warp_m * 32 + mf * 16 + g;
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float v = fB[(r + (e & 1) * 8) * Cfg::BP + ks * 8 + q + (e >> 1) * 4];
                                ahi[mf][e] = f32_to_tf32(v);
                                alo[mf][e] = f32_to_tf32(v - __uint_as_float(ahi[mf][e]));
                            }
                        }
#pragma unroll
                        for (int nf = 0; nf < 4; ++nf) {
                            const int n = warp_n * 32 + nf * 8 + g;
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const float v = fA[(ks * 8 + q + e * 4) * Cfg::AP + n];
                                bhi[nf][e] = f32_to_tf32(v);
                                blo[nf][e] = f32_to_tf32(v - __uint_as_float(bhi[nf][e]));
                            }
                        }
#pragma unroll
                        for (int mf = 0; mf < 2; ++mf)
#pragma unroll
                            for (int nf = 0; nf < 4; ++nf) {
                                mma_tf32_1688(acc[mf][nf], alo[mf], bhi[nf]);
                                mma_tf32_1688(acc[mf][nf], ahi[mf], blo[nf]);
                                mma_tf32_1688(acc[mf][nf], ahi[mf], bhi[nf]);
                            }
                    }
                }
            }

            // ---- fold this adapter's delta into the W tile held in shared memory (each element has one owner thread)
            if constexpr (ES == 2) {
                const int warp_m = warp & 3, warp_n = warp >> 2;
#pragma unroll
                for (int mf = 0; mf < 2; ++mf)
#pragma unroll
                    for (int hr = 0; hr < 2; ++hr) {
                        const int r = warp_m * 32 + mf * 16 + (lane >> 2) + hr * 8;
#pragma unroll
                        for (int nf = 0; nf < 8; ++nf) {
                            const int c = warp_n * 64 + nf * 8 + (lane & 3) * 2;
                            __half2* wp = reinterpret_cast<__half2*>(sW + w_off<T>(r, c >> 3) + (c & 7) * 2);
                            const float2 w = __half22float2(*wp);
                            float d0 = __half2float(__float2half_rn(acc[mf][nf][hr * 2]));
                            float d1 = __half2float(__float2half_rn(acc[mf][nf][hr * 2 + 1]));
                            d0 = __half2float(__float2half_rn(d0 * s));
                            d1 = __half2float(__float2half_rn(d1 * s));
                            *wp = __floats2half2_rn(w.x + d0, w.y + d1);
                        }
                    }
            } else {
                const int warp_m = warp & 1, warp_n = warp >> 1;
#pragma unroll
                for (int mf = 0; mf < 2; ++mf)
#pragma unroll
                    for (int hr = 0; hr < 2; ++hr) {
                        const int r = warp_m * 32 + mf * 16 + (lane >> 2) + hr * 8;
#pragma unroll
                        for (int nf = 0; nf < 4; ++nf) {
                            const int c = warp_n * 32 + nf * 8 + (lane & 3) * 2;
                            float2* wp = reinterpret_cast<float2*>(sW + w_off<T>(r, c >> 2) + (c & 3) * 4);
                            float2 w = *wp;
                            w.x = __fadd_rn(w.x, __fmul_rn(acc[mf][nf][hr * 2], s));
                            w.y = __fadd_rn(w.y, __fmul_rn(acc[mf][nf][hr * 2 + 1], s));
                            *wp = w;
                        }
                    }
            }
        }
        __syncthreads();

        // ---- write-back, 16 bytes per thread, whole rows of the tile contiguous
        T* Wdst = t.W;
        for (int idx = tid; idx < TM * W_CHUNKS_ROW; idx += LM_THREADS) {
            const int r = idx / W_CHUNKS_ROW, c = idx - r * W_CHUNKS_ROW;
            const int gr = t.row0 + r, gc = t.col0 + c * EPC;
            if (gr < t.out_f && gc < t.in_f) {
                const uint4 v = *reinterpret_cast<const uint4*>(sW + w_off<T>(r, c));
                *reinterpret_cast<uint4*>(Wdst + (size_t)gr * t.in_f + gc) = v;
            }
        }
    }
    cp_async_wait<0>();
}

// ---- fp16 weights, rank-r product on the tcgen05 tensor path -------------------------------------------------------
// Same ring, same tile walk and the same rounding as lora_merge_kernel<__half>; the difference is where the product
// is computed. The B tile ([128 rows][64 k], K-major) and the A tile (two [64 k][64 n] MN-major blocks) sit in shared
// memory in the 128-byte-swizzled layouts tcgen05.mma reads, one elected thread issues 128x64x16 MMAs into a 128-column
// TMEM accumulator, and all eight warps read the accumulator back (a thread owns one tile row: tcgen05.ld 32x32b) and
// fold it into the W tile in shared memory with 16-byte accesses. The CUDA cores no longer run ldmatrix/mma.sync.
__global__ void __launch_bounds__(LM_THREADS, 1) lora_merge_f16_tc05_kernel(const katz_lora_layer* __restrict__ layers,
                                                                           const int* __restrict__ tile_start, int n_layers,
                                                                           int total_tiles, float sign, int counts_in_smem,
                                                                           int* __restrict__ status) {
    // Writes weights, which later kernels may fetch before their own dependency wait: dependents are released only by this
    // kernel's completion (no griddepcontrol.launch_dependents).
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    using namespace tc05;
    using T = __half;
    using Cfg = LmCfg<__half>;
    constexpr int TM = Cfg::TM, NST = Cfg::NST, EPC = 8, W_CHUNKS_ROW = LM_TN / EPC;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* xB = smem + NST * Cfg::STAGE;
    unsigned char* xA = xB + Cfg::B_BYTES;
    __shared__ unsigned short s_count[LM_MAX_LAYERS_SMEM];
    __shared__ TileRef<T> s_ref[NST];
    __shared__ __align__(8) uint64_t s_bar;
    __shared__ uint32_t s_tmem;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        mbar_init(smem_u32(&s_bar), 1);
        fence_barrier_init();
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(&s_tmem), 128);
        tmem_relinquish();
    }
    if (counts_in_smem)
        for (int i = tid; i < n_layers; i += LM_THREADS)
            s_count[i] = (unsigned short)((i + 1 < n_layers ? tile_start[i + 1] : total_tiles) - tile_start[i]);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = s_tmem;
    const uint32_t bar = smem_u32(&s_bar);
    uint32_t bar_phase = 0;
    bool ok = true;
    int cur_li = 0, cur_start = 0;

    auto issue = [&](int j) {
        const int tile = blockIdx.x + j * gridDim.x;
        if (tile < total_tiles) {
            unsigned char* sW = smem + (j % NST) * Cfg::STAGE;
            if (counts_in_smem) {
                while (tile >= cur_start + (int)s_count[cur_li]) {
                    cur_start += s_count[cur_li];
                    ++cur_li;
                }
            } else {
                cur_li = find_layer(tile_start, n_layers, tile);
                cur_start = tile_start[cur_li];
            }
            const TileRef<T> t = decode_tile<T>(layers, cur_li, cur_start, tile);
            if (tid == 0) s_ref[j % NST] = t;
            const T* Wsrc = t.L->W0 ? reinterpret_cast<const T*>(t.L->W0) : t.W;
            for (int idx = tid; idx < TM * W_CHUNKS_ROW; idx += LM_THREADS) {
                const int r = idx / W_CHUNKS_ROW, c = idx - r * W_CHUNKS_ROW;
                const int gr = t.row0 + r, gc = t.col0 + c * EPC;
                const bool in = gr < t.out_f && gc < t.in_f;
                const T* src = in ? Wsrc + (size_t)gr * t.in_f + gc : Wsrc;
                cp_async16(smem_u32(sW + w_off<T>(r, c)), src, in ? 16 : 0);
            }
            if (t.n_lora > 0)
                load_adapter_tiles<T, true, true>(t, 0, 0, sW + Cfg::W_BYTES, sW + Cfg::W_BYTES + Cfg::B_BYTES);
        }
        cp_async_commit();
    };

#pragma unroll
    for (int j = 0; j < NST - 1; ++j) issue(j);

    const int q = warp & 3, half = warp >> 2;          // TMEM lane quarter, 64-column half of the tile
    const int row = q * 32 + lane;
    for (int j = 0;; ++j) {
        const int tile = blockIdx.x + j * gridDim.x;
        if (tile >= total_tiles) break;
        cp_async_wait<NST - 2>();
        fence_proxy_async();           // the copied tiles are about to be read by the tensor core (async proxy)
        __syncthreads();
        issue(j + NST - 1);

        unsigned char* sW = smem + (j % NST) * Cfg::STAGE;
        const TileRef<T> t = s_ref[j % NST];

        for (int l = 0; l < t.n_lora; ++l) {
            const int rank = l == 0 ? t.rank0 : t.L->rank[l];
            const float s = (l == 0 ? t.scale0 : t.L->scale[l]) * sign;
            for (int k0 = 0; k0 < rank; k0 += LM_MAXR) {
                uint32_t sBa, sAa;
                if (l == 0 && k0 == 0) {
                    sBa = smem_u32(sW + Cfg::W_BYTES);
                    sAa = sBa + Cfg::B_BYTES;
                } else {
                    __syncthreads();
                    load_adapter_tiles<T, false, true>(t, l, k0, xB, xA);
                    fence_proxy_async();
                    __syncthreads();
                    sBa = smem_u32(xB);
                    sAa = smem_u32(xA);
                }
                const int kpad = (min(LM_MAXR, rank - k0) + 15) & ~15;
                if (tid == 0) {
                    fence_after_sync();
                    constexpr uint32_t idesc = idesc_f16(128, 64) | (1u << 16);     // B operand MN-major
#pragma unroll
                    for (int nb = 0; nb < 2; ++nb)
                        for (int ks = 0; ks < kpad / 16; ++ks)
                            umma_f16(tmem_base + nb * 64, smem_desc_sw128(sBa) + 2 * ks,
                                     smem_desc_sw128(sAa + nb * 8192 + ks * 2048), idesc, (k0 | ks) != 0);
                    umma_commit(bar);
                }
                ok = ok && mbar_wait(bar, bar_phase);
                bar_phase ^= 1;
                fence_after_sync();
            }
            ok = __syncthreads_and(ok);        // block-uniform: either every warp goes on or every warp unwinds
            if (!ok) break;
            // fold: thread = tile row, 64 columns of this warp's half, 8 columns (16 bytes of W) at a time
#pragma unroll
            for (int c = 0; c < 64; c += 32) {
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + half * 64 + c, r);
                tmem_ld_wait();
#pragma unroll
                for (int g8 = 0; g8 < 4; ++g8) {
                    const int chunk = (half * 64 + c + g8 * 8) >> 3;
                    uint4* wp = reinterpret_cast<uint4*>(sW + w_off<T>(row, chunk));
                    uint4 w = *wp;
                    uint32_t wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 wf = unpack_half2(wv[e]);
                        float d0 = __half2float(__float2half_rn(__uint_as_float(r[g8 * 8 + 2 * e])));
                        float d1 = __half2float(__float2half_rn(__uint_as_float(r[g8 * 8 + 2 * e + 1])));
                        d0 = __half2float(__float2half_rn(d0 * s));
                        d1 = __half2float(__float2half_rn(d1 * s));
                        wv[e] = pack_half2(wf.x + d0, wf.y + d1);
                    }
                    *wp = make_uint4(wv[0], wv[1], wv[2], wv[3]);
                }
            }
            fence_before_sync();       // accumulator reads done before the next MMA may overwrite it (after a barrier)
        }
        if (!ok) break;
        __syncthreads();

        T* Wdst = t.W;
        for (int idx = tid; idx < TM * W_CHUNKS_ROW; idx += LM_THREADS) {
            const int r = idx / W_CHUNKS_ROW, c = idx - r * W_CHUNKS_ROW;
            const int gr = t.row0 + r, gc = t.col0 + c * EPC;
            if (gr < t.out_f && gc < t.in_f) {
                const uint4 v = *reinterpret_cast<const uint4*>(sW + w_off<T>(r, c));
                *reinterpret_cast<uint4*>(Wdst + (size_t)gr * t.in_f + gc) = v;
            }
        }
    }
    cp_async_wait<0>();
    if (!ok && tid == 0) atomicExch(status, 21);
    fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        fence_after_sync();
        tmem_dealloc(tmem_base, 128);
    }
}

// ---- fp16, warp-specialised, TMA-tiled ---------------------------------------------------------------------------------
// The fast path for the common request: every layer has at most one adapter of rank <= 64. W moves by tiled TMA, one
// request per 128x64 box, through per-layer tensor maps that the host encodes once (the weights do not move between
// requests); 256-byte bulk copies per row were request-rate bound in the TMA unit and slower than plain 16-byte loads.
// Tiles are dealt to the persistent CTAs round-robin in chunks of 4 consecutive tiles, which walk along one 128-row band
// of one layer: the layer's table entry and the adapter's B tile are read once per chunk, while neighbouring CTAs
// still stream neighbouring addresses (whole contiguous ranges per CTA measured 35% slower, single tiles 30%: the
// first loses DRAM locality, the second re-reads B and the table entry for every tile). A pure restore (no adapters)
// has nothing to reuse and runs with chunks of 1.
// Four roles, each with its own ring so that no role waits for another's latency:
//   * warps 0-3 (one thread per tile row): read the row's delta from TMEM, fold it into the row of W in shared memory
//     with the reference's rounding, then thread 0 sends the tile back with TMA stores (clipped at the matrix edge);
//   * warp 4, one thread: starts the TMA loads of the pristine W tile (ring of 4 x 32 KB, two swizzled 128x64 boxes per
//     tile; boxes past the matrix edge are zero-filled by the TMA unit);
//   * warp 5, one thread: delta = B A as 128x64x16 tcgen05.mma instructions into one of two TMEM accumulators; the
//     instructions' completion frees the adapter stages;
//   * warps 6-9: copy the adapter's A tile (ring of 3) and, at the start of a band, its B tile (2 buffers) with 16-byte
//     async copies into the layouts tcgen05.mma reads.
// A W stage is reused once the TMA store has read it (cp.async.bulk.wait_group.read), so loads of tiles j+1..j+3, the
// product of tile j+1 and the write-back of tile j are in flight together.
// MAXL = adapters per layer the launch can take (1 or 2: one rank <= 64 product per adapter and tile, all accumulated in
// the tile's TMEM accumulator; the adapters of a layer share one scale). With two adapters the B buffers double and the W
// ring gives up a stage to make room.
constexpr int WS_NA = 3;                        // A ring
constexpr int WS_W_BYTES = 32768;
constexpr int WS_A_BYTES = 16384;
constexpr int WS_B_BYTES = 16384;
template <int MAXL>
struct WsCfg {
    static constexpr int NW = MAXL == 1 ? 4 : 3;                 // W ring
    static constexpr int NB = 2 * MAXL;                          // B buffers: two bands in flight x adapters
    static constexpr int SMEM = NW * WS_W_BYTES + WS_NA * WS_A_BYTES + NB * WS_B_BYTES + 1024;
};
constexpr int WS_THREADS = 320;
constexpr int WS_PRODUCERS = 128;
constexpr int WS_CHUNK = 4;                     // consecutive tiles per CTA turn
constexpr int WS_MAX_LAYERS_SMEM = 2048;       // tile_start cached in shared memory up to this many layers

struct WsTile {
    int li, row0, col0, in_f, n_lora;
    float scale;
};

// One role's view of the layer that owns the current tile; the table entry is re-read only when the layer changes.
template <int MAXL>
struct WsLayer {
    int li = -1, start = 0, end = 0;
    int in_f = 0, out_f = 0, n_lora = 0, tiles_n = 1;
    int rank[MAXL];
    float scale = 0.f;
    const __half* B[MAXL];
    const __half* A[MAXL];
    bool has_w0 = false;
    __device__ __forceinline__ void seek(const katz_lora_layer* __restrict__ layers, const int* tile_start, int n_layers,
                                         int total_tiles, int tile) {
        if (li >= 0 && tile >= start && tile < end) return;
        li = find_layer(tile_start, n_layers, tile);
        start = tile_start[li];
        end = li + 1 < n_layers ? tile_start[li + 1] : total_tiles;
        const katz_lora_layer* L = layers + li;
        in_f = L->in_features;
        out_f = L->out_features;
        n_lora = min(L->n_lora, MAXL);
        scale = L->scale[0];
#pragma unroll
        for (int a = 0; a < MAXL; ++a) {
            rank[a] = L->rank[a];
            B[a] = reinterpret_cast<const __half*>(L->B[a]);
            A[a] = reinterpret_cast<const __half*>(L->A[a]);
        }
        has_w0 = L->W0 != nullptr;
        tiles_n = (in_f + 127) >> 7;
    }
};

template <int MAXL>
__global__ void __launch_bounds__(WS_THREADS, 1) lora_merge_f16_ws_kernel(const katz_lora_layer* __restrict__ layers,
                                                                         const CUtensorMap* __restrict__ maps,
                                                                         const int* __restrict__ tile_start, int n_layers,
                                                                         int total_tiles, float sign,
                                                                         int* __restrict__ status, int CH) {
    // This kernel writes weights that the next kernels read as operands they may fetch before their own dependency wait:
    // its dependents are released only by its completion (no griddepcontrol.launch_dependents here).
    pdl_wait();      // nothing below may touch global memory before the kernels this launch depends on are done
    using namespace tc05;
    using T = __half;
    constexpr int WS_NW = WsCfg<MAXL>::NW;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* smem_a = smem + WS_NW * WS_W_BYTES;
    unsigned char* smem_b = smem_a + WS_NA * WS_A_BYTES;
    __shared__ WsTile s_tile[WS_NW];
    // per A stage: {adapters of the tile, rank of this stage's adapter, B buffer, bit 0: first tile of a band, bit 1: first
    // adapter of the tile, bit 2: last adapter of the tile}
    __shared__ int4 s_ab[WS_NA];
    __shared__ __align__(8) uint64_t s_bars[2 * WS_NW + 2 * WS_NA + 2 + 4];
    __shared__ uint32_t s_tmem;
    __shared__ int s_start[WS_MAX_LAYERS_SMEM];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (n_layers <= WS_MAX_LAYERS_SMEM) {
        for (int i = tid; i < n_layers; i += WS_THREADS) s_start[i] = tile_start[i];
        tile_start = s_start;
    }
    const uint32_t wfull0 = smem_u32(s_bars), wempty0 = wfull0 + 8 * WS_NW, afull0 = wempty0 + 8 * WS_NW,
                   aempty0 = afull0 + 8 * WS_NA, bempty0 = aempty0 + 8 * WS_NA, dfull0 = bempty0 + 16, dempty0 = dfull0 + 16;
    if (tid == 0) {
        for (int s = 0; s < WS_NW; ++s) {
            mbar_init(wfull0 + 8 * s, 1);          // the loader's expect_tx arrival; the TMA bytes complete it
            mbar_init(wempty0 + 8 * s, 1);         // the storing thread, once the TMA store has read the stage
        }
        for (int s = 0; s < WS_NA; ++s) {
            mbar_init(afull0 + 8 * s, 1 + WS_PRODUCERS);   // one plain arrival (publishes s_ab) + one async-copy arrival each
            mbar_init(aempty0 + 8 * s, 1);                 // tcgen05.commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bempty0 + 8 * b, 1);         // tcgen05.commit at the end of the band that used the buffers
            mbar_init(dfull0 + 8 * b, 1);          // delta accumulator ready (tcgen05.commit)
            mbar_init(dempty0 + 8 * b, 4);         // delta accumulator read (one arrival per fold warp)
        }
        fence_barrier_init();
    }
    if (warp == 5) {
        tmem_alloc(smem_u32(&s_tmem), 256);
        tmem_relinquish();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = s_tmem;
    // chunks of CH consecutive tiles are dealt round-robin: tile of this CTA's j-th step, or -1 past the end
    auto tile_of = [&](int j) {
        const int t = (blockIdx.x + (j / CH) * gridDim.x) * CH + j % CH;
        return t < total_tiles ? t : -1;
    };
    bool ok = true;

    if (warp < 4) {
        // ------------------------------------------------------------------------------------ fold + write-back (128 threads)
        const int row = tid;                      // TMEM lane = tile row; warp w reads lane quarter w
        for (int j = 0, tile; (tile = tile_of(j)) >= 0; ++j) {
            const int s = j % WS_NW, b = j & 1;
            ok = mbar_wait(wfull0 + 8 * s, (j / WS_NW) & 1) && mbar_wait(dfull0 + 8 * b, (j >> 1) & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            fence_after_sync();
            const WsTile t = s_tile[s];
            unsigned char* wtile = smem + s * WS_W_BYTES;
            if (t.n_lora > 0) {
                const float sc = t.scale * sign;
                uint32_t r[128];
#pragma unroll
                for (int c = 0; c < 128; c += 32) tmem_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + b * 128 + c, r + c);
                tmem_ld_wait();
                fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(dempty0 + 8 * b);
#pragma unroll
                for (int ch = 0; ch < 16; ++ch) {
                    // column chunk ch of this row: box ch/8, 128-byte row, 16-byte chunks XOR-swizzled by the row
                    uint4* wp = reinterpret_cast<uint4*>(wtile + (ch >> 3) * 16384 + row * 128 + (((ch & 7) ^ (row & 7)) << 4));
                    uint4 w = *wp;
                    __half2* wv = reinterpret_cast<__half2*>(&w);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        // half(acc) -> half(. * scale) -> half(W + .): the fp32 sum of two halfs rounds to the same half as
                        // the half-precision add (24 >= 2*11+2 significand bits), so the last step is one hadd2
                        const float2 d = __half22float2(__floats2half2_rn(__uint_as_float(r[ch * 8 + 2 * e]),
                                                                          __uint_as_float(r[ch * 8 + 2 * e + 1])));
                        wv[e] = __hadd2(wv[e], __floats2half2_rn(__fmul_rn(d.x, sc), __fmul_rn(d.y, sc)));
                    }
                    *wp = w;
                }
                fence_proxy_async();              // this thread's row update -> visible to the TMA store
            } else {
                __syncwarp();
                if (lane == 0) mbar_arrive(dempty0 + 8 * b);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");     // named barrier: the four fold warps only
            if (tid == 0) {
                const CUtensorMap* m = maps + 2 * t.li + 1;
                tma_store_2d(m, t.col0, t.row0, smem_u32(wtile));
                if (t.col0 + 64 < t.in_f) tma_store_2d(m, t.col0 + 64, t.row0, smem_u32(wtile) + 16384);
                bulk_commit();
                if (j > 0) {
                    bulk_wait_read<1>();          // the previous tile's store has read its stage
                    mbar_arrive(wempty0 + 8 * ((j - 1) % WS_NW));
                }
            }
        }
        if (tid == 0) bulk_wait<0>();
        if (!ok && lane == 0) atomicExch(status, 33);
    } else if (warp == 4) {
        // ------------------------------------------------------------------------------------ W loader (one thread)
        if (elect_one()) {
            WsLayer<MAXL> lay;
            for (int j = 0, tile; (tile = tile_of(j)) >= 0; ++j) {
                const int s = j % WS_NW;
                if (!mbar_wait(wempty0 + 8 * s, ((j / WS_NW) & 1) ^ 1)) { ok = false; break; }
                lay.seek(layers, tile_start, n_layers, total_tiles, tile);
                const int rel = tile - lay.start, tm = rel / lay.tiles_n;
                WsTile t;
                t.li = lay.li;
                t.in_f = lay.in_f;
                t.n_lora = lay.n_lora;
                t.scale = lay.scale;
                t.row0 = tm * 128;
                t.col0 = (rel - tm * lay.tiles_n) * 128;
                s_tile[s] = t;
                const CUtensorMap* m = maps + 2 * lay.li + (lay.has_w0 ? 0 : 1);
                const bool two = t.col0 + 64 < t.in_f;
                const uint32_t fb = wfull0 + 8 * s, dst = smem_u32(smem + s * WS_W_BYTES);
                mbar_expect_tx(fb, two ? 32768u : 16384u);
                tma_load_2d(dst, m, t.col0, t.row0, fb);
                if (two) tma_load_2d(dst + 16384, m, t.col0 + 64, t.row0, fb);
            }
            if (!ok) atomicExch(status, 31);
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------------------------------ MMA issuer (one thread)
        // Driven by what the adapter warps publish per A stage: one stage per (tile, adapter), or one empty stage for a
        // tile without adapters. The products of a tile's adapters accumulate in the same TMEM tile.
        if (elect_one()) {
            int ja = 0, bands_seen = 0;
            for (int j = 0, tile; (tile = tile_of(j)) >= 0 && ok; ++j) {
                const int b = j & 1;
                if (!mbar_wait(dempty0 + 8 * b, ((j >> 1) & 1) ^ 1)) { ok = false; break; }
                for (bool last = false; !last; ++ja) {
                    const int s = ja % WS_NA;
                    if (!mbar_wait(afull0 + 8 * s, (ja / WS_NA) & 1)) { ok = false; break; }
                    const int4 info = s_ab[s];
                    last = (info.w & 4) != 0;
                    if (info.x > 0) {
                        // a new band starts: once everything issued so far is complete, the previous band's B buffers are free
                        if ((info.w & 3) == 3 && bands_seen++ > 0) umma_commit(bempty0 + 8 * ((info.z / MAXL) ^ 1));
                        fence_proxy_async();          // async-copy writes of B/A -> tensor-core reads
                        fence_after_sync();
                        const uint32_t sBa = smem_u32(smem_b + info.z * WS_B_BYTES), sAa = smem_u32(smem_a + s * WS_A_BYTES);
                        const int kpad = (info.y + 15) & ~15;
                        const bool first = (info.w & 2) != 0;
                        constexpr uint32_t idesc = idesc_f16(128, 64) | (1u << 16);     // B operand MN-major
#pragma unroll
                        for (int nb = 0; nb < 2; ++nb)
                            for (int ks = 0; ks < kpad / 16; ++ks)
                                umma_f16(tmem_base + b * 128 + nb * 64, smem_desc_sw128(sBa) + 2 * ks,
                                         smem_desc_sw128(sAa + nb * 8192 + ks * 2048), idesc, !(first && ks == 0));
                    }
                    if (last) umma_commit(dfull0 + 8 * b);      // with no MMA outstanding this arrives at once (plain restore tiles)
                    umma_commit(aempty0 + 8 * s);
                }
            }
            if (!ok) atomicExch(status, 32);
        }
    } else {
        // ------------------------------------------------------------------------------------ adapter tiles (128 threads)
        const int pt = tid - 192;
        WsLayer<MAXL> lay;
        int band = -1, prev_li = -1, prev_row0 = -1;      // bands with an adapter so far; B buffers = (band & 1) * MAXL + adapter
        int ja = 0;
        for (int j = 0, tile; (tile = tile_of(j)) >= 0 && ok; ++j) {
            lay.seek(layers, tile_start, n_layers, total_tiles, tile);
            const int rel = tile - lay.start, tm = rel / lay.tiles_n;
            const int row0 = tm * 128, col0 = (rel - tm * lay.tiles_n) * 128;
            const int nsub = lay.n_lora > 0 ? lay.n_lora : 1;
            bool new_band = false;
            if (lay.n_lora > 0) {
                new_band = lay.li != prev_li || row0 != prev_row0;
                prev_li = lay.li;
                prev_row0 = row0;
                if (new_band) {
                    ++band;
                    // the buffers are free once the products of the band before last are complete
                    if (!mbar_wait(bempty0 + 8 * (band & 1), ((band >> 1) & 1) ^ 1)) { ok = false; break; }
                }
            }
#pragma unroll 1
            for (int a = 0; a < nsub; ++a, ++ja) {
                const int s = ja % WS_NA;
                if (!mbar_wait(aempty0 + 8 * s, ((ja / WS_NA) & 1) ^ 1)) { ok = false; break; }
                const int rank = lay.n_lora > 0 ? lay.rank[a < MAXL ? a : 0] : 0, kpad = (rank + 15) & ~15;
                const __half* Bm = lay.B[a < MAXL ? a : 0];
                const __half* Am = lay.A[a < MAXL ? a : 0];
                const int bbuf = (band & 1) * MAXL + a;
                const uint32_t fb = afull0 + 8 * s;
                if (lay.n_lora > 0 && new_band) {
                    const int rows = min(128, lay.out_f - row0);
                    const int c = pt & 7;
                    if (c < (kpad >> 3)) {
                        const uint32_t sB = smem_u32(smem_b + bbuf * WS_B_BYTES);
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int r = (pt >> 3) + 16 * i;
                            const bool in = (c * 8) < rank && r < rows;
                            const T* src = in ? Bm + (size_t)(row0 + r) * rank + c * 8 : Bm;
                            cp_async16(sB + b_off<T>(r, c), src, in ? 16 : 0);
                        }
                    }
                }
                if (pt == 0) {
                    s_ab[s] = make_int4(lay.n_lora, rank, bbuf, (new_band ? 1 : 0) | (a == 0 ? 2 : 0) | (a == nsub - 1 ? 4 : 0));
                    mbar_arrive(fb);
                }
                if (lay.n_lora > 0) {
                    const int cols = min(128, lay.in_f - col0);
                    const int c = pt & 15;
                    const bool col_in = (c * 8) < cols;
                    const uint32_t sA = smem_u32(smem_a + s * WS_A_BYTES);
                    const T* src0 = Am + col0 + c * 8;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int r = (pt >> 4) + 8 * i;
                        if (r < kpad) {
                            const bool in = r < rank && col_in;
                            cp_async16(sA + a_off<T, true>(r, c), in ? src0 + (size_t)r * lay.in_f : Am, in ? 16 : 0);
                        }
                    }
                }
                cp_async_mbar_arrive_noinc(fb);
            }
        }
        if (!ok && lane == 0) atomicExch(status, 34);
        cp_async_wait<0>();
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 5) {
        fence_after_sync();
        tmem_dealloc(tmem_base, 256);
    }
}

int* tc05_status_device_ptr();   // gemm_tc05.cu
// lora_merge_f32.cu: the fp32 fast path (tiles of 128 x 64, bf16x3 products on tcgen05)
int lora_merge_f32_ws_launch(const katz_lora_layer* d_layers, const void* d_tile_maps, const int* d_tile_start, int n_layers,
                             int total_tiles, float sign, int no_adapters, int grid, cudaStream_t st);

static int lm_sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
    }
    return n;
}

}  // namespace katz

using namespace katz;

extern "C" int katz_lora_tile_rows(int w_dtype) { return w_dtype == KATZ_DTYPE_F16 ? LmCfg<__half>::TM : LmCfg<float>::TM; }
extern "C" int katz_lora_tile_cols(void) { return LM_TN; }
// Tile geometry of the TMA-tiled fast paths (KATZ_LORA_UNIFORM_TILES*): 128 x 128 for fp16 weights, 128 x 64 for fp32.
extern "C" int katz_lora_fast_tile_rows(int w_dtype) { (void)w_dtype; return 128; }
extern "C" int katz_lora_fast_tile_cols(int w_dtype) { return w_dtype == KATZ_DTYPE_F16 ? 128 : 64; }

extern "C" int katz_lora_merge(const katz_lora_layer* d_layers, const int* d_tile_start, int n_layers, int total_tiles,
                               int w_dtype, float sign, int max_tiles_per_layer, int flags, const void* d_tile_maps,
                               void* stream) {
    KATZ_CHECK_ARG(d_layers && d_tile_start, KATZ_EINVAL);
    KATZ_CHECK_ARG(n_layers > 0 && total_tiles > 0, KATZ_ESIZE);
    KATZ_CHECK_ARG(w_dtype == KATZ_DTYPE_F16 || w_dtype == KATZ_DTYPE_F32, KATZ_EINVAL);
    KATZ_CHECK_ARG(sign == 1.0f || sign == -1.0f, KATZ_EINVAL);
    cudaStream_t st = (cudaStream_t)stream;
    static bool attr_set_dev[KATZ_MAX_DEVICES] = {false};
    bool& attr_set = attr_set_dev[current_device_index()];
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(lora_merge_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, LmCfg<__half>::SMEM);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(lora_merge_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, LmCfg<float>::SMEM);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    const int grid = total_tiles < lm_sm_count() ? total_tiles : lm_sm_count();
    const int in_smem = (n_layers <= LM_MAX_LAYERS_SMEM && max_tiles_per_layer > 0 && max_tiles_per_layer < 65536) ? 1 : 0;
    static int use_tc05 = -1;
    if (use_tc05 < 0) {
        const char* e = getenv("KATZ_LORA_MMA");
        use_tc05 = (e && e[0] == '1') ? 0 : 1;
    }
    if (w_dtype == KATZ_DTYPE_F32 && use_tc05 && (flags & KATZ_LORA_UNIFORM_TILES) && d_tile_maps) {
        // fp32 fast path: d_tile_start / total_tiles count tiles of katz_lora_fast_tile_rows x katz_lora_fast_tile_cols
        KATZ_CHECK_ARG((reinterpret_cast<uintptr_t>(d_tile_maps) & 63) == 0, KATZ_EALIGN);
        return lora_merge_f32_ws_launch(d_layers, d_tile_maps, d_tile_start, n_layers, total_tiles, sign,
                                        (flags & KATZ_LORA_NO_ADAPTERS) ? 1 : 0, grid, st);
    }
    if (w_dtype == KATZ_DTYPE_F16 && use_tc05 && (flags & (KATZ_LORA_UNIFORM_TILES | KATZ_LORA_UNIFORM_TILES_2)) && d_tile_maps) {
        KATZ_CHECK_ARG((reinterpret_cast<uintptr_t>(d_tile_maps) & 63) == 0, KATZ_EALIGN);
        static bool attr3_dev[KATZ_MAX_DEVICES] = {false};
        bool& attr3 = attr3_dev[current_device_index()];
        if (!attr3) {
            cudaError_t e = cudaFuncSetAttribute(lora_merge_f16_ws_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, WsCfg<1>::SMEM);
            if (e != cudaSuccess) return (int)e;
            e = cudaFuncSetAttribute(lora_merge_f16_ws_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, WsCfg<2>::SMEM);
            if (e != cudaSuccess) return (int)e;
            attr3 = true;
        }
        int* status = tc05_status_device_ptr();
        if (!status) return KATZ_ENOTREADY;
        const CUtensorMap* maps = reinterpret_cast<const CUtensorMap*>(d_tile_maps);
        const int ch = (flags & KATZ_LORA_NO_ADAPTERS) ? 1 : WS_CHUNK;
        if (flags & KATZ_LORA_UNIFORM_TILES)
            launch_k(lora_merge_f16_ws_kernel<1>, grid, WS_THREADS, WsCfg<1>::SMEM, st, d_layers, maps, d_tile_start, n_layers,
                     total_tiles, sign, status, ch);
        else
            launch_k(lora_merge_f16_ws_kernel<2>, grid, WS_THREADS, WsCfg<2>::SMEM, st, d_layers, maps, d_tile_start, n_layers,
                     total_tiles, sign, status, ch);
    } else if (w_dtype == KATZ_DTYPE_F16 && use_tc05) {
        static bool attr2_dev[KATZ_MAX_DEVICES] = {false};
        bool& attr2 = attr2_dev[current_device_index()];
        if (!attr2) {
            cudaError_t e = cudaFuncSetAttribute(lora_merge_f16_tc05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 LmCfg<__half>::SMEM + 1024);
            if (e != cudaSuccess) return (int)e;
            attr2 = true;
        }
        int* status = tc05_status_device_ptr();
        if (!status) return KATZ_ENOTREADY;
        launch_k(lora_merge_f16_tc05_kernel, grid, LM_THREADS, LmCfg<__half>::SMEM + 1024, st, d_layers, d_tile_start, n_layers,
                                                                                          total_tiles, sign, in_smem, status);
    } else if (w_dtype == KATZ_DTYPE_F16)
        launch_k(lora_merge_kernel<__half>, grid, LM_THREADS, LmCfg<__half>::SMEM, st, d_layers, d_tile_start, n_layers,
                 total_tiles, sign, in_smem);
    else
        launch_k(lora_merge_kernel<float>, grid, LM_THREADS, LmCfg<float>::SMEM, st, d_layers, d_tile_start, n_layers,
                 total_tiles, sign, in_smem);
    KATZ_LAUNCH_RET();
}

// Tensor maps of the fast path, two per layer (128 bytes each): [2i] the pristine copy W0 (W when there is none), [2i+1]
// the live W; 128-row x 64-column boxes with the 128-byte swizzle. They depend only on the weight pointers and shapes,
// so a caller encodes them once and keeps them in device memory.
static int encode_tile_maps(const katz_lora_layer* h_layers, int n_layers, int w_dtype, void* h_maps);

extern "C" int katz_lora_encode_tile_maps(const katz_lora_layer* h_layers, int n_layers, void* h_maps) {
    return encode_tile_maps(h_layers, n_layers, KATZ_DTYPE_F16, h_maps);
}

extern "C" int katz_lora_encode_tile_maps_dtype(const katz_lora_layer* h_layers, int n_layers, int w_dtype, void* h_maps) {
    KATZ_CHECK_ARG(w_dtype == KATZ_DTYPE_F16 || w_dtype == KATZ_DTYPE_F32, KATZ_EINVAL);
    return encode_tile_maps(h_layers, n_layers, w_dtype, h_maps);
}

static int encode_tile_maps(const katz_lora_layer* h_layers, int n_layers, int w_dtype, void* h_maps) {
    KATZ_CHECK_ARG(h_layers && h_maps, KATZ_EINVAL);
    KATZ_CHECK_ARG(n_layers > 0, KATZ_ESIZE);
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn enc = nullptr;
    if (!enc) {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            return KATZ_ENOTREADY;
        enc = reinterpret_cast<EncodeFn>(f);
    }
    CUtensorMap* out = reinterpret_cast<CUtensorMap*>(h_maps);
    for (int i = 0; i < n_layers; ++i) {
        const katz_lora_layer& L = h_layers[i];
        KATZ_CHECK_ARG(L.W && aligned16(L.W) && (!L.W0 || aligned16(L.W0)), KATZ_EALIGN);
        const bool f32 = w_dtype == KATZ_DTYPE_F32;
        KATZ_CHECK_ARG(L.out_features > 0 && L.in_features > 0 && L.in_features % (f32 ? 4 : 8) == 0, KATZ_ESIZE);
        cuuint64_t dims[2] = {(cuuint64_t)L.in_features, (cuuint64_t)L.out_features};
        cuuint64_t strides[1] = {(cuuint64_t)L.in_features * (f32 ? 4 : 2)};
        cuuint32_t box[2] = {f32 ? 32u : 64u, 128};      // 128 bytes per box row either way
        cuuint32_t es[2] = {1, 1};
        for (int k = 0; k < 2; ++k) {
            void* base = (k == 0 && L.W0) ? const_cast<void*>(L.W0) : L.W;
            CUtensorMap tmp;
            CUresult r = enc(&tmp, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return KATZ_EINVAL;
            memcpy(out + 2 * i + k, &tmp, sizeof(CUtensorMap));      // the caller's buffer need not be 64-byte aligned
        }
    }
    return KATZ_OK;
}

// Host-side validation of a whole table in one call. Returns 0, or the negative argument error of the first bad entry
// with its index in *bad_index (when given).
extern "C" int katz_lora_table_check(const katz_lora_layer* h_layers, int n_layers, int w_dtype, int* bad_index) {
    KATZ_CHECK_ARG(h_layers, KATZ_EINVAL);
    for (int i = 0; i < n_layers; ++i) {
        const int rc = katz_lora_layer_check(h_layers + i, w_dtype);
        if (rc != KATZ_OK) {
            if (bad_index) *bad_index = i;
            return rc;
        }
    }
    return KATZ_OK;
}

// Host-side validation of one table entry (the table itself lives in device memory, so the caller validates before
// uploading). Returns 0 or a negative argument error.
extern "C" int katz_lora_layer_check(const katz_lora_layer* h, int w_dtype) {
    KATZ_CHECK_ARG(h, KATZ_EINVAL);
    KATZ_CHECK_ARG(w_dtype == KATZ_DTYPE_F16 || w_dtype == KATZ_DTYPE_F32, KATZ_EINVAL);
    const int epc = w_dtype == KATZ_DTYPE_F16 ? 8 : 4;
    KATZ_CHECK_ARG(h->W && aligned16(h->W) && (!h->W0 || aligned16(h->W0)), KATZ_EALIGN);
    KATZ_CHECK_ARG(h->out_features > 0 && h->in_features > 0 && h->in_features % epc == 0, KATZ_ESIZE);
    KATZ_CHECK_ARG(h->n_lora >= 0 && h->n_lora <= KATZ_LORA_MAX_ADAPTERS, KATZ_ESIZE);
    for (int i = 0; i < h->n_lora; ++i) {
        KATZ_CHECK_ARG(h->A[i] && h->B[i] && aligned16(h->A[i]) && aligned16(h->B[i]), KATZ_EALIGN);
        KATZ_CHECK_ARG(h->rank[i] > 0 && h->rank[i] % 8 == 0, KATZ_ESIZE);
    }
    return KATZ_OK;
}
