// LoRA merge for fp32 weights and fp32 adapters on the tcgen05 tensor path: W = (W0 ? W0 : W) + sign * scale * B A, one
// launch for every layer of the table, bound by reading and writing W (2 x 4 bytes per element).
//
// The reference's CPU-runnable configuration keeps W, up and down in fp32 (lora_utils.py:29-33 with fp32 tensors):
// the rank-r product must then carry fp32 accuracy, which one pass of a 16-bit tensor-core format does not. Each fp32
// operand is split into three bf16 terms (x = x1 + x2 + x3 exactly, 8 significand bits each, same exponent range as fp32) and the
// product is the sum of the six partial products whose weight is above 2^-24: B1A1 + B1A2 + B2A1 + B2A2 + B1A3 + B3A1, all
// accumulated in the same fp32 accumulator in tensor memory (24 tcgen05.mma of 128 x 64 x 16 per tile at rank 64). The
// dropped terms are below 2^-23 of |B||A|: the delta matches an fp32 matrix product to parts in 1e-7.
//
// Same persistent, warp-specialised structure as the fp16 kernel (lora_merge.cu): tiles of 128 rows x 64 columns (32 KB
// of fp32) walk along one 128-row band of a layer in chunks;
//   * warps 0-3, one thread per tile row: read the row's delta from TMEM, fold `W + delta * scale` into the row of W in
//     shared memory, thread 0 sends the tile back with TMA stores;
//   * warp 4, one thread: TMA loads of the pristine W tile (two swizzled 128 x 32 fp32 boxes) into a ring of three;
//   * warp 5, one thread: the 24 tcgen05.mma per tile into one of two TMEM accumulators;
//   * warps 6-13: read the adapter's fp32 A tile (per tile) and B tile (per band) from global memory, split them into the three
//     bf16 terms and store those in the shared-memory layouts tcgen05.mma reads.
// Every mbarrier wait is bounded; a time-out records the library's status word and the CTA unwinds.
#include <cuda_bf16.h>

#include "tc05.cuh"
#include "katz_b200.h"

namespace katz {

using namespace tc05;

int* tc05_status_device_ptr();   // gemm_tc05.cu

constexpr int F32_NW = 3;                        // W ring
constexpr int F32_NA = 3;                        // A ring (three bf16 terms per stage): the splitting warps run two tiles ahead
constexpr int F32_NB = 1;                        // B term sets (a second one would cost two A stages: measured slower)
constexpr int F32_W_BYTES = 32768;               // 128 rows x 64 fp32
constexpr int F32_AT_BYTES = 8192;               // one bf16 term of A: 64 k-rows x 64 columns
constexpr int F32_A_BYTES = 3 * F32_AT_BYTES;
constexpr int F32_BT_BYTES = 16384;              // one bf16 term of B: 128 rows x 64 k
constexpr int F32_B_BYTES = 3 * F32_BT_BYTES;
constexpr int F32_SMEM = F32_NW * F32_W_BYTES + F32_NA * F32_A_BYTES + F32_NB * F32_B_BYTES + 1024;
constexpr int F32_THREADS = 448;
constexpr int F32_PRODUCERS = 256;

struct F32Tile {
    int li, row0, col0, in_f, n_lora;
    float scale;
};

__device__ __forceinline__ int f32_find_layer(const int* tile_start, int n_layers, int tile) {
    int lo = 0, hi = n_layers - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (tile_start[mid] <= tile) lo = mid;
        else hi = mid - 1;
    }
    return lo;
}

struct F32Layer {
    int li = -1, start = 0, end = 0;
    int in_f = 0, out_f = 0, n_lora = 0, rank = 0, tiles_n = 1;
    float scale = 0.f;
    const float* B = nullptr;
    const float* A = nullptr;
    bool has_w0 = false;
    __device__ __forceinline__ void seek(const katz_lora_layer* __restrict__ layers, const int* tile_start, int n_layers,
                                         int total_tiles, int tile) {
        if (li >= 0 && tile >= start && tile < end) return;
        li = f32_find_layer(tile_start, n_layers, tile);
        start = tile_start[li];
        end = li + 1 < n_layers ? tile_start[li + 1] : total_tiles;
        const katz_lora_layer* L = layers + li;
        in_f = L->in_features;
        out_f = L->out_features;
        n_lora = L->n_lora;
        rank = L->rank[0];
        scale = L->scale[0];
        B = reinterpret_cast<const float*>(L->B[0]);
        A = reinterpret_cast<const float*>(L->A[0]);
        has_w0 = L->W0 != nullptr;
        tiles_n = (in_f + 63) >> 6;
    }
};

// x -> three bf16 terms, packed two elements per 32-bit word. The terms are TRUNCATIONS (the upper 16 bits of the fp32
// word), not roundings: x1 = hi16(x), x2 = hi16(x - x1), x3 = hi16(x - x1 - x2), each difference exact, so x1 + x2 + x3
// reproduces all 24 significand bits of x and the split costs a mask, a subtraction and a byte permute per term instead of
// conversions (the four splitting warps are what the kernel waits for).
__device__ __forceinline__ uint32_t hi16_pair(float lo, float hi) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(r) : "r"(__float_as_uint(lo)), "r"(__float_as_uint(hi)));
    return r;
}
__device__ __forceinline__ float drop_hi16(float x) { return x - __uint_as_float(__float_as_uint(x) & 0xffff0000u); }
__device__ __forceinline__ void split3(float x0, float x1, uint32_t& t1, uint32_t& t2, uint32_t& t3) {
    t1 = hi16_pair(x0, x1);
    const float r0 = drop_hi16(x0), r1 = drop_hi16(x1);
    t2 = hi16_pair(r0, r1);
    const float s0 = drop_hi16(r0), s1 = drop_hi16(r1);
    t3 = hi16_pair(s0, s1);
}

// eight consecutive fp32 values (already loaded) -> one 16-byte chunk of each term
__device__ __forceinline__ void split_chunk(const float4& v0, const float4& v1, uint4& o1, uint4& o2, uint4& o3) {
    split3(v0.x, v0.y, o1.x, o2.x, o3.x);
    split3(v0.z, v0.w, o1.y, o2.y, o3.y);
    split3(v1.x, v1.y, o1.z, o2.z, o3.z);
    split3(v1.z, v1.w, o1.w, o2.w, o3.w);
}
__device__ __forceinline__ void load8(const float* src, bool in, float4& v0, float4& v1) {
    v0 = make_float4(0.f, 0.f, 0.f, 0.f);
    v1 = v0;
    if (in) {
        v0 = __ldg(reinterpret_cast<const float4*>(src));
        v1 = __ldg(reinterpret_cast<const float4*>(src + 4));
    }
}

// kind::f16 instruction descriptor with bf16 operands, fp32 accumulate, B operand MN-major
__host__ __device__ constexpr uint32_t idesc_bf16_bmn(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__global__ void __launch_bounds__(F32_THREADS, 1) lora_merge_f32_ws_kernel(const katz_lora_layer* __restrict__ layers,
                                                                          const CUtensorMap* __restrict__ maps,
                                                                          const int* __restrict__ tile_start, int n_layers,
                                                                          int total_tiles, float sign, int* __restrict__ status,
                                                                          int CH) {
    // Writes weights, which later kernels may fetch before their own dependency wait: dependents are released only by this
    // kernel's completion (no griddepcontrol.launch_dependents).
    pdl_wait();
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* smem_a = smem + F32_NW * F32_W_BYTES;
    unsigned char* smem_b = smem_a + F32_NA * F32_A_BYTES;
    __shared__ F32Tile s_tile[F32_NW];
    __shared__ int4 s_ab[F32_NA];                // {adapters of the tile, rank, -, first tile of a band}
    __shared__ __align__(8) uint64_t s_bars[2 * F32_NW + 2 * F32_NA + F32_NB + 4];
    __shared__ uint32_t s_tmem;
    // (the tile -> layer table stays in global memory: it is searched only when a role crosses into another layer, and
    // shared memory is full: three W stages, three A stages and one set of B terms)

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t wfull0 = smem_u32(s_bars), wempty0 = wfull0 + 8 * F32_NW, afull0 = wempty0 + 8 * F32_NW,
                   aempty0 = afull0 + 8 * F32_NA, bempty0 = aempty0 + 8 * F32_NA, dfull0 = bempty0 + 8 * F32_NB, dempty0 = dfull0 + 16;
    if (tid == 0) {
        for (int s = 0; s < F32_NW; ++s) {
            mbar_init(wfull0 + 8 * s, 1);          // the loader's expect_tx arrival; the TMA bytes complete it
            mbar_init(wempty0 + 8 * s, 1);         // the storing thread, once the TMA store has read the stage
        }
        for (int s = 0; s < F32_NA; ++s) {
            mbar_init(afull0 + 8 * s, F32_PRODUCERS);      // every producer thread, after its stores and its proxy fence
            mbar_init(aempty0 + 8 * s, 1);                 // tcgen05.commit
        }
        for (int b = 0; b < F32_NB; ++b) mbar_init(bempty0 + 8 * b, 1);      // tcgen05.commit once the band's products are complete
        for (int b = 0; b < 2; ++b) {
            mbar_init(dfull0 + 8 * b, 1);          // delta accumulator ready (tcgen05.commit)
            mbar_init(dempty0 + 8 * b, 4);         // delta accumulator read (one arrival per fold warp)
        }
        fence_barrier_init();
    }
    if (warp == 5) {
        tmem_alloc(smem_u32(&s_tmem), 128);
        tmem_relinquish();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = s_tmem;
    auto tile_of = [&](int j) {
        const int t = (blockIdx.x + (j / CH) * gridDim.x) * CH + j % CH;
        return t < total_tiles ? t : -1;
    };
    bool ok = true;

    if (warp < 4) {
        // ------------------------------------------------------------------------------------ fold + write-back (128 threads)
        const int row = tid;
        for (int j = 0; tile_of(j) >= 0; ++j) {
            const int s = j % F32_NW, b = j & 1;
            ok = mbar_wait(wfull0 + 8 * s, (j / F32_NW) & 1) && mbar_wait(dfull0 + 8 * b, (j >> 1) & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            fence_after_sync();
            const F32Tile t = s_tile[s];
            unsigned char* wtile = smem + s * F32_W_BYTES;
            if (t.n_lora > 0) {
                const float sc = t.scale * sign;
                uint32_t r[64];
                tmem_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + b * 64, r);
                tmem_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + b * 64 + 32, r + 32);
                tmem_ld_wait();
                fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(dempty0 + 8 * b);
#pragma unroll
                for (int ch = 0; ch < 16; ++ch) {
                    // fp32 chunk ch (4 columns) of this row: box ch/8, 128-byte row, 16-byte chunks XOR-swizzled by the row
                    float4* wp = reinterpret_cast<float4*>(wtile + (ch >> 3) * 16384 + row * 128 + (((ch & 7) ^ (row & 7)) << 4));
                    float4 w = *wp;
                    // `W += (up @ down) * scale` in fp32: the product's scaling and the addition round separately
                    w.x = __fadd_rn(w.x, __fmul_rn(__uint_as_float(r[ch * 4 + 0]), sc));
                    w.y = __fadd_rn(w.y, __fmul_rn(__uint_as_float(r[ch * 4 + 1]), sc));
                    w.z = __fadd_rn(w.z, __fmul_rn(__uint_as_float(r[ch * 4 + 2]), sc));
                    w.w = __fadd_rn(w.w, __fmul_rn(__uint_as_float(r[ch * 4 + 3]), sc));
                    *wp = w;
                }
                fence_proxy_async();
            } else {
                __syncwarp();
                if (lane == 0) mbar_arrive(dempty0 + 8 * b);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (tid == 0) {
                const CUtensorMap* m = maps + 2 * t.li + 1;
                tma_store_2d(m, t.col0, t.row0, smem_u32(wtile));
                if (t.col0 + 32 < t.in_f) tma_store_2d(m, t.col0 + 32, t.row0, smem_u32(wtile) + 16384);
                bulk_commit();
                if (j > 0) {
                    bulk_wait_read<1>();
                    mbar_arrive(wempty0 + 8 * ((j - 1) % F32_NW));
                }
            }
        }
        if (tid == 0) bulk_wait<0>();
        if (!ok && lane == 0) atomicExch(status, 43);
    } else if (warp == 4) {
        // ------------------------------------------------------------------------------------ W loader (one thread)
        if (elect_one()) {
            F32Layer lay;
            for (int j = 0, tile; (tile = tile_of(j)) >= 0; ++j) {
                const int s = j % F32_NW;
                if (!mbar_wait(wempty0 + 8 * s, ((j / F32_NW) & 1) ^ 1)) { ok = false; break; }
                lay.seek(layers, tile_start, n_layers, total_tiles, tile);
                const int rel = tile - lay.start, tm = rel / lay.tiles_n;
                F32Tile t;
                t.li = lay.li;
                t.in_f = lay.in_f;
                t.n_lora = lay.n_lora;
                t.scale = lay.scale;
                t.row0 = tm * 128;
                t.col0 = (rel - tm * lay.tiles_n) * 64;
                s_tile[s] = t;
                const CUtensorMap* m = maps + 2 * lay.li + (lay.has_w0 ? 0 : 1);
                const bool two = t.col0 + 32 < t.in_f;
                const uint32_t fb = wfull0 + 8 * s, dst = smem_u32(smem + s * F32_W_BYTES);
                mbar_expect_tx(fb, two ? 32768u : 16384u);
                tma_load_2d(dst, m, t.col0, t.row0, fb);
                if (two) tma_load_2d(dst + 16384, m, t.col0 + 32, t.row0, fb);
            }
            if (!ok) atomicExch(status, 41);
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------------------------------ MMA issuer (one thread)
        if (elect_one()) {
            int bands = 0;
            for (int j = 0; tile_of(j) >= 0; ++j) {
                const int s = j % F32_NA, b = j & 1;
                if (!mbar_wait(afull0 + 8 * s, (j / F32_NA) & 1)) { ok = false; break; }
                if (!mbar_wait(dempty0 + 8 * b, ((j >> 1) & 1) ^ 1)) { ok = false; break; }
                const int4 info = s_ab[s];
                if (info.x > 0) {
                    fence_after_sync();
                    if (info.w) ++bands;
                    const int bset = (bands - 1) % F32_NB;
                    const uint32_t sB = smem_u32(smem_b + bset * F32_B_BYTES), sA = smem_u32(smem_a + s * F32_A_BYTES);
                    const int ksteps = ((info.y + 15) & ~15) >> 4;
                    constexpr uint32_t idesc = idesc_bf16_bmn(128, 64);
                    // (B term, A term) pairs whose product is kept, largest first
                    constexpr int TB[6] = {0, 0, 1, 1, 0, 2}, TA[6] = {0, 1, 0, 1, 2, 0};
                    bool first = true;
#pragma unroll
                    for (int q = 0; q < 6; ++q) {
                        for (int ks = 0; ks < ksteps; ++ks) {
                            umma_f16(tmem_base + b * 64, smem_desc_sw128(sB + TB[q] * F32_BT_BYTES) + 2 * ks,
                                     smem_desc_sw128(sA + TA[q] * F32_AT_BYTES + ks * 2048), idesc, first ? 0u : 1u);
                            first = false;
                        }
                    }
                    if (info.z) umma_commit(bempty0 + 8 * bset);      // last tile of the band: its completion frees the set
                }
                umma_commit(dfull0 + 8 * b);
                umma_commit(aempty0 + 8 * s);
            }
            if (!ok) atomicExch(status, 42);
        }
    } else {
        // ------------------------------------------------------------------------------------ adapter terms (128 threads)
        const int pt = tid - 192;
        F32Layer lay;
        int band = -1, prev_li = -1, prev_row0 = -1;
        for (int j = 0, tile; (tile = tile_of(j)) >= 0; ++j) {
            const int s = j % F32_NA;
            if (!mbar_wait(aempty0 + 8 * s, ((j / F32_NA) & 1) ^ 1)) { ok = false; break; }
            lay.seek(layers, tile_start, n_layers, total_tiles, tile);
            const int rel = tile - lay.start, tm = rel / lay.tiles_n;
            const int row0 = tm * 128, col0 = (rel - tm * lay.tiles_n) * 64;
            const int rank = lay.rank, kpad = (rank + 15) & ~15;
            const uint32_t fb = afull0 + 8 * s;
            bool new_band = false, last_of_band = false;
            if (lay.n_lora > 0) {
                new_band = lay.li != prev_li || row0 != prev_row0;
                prev_li = lay.li;
                prev_row0 = row0;
                // is the NEXT tile of this CTA in another band (or is there none)? then this tile's products free the B terms
                const int nxt = tile_of(j + 1);
                if (nxt < 0) last_of_band = true;
                else if (nxt >= lay.end) last_of_band = true;
                else last_of_band = ((nxt - lay.start) / lay.tiles_n) != tm;
                if (new_band) {
                    ++band;
                    const int rows = min(128, lay.out_f - row0);
                    const int c = pt & 7;                  // 8-element chunk of the rank
                    // every load of this thread is requested before the first is consumed, and before the wait for the
                    // one set of B terms to be free (the previous band's products complete): the latency hides under it
                    float4 v0[4], v1[4];
                    if (c * 8 < kpad) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int r = (pt >> 3) + 32 * i;
                            load8(lay.B + (size_t)(row0 + r) * rank + c * 8, (c * 8) < rank && r < rows, v0[i], v1[i]);
                        }
                    }
                    // the set is free once the products of the band before last are complete
                    if (band >= F32_NB && !mbar_wait(bempty0 + 8 * (band % F32_NB), ((band / F32_NB) - 1) & 1)) { ok = false; break; }
                    unsigned char* sBset = smem_b + (band % F32_NB) * F32_B_BYTES;
                    if (c * 8 < kpad) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int r = (pt >> 3) + 32 * i;
                            uint4 o1, o2, o3;
                            split_chunk(v0[i], v1[i], o1, o2, o3);
                            const uint32_t off = r * 128 + ((c ^ (r & 7)) << 4);
                            *reinterpret_cast<uint4*>(sBset + off) = o1;
                            *reinterpret_cast<uint4*>(sBset + F32_BT_BYTES + off) = o2;
                            *reinterpret_cast<uint4*>(sBset + 2 * F32_BT_BYTES + off) = o3;
                        }
                    }
                }
                const int cols = min(64, lay.in_f - col0);
                const int c = pt & 7;                      // 8-column chunk of the tile
                unsigned char* sA = smem_a + s * F32_A_BYTES;
                float4 v0[2], v1[2];
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int r = (pt >> 3) + 32 * i;      // k-row
                    load8(lay.A + (size_t)r * lay.in_f + col0 + c * 8, r < rank && (c * 8) < cols, v0[i], v1[i]);
                }
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int r = (pt >> 3) + 32 * i;
                    if (r < kpad) {
                        uint4 o1, o2, o3;
                        split_chunk(v0[i], v1[i], o1, o2, o3);
                        const uint32_t off = r * 128 + ((c ^ (r & 7)) << 4);
                        *reinterpret_cast<uint4*>(sA + off) = o1;
                        *reinterpret_cast<uint4*>(sA + F32_AT_BYTES + off) = o2;
                        *reinterpret_cast<uint4*>(sA + 2 * F32_AT_BYTES + off) = o3;
                    }
                }
            }
            if (pt == 0) s_ab[s] = make_int4(lay.n_lora, rank, last_of_band ? 1 : 0, new_band ? 1 : 0);
            fence_proxy_async();          // this thread's term stores -> visible to the tensor core
            mbar_arrive(fb);
        }
        if (!ok && lane == 0) atomicExch(status, 44);
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 5) {
        fence_after_sync();
        tmem_dealloc(tmem_base, 128);
    }
}

// Tiles per CTA turn. The SDXL targets are 640, 1280, 2560 or 5120 columns wide (10, 20, 40, 80 tiles per band), so turns of
// 10 never straddle two bands and the B terms are split once per turn (8: 3.61 ms, 10: 3.49 ms, 16: 3.96 ms for the
// 700-layer set).
constexpr int F32_CHUNK = 10;

// Launcher used by katz_lora_merge (lora_merge.cu) for fp32 tables with at most one adapter of rank <= 64 per layer.
int lora_merge_f32_ws_launch(const katz_lora_layer* d_layers, const void* d_tile_maps, const int* d_tile_start, int n_layers,
                             int total_tiles, float sign, int no_adapters, int grid, cudaStream_t st) {
    static bool attr_dev[KATZ_MAX_DEVICES] = {false};
    bool& attr = attr_dev[current_device_index()];
    if (!attr) {
        cudaError_t e = cudaFuncSetAttribute(lora_merge_f32_ws_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F32_SMEM);
        if (e != cudaSuccess) return (int)e;
        attr = true;
    }
    int* status = tc05_status_device_ptr();
    if (!status) return KATZ_ENOTREADY;
    launch_k(lora_merge_f32_ws_kernel, grid, F32_THREADS, F32_SMEM, st, d_layers, reinterpret_cast<const CUtensorMap*>(d_tile_maps),
             d_tile_start, n_layers, total_tiles, sign, status, no_adapters ? 1 : F32_CHUNK);
    KATZ_LAUNCH_RET();
}

}  // namespace katz
