/*
 * katz_b200 C ABI: the boundary a host program binds (ctypes / cffi / a TORCH_LIBRARY shim) to run the SDXL UNet
 * denoising step with adapters on one B200. It stands where the reference's `fast_kernel` torch extension and the
 * PyTorch library calls around it stand. Citations are file:line inside the reference project.
 *
 * Conventions (all entry points):
 *   - plain pointers and sizes; every pointer is DEVICE memory unless the name starts with `h_`;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream); nothing synchronises, nothing
 *     allocates unless the comment says so, so calls can be captured into a CUDA graph;
 *   - return value: 0 = launched; < 0 = argument error (KATZ_E*), nothing launched; > 0 = a cudaError_t;
 *   - activations are fp16, NHWC / token-major ([B, H*W, C]); weights are fp16 [N, K] row-major; convolution weights
 *     are [Cout, ky, kx, Cin] (torch's [Cout, Cin, ky, kx] permuted once at load time).
 */
#ifndef KATZ_B200_H_
#define KATZ_B200_H_

#ifdef __cplusplus
extern "C" {
#endif

#define KATZ_ABI_VERSION 1

#define KATZ_E_INVAL (-1)    /* null pointer / bad enum */
#define KATZ_E_ALIGN (-2)    /* pointer or stride not aligned as the kernel needs */
#define KATZ_E_SIZE (-3)     /* shape outside what the kernel supports */
#define KATZ_E_NOTREADY (-4) /* driver entry point or device set-up missing */
#define KATZ_E_DEVICE (-5)   /* a bounded device-side wait gave up */

#define KATZ_DTYPE_F16 0
#define KATZ_DTYPE_F32 1

#define KATZ_ACT_NONE 0
#define KATZ_ACT_SILU 1

int katz_abi_version(void);
/* Name of the GPU architecture the library was built for ("sm_100a"). */
const char* katz_build_arch(void);

/* ------------------------------------------------------------------------------------------------ LoRA merge ---- */
#define KATZ_LORA_MAX_ADAPTERS 4

/* One targeted linear. W is the live weight [out, in]; W0 (optional) the pristine copy it is rebuilt from.
 * B[i] = lora up [out, rank[i]], A[i] = lora down [rank[i], in], same dtype as W; scale[i] = alpha_i / rank_i * user
 * scale (the reference hard-codes 20000/64, lora_utils.py:22). */
typedef struct katz_lora_layer {
    void* W;
    const void* W0;
    const void* B[KATZ_LORA_MAX_ADAPTERS];
    const void* A[KATZ_LORA_MAX_ADAPTERS];
    int rank[KATZ_LORA_MAX_ADAPTERS];
    float scale[KATZ_LORA_MAX_ADAPTERS];
    int out_features;
    int in_features;
    int n_lora;
    int reserved_;
} katz_lora_layer;

/* Tile geometry the caller needs to build `d_tile_start`: layer i owns
 * ceil(out/tile_rows) * ceil(in/tile_cols) consecutive tiles starting at tile_start[i]. */
int katz_lora_tile_rows(int w_dtype);
int katz_lora_tile_cols(void);
/* Host-side validation of one table entry before it is uploaded. */
int katz_lora_layer_check(const katz_lora_layer* h_layer, int w_dtype);
/* The same over a whole host table; *bad_index (optional) receives the index of the first bad entry. */
int katz_lora_table_check(const katz_lora_layer* h_layers, int n_layers, int w_dtype, int* bad_index);
/* W = (W0 ? W0 : W) + sign * sum_i scale_i * B_i @ A_i over every layer of the table, one launch.
 * Replaces lora_utils.patch_on_lora's loop (lora_utils.py:28-33), StableDiffusionXLControlNetPipelineKatz.patch_on_lora
 * (pipelines/controlnet/pipeline_controlnet_sd_xl_katz.py:1741-1747) and, with n_lora = 0 and W0 set, the restore
 * `unet.load_state_dict(deepcopy(default_unet_state_dict))` (sdxl_unet_server.py:217). sign = -1 with W0 = NULL is the
 * subtractive unmerge of LoRACompatibleLinear._unfuse_lora (diffusers/models/lora.py:427-449).
 * `max_tiles_per_layer` (the largest per-layer tile count, or 0 if unknown) lets the kernel keep the tile -> layer table
 * in shared memory. `flags`: KATZ_LORA_UNIFORM_TILES promises that every layer has at most one adapter and that its rank
 * is at most 64. With the flag, fp16 weights and `d_tile_maps` (device copy of what katz_lora_encode_tile_maps wrote, 64-byte
 * aligned) the TMA-tiled warp-specialised kernel runs; otherwise, or with d_tile_maps NULL, the general kernel. */
#define KATZ_LORA_UNIFORM_TILES 1
/* KATZ_LORA_NO_ADAPTERS additionally promises n_lora == 0 in every layer (a pure restore): a scheduling hint only. */
#define KATZ_LORA_NO_ADAPTERS 2
/* KATZ_LORA_UNIFORM_TILES_2 (instead of KATZ_LORA_UNIFORM_TILES) promises at most TWO adapters per layer, each of rank at
 * most 64, with scale[1] == scale[0] wherever a layer has two: the same kernel accumulates both rank-r products in one
 * tensor-memory tile (the sum of the products is rounded once, where the reference rounds after each adapter). */
#define KATZ_LORA_UNIFORM_TILES_2 4
int katz_lora_merge(const katz_lora_layer* d_layers, const int* d_tile_start, int n_layers, int total_tiles, int w_dtype,
                    float sign, int max_tiles_per_layer, int flags, const void* d_tile_maps, void* stream);

/* Encodes, on the host, the TMA tensor maps of the fp16 fast path: 2 x 128 bytes per layer into h_maps ([2i] = W0, or W
 * when W0 is NULL; [2i+1] = W). They depend only on the weight pointers and shapes: encode once per weight set, upload,
 * and pass the device copy to katz_lora_merge. No reference counterpart (the reference merges layer by layer in
 * PyTorch, lora_utils.py:29-33). */
int katz_lora_encode_tile_maps(const katz_lora_layer* h_layers, int n_layers, void* h_maps);
/* The fast paths for either weight type. fp32 weights with fp32 adapters (the reference's CPU-runnable configuration,
 * lora_utils.py:29-33 on fp32 tensors): KATZ_LORA_UNIFORM_TILES, maps from katz_lora_encode_tile_maps_dtype(KATZ_DTYPE_F32) and a
 * `d_tile_start` / `total_tiles` counted in tiles of katz_lora_fast_tile_rows x katz_lora_fast_tile_cols (128 x 64 for fp32,
 * 128 x 128 for fp16, which equals katz_lora_tile_rows x katz_lora_tile_cols there) select the kernel that forms the rank-r
 * product from three bf16 terms per operand on the tensor cores (fp32-accurate to parts in 1e-7). */
int katz_lora_fast_tile_rows(int w_dtype);
int katz_lora_fast_tile_cols(int w_dtype);
int katz_lora_encode_tile_maps_dtype(const katz_lora_layer* h_layers, int n_layers, int w_dtype, void* h_maps);

/* -------------------------------------------------------------------------------------- fast_kernel drop-ins ---- */
/* fast_kernel::group_norm_fp16 (fast_kernel/csrc/group_norm.cuh:7-15, group_norm.cu:224-274), channels-last input.
 * `scratch` (256-byte aligned, katz_group_norm_scratch_bytes() bytes) holds per-image ticket counters in its first 1024
 * bytes, then the statistics and per-slab partial sums. The caller zero-fills it ONCE before its first use; every call
 * leaves the counters at zero again, the rest undefined. One scratch buffer serves one stream at a time. */
long long katz_group_norm_scratch_bytes(int B, int HW, int C, int G);
int katz_group_norm_nhwc_f16(const void* x, void* y, const void* gamma, const void* beta, int B, int HW, int C, int G,
                             float eps, int act, void* scratch, long long scratch_bytes, void* stream);
/* The same GroupNorm in two halves, for a tensor that is row-split across GPUs: `stats` leaves the shard's
 * (sum, sum of squares) per (batch, group) as fp64 in sums[B, G, 2]; the caller sums those across ranks; `apply`
 * normalises the shard with the global sums and n_total = (total rows) * (C / G). Needs C % 8 == 0. */
int katz_group_norm_stats_nhwc_f16(const void* x, double* sums, int B, int HW, int C, int G, void* scratch,
                                   long long scratch_bytes, void* stream);
int katz_group_norm_apply_nhwc_f16(const void* x, void* y, const double* sums, int n_parts, const void* gamma,
                                   const void* beta, int B, int HW, int C, int G, double n_total, float eps, int act,
                                   void* stream);
/* katz_group_norm_nhwc_f16 for callers that cannot allocate device memory (no counterpart in the reference: its op
 * takes scratch from torch's allocator). A serving process that gave all device memory to another allocator at
 * start-up, or a plugin inside a runtime that forbids allocations after initialisation, has no buffer to pass as
 * `scratch`; here the partial sums live in a fixed 512 KiB array inside the library's device image, held by every GPU
 * that loads the library until the process exits. The call itself allocates nothing.
 *   - Limit: shapes with katz_group_norm_scratch_bytes(B, HW, C, G) > katz_group_norm_static_scratch_bytes() return
 *     KATZ_E_SIZE; C must be a multiple of 8.
 *   - The first call on each device looks up the array's device address (that device must be current); make that
 *     first call outside any stream capture.
 *   - All calls on a device share the one array: calls that may overlap on the GPU (different streams without an
 *     ordering between them) race. Calls that are ordered need nothing cleared between them: each overwrites what it
 *     reads and leaves the ticket counters at the head of the array at zero. After such a race, or after a launch
 *     that was aborted, the counters may be left non-zero and later calls would then be wrong: call
 *     katz_group_norm_static_scratch_reset(stream) (a 1 KiB memset in stream order; it allocates nothing either). */
long long katz_group_norm_static_scratch_bytes(void);
int katz_group_norm_static_scratch_reset(void* stream);
int katz_group_norm_nhwc_f16_noalloc(const void* x, void* y, const void* gamma, const void* beta, int B, int HW, int C,
                                     int G, float eps, int act, void* stream);
/* Same op for a channels-first tensor (the `channels_first` branch of group_norm.cu:162-206). */
int katz_group_norm_nchw_f16(const void* x, void* y, const void* gamma, const void* beta, int B, int HW, int C, int G,
                             float eps, int act, void* stream);
/* fast_kernel::fast_gelu_mul_fp16 (fast_kernel/csrc/gelu.cuh:44-59): out = fast_gelu(x) * m, n elements. */
int katz_fast_gelu_mul_f16(const void* x, const void* m, void* out, long long n, void* stream);

/* --------------------------------------------------------------------------------------------- UNet step ops ---- */
/* nn.LayerNorm(C, eps, affine) over `rows` rows (diffusers/models/attention.py:195,225,253). */
int katz_layer_norm_f16(const void* x, void* y, const void* gamma, const void* beta, int rows, int C, float eps,
                        void* stream);
/* Unfused GEGLU gating of the torch path (diffusers/models/activations.py:146-149): hg = [M, 2F] (row stride ld),
 * out[M, F] = hg[:, :F] * gelu_erf(hg[:, F:]). */
int katz_geglu_erf_f16(const void* hg, void* out, long long M, int F, int ld, void* stream);

/* C[M,N] = A[M,K] @ W[N,K]^T (+bias[N]) (+rowvec[m / rows_per_batch, n]) -> act -> (+residual[M,N]) * out_scale.
 * nn.Linear as used by Attention / FeedForward / Transformer2DModel (attention_processor.py:1256-1284,
 * attention.py:649, transformer_2d.py:404-409,479-527) and TimestepEmbedding (embeddings.py:190-235).
 * `_mma` is the general-shape kernel on the legacy mma.sync path. */
int katz_linear_f16_mma(const void* A, int lda, const void* W, void* C, int ldc, int M, int N, int K, const void* bias,
                        const void* rowvec, int ld_rowvec, int rows_per_batch, const void* residual, int ldr, int act,
                        float out_scale, void* stream);

/* Same contract as katz_linear_f16_mma on the tcgen05 path (TMA operands, TMEM accumulator). Needs K % 64 == 0,
 * N % 8 == 0, 16-byte aligned pointers and lda/ldc/ldr/ld_rowvec multiples of 8; other shapes return KATZ_E_SIZE /
 * KATZ_E_ALIGN and belong to the _mma entry point. */
int katz_linear_f16(const void* A, int lda, const void* W, void* C, int ldc, int M, int N, int K, const void* bias,
                    const void* rowvec, int ld_rowvec, int rows_per_batch, const void* residual, int ldr, int act,
                    float out_scale, void* stream);
/* Feed-forward projection with the GEGLU gate fused into the epilogue (FeedForward / GEGLU,
 * diffusers/models/attention.py:608-664, activations.py:146-149): W is the unsplit `proj` weight [2F, K], bias [2F];
 * C[M, F] = half(A W[:F]^T + b[:F]) * half(gelu_erf(half(A W[F:]^T + b[F:]))), rounded to half where the reference's
 * fp16 tensors round. Same shape rules as katz_linear_f16, F % 16 == 0. */
int katz_linear_geglu_f16(const void* A, int lda, const void* W, void* C, int ldc, int M, int F, int K, const void* bias,
                          void* stream);

/* LayerNorm folded into the linear layer that consumes it (nn.LayerNorm before to_q/to_k/to_v, attn2.to_q and the GEGLU
 * projection: diffusers/models/attention.py:195,225,253 followed by attention_processor.py:1256-1258 / activations.py:145).
 * LN(x) W^T = rstd * (x W'^T) - rstd * mean * c1 + c2 with W' = W diag(gamma), c1[n] = sum_k W'[n,k] and
 * c2[n] = sum_k W[n,k] beta[k] + bias[n]: the GEMM reads the RAW rows x and the epilogue applies the two row scalars.
 *  - katz_ln_fold_f16 prepares W' (fp16, [N,K]) and c12 ([N] pairs of fp32 (c1, c2)) from W, gamma, beta (bias optional). Run
 *    it whenever W changes (a LoRA merge or restore).
 *  - A producer call passes extras.stats_out: float2 [ceil(N/32)][M], per 32-column chunk of its output and row the
 *    (sum, sum of squares) of the fp16 values it stored.
 *  - The consumer call passes W' as W and extras.ln_stats (= the producer's stats_out, ln_slots = its chunk count, which must
 *    cover exactly this call's K columns), ln_c12 and ln_eps; bias, rowvec, residual must be NULL, act 0, out_scale 1.
 * Both may be set in one call. The same shapes and alignments as katz_linear_f16 / katz_linear_geglu_f16. */
typedef struct katz_linear_extras {
    const void* ln_stats;
    const void* ln_c12;
    int ln_slots;
    float ln_eps;
    void* stats_out;
} katz_linear_extras;
int katz_ln_fold_f16(const void* W, const void* gamma, const void* beta, const void* bias, void* Wf, void* c12, int N, int K,
                     void* stream);
int katz_linear_ex_f16(const void* A, int lda, const void* W, void* C, int ldc, int M, int N, int K, const void* bias,
                       const void* rowvec, int ld_rowvec, int rows_per_batch, const void* residual, int ldr, int act,
                       float out_scale, const katz_linear_extras* ex, void* stream);
int katz_linear_geglu_ex_f16(const void* A, int lda, const void* W, void* C, int ldc, int M, int F, int K, const void* bias,
                             const katz_linear_extras* ex, void* stream);
/* 3x3 NHWC convolution, stride 1 or 2, horizontal padding 1, on the tcgen05 path (nn.Conv2d of ResnetBlock2D,
 * resnet.py:378,408; Downsample2D, downsampling.py). X[B,Hin,Win,Cin], W[Cout,3,3,Cin], Y[B,Hout,Wout,Cout] with
 * Hout = (Hin + 2*pad_h - 3)/stride + 1 and Wout = (Win - 1)/stride + 1: pad_h = 1 is the usual padding, pad_h = 0 is for
 * a row shard whose input already carries its halo rows (latent-row parallelism). Needs Cin % 64 == 0, Cout % 8 == 0
 * and Wout a power of two >= 8 or a multiple of 128 (stride 2: Win even). Epilogue as katz_conv2d_nhwc_f16_mma. */
int katz_conv3x3_nhwc_f16(const void* X, const void* W, void* Y, int B, int Hin, int Win, int Cin, int Cout, int stride,
                          int pad_h, const void* bias, const void* rowvec, int ld_rowvec, const void* residual, int act,
                          float out_scale, void* stream);
/* Status word of the tcgen05 kernels: 0, or which bounded device-side wait gave up (1 producer, 2 MMA issuer,
 * 3 epilogue). Reading it synchronises the device; clear it before the next launch. */
int katz_tc05_status(void);
int katz_tc05_clear_status(void);
/* Nearest-neighbour 2x upsample, NHWC (Upsample2D.forward, diffusers/models/upsampling.py:165-172). */
int katz_upsample_nearest2x_nhwc_f16(const void* x, void* y, int B, int H, int W, int C, void* stream);

/* NHWC convolution as implicit GEMM. Input is X[B, Hs, Ws, C1] (optionally channel-concatenated with
 * X2[B, Hs, Ws, C2], the skip connection of CrossAttnUpBlock2D/UpBlock2D, unet_2d_blocks.py:2473,2608); with
 * `upsample` the input is read through a nearest-neighbour 2x upsample (Upsample2D, upsampling.py:141-186) and
 * Hin, Win are the upsampled sizes. Epilogue as katz_linear_f16 with rows_per_batch = Hout*Wout (the time-embedding
 * add of ResnetBlock2D, resnet.py:381-390, and its shortcut add, resnet.py:410-413). */
int katz_conv2d_nhwc_f16_mma(const void* X, const void* X2, const void* W, void* Y, int B, int Hin, int Win, int C1,
                             int C2, int Cout, int ksize, int stride, int pad_h, int pad_w, int upsample, const void* bias,
                             const void* rowvec, int ld_rowvec, const void* residual, int act, float out_scale,
                             void* stream);

/* 3x3 convolution, padding 1 (vertical padding `pad_h`: 0 for a row shard that carries its halo rows), stride 1 or 2, for
 * NHWC tensors with Cin in {8, 16, 32} and Cout a multiple of 8: the first five layers of
 * ControlNetConditioningEmbedding (controlnet.py:113-127), which the reference runs through nn.Conv2d. W is [Cout, 3, 3, Cin]; bias (optional) and
 * SiLU (act = 1) in the epilogue. A direct convolution from a shared-memory patch: these layers move a 1024 x 1024
 * image and have too few channels to fill the implicit-GEMM tiles. */
int katz_conv3x3_small_nhwc_f16(const void* X, const void* W, void* Y, int B, int Hin, int Win, int Cin, int Cout,
                                int stride, int pad_h, const void* bias, int act, void* stream);

/* softmax(Q K^T * scale) V per (batch, head), head_dim 64, no mask (F.scaled_dot_product_attention as called at
 * attention_processor.py:1276). Q/K/V/O are [B, S, ld*] token-major with head h at columns [64h, 64h+64);
 * bs* are batch strides in elements. With 0 < kv_chunk_rows < Sk (a multiple of 64) key/value row j is read from
 * chunk j / kv_chunk_rows at element offset chunk * kv_chunk_stride: the layout an all-gather of per-rank K/V shards
 * leaves when the latent is row-split; 0 means one contiguous run. */
int katz_attention_f16_mma(const void* Q, const void* K, const void* V, void* O, int B, int H, int Sq, int Sk,
                           int head_dim, int ldq, int ldk, int ldv, int ldo, long long bsq, long long bsk,
                           long long bsv, long long bso, float scale, int kv_chunk_rows, long long kv_chunk_stride,
                           void* stream);

/* Same contract on the tcgen05 path (TMA-fed, S and O accumulators in TMEM, one query row per softmax thread). Needs
 * ld* and bs* multiples of 8, 16-byte aligned pointers, and kv_chunk_rows a multiple of 128 when chunked; other
 * layouts belong to the _mma entry point. */
int katz_attention_f16(const void* Q, const void* K, const void* V, void* O, int B, int H, int Sq, int Sk, int head_dim,
                       int ldq, int ldk, int ldv, int ldo, long long bsq, long long bsk, long long bsv, long long bso,
                       float scale, int kv_chunk_rows, long long kv_chunk_stride, void* stream);

/* The same kernel with the wave tail cut (same reference call, attention_processor.py:1276): an SM holds two CTAs of
 * this kernel, and the query tiles beyond a whole number of rounds of 2 x SMs CTAs make a last round that costs as
 * much as a full one. With scratch memory, query tiles of 16 or more key tiles (2048 keys) that fall into that last
 * round are cut along the key axis into short CTAs that are dispatched first; each leaves its unnormalised result in
 * `scratch` and the last one of a tile to finish adds the parts in index order (bit-reproducible). Shorter tiles are
 * launched exactly as katz_attention_f16 launches them. `scratch` (16-byte aligned;
 * katz_attention_split_scratch_bytes() bytes are always enough) must be zero when first used; every launch leaves its
 * first 4096 bytes (the tickets) zero again. Launches that share a scratch buffer must be ordered on one stream. */
long long katz_attention_split_scratch_bytes(void);
int katz_attention_split_f16(const void* Q, const void* K, const void* V, void* O, int B, int H, int Sq, int Sk,
                             int head_dim, int ldq, int ldk, int ldv, int ldo, long long bsq, long long bsk, long long bsv,
                             long long bso, float scale, int kv_chunk_rows, long long kv_chunk_stride, void* scratch,
                             long long scratch_bytes, void* stream);

/* The same kernel for a row shard whose K/V chunks are pushed by peers (katz_peer_push) into this GPU's arena: chunk
 * `self_chunk` is this rank's own shard and is walked first; before its first tile of any other chunk r the kernel waits
 * (bounded: about a second, then a non-zero katz_tc05_status() and no valid output) until peer_ctrl[64 + r] has reached
 * peer_ctrl[0], the number of the exchange that delivered the chunks. `peer_ctrl` points at the control words of this
 * rank's arena; the kernel must follow the katz_peer_push of the same K/V on the same stream. `scratch` may be NULL.
 * No reference counterpart (the reference has no row split). */
int katz_attention_peer_f16(const void* Q, const void* K, const void* V, void* O, int B, int H, int Sq, int Sk,
                            int head_dim, int ldq, int ldk, int ldv, int ldo, long long bsq, long long bsk, long long bsv,
                            long long bso, float scale, int kv_chunk_rows, long long kv_chunk_stride, void* scratch,
                            long long scratch_bytes, const void* peer_ctrl, int self_chunk, void* stream);

/* dst = src + half(sum_i scales[i] * residuals[i]) — ControlNet residual intake (unet_2d_condition.py:1281-1292; the
 * sum / mean over nets of :1418-1439). `h_residuals` and `h_scales` are HOST arrays of n_res entries (device pointers
 * inside). */
int katz_residual_intake_f16(const void* src, void* dst, const void* const* h_residuals, const float* h_scales,
                             int n_res, long long n, void* stream);
/* Latent-row split: the input of a row shard's 3x3 convolution in one pass. x[B,h,W,C] plus the all-gather of every
 * rank's first and last row (edges[P][2][B][W][C], NULL when world == 1) -> out[B, h+top+bottom, W, C] with the
 * neighbours' rows attached (zeros at the image edge), or with upsample = 1 (top = bottom = 1) -> out[B, 2h+2, 2W, C]:
 * rows [1, 2h+3) of the nearest-2x upsample of the padded shard. No reference counterpart (the reference has no row
 * split). */
int katz_halo_assemble_f16(const void* x, const void* edges, void* out, int B, int h, int W, int C, int top, int bottom,
                           int upsample, int rank, int world, void* stream);
/* ---- peer-memory all-gather (latent-row split over several GPUs, one process per GPU) ---------------------------------
 * No reference counterpart: the reference's 2-GPU mode exchanges tensors through torch.distributed
 * (sdxl_unet_server.py:199-215). Each process allocates one arena (katz_peer_arena_alloc: cudaMalloc, first
 * katz_peer_ctrl_bytes() bytes are zeroed control words), exports it (katz_peer_ipc_export, a
 * katz_peer_ipc_handle_bytes()-byte handle to send to the other processes by any means) and maps the others'
 * (katz_peer_ipc_open). katz_peer_allgather copies a block of `rows` rows of `row_bytes` bytes (multiple of 16;
 * `src_pitch_bytes` apart in the source, so a column slice needs no contiguous copy) from `src` into
 * arena[p] + dst_off + rank*rows*row_bytes, packed, on EVERY rank p with plain stores over NVLink, then returns (in stream order) once
 * every rank's block has arrived in this rank's arena. h_bases[world]: the arenas as mapped in this process, own arena at
 * index `rank`. Every rank must issue the same sequence of calls; consecutive calls must use different dst_off. Waits
 * are bounded: katz_peer_status(arena) is 0, or 100 + the rank whose block never arrived. */
int katz_peer_ctrl_bytes(void);
int katz_peer_arena_alloc(long long bytes, void** ptr);
int katz_peer_arena_free(void* ptr);
int katz_peer_ipc_handle_bytes(void);
int katz_peer_ipc_export(void* ptr, void* handle_out);
int katz_peer_ipc_open(const void* handle, void** ptr);
int katz_peer_ipc_close(void* ptr);
int katz_peer_allgather(const void* src, long long rows, long long row_bytes, long long src_pitch_bytes, long long dst_off,
                        const unsigned long long* h_bases, int rank, int world, void* stream);
/* The same push without the wait: the block goes to slot `rank` of every arena and the flags are raised; a consumer
 * that waits for the flags itself (katz_attention_peer_f16) follows on the same stream. */
int katz_peer_push(const void* src, long long rows, long long row_bytes, long long src_pitch_bytes, long long dst_off,
                   const unsigned long long* h_bases, int rank, int world, void* stream);
int katz_peer_status(const void* arena);
/* Put the status word back to zero (for instance after a warm-up during which the ranks were not yet in step). */
int katz_peer_clear_status(void* arena);
/* get_timestep_embedding (diffusers/models/embeddings.py:26-66), flip_sin_to_cos, shift 0: out[rows, dim] fp16. */
int katz_timestep_embedding_f16(const float* t, void* out, int rows, int dim, int ld_out, void* stream);
int katz_silu_f16(const void* x, void* y, long long n, void* stream);
/* y[r, 0..cols) = softmax(x[r, 0..cols)) in fp32 arithmetic, fp16 in and out, rows `ld_x` / `ld_y` elements apart; y may be
 * x. The probabilities of an attention whose scores come from a GEMM: the VAE decoder's one-head attention over all
 * pixels (diffusers/models/attention_processor.py:1276 with a 512-channel head; unet_2d_blocks.py:681-694).
 * cols: a multiple of 8, at most 16384; ld_x, ld_y: multiples of 8; x, y 16-byte aligned. */
int katz_softmax_rows_f16(const void* x, void* y, int rows, int cols, long long ld_x, long long ld_y, void* stream);
int katz_add_f16(const void* a, const void* b, void* y, long long n, void* stream);
/* y[rows, C1+C2] = x1[rows, C1] ++ x2[rows, C2]: torch.cat([hidden, skip], dim=1) of the up blocks
 * (diffusers/models/unets/unet_2d_blocks.py:2473,2608) in NHWC. */
int katz_concat_channels_f16(const void* x1, const void* x2, void* y, long long rows, int C1, int C2, void* stream);
/* Layout moves at the model boundary: NCHW (C channels) <-> NHWC with Cpad >= C channels (extra channels zero). */
int katz_nchw_to_nhwc_f16(const void* x, void* y, int B, int C, int HW, int Cpad, void* stream);
int katz_nhwc_to_nchw_f16(const void* x, void* y, int B, int C, int HW, int Cpad, void* stream);

/* torch evaluates `tensor / host_scalar` and `host_scalar * half_tensor` differently on its two devices; `mode` picks
 * which one is reproduced bit for bit: 0 = torch on CUDA (the reference's serving path: multiply by the fp32
 * reciprocal; fp32 sigma times the fp16 prediction), 1 = torch on CPU (true division; sigma rounded to fp16 first). */
#define KATZ_ROUNDING_TORCH_CUDA 0
#define KATZ_ROUNDING_TORCH_CPU 1
/* EulerDiscreteScheduler.scale_model_input (schedulers/scheduling_euler_discrete.py:294-295): out = half(x / sqrt(sigma^2+1)),
 * written `copies` times back to back (the CFG batch). x is the fp16 latent. */
int katz_euler_scale_input(const void* x, void* out, long long n, float sigma, int copies, int mode, void* stream);
/* CFG combine (pipeline_controlnet_sd_xl_katz.py:1649-1655) + EulerDiscreteScheduler.step (:498-537, epsilon
 * prediction, s_churn 0) in place on the fp16 latent x. eps_cond may be NULL (no guidance). */
int katz_euler_cfg_step(void* x, const void* eps_uncond, const void* eps_cond, long long n, float guidance, float sigma,
                        float sigma_next, int mode, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KATZ_B200_H_ */
