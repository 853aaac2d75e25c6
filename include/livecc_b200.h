/*
 * livecc_b200.h — C ABI of liblivecc_sm100a.so, the B200-native (sm_100a) kernels and model runtime
 * behind LiveCC's per-chunk encode -> prefill -> decode hot path.
 *
 * The reference (showlab/livecc) has no native/FFI boundary of its own: the path sits behind Python
 * surfaces (REF/demo/infer.py:43-50,165-174 -> transformers Qwen2VLForConditionalGeneration). This
 * header is therefore the boundary *we* define one level below that surface;
 * each entry point cites the reference interface (file:line) whose arithmetic it replaces.
 *   mq2vl.py     = transformers/models/qwen2_vl/modeling_qwen2_vl.py   (transformers 5.5.0)
 *   gen/utils.py = transformers/generation/utils.py
 *   REF/         = showlab/livecc
 *
 * Conventions
 *   - All data pointers are DEVICE pointers owned by the caller (PyTorch storage in our host code);
 *     the library never allocates device memory.
 *   - Every call is asynchronous on `stream`; nothing synchronises the device.
 *   - Return value: 0 on success, negative on error; lcc_last_error(ctx) returns a message.
 *   - A ctx is bound to one device and one host thread at a time; no hidden globals.
 *   - bf16 everywhere unless the name says otherwise; "bf16 rounding points" follow the reference's
 *     eager graph (one torch op = one rounding).
 *   - The paged KV cache uses pages of LCC_PAGE_SIZE tokens; a layer's K (or V) pool is
 *     [num_pages, kv_heads, LCC_PAGE_SIZE, 128] bf16.
 */
#ifndef LIVECC_B200_H
#define LIVECC_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LCC_ABI_VERSION 11
#define LCC_PAGE_SIZE 64

typedef struct lcc_ctx lcc_ctx;
typedef struct lcc_model lcc_model;
typedef void* lcc_stream_t; /* cudaStream_t */

/* GEMM epilogues (lcc_gemm_bf16) */
#define LCC_EPI_NONE 0            /* C = bf16(acc) */
#define LCC_EPI_BIAS 1            /* C = bf16(acc + bias) */
#define LCC_EPI_BIAS_QUICKGELU 2  /* ViT fc1: mq2vl.py:329-337 */
#define LCC_EPI_BIAS_GELU 3       /* merger mlp[0..1]: mq2vl.py:317-326 */
#define LCC_EPI_RESIDUAL 4        /* o_proj / down_proj + residual: mq2vl.py:645-660 */
#define LCC_EPI_BIAS_RESIDUAL 5   /* ViT proj / fc2 + residual: mq2vl.py:479-487 */
#define LCC_EPI_SWIGLU 6          /* gate|up (16-row interleaved) -> silu(gate)*up: mq2vl.py:502-504 */

/* Device-side per-stream scalars (int32[LCC_SC_COUNT]); they replace the host-side loop state of
 * GenerationMixin._sample (gen/utils.py:2743-2805) so that a generate() call needs no host sync. */
#define LCC_SC_KV_LEN 0       /* tokens in the KV cache */
#define LCC_SC_ROPE_POS 1     /* position id of the next token to forward = kv_len + rope_delta (mq2vl.py:1212-1222) */
#define LCC_SC_FINISHED 2     /* non-zero once EOS was produced or max_new_tokens reached */
#define LCC_SC_N_GENERATED 3  /* tokens generated in this generate() call */
#define LCC_SC_SEQ_LEN 4      /* ids in the sequence buffer (history + generated) */
#define LCC_SC_LAST_TOKEN 5
#define LCC_SC_VIDEO_TOKENS 6 /* number of video placeholder ids seen by the last lcc_prefill (mq2vl.py:1169-1175 check) */
#define LCC_SC_NATIVE_ERROR 7 /* non-zero: a bounded wait inside the persistent decode kernel gave up (results invalid) */
#define LCC_SC_COUNT 8

int lcc_abi_version(void);

/* ---- context ---------------------------------------------------------------------------- */
/* lcc_create returns NULL unless `device` is an sm_100 GPU (there is no fallback path). */
lcc_ctx* lcc_create(int device);
void lcc_destroy(lcc_ctx* ctx);
const char* lcc_last_error(lcc_ctx* ctx);
int lcc_num_sms(lcc_ctx* ctx);
/* Kernel launches issued by this library in this process so far (launches recorded into a CUDA graph count once,
 * at capture). */
uint64_t lcc_launch_count(void);

/* ---- op level (each is unit-tested against the oracle) ---------------------------------- */

/* C[M,N] = epilogue(A[M,K] x B[N,K]^T), bf16 in, fp32 accumulate (tcgen05/TMEM), bf16 out.
 * Replaces every nn.Linear / Conv3d-as-GEMM call with M >= 16 on the path:
 * mq2vl.py:304-310 (patch embed), :385,:401-403,:456 (ViT qkv/proj), :329-337 (ViT MLP),
 * :317-326 (merger), :539-541,:559-565,:593 (decoder q/k/v/o), :502-504 (MLP).
 * K, N and all leading dimensions must be multiples of 8 elements. block_n (N tile): 0 = dispatch rule, else a multiple of 16 in [32,256] (SwiGLU: of 32);
 * a negative value selects the CTA-pair kernel (cta_group::2, 256 x |block_n| tiles, |block_n| a multiple of 32).
 * splitk_ws: optional fp32 scratch (>= 8*M*N*4 bytes) that allows split-K for M <= 384 when the tile count cannot
 * occupy the SMs; used for K >= 8192 by default (LIVECC_B200_GEMM_SPLITK=1 forces it for every eligible shape, =0 disables). NULL = never. */
int lcc_gemm_bf16(lcc_ctx* ctx, const void* A, int lda, const void* B, int ldb, void* C, int ldc,
                  int M, int N, int K, const void* bias, const void* residual, int ldr, int epilogue,
                  int block_n, void* splitk_ws, int64_t splitk_ws_bytes, lcc_stream_t stream);

/* hidden_states.to(bf16) of the f32 patch rows (mq2vl.py:309). */
int lcc_cast_f32_bf16(lcc_ctx* ctx, const float* in, void* out, int64_t n, lcc_stream_t stream);

/* nn.LayerNorm(dim, eps) over rows (ViT norm1/norm2/ln_q, mq2vl.py:464-465,317). */
int lcc_layernorm(lcc_ctx* ctx, const void* x, int ldx, const void* w, const void* b, void* y, int ldy,
                  int rows, int dim, float eps, lcc_stream_t stream);

/* Qwen2VLRMSNorm over rows (mq2vl.py:126-131). */
int lcc_rmsnorm(lcc_ctx* ctx, const void* x, int ldx, const void* w, void* y, int ldy, int rows, int dim,
                float eps, lcc_stream_t stream);

/* ViT 2-D rotary: table for a (t,h,w) grid in merge-window patch order (rot_pos_emb, mq2vl.py:725-752;
 * inv_freq[head_dim/4] fp32 from VisionRotaryEmbedding :271-284), then in-place application to the
 * q and k thirds of qkv [N, 3*heads*head_dim] (apply_rotary_pos_emb_vision, :257-268). */
int lcc_vit_rope_table(lcc_ctx* ctx, float* cos_t, float* sin_t, int t, int h, int w, int merge,
                       int head_dim, const float* inv_freq, lcc_stream_t stream);
int lcc_vit_rope_apply(lcc_ctx* ctx, void* qkv, int ld, const float* cos_t, const float* sin_t, int N,
                       int heads, int head_dim, lcc_stream_t stream);

/* VisionAttention core (mq2vl.py:392-454): non-causal attention inside each cu_seqlens segment,
 * q/k/v read from qkv [n_rows, 3*heads*80] (already rotated), out [n_rows, heads*80]. cu_seqlens: device
 * int32[nseg+1] with cu_seqlens[nseg] == n_rows. impl: LCC_VIT_ATTN_DEFAULT, or force one kernel family. */
#define LCC_VIT_ATTN_DEFAULT 0
#define LCC_VIT_ATTN_MMA 1 /* mma.sync flash kernels */
#define LCC_VIT_ATTN_TC 2  /* tcgen05 + TMEM kernel */
int lcc_vit_attention(lcc_ctx* ctx, const void* qkv, int ld, int64_t n_rows, void* out, int o_ld,
                      const int32_t* cu_seqlens, int nseg, int max_seg_len, int heads, int head_dim, int impl,
                      lcc_stream_t stream);

/* embed_tokens gather + masked_scatter of the video features (mq2vl.py:1255-1272).
 * ids: device int64[S]; video_embeds: bf16 [n_video_rows, H] or NULL (then placeholders keep their text embedding,
 * as in the reference when no pixel values are passed); placeholders beyond n_video_rows also keep their text
 * embedding (nothing is read out of bounds; the caller compares the count and raises like mq2vl.py:1169-1175).
 * rank_ws: device int32[S+1] scratch (last entry receives the video-token count). */
int lcc_embed_gather(lcc_ctx* ctx, const int64_t* ids, const void* table, const void* video_embeds,
                     int n_video_rows, int64_t video_token_id, void* out, int32_t* rank_ws, int S, int H, int64_t vocab,
                     lcc_stream_t stream);

/* M-RoPE (mq2vl.py:188-201,212-254) on the q and k parts of qkv [S, (Hq+2Hkv)*128] (q rotated in
 * place) and append of rotated k / v to the paged cache at positions kv_start..kv_start+S-1
 * (DynamicLayer.update, cache_utils.py:102-121). pos3: device int32[3,S]; inv_freq: device f32[64]. */
int lcc_mrope_kv_write(lcc_ctx* ctx, void* qkv, int ld, const int32_t* pos3, int S, const float* inv_freq,
                       int sec_t, int sec_h, int Hq, int Hkv, void* k_cache, void* v_cache,
                       const int32_t* page_table, int kv_start, lcc_stream_t stream);

/* Causal GQA attention of S new tokens over past+S cached tokens (Qwen2VLAttention core,
 * mq2vl.py:572-594; eager_attention_forward :353-375). q: rotated rows of qkv; out [S, Hq*128].
 * part_o / part_ml: optional split-KV scratch, f32[part_rows,128] and f32[part_rows,2] with
 * part_rows >= nsplit*S*Hq (nsplit <= 8); NULL => no KV split. impl: LCC_ATTN_DEFAULT | LCC_ATTN_MMA | LCC_ATTN_TC.
 * The V slots of the last page behind token past+S-1 must hold finite values (lcc_mrope_kv_write zeroes them). */
#define LCC_ATTN_DEFAULT 0
#define LCC_ATTN_MMA 1 /* mma.sync flash kernel */
#define LCC_ATTN_TC 2  /* tcgen05 + TMEM kernel */
int lcc_attn_prefill(lcc_ctx* ctx, const void* q, int q_ld, const void* k_cache, const void* v_cache,
                     const int32_t* page_table, int Hq, int Hkv, int S, int past, void* out, int o_ld,
                     float* part_o, float* part_ml, int64_t part_rows, int impl, lcc_stream_t stream);

/* One-token attention: RoPE of q, RoPE + append of the new k/v at slot scalars[LCC_SC_KV_LEN],
 * split-KV attention over the paged cache and merge. qkv: raw projections(+bias) of the new token.
 * part_o: f32[nsplit,Hq,128], part_ml: f32[nsplit,Hq,2] scratch; counters: int32[Hkv], zero-initialised
 * once by the caller (the kernel leaves them zero); out: bf16[Hq*128]. */
int lcc_attn_decode(lcc_ctx* ctx, void* qkv, void* k_cache, void* v_cache, const int32_t* page_table,
                    const int32_t* scalars, const float* inv_freq, int Hq, int Hkv, int nsplit, float* part_o,
                    float* part_ml, int32_t* counters, void* out, lcc_stream_t stream);

/* Decode-step projections (M = 1), each fused with its neighbours in the layer
 * (Qwen2VLDecoderLayer.forward, mq2vl.py:613-662). `scalars` may be NULL (no early-exit flag). */
int lcc_gemv_norm_bias(lcc_ctx* ctx, const void* W, int ldw, const void* x, const void* norm_w, float eps,
                       const void* bias, void* out, int N, int K, const int32_t* scalars, lcc_stream_t stream);
int lcc_gemv_residual(lcc_ctx* ctx, const void* W, int ldw, const void* x, void* h_inout, int N, int K,
                      const int32_t* scalars, lcc_stream_t stream);
int lcc_gemv_norm_swiglu(lcc_ctx* ctx, const void* W_gate_up, int ldw, const void* x, const void* norm_w,
                         float eps, void* act, int N2, int K, const int32_t* scalars, lcc_stream_t stream);
/* final norm + lm_head on one token -> fp32 logits (mq2vl.py:905,1437-1438; gen/utils.py:2762). */
int lcc_gemv_norm_logits(lcc_ctx* ctx, const void* W, int ldw, const void* x, const void* norm_w, float eps,
                         float* logits, float* logits_copy, int N, int K, const int32_t* scalars,
                         lcc_stream_t stream);

/* Logits processing + greedy token selection + stream bookkeeping (gen/utils.py:2762-2805;
 * logits_process.py:407-410; REF/demo/infer.py:10-23). */
typedef struct {
    float repetition_penalty; /* 1.0 = off */
    int32_t thr_token;        /* ThresholdLogitsProcessor token id, < 0 = off */
    float thr_base, thr_step;
    int32_t eos_token_id;
    int32_t max_new_tokens;
    float inv_repetition_penalty; /* fp32(1.0 / (double)penalty): torch's CUDA `tensor / python_float` multiplies by
                                     this value (measured: tools/penalty_probe.py); 0 = derive as 1.0f / repetition_penalty */
    int32_t eos_token_id2;        /* second stop id (generation_config.json eos_token_id = [151645, 151643] in the
                                     Qwen2-VL family; gen/utils.py stops on any of them), < 0 = none */
} lcc_sampling;

int lcc_sample_greedy(lcc_ctx* ctx, const float* logits_raw, float* logits_proc, int V, int64_t* seq,
                      int32_t* scalars, const lcc_sampling* sp, int advance_kv, const void* embed, void* h,
                      int H, lcc_stream_t stream);

/* ---- model level (native runtime: one call launches a whole phase) ---------------------- */
typedef struct {
    /* vision (Qwen2VLVisionConfig) */
    int32_t vit_depth, vit_dim, vit_heads, vit_mlp, patch_dim, merge, vit_out;
    /* text (Qwen2VLTextConfig) */
    int32_t hidden, inter, layers, q_heads, kv_heads, vocab;
    float rms_eps, rope_theta;
    int32_t mrope_t, mrope_h; /* mrope_section[0], [1] */
    int64_t video_token_id;
} lcc_model_config;

typedef struct {
    const void *norm1_w, *norm1_b, *norm2_w, *norm2_b;
    const void *qkv_w, *qkv_b, *proj_w, *proj_b, *fc1_w, *fc1_b, *fc2_w, *fc2_b;
} lcc_vit_block_weights;

typedef struct {
    const void *ln1_w, *qkv_w, *qkv_b, *o_w, *ln2_w, *gate_up_w /* 16-row interleaved */, *down_w;
} lcc_layer_weights;

typedef struct {
    const void* patch_w; /* [vit_dim, patch_dim] */
    const lcc_vit_block_weights* vit_blocks;
    const void *merger_ln_w, *merger_ln_b, *merger_fc1_w, *merger_fc1_b, *merger_fc2_w, *merger_fc2_b;
    const void* embed; /* [vocab, hidden] */
    const lcc_layer_weights* layers;
    const void* final_norm_w;
    const void* lm_head; /* [vocab, hidden] */
    /* fp32 rotary tables computed by the host exactly as the reference does:
     * text_inv_freq[64]  = 1/theta^(2i/128)            (mq2vl.py:175-183)
     * vit_inv_freq[hd/4] = 1/10000^(2i/(hd/2))         (mq2vl.py:274-279) */
    const float* text_inv_freq;
    const float* vit_inv_freq;
} lcc_model_weights;

/* One video stream's device state (all caller-owned). */
typedef struct {
    void* k_pool;               /* [layers][num_pages][kv_heads][LCC_PAGE_SIZE][128] bf16 */
    void* v_pool;
    int64_t layer_stride;       /* elements between consecutive layers of a pool */
    const int32_t* page_table;  /* device int32: logical page -> physical page */
    int32_t* scalars;           /* device int32[LCC_SC_COUNT] */
    int64_t* seq;               /* device int64[cap]: input ids then generated ids */
} lcc_stream_state;

lcc_model* lcc_model_create(lcc_ctx* ctx, const lcc_model_config* cfg, const lcc_model_weights* w);
void lcc_model_destroy(lcc_model* m);

/* Scratch bytes needed by the calls below for at most `max_patches` ViT rows / `max_tokens` prefill rows,
 * and binding of a caller-owned scratch buffer of that size to the model. */
size_t lcc_workspace_bytes(const lcc_model* m, int max_patches, int max_tokens);
int lcc_model_bind_workspace(lcc_model* m, void* ws, size_t ws_bytes, int max_patches, int max_tokens);

/* Qwen2VisionTransformerPretrainedModel.forward (mq2vl.py:757-795) for one video of grid (t,h,w):
 * pixel_values f32 [t*h*w, patch_dim] -> out bf16 [t*h*w/merge^2, vit_out]. */
int lcc_vit_forward(lcc_model* m, const float* pixel_values, int t, int h, int w, void* out,
                    lcc_stream_t stream);

/* Same, starting from the resized uint8 frames [T,3,H,W] on the device (H, W multiples of 28): the
 * rescale/normalize/patchify of Qwen2VLVideoProcessor._preprocess (video_processing_qwen2_vl.py:240-272) and the
 * bf16 cast of PatchEmbed (mq2vl.py:309) are fused into one kernel; bit-identical to the f32 path.
 * mean255/std255: HOST float[3] = fp32(image_mean)*255, fp32(image_std)*255 (image_processing_backends.py:301-304). */
int lcc_vit_forward_frames(lcc_model* m, const uint8_t* frames, int T, int H, int W, const float* mean255,
                           const float* std255, void* out, lcc_stream_t stream);

/* Prefill of S new tokens (Qwen2VLModel.forward + lm_head on the last token, mq2vl.py:1230-1300,
 * 828-910, 1437) followed by the first token selection. ids: device int64[S] (the new tokens);
 * pos3: device int32[3,S]; video_embeds: bf16 [n_video_rows, hidden] or NULL; past = tokens already
 * cached. Host must have set scalars {KV_LEN = past+S, ROPE_POS, FINISHED=0, N_GENERATED=0, SEQ_LEN}.
 * slot (0..7): which row of the decode-step buffers receives the first token's embedding and logits; 0 for the
 * one-stream path, b for stream b of a lcc_decode_batch group. */
int lcc_prefill(lcc_model* m, const lcc_stream_state* st, const int64_t* ids, const int32_t* pos3, int S,
                int past, const void* video_embeds, int n_video_rows, const lcc_sampling* sp, int slot, lcc_stream_t stream);

/* n_steps x (one-token forward + token selection) (the loop body of _sample, gen/utils.py:2743-2805).
 * No-ops once scalars[LCC_SC_FINISHED] is set. Capturable in a CUDA graph. nsplit: KV splits (1..64). */
int lcc_decode_steps(lcc_model* m, const lcc_stream_state* st, int n_steps, int nsplit, const lcc_sampling* sp,
                     lcc_stream_t stream);

/* Batched decode (the reference demo admits 5 concurrent sessions on one model,
 * REF/demo/app.py:178): n_steps x (one persistent kernel = every decoder layer + lm_head for all n_streams <= 8 streams,
 * each weight byte read once per step, then one token selection per stream). states[b] must have been prefilled with
 * slot = b and share one page pool. A stream's ids and logits are bit-identical to decoding it alone (same kernel,
 * same reduction order). lcc_decode_steps (one stream) uses the per-op kernels unless LIVECC_B200_MEGA=1: they are ~5 % faster
 * for a single stream (measured); with 2..8 streams the persistent kernel reads every weight byte once per step for all. */
int lcc_decode_batch(lcc_model* m, const lcc_stream_state* states, int n_streams, int n_steps, const lcc_sampling* sp,
                     lcc_stream_t stream);
/* Test hook: run layers [layer_begin, layer_end) and the phases in phase_mask (1 qkv, 2 attention, 4 o_proj,
 * 8 gate/up, 16 down_proj) of the persistent decode kernel, optionally the lm_head, without token selection. */
int lcc_decode_mega_debug(lcc_model* m, const lcc_stream_state* states, int n_streams, int layer_begin, int layer_end,
                          int phase_mask, int do_head, lcc_stream_t stream);

/* ---- frame ingest ------------------------------------------------------------------------------
 * transforms.functional.resize(clip, [H, W], interpolation=BICUBIC, antialias=True) on a uint8 TCHW clip
 * (REF/livecc-utils/src/livecc_utils/video_process_patch.py:101-106 and :150-155), bit-identical to torchvision 0.26 /
 * ATen's CPU kernel: float32 width pass, float32 height pass, clamp, round half to even, uint8. */
/* Window/weight table of one axis (ATen _compute_indices_min_size_weights_aa<float>, Keys cubic a = -0.5), host only:
 * lcc_resize_aa_taps = max window length; xmin/xsize: int32[out_size]; weights: float[taps][out_size] (tap-major). */
int lcc_resize_aa_taps(int in_size, int out_size);
int lcc_resize_aa_table(int in_size, int out_size, int32_t* xmin, int32_t* xsize, float* weights);
/* A plan owns the device copy of both axes' tables for (h, w) -> (H, W). rows_per_cta: 0 = choose (tuning hook).
 * NULL (and lcc_last_error) when a window does not fit in shared memory or a size is out of range. */
typedef struct lcc_resize_plan lcc_resize_plan;
lcc_resize_plan* lcc_resize_plan_create(lcc_ctx* ctx, int h, int w, int H, int W, int rows_per_cta);
void lcc_resize_plan_destroy(lcc_resize_plan* plan);
int lcc_resize_plan_info(const lcc_resize_plan* plan, int* rows_per_cta, int* max_rows, int64_t* smem_bytes);
/* src: device uint8 [planes, h, w] (planes = T*C), dst: device uint8 [planes, H, W]. One kernel. */
int lcc_resize_bicubic_aa_u8(lcc_ctx* ctx, const lcc_resize_plan* plan, const uint8_t* src, int planes, uint8_t* dst,
                             lcc_stream_t stream);

/* ---- hybrid sequence models: decoder-only language models whose layers mix tokens with a state-space recurrence, gated
 * linear attention, retention, a gated delta rule, chunk-local attention, latent attention or sliding-window attention. A layer is
 *     x <- norm1(alpha * x + mixer(x)),  then (if it has a feed-forward)  x <- norm2(alpha * x + ff(x))       (post-norm)
 * or, in a model with LCC_BLOCK_PRENORM_HC, pre-norm sublayers on several residual streams (see LCC_BLOCK_PRENORM_HC),
 * or, with LCC_BLOCK_PARALLEL, x <- x + mixer(norm1(x)) + ff(norm1(x)),
 * or, with LCC_BLOCK_BRANCHNORM, x <- x + norm1(mixer(x + canon(x))), then x <- x + norm2(ff(x)) (the norm sits on the sublayer's
 * output; canon is a short causal convolution over time on every channel of the residual stream);
 * the feed-forward is dense (gated gelu, or two matrices around a gelu) or routed (LCC_FF_MOE);
 * with the residual stream(s), every norm, every score, every router and every recurrent state in fp32. One library serves two storage
 * types: LCC_DT_BF16 (bf16 weights, activations and K/V pages; fp32 accumulation) and LCC_DT_F32 (everything fp32, plain
 * FMAs). The caller owns all memory: weights, workspace, K/V pages and the fp32 recurrent-state slots of every sequence. */
#define LCC_DT_BF16 0
#define LCC_DT_F32 1
#define LCC_MIX_SSD 1      /* scalar-decay state-space layer: in-proj -> causal conv + silu -> recurrence -> gated grouped norm -> out-proj */
#define LCC_MIX_PARALLEL 2 /* chunk-local sink attention (left) beside gated linear attention (right), averaged after a norm each */
#define LCC_MIX_RETENTION 3 /* rotary q/k -> linear attention with a fixed decay per head, no normaliser -> unit-rms heads x silu gate -> out-proj */
#define LCC_MIX_LATENT 4    /* causal softmax attention over a cached low-rank latent + one shared rotary key part, per-head sink and sigmoid gate */
#define LCC_MIX_ATTENTION 5 /* softmax attention over paged K/V: per-head q/k RMS norm, rotary positions on part of a head, a sliding
                               window and / or chunks, optional sink, values projected or taken from the keys as projected, output
                               gate per head or per channel (every option a field of the layer) */
#define LCC_MIX_DELTA 6     /* gated delta rule with a decay per key channel: q/k/v through a short causal convolution + silu, unit-length q
                               and k, S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q; unit-rms heads x weight x sigmoid
                               gate -> out-proj (decays and output gate come through low-rank bottlenecks) */
#define LCC_FF_GLU 0        /* dense gated feed-forward: gelu_tanh(gate) * up */
#define LCC_FF_MOE 1        /* routed experts (sigmoid or softmax router, top-k of score + correction, optionally inside the best groups
                               of neighbouring experts; relu^2 or clamped gated experts; identity experts) + gated shared expert */
#define LCC_FF_MLP 2        /* dense two-matrix feed-forward: down(gelu_tanh(up x)) */
#define LCC_BLOCK_POSTNORM 0 /* x <- norm(alpha * x + sublayer(x)) */
#define LCC_BLOCK_PRENORM_HC 1 /* `streams` residual streams x_s; per sublayer: u = sum_s in[s] x_s; y = sublayer(norm(u));
                                  x_t <- sum_s mix[s][t] x_s + out[t] y. The model's output is the sum of the streams. */
#define LCC_BLOCK_PARALLEL 2   /* h = norm1(x); x <- x + mixer(h) + ff(h): one norm, both sublayers read it, one fp32 residual sum */
#define LCC_BLOCK_BRANCHNORM 3 /* x <- x + norm1(mixer(x + canon(x))); x <- x + norm2(ff(x)): sublayers read the residual stream itself */
#define LCC_NORM_RMS 0         /* x / sqrt(mean(x^2) + eps) * w */
#define LCC_NORM_DYT 1         /* tanh(alpha * x) * w + b: no statistics of the row (Dynamic Tanh) */
#define LCC_ROUTER_SIGMOID 0
#define LCC_ROUTER_SOFTMAX 1   /* scores = softmax over all router outputs (identity experts included) */
#define LCC_ROUTER_TOPK_SOFTMAX 2 /* the e_top largest logits are chosen; weights = softmax over the chosen logits only */
#define LCC_EXPERT_RELU2 0     /* down(relu(up x)^2) */
#define LCC_EXPERT_CLAMP_GLU 1 /* g = min(gate x, limit), u = clamp(up x, +-limit); down(g * sigmoid(1.702 g) * (u + 1)); e_up rows [gate | up] */
#define LCC_EXPERT_SILU_GLU 2  /* down(silu(gate x) * (up x)); e_up rows as for LCC_EXPERT_CLAMP_GLU */
#define LCC_GATE_NONE 0
#define LCC_GATE_HEAD 1        /* one sigmoid gate per (row, head) */
#define LCC_GATE_CHANNEL 2     /* one sigmoid gate per (row, head, value channel) */

typedef struct {
    int32_t type; /* LCC_MIX_* */
    int32_t ff;   /* feed-forward width, 0 = the layer has none */
    /* LCC_MIX_SSD: heads x vdim value channels, `state` key channels shared by heads / groups heads, `conv` taps */
    int32_t s_heads, s_vdim, s_state, s_groups, s_conv, s_norm_groups;
    /* LCC_MIX_PARALLEL, left: Hq query heads over G key/value heads, key size dim, value size vdim, chunk (<= 0: none) */
    int32_t l_heads, l_kv_heads, l_dim, l_vdim, l_chunk;
    float l_scale;
    /* LCC_MIX_PARALLEL, right: heads x dim key channels, heads x vdim value channels, decay bottleneck rank, temperature tau */
    int32_t r_heads, r_dim, r_vdim, r_rank;
    float r_tau;
    /* LCC_MIX_RETENTION: heads x dim key channels (the first t_rot_dims of each head rotated), heads x vdim value channels */
    int32_t t_heads, t_dim, t_vdim, t_rot_dims;
    /* LCC_MIX_LATENT: per head a_dim unrotated + a_rot_dim rotated query channels, value size a_vdim; the cache holds
     * a_rank latent channels + a_rot_dim rotated key channels per token; a_kv_from >= 0: this layer has no cache of its own
     * and reads that layer's */
    int32_t a_heads, a_dim, a_rot_dim, a_vdim, a_rank, a_kv_from;
    float a_scale;
    /* a_q_rank > 0: the queries come through a latent of that many channels (a_in rows [q latent | latent, key part | gate], RMS norm
     * with a_q_norm_f32, then a_uq); a_window > 0: a row at position i sees j with i - j < a_window; a_gate: a_in ends with one gate
     * row per head; a_sink_f32 NULL: ordinary softmax */
    int32_t a_q_rank, a_window, a_gate;
    float rot_mag;  /* factor on cos and sin of the rotation (1 without long-context scaling) */
    /* LCC_MIX_ATTENTION: m_heads query heads over m_kv_heads key/value heads; per-head RMS norm of q and k (weights [m_dim], shared by
     * the heads); the first m_rot_dims channels of a head rotated (m_rot_pairs: channel 2i with 2i+1, else i with i + dims/2);
     * a row at position i sees j <= i with i - j < m_window (m_window <= 0: no window) inside its chunk of m_chunk positions
     * (<= 0: none); m_sink: a zero-logit sink in the softmax denominator; m_value_keys: the values are the keys as projected
     * (before norm and rotation; the layer has no value projection); m_gate: LCC_GATE_* */
    int32_t m_heads, m_kv_heads, m_dim, m_vdim, m_window, m_chunk, m_rot_dims, m_rot_pairs, m_sink, m_value_keys, m_gate;
    float m_scale;
    /* m_unit_norm: q and k heads are divided by their rms without a weight (m_qnorm_f32 / m_knorm_f32 NULL); m_temp_f32: one factor
     * per query head on the scores; m_vmix_role: 0 none, 1 the layer's values as projected are kept for later layers of the step, 2 the
     * cached values are (1 - m_vmix) * v + m_vmix * the kept values of the same token */
    int32_t m_unit_norm, m_vmix_role;
    float m_vmix;
    /* LCC_MIX_DELTA: d_heads value heads of d_vdim channels over d_kv_heads query/key heads of d_dim channels, d_conv taps, bottleneck
     * ranks of the decay and of the output gate */
    int32_t d_heads, d_kv_heads, d_dim, d_vdim, d_conv, d_rank_a, d_rank_g;
    /* feed-forward: ff_kind LCC_FF_*; MoE: e_experts experts of width e_ff, e_top per token, weights = score * e_scale,
     * shared expert of width e_shared_ff (0 = none) */
    int32_t ff_kind, e_experts, e_top, e_ff, e_shared_ff;
    float e_scale;
    /* e_router_kind LCC_ROUTER_*; the last e_identity router outputs (beyond the e_experts real ones) stand for experts that return
     * their input; e_groups > 0: the router outputs form e_groups equal groups of neighbours and only the e_keep groups with the
     * largest choice score can be chosen; e_act LCC_EXPERT_*, e_limit its clamp */
    int32_t e_router_kind, e_identity, e_groups, e_keep, e_act;
    int32_t e_up_il16; /* LCC_EXPERT_CLAMP_GLU: non-zero when each expert's gate and up rows are interleaved in groups of 16 (16 gate
                          rows, then the 16 matching up rows; e_ff a multiple of 16) instead of [gate: e_ff | up: e_ff] */
    float e_limit;
    float norm1_alpha; /* LCC_NORM_DYT: the scalar inside tanh */
    /* weights: matrices [out, in] in the model's storage type; everything named *_f32 is fp32 */
    const float *norm1_f32, *norm2_f32;
    const float* canon_w_f32;  /* LCC_BLOCK_BRANCHNORM: [width, canon_taps] taps of the convolution in front of the mixer (NULL: none) */
    const float* m_temp_f32;   /* [m_heads] or NULL */
    const void* a_uq;          /* [heads*(dim+rot_dim), a_q_rank] */
    const float* a_q_norm_f32; /* [a_q_rank] */
    const void* d_in;          /* rows [q: G*dim | k: G*dim | v: heads*vdim | beta: heads | decay-down: rank_a | gate-down: rank_g] x width,
                                  every block padded with zero rows to a multiple of 8, so that each starts at a multiple of 8 */
    const float* d_conv_w_f32; /* [channels, d_conv]: the q, k, v blocks of d_in with their padding (zero taps there) */
    const void* d_a_up;        /* [heads*dim, rank_a] */
    const float *d_dt_bias_f32, *d_a_log_f32; /* [heads*dim], [heads] */
    const void* d_g_up;        /* [heads*vdim, rank_g] */
    const float* d_norm_f32;   /* [vdim], shared by the heads */
    const void* d_out;         /* [width, heads*vdim] */
    const float* norm1_bias_f32; /* LCC_NORM_DYT: [width] */
    const void* m_in;          /* [Hq*dim + G*dim (+ G*vdim) + gate rows, width], rows [q | k | (v) | gate] */
    const float *m_qnorm_f32, *m_knorm_f32; /* [dim] each */
    const void* m_out;         /* [width, Hq*vdim] */
    const void* s_in;          /* [2*inner + 2*groups*state + heads, width], rows [z | x | B | C | dt] */
    const float *s_conv_w_f32, *s_conv_b_f32; /* [inner + 2*groups*state, conv], [..] */
    const float *s_dt_bias_f32, *s_a_log_f32, *s_skip_f32, *s_norm_f32; /* [heads] x3, [inner] */
    const void* s_out;         /* [width, inner] */
    const void* l_in;          /* [Hq*dim + G*dim + G*vdim + Hq, width], rows [q | k | v | gate] */
    const float* l_in_bias_f32; /* same length, zeros for the gate rows */
    const void* l_in_bias;      /* optional copy in the storage type, padded like the matrix rows (tensor-core epilogue) */
    const float *l_qnorm_f32, *l_knorm_f32; /* [Hq*dim], [G*dim] */
    const void* l_out;         /* [width, Hq*vdim] */
    const float* l_branch_norm_f32; /* [width] */
    const void* r_in;          /* [2*heads*dim + 2*heads*vdim + rank, width], rows [q | k | v | gate | decay-down] */
    const void* r_decay_up;    /* [heads*dim, rank] */
    const float* r_decay_bias_f32; /* [heads*dim] */
    const float* r_norm_f32;   /* [vdim], shared by the heads */
    const void* r_out;         /* [width, heads*vdim] */
    const float* r_branch_norm_f32; /* [width] */
    const void* ff_in;         /* LCC_FF_GLU: [2*ff, width], rows [gate | up]; act = gelu_tanh(gate) * up. LCC_FF_MLP: [ff, width] */
    const void* ff_out;        /* [width, ff] */
    const float* rot_inv_freq_f32; /* [rot dims / 2]: rotation frequencies of this layer's mixer, computed by the host */
    const void* t_in;          /* [2*heads*dim + 2*heads*vdim, width], rows [q | k | v | gate] */
    const float* t_log_decay_f32; /* [heads]: log of the per-head decay */
    const float* t_norm_f32;   /* [vdim]: weight of the per-head unit norm (ones when the design has none) */
    const void* t_out;         /* [width, heads*vdim] */
    const void* a_in;          /* [heads*(dim+rot_dim) (+ rank + rot_dim) + heads, width], rows [q | latent, key part | gate];
                                  a layer that reads another layer's cache has no middle block */
    const float* a_latent_norm_f32; /* [rank] */
    const void* a_uk_t;        /* [heads][rank][dim]: each head's key up-projection, transposed (query absorption) */
    const void* a_uv;          /* [heads*vdim, rank] */
    const float* a_sink_f32;   /* [heads] sink logits */
    const void* a_out;         /* [width, heads*vdim] */
    const void* e_router;      /* [experts + identity (+1), width]: router rows, then the shared expert's gate row */
    const float* e_correction_f32; /* [experts + identity]: added to the scores for the choice only (NULL: zeros) */
    const void* e_up;          /* [experts][e_ff, width]; LCC_EXPERT_CLAMP_GLU: [experts][2*e_ff, width], rows [gate | up] */
    const void* e_down;        /* [experts][width, e_ff] */
    const void* e_shared_up;   /* [e_shared_ff, width] */
    const void* e_shared_down; /* [width, e_shared_ff] */
    const float *hc1_f32, *hc2_f32; /* LCC_BLOCK_PRENORM_HC: [in: s | out: s | mix: s*s, indexed from*s + to] per sublayer */
} lcc_seq_layer;

typedef struct {
    int32_t width, vocab, n_layers, dtype;
    int32_t rows_padded8; /* non-zero: every matrix is allocated with its row count rounded up to 8 (zero rows), so that a
                             ragged projection can run as an 8-aligned tensor-core GEMM into its padded output buffer */
    float eps, alpha, embed_scale, logit_softcap; /* logit_softcap <= 0: none */
    int32_t block;   /* LCC_BLOCK_* */
    int32_t streams; /* residual streams of LCC_BLOCK_PRENORM_HC (>= 1) */
    int32_t norm_kind; /* LCC_NORM_*: the block norms and the final norm */
    int32_t canon_taps; /* LCC_BLOCK_BRANCHNORM: taps of the convolution in front of every mixer (<= 8) */
    float final_norm_alpha; /* LCC_NORM_DYT */
    float logit_scale;      /* logits are multiplied by it (0 reads as 1) */
    const float* final_norm_bias_f32; /* LCC_NORM_DYT: [width] */
    const void* embed;          /* [vocab, width] */
    const float* inv_freq_f32;  /* [width/2]: sinusoidal position frequencies, computed by the host; NULL: the embedding has no position term */
    const float* final_norm_f32;
    const void* head;           /* [vocab, width] */
    const lcc_seq_layer* layers;
} lcc_seq_model_desc;

/* One sequence's part of a step: n_new tokens that follow `past` cached ones. layer_state[i]: this sequence's fp32 state
 * slot of layer i (SSD: [conv carry: channels x (conv-1)] then [heads x vdim x state]; PARALLEL: [heads x vdim x dim] of
 * the right mixer; RETENTION: [heads x vdim x dim]; DELTA: [conv carry: (padded q, k, v channels) x (conv-1)] then [heads x vdim x dim]; in a
 * LCC_BLOCK_BRANCHNORM model every layer's slot starts with [width x (canon_taps-1)], the last inputs of the convolution in front of
 * the mixer), zero at the start of a sequence. k_pages[i] / v_pages[i]: the layer's page pools
 * [page][kv_heads][page_size][dim|vdim] (NULL for layers without attention); a LATENT layer has K pages only,
 * [page][1][page_size][rank + rot_dim], and a layer that reads another layer's cache is given that layer's pool.
 * page_table: logical -> physical page.
 * scalars (optional, device int32[LCC_SC_COUNT]): when given, kernels read the number of cached tokens from scalars[LCC_SC_KV_LEN]
 * and the ids from ids[scalars[LCC_SC_SEQ_LEN] - n_new ...], and do nothing once scalars[LCC_SC_FINISHED] is set, so that a
 * decode step can be replayed from a CUDA graph; otherwise `past` and ids[0..n_new) are used. */
typedef struct {
    int32_t n_new, past;
    const int64_t* ids;
    const int32_t* page_table;
    int32_t* scalars;
    float* const* layer_state;
    void* const* k_pages;
    void* const* v_pages;
} lcc_seq_entry;

typedef struct lcc_seq_model lcc_seq_model;
/* sizeof(lcc_seq_layer) (which = 0), sizeof(lcc_seq_model_desc) (1), sizeof(lcc_seq_entry) (2): a binding checks its own layout against them */
size_t lcc_seq_struct_bytes(int which);
lcc_seq_model* lcc_seq_model_create(lcc_ctx* ctx, const lcc_seq_model_desc* desc);
void lcc_seq_model_destroy(lcc_seq_model* m);
size_t lcc_seq_workspace_bytes(const lcc_seq_model* m, int max_tokens, int max_want);
int lcc_seq_bind_workspace(lcc_seq_model* m, void* ws, size_t ws_bytes, int max_tokens, int max_want);
/* fp32 elements of one sequence's state slot of layer i (0 for none). */
int64_t lcc_seq_layer_state_floats(const lcc_seq_model* m, int layer);
/* One step over the concatenated new tokens of all entries (linear layers and row ops run over all rows at once, the
 * sequence mixers per entry). want_rows: device int32[n_want] row indices into the concatenation whose logits are
 * wanted; logits: device fp32 [n_want, vocab] (soft cap applied); logits_copy: optional second copy. layer_dump: optional
 * device fp32 [n_layers, rows, width], the residual stream after every layer. */
int lcc_seq_forward(lcc_seq_model* m, const lcc_seq_entry* entries, int n_entries, int page_size, const int32_t* want_rows,
                    int n_want, float* logits, float* logits_copy, float* layer_dump, lcc_stream_t stream);

/* Debug/parity hooks: byte offsets of buffers inside the bound workspace. */
#define LCC_WS_PREFILL_HIDDEN 0 /* bf16 [S, hidden] residual stream of the last prefill */
#define LCC_WS_LOGITS 1         /* f32 [8][vocab] raw logits of the last token selection (row = slot) */
#define LCC_WS_DECODE_HIDDEN 2  /* bf16 [8][hidden] embedding row / residual stream of the decode step (row = slot) */
#define LCC_WS_DECODE_QKV 3     /* bf16 [8][(Hq+2Hkv)*128] */
#define LCC_WS_DECODE_ATTN 4    /* bf16 [8][Hq*128] */
#define LCC_WS_DECODE_ACT 5     /* bf16 [8][inter] */
#define LCC_WS_LOGITS_PROC 6    /* f32 [8][vocab] processed logits */
#define LCC_WS_MEGA_ERROR 7     /* int32: sticky error flag of the persistent decode kernel (0 = ok) */
#define LCC_WS_MEGA_TRACE 8     /* u64 [256][64]: per-CTA globaltimer stamps when LIVECC_B200_MEGA_TRACE=1 */
size_t lcc_ws_offset(const lcc_model* m, int which);

#ifdef __cplusplus
}
#endif
#endif /* LIVECC_B200_H */
