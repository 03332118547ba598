/*
 * neon_decoder.h - C ABI of the gpt-oss-shaped decoder stack built around the MoE layer of
 * neon_moe.h (same shared library): token embedding, per layer RMSNorm -> QKV projection ->
 * YaRN rotary embedding -> KV-cache append -> grouped-query attention with per-head sink
 * logits (sliding window on even layers) -> output projection -> residual -> RMSNorm -> MoE
 * -> residual, then final RMSNorm -> unembedding -> argmax.  One call advances every
 * sequence of a small decode batch by one token.
 *
 * Relation to the reference engine: none of this exists there (the engine has no language
 * model code).  The calling conventions are those of neon_moe.h, which follow the engine's
 * "system" classes (construction owns device buffers, NeonEngine/src/water_physics.cpp:23-123;
 * stream-ordered execution, NeonEngine/src/water_physics.hpp:66; explicit host read-back,
 * NeonEngine/src/water_app.cpp:601-612).
 *
 * Conventions (this library's own):
 *   - bf16 tensors are raw 16-bit patterns; the residual stream, q and logits are fp32;
 *     normalised activations, attention outputs and the K/V cache are bf16 (round to nearest even).
 *   - RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w.
 *   - QKV weight rows: n_q_heads*64 query rows, then n_kv_heads*64 key rows, then value rows.
 *   - Rotary embedding pairs element i with i + 32 of a head ("rotate half"); YaRN
 *     (NTK-by-parts): inv_freq_i = (1-r_i)/ (factor*theta^(2i/64)) + r_i / theta^(2i/64) with
 *     r_i = 1 - clamp((i - low)/(high - low), 0, 1), low/high from beta_fast/beta_slow and
 *     orig_ctx as in the YaRN paper; cos and sin are multiplied by 0.1*ln(factor) + 1.
 *   - Attention scores are q.k/8; the softmax denominator includes exp(sink[head]); layers with
 *     even index attend to the last `window` positions only, odd layers to the whole cache.
 *   - K/V cache per layer (internal): keys bf16 [max_batch][n_kv_heads][max_ctx][64], values
 *     transposed [max_batch][n_kv_heads][64][max_ctx].
 *   - The MoE of a layer receives the bf16 normalised activations; its config is
 *     {hidden, inter, n_experts, top_k, swiglu_limit, swiglu_alpha} (neon_moe.h).
 *
 * All functions return 0 or a NEON_MOE_E* code (neon_moe.h); none throws or aborts.
 */
#ifndef NEON_DECODER_H
#define NEON_DECODER_H

#include <stdint.h>

#include "neon_moe.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct neon_decoder_handle neon_decoder_handle;

typedef struct neon_decoder_config {
    int n_layers;        /* 24                                                       */
    int hidden;          /* 2880, multiple of 64                                     */
    int n_q_heads;       /* 64; n_q_heads / n_kv_heads in {1,2,4,8}                  */
    int n_kv_heads;      /* 8                                                        */
    int head_dim;        /* 64 (only value supported)                                */
    int vocab;           /* 201088                                                   */
    int max_batch;       /* sequences per step, <= 8                                 */
    int max_ctx;         /* cache positions per sequence (4096), multiple of 8       */
    int window;          /* sliding window of even layers (128); 0 = none anywhere   */
    float rope_theta;    /* 150000                                                   */
    float rope_factor;   /* 32 (1 = plain rotary embedding)                          */
    float rope_orig_ctx; /* 4096                                                     */
    float rope_beta_fast;/* 32                                                       */
    float rope_beta_slow;/* 1                                                        */
    float rms_eps;       /* 1e-5                                                     */
    int inter;           /* MoE intermediate size (2880)                             */
    int n_experts;       /* 32                                                       */
    int top_k;           /* 4                                                        */
    float swiglu_limit;  /* 7.0                                                      */
    float swiglu_alpha;  /* 1.702                                                    */
    int device;          /* CUDA device ordinal                                      */
} neon_decoder_config;

/* Allocates caches, activations and one MoE layer handle per layer on cfg->device. */
int neon_decoder_create(const neon_decoder_config* cfg, neon_decoder_handle** out);
int neon_decoder_destroy(neon_decoder_handle* h);
const char* neon_decoder_last_error(const neon_decoder_handle* h);

/* embed, unembed: bf16 [vocab, hidden]; final_norm: bf16 [hidden].  Copied. */
int neon_decoder_set_embeddings(neon_decoder_handle* h, const void* embed, const void* unembed,
                                const void* final_norm, int on_device);

/* Attention block of one layer (all bf16, copied): ln1 [H]; wqkv [(nq+2nkv)*64, H]; bqkv
 * [(nq+2nkv)*64]; sinks [nq]; wo [H, nq*64]; bo [H]; ln2 [H]. */
int neon_decoder_set_attention(neon_decoder_handle* h, int layer, const void* ln1, const void* wqkv,
                               const void* bqkv, const void* sinks, const void* wo, const void* bo,
                               const void* ln2, int on_device);

/* MoE block of one layer; arguments as neon_moe_set_weights. */
int neon_decoder_set_moe(neon_decoder_handle* h, int layer, const void* router_w, const void* router_b,
                         const uint8_t* gate_up_blocks, const uint8_t* gate_up_scales, const void* gate_up_bias,
                         const uint8_t* down_blocks, const uint8_t* down_scales, const void* down_bias,
                         int on_device);

/* Fills cache positions [0, n_pos) of one layer for sequences [0, batch): k, v bf16
 * [batch, n_pos, n_kv_heads, 64] (keys already rotated). */
int neon_decoder_load_kv(neon_decoder_handle* h, int layer, const void* k, const void* v, int batch,
                         int n_pos, int on_device);

/* One decode step for `batch` sequences, enqueued on cuda_stream.  Device pointers:
 * tokens int32 [batch]; positions int32 [batch] (each < max_ctx; the new K/V go to that cache
 * slot and attention covers positions <= it); logits fp32 [batch, vocab] or NULL (internal
 * buffer); next_tokens int32 [batch] or NULL.  Token ids and positions outside their ranges are
 * clamped into range by the kernels (they live in device memory, so the host cannot check them).  The second call with the same arguments is
 * captured into a CUDA graph and replayed from then on (option use_graphs). */
int neon_decoder_step(neon_decoder_handle* h, const int32_t* tokens, const int32_t* positions, int batch,
                      float* logits, int32_t* next_tokens, void* cuda_stream);

/* Same with HOST arrays; copies tokens/positions in, next_tokens out, and waits. */
int neon_decoder_step_host(neon_decoder_handle* h, const int32_t* tokens, const int32_t* positions,
                           int batch, int32_t* next_tokens, void* cuda_stream);

/* Test/debug read-back (blocking) of an internal buffer of the last step into host memory.
 * name: "x" fp32 [B,H] residual stream after the last layer; "xn" bf16 [B,H] last normalised
 * activations (the final norm's output); "qkv" fp32 [B,(nq+2nkv)*64] of the last layer
 * (q rotated, k/v as projected); "attn" bf16 [B,nq*64]; "moe_in" bf16 [B,H] of the last layer;
 * "moe_out" fp32 [B,H]; "logits" fp32 [B,vocab]; "inv_freq" fp32 [32]. */
int neon_decoder_read(neon_decoder_handle* h, const char* name, void* dst, uint64_t bytes);

/* Options: "use_graphs" (default 1), "pdl" (programmatic dependent launch, a bit per
 * kernel kind: 1 GEMV, 2 RMSNorm, 4 rotary/cache, 8 attention, 16 merge, 32 others; default 29), "moe.<option>" (passed to every layer, see neon_moe.h), "stop_after_layer" (debug: run only the first n layers
 * and skip the head; 0 = all). */
int neon_decoder_set_option(neon_decoder_handle* h, const char* name, int64_t value);

/* Kernels this library launched for the handle so far (MoE layers included). */
int64_t neon_decoder_launch_count(const neon_decoder_handle* h);

/* Bytes of weights and cache one decode step must read at least: attention and unembedding
 * weights, the K/V positions in range, and (MoE) the distinct experts the last step touched
 * are reported separately: bytes3 = {dense_weights, kv, moe_per_expert}. */
int neon_decoder_step_bytes(neon_decoder_handle* h, const int32_t* positions_host, int batch, double* bytes3);

#ifdef __cplusplus
}
#endif
#endif /* NEON_DECODER_H */
