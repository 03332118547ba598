// Host side of the decoder stack declared in include/neon_decoder.h: owns the dense weights,
// the K/V caches and one MoE layer handle (neon_moe.h) per layer, and enqueues one decode
// step as a fixed kernel sequence (replayed as a CUDA graph once the arguments repeat).
// No CPU fallback exists: a step launches CUDA kernels or fails with an error code.
#include "../../include/neon_decoder.h"

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>
#include <algorithm>
#include <string>
#include <vector>

#include "decoder_kernels.cuh"

using namespace neon;

namespace {
thread_local std::string g_dec_create_error;

struct LayerW {
    uint16_t *ln1 = nullptr, *wqkv = nullptr, *bqkv = nullptr, *sinks = nullptr, *wo = nullptr, *bo = nullptr, *ln2 = nullptr;
    uint16_t *kc = nullptr, *vc = nullptr;
    neon_moe_handle* moe = nullptr;
    bool has_attn = false, has_moe = false;
};
}  // namespace

struct neon_decoder_handle {
    neon_decoder_config cfg{};
    std::string err;
    std::vector<LayerW> layers;
    uint16_t *embed = nullptr, *unembed = nullptr, *final_norm = nullptr;
    bool has_embed = false;
    float *x = nullptr, *qkv = nullptr, *moe_out = nullptr, *logits = nullptr, *part = nullptr, *inv_freq = nullptr;
    float* oproj = nullptr;  // K-split parts of the attention output projection
    int qkv_split = 1, o_split = 1;
    uint16_t *xn = nullptr, *xn2 = nullptr, *attn = nullptr;
    int32_t *tok_dev = nullptr, *pos_dev = nullptr, *next_dev = nullptr;
    float mscale = 1.f;
    int64_t launches = 0;
    int use_graphs = 1, stop_after = 0;
    int pdl = 29;  // programmatic dependent launch per kernel kind (PdlBit); RMSNorm measured slower with it
    cudaStream_t own_stream = nullptr, last_stream = nullptr;
    // one cached graph
    struct {
        const int32_t *tokens = nullptr, *positions = nullptr;
        float* logits = nullptr;
        int32_t* next = nullptr;
        int batch = 0, seen = 0;
        int64_t launches = 0;
        cudaGraphExec_t exec = nullptr;
    } g;
};

namespace {

int dfail(neon_decoder_handle* h, int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (h) h->err = buf; else g_dec_create_error = buf;
    return code;
}

#define DCU(h, call)                                                                              \
    do {                                                                                          \
        cudaError_t e_ = (call);                                                                  \
        if (e_ != cudaSuccess) return dfail(h, NEON_MOE_ECUDA, "%s: %s", #call, cudaGetErrorString(e_)); \
    } while (0)

int dalloc(neon_decoder_handle* h, void** p, size_t bytes) {
    DCU(h, cudaMalloc(p, std::max<size_t>(bytes, 16)));
    return NEON_MOE_OK;
}
#define DALLOC(h, ptr, bytes)                                          \
    do {                                                               \
        int rc_ = dalloc(h, reinterpret_cast<void**>(&(ptr)), bytes);  \
        if (rc_) return rc_;                                           \
    } while (0)

int copy_in(neon_decoder_handle* h, void* dst, const void* src, size_t bytes, int on_device) {
    if (!src) return dfail(h, NEON_MOE_EINVAL, "null tensor");
    DCU(h, cudaMemcpy(dst, src, bytes, on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice));
    return NEON_MOE_OK;
}

void drop_graph(neon_decoder_handle* h) {
    if (h->g.exec) cudaGraphExecDestroy(h->g.exec);
    h->g = {};
}

// YaRN (NTK-by-parts) inverse frequencies for head_dim 64, computed in double.
void yarn_inv_freq(const neon_decoder_config& c, float* inv, float* mscale) {
    const int d = c.head_dim, half = d / 2;
    const double theta = c.rope_theta, factor = c.rope_factor;
    const double kPi = 3.14159265358979323846;
    auto corr_dim = [&](double n_rot) { return d * std::log(c.rope_orig_ctx / (n_rot * 2.0 * kPi)) / (2.0 * std::log(theta)); };
    double low = 0, high = 0;
    if (factor > 1.0) {
        low = std::max(std::floor(corr_dim(c.rope_beta_fast)), 0.0);
        high = std::min(std::ceil(corr_dim(c.rope_beta_slow)), (double)(d - 1));
        if (high == low) high += 0.001;
    }
    for (int i = 0; i < half; ++i) {
        const double freq = std::pow(theta, 2.0 * i / d);
        double v = 1.0 / freq;
        if (factor > 1.0) {
            const double ramp = std::min(std::max((i - low) / (high - low), 0.0), 1.0);
            const double keep = 1.0 - ramp;  // 1: high-frequency dimension, left as is
            v = (1.0 / (factor * freq)) * (1.0 - keep) + (1.0 / freq) * keep;
        }
        inv[i] = (float)v;
    }
    *mscale = factor > 1.0 ? (float)(0.1 * std::log(factor) + 1.0) : 1.f;
}

// Launch with programmatic stream serialization (option "pdl"): the kernel may be scheduled
// while its predecessor drains; every kernel waits for its predecessor before it reads or writes
// anything a predecessor touches.
template <typename... KArgs, typename... Args>
void launch_pdl(neon_decoder_handle* h, bool pdl, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    h->launches++;
}

enum PdlBit { kPdlGemv = 1, kPdlNorm = 2, kPdlRope = 4, kPdlAttn = 8, kPdlMerge = 16, kPdlOther = 32 };

template <typename... KArgs, typename... Args>
void launch(neon_decoder_handle* h, int bit, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
            Args... args) {
    launch_pdl(h, (h->pdl & bit) != 0, kernel, grid, block, smem, st, args...);
}

int launch_gemv(neon_decoder_handle* h, const uint16_t* W, const uint16_t* bias, const uint16_t* x, int B, int rows, int K,
                int accumulate, float* out, cudaStream_t st) {
    if (K % 32) return dfail(h, NEON_MOE_EINVAL, "GEMV depth %d is not a multiple of 32", K);
    const size_t smem = (size_t)8 * (K + gemv_row_pad(K)) * 2 + 8 * 128 * sizeof(float);
    if (smem > 72 * 1024) return dfail(h, NEON_MOE_EINVAL, "GEMV operand of %zu bytes does not fit shared memory", smem);
    static bool configured[64] = {};
    if (!configured[h->cfg.device & 63]) {
        DCU(h, cudaFuncSetAttribute(gemv_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024));
        configured[h->cfg.device & 63] = true;
    }
    const int grid = std::min((rows + 15) / 16, 148 * 2);
    launch_pdl(h, (h->pdl & kPdlGemv) != 0, gemv_mma_kernel, dim3(grid), dim3(256), smem, st, W, bias, x, B, rows, K, accumulate, out);
    return NEON_MOE_OK;
}

int launch_gemv_split(neon_decoder_handle* h, const uint16_t* W, const uint16_t* bias, const uint16_t* x, int B, int rows, int K,
                      int splits, float* parts, long long part_stride, cudaStream_t st) {
    if (K % 32) return dfail(h, NEON_MOE_EINVAL, "GEMV depth %d is not a multiple of 32", K);
    const int nkb = K / 32;
    if ((nkb + splits - 1) / splits > 8 * kGemvSplitU) return dfail(h, NEON_MOE_EINVAL, "GEMV depth %d needs more K-splits", K);
    launch_pdl(h, (h->pdl & kPdlGemv) != 0, gemv_mma_split_kernel, dim3((rows + 15) / 16, splits), dim3(256), 0, st, W, bias, x,
               B, rows, K, parts, part_stride);
    return NEON_MOE_OK;
}

int launch_attention(neon_decoder_handle* h, const LayerW& L, int layer, int B, const int32_t* pos, cudaStream_t st) {
    const auto& c = h->cfg;
    const int window = (c.window > 0 && layer % 2 == 0) ? c.window : 0;
    // chunks start at the window start rounded down to a multiple of 8
    const int span = window > 0 ? std::min(window + 7, c.max_ctx) : c.max_ctx;
    const int splits = (span + kAttnChunk - 1) / kAttnChunk;
    const int G = c.n_q_heads / c.n_kv_heads;
    const dim3 grid(c.n_kv_heads, B, splits);
    const float scale = 1.f / std::sqrt((float)c.head_dim);
#define ATTN_CASE(GG)                                                                                               \
    case GG:                                                                                                        \
        launch(h, kPdlAttn, attn_partial_kernel<GG>, grid, dim3(256), 0, st, (const float*)h->qkv, (const uint16_t*)L.kc,     \
               (const uint16_t*)L.vc, pos, c.n_q_heads, c.n_kv_heads, c.max_ctx, window, scale, splits, h->part);   \
        break;
    switch (G) {
        ATTN_CASE(1) ATTN_CASE(2) ATTN_CASE(4) ATTN_CASE(8)
        default: return dfail(h, NEON_MOE_EINVAL, "unsupported query group size %d", G);
    }
#undef ATTN_CASE
    launch(h, kPdlMerge, attn_merge_kernel, dim3(c.n_q_heads, B), dim3(64), 0, st, (const float*)h->part, (const uint16_t*)L.sinks,
           c.n_q_heads, splits, h->attn);
    return NEON_MOE_OK;
}

int step_eager(neon_decoder_handle* h, const int32_t* tokens, const int32_t* positions, int B, float* logits, int32_t* next,
               cudaStream_t st) {
    const auto& c = h->cfg;
    const int H = c.hidden, QKV = (c.n_q_heads + 2 * c.n_kv_heads) * c.head_dim, QD = c.n_q_heads * c.head_dim;
    launch(h, kPdlOther, embed_kernel, dim3(B), dim3(256), 0, st, (const uint16_t*)h->embed, tokens, H, c.vocab, h->x);
    const int n_layers = h->stop_after > 0 ? std::min(h->stop_after, c.n_layers) : c.n_layers;
    const float* pending = nullptr;  // MoE output of the previous layer, added by the next RMSNorm kernel
    for (int l = 0; l < n_layers; ++l) {
        LayerW& L = h->layers[l];
        launch(h, kPdlNorm, rmsnorm_kernel, dim3(B), dim3(1024), 0, st, h->x, pending, pending ? 1 : 0, 0ll,
               (const uint16_t*)L.ln1, H, c.rms_eps, h->xn);
        int rc = launch_gemv_split(h, L.wqkv, L.bqkv, h->xn, B, QKV, H, h->qkv_split, h->qkv, (long long)B * QKV, st);
        if (rc) return rc;
        launch(h, kPdlRope, rope_cache_kernel, dim3(c.n_q_heads + 2 * c.n_kv_heads, B), dim3(64), 0, st, h->qkv, h->qkv_split,
               (long long)B * QKV, (const float*)h->inv_freq, positions, c.n_q_heads, c.n_kv_heads, h->mscale, c.max_ctx, L.kc,
               L.vc);
        rc = launch_attention(h, L, l, B, positions, st);
        if (rc) return rc;
        rc = launch_gemv_split(h, L.wo, L.bo, h->attn, B, H, QD, h->o_split, h->oproj, (long long)B * H, st);
        if (rc) return rc;
        // residual add of the projection's parts, then the second norm
        launch(h, kPdlNorm, rmsnorm_kernel, dim3(B), dim3(1024), 0, st, h->x, (const float*)h->oproj, h->o_split,
               (long long)B * H, (const uint16_t*)L.ln2, H, c.rms_eps, h->xn2);
        const int64_t before = neon_moe_launch_count(L.moe);
        rc = neon_moe_forward(L.moe, h->xn2, B, nullptr, h->moe_out, nullptr, nullptr, st);
        if (rc) return dfail(h, rc, "layer %d MoE: %s", l, neon_moe_last_error(L.moe));
        h->launches += neon_moe_launch_count(L.moe) - before;
        pending = h->moe_out;
    }
    if (h->stop_after > 0) {
        launch(h, kPdlOther, add_kernel, dim3((B * H + 255) / 256), dim3(256), 0, st, h->x, pending, B * H);
        return NEON_MOE_OK;
    }
    launch(h, kPdlNorm, rmsnorm_kernel, dim3(B), dim3(1024), 0, st, h->x, pending, pending ? 1 : 0, 0ll,
           (const uint16_t*)h->final_norm, H, c.rms_eps, h->xn);
    float* lg = logits ? logits : h->logits;
    int rc = launch_gemv(h, h->unembed, nullptr, h->xn, B, c.vocab, H, 0, lg, st);
    if (rc) return rc;
    if (next) launch(h, kPdlOther, argmax_kernel, dim3(B), dim3(1024), 0, st, (const float*)lg, c.vocab, next);
    DCU(h, cudaGetLastError());
    return NEON_MOE_OK;
}

int check_ready(neon_decoder_handle* h) {
    if (!h->has_embed) return dfail(h, NEON_MOE_ESTATE, "step before set_embeddings");
    for (size_t l = 0; l < h->layers.size(); ++l)
        if (!h->layers[l].has_attn || !h->layers[l].has_moe)
            return dfail(h, NEON_MOE_ESTATE, "step before layer %zu has its weights", l);
    return NEON_MOE_OK;
}

}  // namespace

extern "C" {

const char* neon_decoder_last_error(const neon_decoder_handle* h) { return h ? h->err.c_str() : g_dec_create_error.c_str(); }
int64_t neon_decoder_launch_count(const neon_decoder_handle* h) { return h ? h->launches : 0; }

int neon_decoder_create(const neon_decoder_config* cfg, neon_decoder_handle** out) {
    if (!cfg || !out) return dfail(nullptr, NEON_MOE_EINVAL, "null argument");
    *out = nullptr;
    const auto& c = *cfg;
    if (c.head_dim != 64) return dfail(nullptr, NEON_MOE_EINVAL, "head_dim must be 64");
    if (c.n_layers <= 0 || c.hidden <= 0 || c.hidden % 64 || c.vocab <= 0 || c.max_ctx <= 0 || c.max_ctx % 8)
        return dfail(nullptr, NEON_MOE_EINVAL, "bad layer count, hidden size, vocabulary or context (a multiple of 8)");
    if (c.max_batch < 1 || c.max_batch > kDecMaxBatch) return dfail(nullptr, NEON_MOE_EINVAL, "max_batch must be 1..8");
    if (c.n_kv_heads <= 0 || c.n_q_heads % c.n_kv_heads) return dfail(nullptr, NEON_MOE_EINVAL, "n_q_heads %% n_kv_heads != 0");
    const int G = c.n_q_heads / c.n_kv_heads;
    if (G != 1 && G != 2 && G != 4 && G != 8) return dfail(nullptr, NEON_MOE_EINVAL, "query group size must be 1, 2, 4 or 8");
    if (c.n_q_heads * c.head_dim > 4096 || c.hidden > 4096)
        return dfail(nullptr, NEON_MOE_EINVAL, "hidden size and query width are limited to 4096 (GEMV shared memory)");
    if (!(c.rope_theta > 1.f) || !(c.rope_factor >= 1.f)) return dfail(nullptr, NEON_MOE_EINVAL, "bad rotary parameters");
    if (cudaSetDevice(c.device) != cudaSuccess) {
        cudaGetLastError();
        return dfail(nullptr, NEON_MOE_ECUDA, "cudaSetDevice(%d) failed", c.device);
    }
    auto* h = new (std::nothrow) neon_decoder_handle;
    if (!h) return dfail(nullptr, NEON_MOE_ECUDA, "out of host memory");
    h->cfg = c;
    h->layers.resize(c.n_layers);
    const int H = c.hidden, B = c.max_batch, QKV = (c.n_q_heads + 2 * c.n_kv_heads) * 64, QD = c.n_q_heads * 64;
    auto bail = [&](int rc) {
        g_dec_create_error = h->err;
        neon_decoder_destroy(h);
        return rc;
    };
#define TRY(expr)                   \
    do {                            \
        int rc__ = (expr);          \
        if (rc__) return bail(rc__); \
    } while (0)
    auto alloc = [&](auto& ptr, size_t bytes) { return dalloc(h, reinterpret_cast<void**>(&ptr), bytes); };
    TRY(alloc(h->embed, (size_t)c.vocab * H * 2));
    TRY(alloc(h->unembed, (size_t)c.vocab * H * 2));
    TRY(alloc(h->final_norm, (size_t)H * 2));
    TRY(alloc(h->x, (size_t)B * H * 4));
    TRY(alloc(h->moe_out, (size_t)B * H * 4));
    // K-split factors of the two small projections: every warp of a CTA gets at most kGemvSplitU k-blocks
    auto split_for = [](int K) { return std::min(4, (K / 32 + 8 * kGemvSplitU - 1) / (8 * kGemvSplitU)); };
    h->qkv_split = split_for(H);
    h->o_split = split_for(QD);
    TRY(alloc(h->qkv, (size_t)h->qkv_split * B * QKV * 4));
    TRY(alloc(h->oproj, (size_t)h->o_split * B * H * 4));
    TRY(alloc(h->logits, (size_t)B * c.vocab * 4));
    TRY(alloc(h->part, (size_t)B * c.n_q_heads * ((c.max_ctx + kAttnChunk - 1) / kAttnChunk) * 66 * 4));
    TRY(alloc(h->inv_freq, 32 * 4));
    TRY(alloc(h->xn, (size_t)B * H * 2));
    TRY(alloc(h->xn2, (size_t)B * H * 2));
    TRY(alloc(h->attn, (size_t)B * QD * 2));
    TRY(alloc(h->tok_dev, B * 4));
    TRY(alloc(h->pos_dev, B * 4));
    TRY(alloc(h->next_dev, B * 4));
    float inv[32];
    yarn_inv_freq(c, inv, &h->mscale);
    if (cudaMemcpy(h->inv_freq, inv, sizeof inv, cudaMemcpyHostToDevice) != cudaSuccess) return bail(dfail(h, NEON_MOE_ECUDA, "inv_freq upload"));
    if (cudaStreamCreateWithFlags(&h->own_stream, cudaStreamNonBlocking) != cudaSuccess) return bail(dfail(h, NEON_MOE_ECUDA, "stream"));
    const size_t cache = (size_t)B * c.max_ctx * c.n_kv_heads * 64 * 2;
    for (int l = 0; l < c.n_layers; ++l) {
        LayerW& L = h->layers[l];
        TRY(alloc(L.ln1, (size_t)H * 2));
        TRY(alloc(L.ln2, (size_t)H * 2));
        TRY(alloc(L.wqkv, (size_t)QKV * H * 2));
        TRY(alloc(L.bqkv, (size_t)QKV * 2));
        TRY(alloc(L.sinks, (size_t)c.n_q_heads * 2));
        TRY(alloc(L.wo, (size_t)H * QD * 2));
        TRY(alloc(L.bo, (size_t)H * 2));
        TRY(alloc(L.kc, cache));
        TRY(alloc(L.vc, cache));
        if (cudaMemset(L.kc, 0, cache) != cudaSuccess || cudaMemset(L.vc, 0, cache) != cudaSuccess)
            return bail(dfail(h, NEON_MOE_ECUDA, "cache clear"));
        neon_moe_config mc{};
        mc.hidden = H; mc.inter = c.inter; mc.n_experts = c.n_experts; mc.top_k = c.top_k;
        mc.swiglu_limit = c.swiglu_limit; mc.swiglu_alpha = c.swiglu_alpha;
        mc.max_tokens = B; mc.ep_rank = 0; mc.ep_size = 1; mc.device = c.device;
        int rc = neon_moe_create(&mc, &L.moe);
        if (rc) return bail(dfail(h, rc, "layer %d MoE: %s", l, neon_moe_last_error(nullptr)));
    }
#undef TRY
    *out = h;
    return NEON_MOE_OK;
}

int neon_decoder_destroy(neon_decoder_handle* h) {
    if (!h) return NEON_MOE_OK;
    cudaSetDevice(h->cfg.device);
    cudaDeviceSynchronize();
    drop_graph(h);
    for (auto& L : h->layers) {
        for (void* p : {(void*)L.ln1, (void*)L.wqkv, (void*)L.bqkv, (void*)L.sinks, (void*)L.wo, (void*)L.bo, (void*)L.ln2,
                        (void*)L.kc, (void*)L.vc})
            if (p) cudaFree(p);
        if (L.moe) neon_moe_destroy(L.moe);
    }
    for (void* p : {(void*)h->embed, (void*)h->unembed, (void*)h->final_norm, (void*)h->x, (void*)h->qkv, (void*)h->moe_out,
                    (void*)h->logits, (void*)h->part, (void*)h->oproj, (void*)h->inv_freq, (void*)h->xn, (void*)h->xn2, (void*)h->attn,
                    (void*)h->tok_dev, (void*)h->pos_dev, (void*)h->next_dev})
        if (p) cudaFree(p);
    if (h->own_stream) cudaStreamDestroy(h->own_stream);
    cudaGetLastError();
    delete h;
    return NEON_MOE_OK;
}

int neon_decoder_set_embeddings(neon_decoder_handle* h, const void* embed, const void* unembed, const void* final_norm,
                                int on_device) {
    if (!h) return NEON_MOE_EINVAL;
    DCU(h, cudaSetDevice(h->cfg.device));
    const size_t n = (size_t)h->cfg.vocab * h->cfg.hidden * 2;
    int rc;
    if ((rc = copy_in(h, h->embed, embed, n, on_device))) return rc;
    if ((rc = copy_in(h, h->unembed, unembed, n, on_device))) return rc;
    if ((rc = copy_in(h, h->final_norm, final_norm, (size_t)h->cfg.hidden * 2, on_device))) return rc;
    h->has_embed = true;
    return NEON_MOE_OK;
}

int neon_decoder_set_attention(neon_decoder_handle* h, int layer, const void* ln1, const void* wqkv, const void* bqkv,
                               const void* sinks, const void* wo, const void* bo, const void* ln2, int on_device) {
    if (!h) return NEON_MOE_EINVAL;
    if (layer < 0 || layer >= h->cfg.n_layers) return dfail(h, NEON_MOE_EINVAL, "layer %d out of range", layer);
    DCU(h, cudaSetDevice(h->cfg.device));
    const auto& c = h->cfg;
    const size_t H = c.hidden, QKV = (size_t)(c.n_q_heads + 2 * c.n_kv_heads) * 64, QD = (size_t)c.n_q_heads * 64;
    LayerW& L = h->layers[layer];
    int rc;
    if ((rc = copy_in(h, L.ln1, ln1, H * 2, on_device))) return rc;
    if ((rc = copy_in(h, L.wqkv, wqkv, QKV * H * 2, on_device))) return rc;
    if ((rc = copy_in(h, L.bqkv, bqkv, QKV * 2, on_device))) return rc;
    if ((rc = copy_in(h, L.sinks, sinks, (size_t)c.n_q_heads * 2, on_device))) return rc;
    if ((rc = copy_in(h, L.wo, wo, H * QD * 2, on_device))) return rc;
    if ((rc = copy_in(h, L.bo, bo, H * 2, on_device))) return rc;
    if ((rc = copy_in(h, L.ln2, ln2, H * 2, on_device))) return rc;
    L.has_attn = true;
    return NEON_MOE_OK;
}

int neon_decoder_set_moe(neon_decoder_handle* h, int layer, const void* router_w, const void* router_b,
                         const uint8_t* gate_up_blocks, const uint8_t* gate_up_scales, const void* gate_up_bias,
                         const uint8_t* down_blocks, const uint8_t* down_scales, const void* down_bias, int on_device) {
    if (!h) return NEON_MOE_EINVAL;
    if (layer < 0 || layer >= h->cfg.n_layers) return dfail(h, NEON_MOE_EINVAL, "layer %d out of range", layer);
    LayerW& L = h->layers[layer];
    int rc = neon_moe_set_weights(L.moe, router_w, router_b, gate_up_blocks, gate_up_scales, gate_up_bias, down_blocks,
                                  down_scales, down_bias, on_device);
    if (rc) return dfail(h, rc, "layer %d MoE: %s", layer, neon_moe_last_error(L.moe));
    L.has_moe = true;
    return NEON_MOE_OK;
}

int neon_decoder_load_kv(neon_decoder_handle* h, int layer, const void* k, const void* v, int batch, int n_pos, int on_device) {
    if (!h) return NEON_MOE_EINVAL;
    const auto& c = h->cfg;
    if (layer < 0 || layer >= c.n_layers) return dfail(h, NEON_MOE_EINVAL, "layer %d out of range", layer);
    if (batch < 0 || batch > c.max_batch || n_pos < 0 || n_pos > c.max_ctx)
        return dfail(h, NEON_MOE_EINVAL, "batch %d / positions %d outside the cache", batch, n_pos);
    if (!k || !v) return dfail(h, NEON_MOE_EINVAL, "null cache tensor");
    DCU(h, cudaSetDevice(c.device));
    LayerW& L = h->layers[layer];
    if (batch && n_pos) {
        const size_t bytes = (size_t)batch * n_pos * c.n_kv_heads * 64 * 2;
        const size_t vecs = bytes / 16;
        const void *ks = k, *vs = v;
        void* tmp = nullptr;
        if (!on_device) {  // stage the host arrays in device memory, then re-tile
            DCU(h, cudaMalloc(&tmp, 2 * bytes));
            cudaError_t e1 = cudaMemcpy(tmp, k, bytes, cudaMemcpyHostToDevice);
            cudaError_t e2 = cudaMemcpy(static_cast<char*>(tmp) + bytes, v, bytes, cudaMemcpyHostToDevice);
            if (e1 != cudaSuccess || e2 != cudaSuccess) {
                cudaFree(tmp);
                return dfail(h, NEON_MOE_ECUDA, "cache upload failed");
            }
            ks = tmp;
            vs = static_cast<char*>(tmp) + bytes;
        }
        k_load_kernel<<<(unsigned)((vecs + 255) / 256), 256>>>(static_cast<const uint4*>(ks), batch, n_pos, c.n_kv_heads,
                                                               c.max_ctx, reinterpret_cast<uint4*>(L.kc));
        v_load_kernel<<<(unsigned)((bytes / 2 + 255) / 256), 256>>>(static_cast<const uint16_t*>(vs), batch, n_pos, c.n_kv_heads,
                                                                    c.max_ctx, L.vc);
        h->launches += 2;
        cudaError_t e = cudaDeviceSynchronize();
        if (tmp) cudaFree(tmp);
        if (e != cudaSuccess) return dfail(h, NEON_MOE_ECUDA, "cache re-tiling failed: %s", cudaGetErrorString(e));
    }
    return NEON_MOE_OK;
}

int neon_decoder_step(neon_decoder_handle* h, const int32_t* tokens, const int32_t* positions, int batch, float* logits,
                      int32_t* next_tokens, void* cuda_stream) {
    if (!h) return NEON_MOE_EINVAL;
    int rc = check_ready(h);
    if (rc) return rc;
    if (batch < 1 || batch > h->cfg.max_batch) return dfail(h, NEON_MOE_EINVAL, "batch %d outside 1..%d", batch, h->cfg.max_batch);
    if (!tokens || !positions) return dfail(h, NEON_MOE_EINVAL, "null tokens/positions");
    DCU(h, cudaSetDevice(h->cfg.device));
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    h->last_stream = st;
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    const bool capturing = cudaStreamIsCapturing(st, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone;
    cudaGetLastError();
    if (!h->use_graphs || capturing) return step_eager(h, tokens, positions, batch, logits, next_tokens, st);
    auto& g = h->g;
    if (!(g.tokens == tokens && g.positions == positions && g.batch == batch && g.logits == logits && g.next == next_tokens)) {
        drop_graph(h);
        g.tokens = tokens; g.positions = positions; g.batch = batch; g.logits = logits; g.next = next_tokens;
    }
    if (!g.exec) {
        if (g.seen++ == 0) return step_eager(h, tokens, positions, batch, logits, next_tokens, st);
        const int64_t before = h->launches;
        DCU(h, cudaStreamBeginCapture(h->own_stream, cudaStreamCaptureModeThreadLocal));
        rc = step_eager(h, tokens, positions, batch, logits, next_tokens, h->own_stream);
        cudaGraph_t graph = nullptr;
        cudaError_t ce = cudaStreamEndCapture(h->own_stream, &graph);
        g.launches = h->launches - before;
        h->launches = before;
        if (rc || ce != cudaSuccess || !graph) {
            if (graph) cudaGraphDestroy(graph);
            cudaGetLastError();
            h->use_graphs = 0;
            return step_eager(h, tokens, positions, batch, logits, next_tokens, st);
        }
        ce = cudaGraphInstantiate(&g.exec, graph, 0);
        cudaGraphDestroy(graph);
        if (ce != cudaSuccess) {
            g.exec = nullptr;
            h->use_graphs = 0;
            cudaGetLastError();
            return step_eager(h, tokens, positions, batch, logits, next_tokens, st);
        }
    }
    DCU(h, cudaGraphLaunch(g.exec, st));
    h->launches += g.launches;
    return NEON_MOE_OK;
}

int neon_decoder_step_host(neon_decoder_handle* h, const int32_t* tokens, const int32_t* positions, int batch,
                           int32_t* next_tokens, void* cuda_stream) {
    if (!h) return NEON_MOE_EINVAL;
    if (batch < 1 || batch > h->cfg.max_batch) return dfail(h, NEON_MOE_EINVAL, "batch %d outside 1..%d", batch, h->cfg.max_batch);
    if (!tokens || !positions || !next_tokens) return dfail(h, NEON_MOE_EINVAL, "null argument");
    DCU(h, cudaSetDevice(h->cfg.device));
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    DCU(h, cudaMemcpyAsync(h->tok_dev, tokens, (size_t)batch * 4, cudaMemcpyHostToDevice, st));
    DCU(h, cudaMemcpyAsync(h->pos_dev, positions, (size_t)batch * 4, cudaMemcpyHostToDevice, st));
    int rc = neon_decoder_step(h, h->tok_dev, h->pos_dev, batch, nullptr, h->next_dev, st);
    if (rc) return rc;
    DCU(h, cudaMemcpyAsync(next_tokens, h->next_dev, (size_t)batch * 4, cudaMemcpyDeviceToHost, st));
    DCU(h, cudaStreamSynchronize(st));
    return NEON_MOE_OK;
}

int neon_decoder_read(neon_decoder_handle* h, const char* name, void* dst, uint64_t bytes) {
    if (!h || !name || !dst) return NEON_MOE_EINVAL;
    const auto& c = h->cfg;
    const size_t B = c.max_batch, H = c.hidden;
    const void* src = nullptr;
    size_t cap = 0;
    if (!strcmp(name, "x")) { src = h->x; cap = B * H * 4; }
    else if (!strcmp(name, "xn")) { src = h->xn; cap = B * H * 2; }
    else if (!strcmp(name, "moe_in")) { src = h->xn2; cap = B * H * 2; }
    else if (!strcmp(name, "moe_out")) { src = h->moe_out; cap = B * H * 4; }
    else if (!strcmp(name, "qkv")) { src = h->qkv; cap = B * (size_t)(c.n_q_heads + 2 * c.n_kv_heads) * 64 * 4; }
    else if (!strcmp(name, "attn")) { src = h->attn; cap = B * (size_t)c.n_q_heads * 64 * 2; }
    else if (!strcmp(name, "logits")) { src = h->logits; cap = B * (size_t)c.vocab * 4; }
    else if (!strcmp(name, "inv_freq")) { src = h->inv_freq; cap = 32 * 4; }
    else return dfail(h, NEON_MOE_EINVAL, "unknown buffer '%s'", name);
    if (bytes > cap) return dfail(h, NEON_MOE_EINVAL, "'%s' holds %zu bytes, %llu asked", name, cap, (unsigned long long)bytes);
    DCU(h, cudaSetDevice(c.device));
    DCU(h, cudaStreamSynchronize(h->last_stream));
    DCU(h, cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost));
    return NEON_MOE_OK;
}

int neon_decoder_set_option(neon_decoder_handle* h, const char* name, int64_t value) {
    if (!h || !name) return NEON_MOE_EINVAL;
    drop_graph(h);
    if (!strcmp(name, "use_graphs")) h->use_graphs = (int)value;
    else if (!strcmp(name, "pdl")) h->pdl = (int)value;
    else if (!strncmp(name, "moe.", 4)) {  // pass an option on to every layer's MoE handle
        for (auto& L : h->layers) {
            int rc = neon_moe_set_option(L.moe, name + 4, value);
            if (rc) return dfail(h, rc, "MoE option: %s", neon_moe_last_error(L.moe));
        }
    }
    else if (!strcmp(name, "stop_after_layer")) h->stop_after = (int)value;
    else return dfail(h, NEON_MOE_EINVAL, "unknown option '%s'", name);
    return NEON_MOE_OK;
}

int neon_decoder_step_bytes(neon_decoder_handle* h, const int32_t* positions_host, int batch, double* bytes3) {
    if (!h || !positions_host || !bytes3) return NEON_MOE_EINVAL;
    const auto& c = h->cfg;
    if (batch < 1 || batch > c.max_batch) return dfail(h, NEON_MOE_EINVAL, "batch %d outside 1..%d", batch, c.max_batch);
    const double H = c.hidden, I = c.inter, QKV = (c.n_q_heads + 2.0 * c.n_kv_heads) * 64, QD = c.n_q_heads * 64.0;
    double dense = (double)c.vocab * H * 2 + batch * H * 2 + H * 2;  // unembedding, embedding rows, final norm
    dense += c.n_layers * ((QKV * H + QKV + H * QD + H + 2 * H + c.n_q_heads) * 2 + (double)c.n_experts * (H + 1) * 2);
    double kv = 0;
    for (int l = 0; l < c.n_layers; ++l)
        for (int b = 0; b < batch; ++b) {
            const int p = positions_host[b];
            const int n = (c.window > 0 && l % 2 == 0) ? std::min(p + 1, c.window) : p + 1;
            kv += (double)n * c.n_kv_heads * 64 * 2 * 2;
        }
    const double per_expert = 2 * I * H / 2 + 2 * I * H / 32 + 2 * I * 2 + H * I / 2 + H * I / 32 + H * 2;
    double moe = 0;
    std::vector<int32_t> count(c.n_experts);
    for (int l = 0; l < c.n_layers; ++l) {
        int n = 0;
        int rc = neon_moe_read_dispatch(h->layers[l].moe, count.data(), nullptr, nullptr, nullptr, &n);
        if (rc) return dfail(h, rc, "layer %d MoE: %s", l, neon_moe_last_error(h->layers[l].moe));
        if (n == 0) continue;
        for (int e = 0; e < c.n_experts; ++e) moe += count[e] > 0 ? per_expert : 0.0;
    }
    bytes3[0] = dense;
    bytes3[1] = kv;
    bytes3[2] = moe;
    return NEON_MOE_OK;
}

}  // extern "C"
