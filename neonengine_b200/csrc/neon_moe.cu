// Host side of libneon_moe.so: the C ABI declared in include/neon_moe.h over the kernels
// in moe_kernels.cuh.  No CPU fallback exists: every compute entry point launches CUDA
// kernels or fails with an error code.
#include "../../include/neon_moe.h"

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <algorithm>
#include <atomic>
#include <string>
#include <vector>

#include "moe_kernels.cuh"
#include "gmm_sm100.cuh"
#include "gmm_pair_sm100.cuh"
#include "ep.cuh"
#include "decode_fused.cuh"
#include "decode_sliced.cuh"
#include "gmm_pair_prefill_sm100.cuh"
#include "mma_rate.cuh"
#include "mma_pair.cuh"

using namespace neon;

namespace {
thread_local std::string g_create_error;

struct DeviceBuf {
    void* p = nullptr;
    size_t bytes = 0;
};
}  // namespace

struct neon_moe_handle {
    neon_moe_config cfg{};
    int n_local = 0, e_lo = 0;
    bool has_weights = false;
    std::string err;
    int64_t launches = 0;
    cudaStream_t last_stream = nullptr;
    cudaStream_t own_stream = nullptr;
    int last_n = 0;
    int n_sms = 148;
    unsigned* route_done = nullptr;  // CTA counter of router_dispatch_kernel
    int fuse_dispatch = 0;          // decode passes: the last router CTA runs the dispatch (measured: no gain over PDL)
    // weights
    uint16_t *router_w = nullptr, *router_b = nullptr, *gu_bias = nullptr, *dn_bias = nullptr;
    uint4 *gu_wq = nullptr, *dn_wq = nullptr;
    uint32_t *gu_sq = nullptr, *dn_sq = nullptr;
    // workspaces
    int32_t *idx = nullptr, *count = nullptr, *offset = nullptr, *perm = nullptr, *inv = nullptr;
    float *route_w = nullptr, *y = nullptr;
    uint16_t *a_hi = nullptr, *a_lo = nullptr;
    int* status = nullptr;
    // tensor-core path: "tc" weights, tensor maps, activation-term planes, token tiles
    int path = 2;                 // 1 = mma.sync kernels, 2 = TMA + tcgen05 block-scaled GEMM
    uint32_t a_tx_bytes = 8192;   // bytes one 128x128 4-bit box adds to its mbarrier
    int max_stages = 0, ctas_per_sm = 1;
    int pdl = 1;                  // programmatic dependent launch between the kernels of a pass
    int tile_override = 0;        // 0 = token-tile size chosen from the batch size; 16 / 32 / 128 force it
    int router_wide_max = 384;    // passes up to this many tokens use the one-CTA-per-token router, which also yields the token
                                  // maxima the stacked-term tiles need (measured 9-13 us faster than the token-blocked router
                                  // plus a separate maxima kernel at 96-256 tokens, equal at 384)
    int graph_max_tokens = 64;    // passes up to this many tokens are replayed from a captured CUDA graph
    int router_mma = 1;           // larger passes route on tensor cores (32 or 128 experts); 0 = the token-blocked CUDA-core router
    int sync_debug = 0;           // synchronise and check after every kernel (slow; names the failing kernel)
    long long* trace = nullptr;
    int trace_which = 0;  // 0 = both products (the down product overwrites), 1 = gate_up only, 2 = down only
    uint8_t *gu_wt = nullptr, *gu_sfa = nullptr, *dn_wt = nullptr, *dn_sfa = nullptr;
    float* x_scale = nullptr;  // per-row scales of the hidden-state terms (stacked mode; the SwiGLU rows use a fixed bound)
    float* x_amax = nullptr;   // largest magnitude per token row
    uint8_t *x_act = nullptr, *a_act = nullptr;  // activation blocks (terms + scales) per (tile, chunk)
    float* a_f32 = nullptr;
    int32_t *tile_expert = nullptr, *tile_row0 = nullptr, *tile_rows = nullptr, *n_tiles = nullptr, *row_tile = nullptr;
    int tile_cap = 0, kp_h = 0, kp_i = 0;
    CUtensorMap tm_gu{}, tm_dn{}, tm_gu2{}, tm_dn2{};  // weight boxes of 128 rows and of 256 rows (two chunks)
    CUtensorMap tm4_gu{}, tm4_dn{}, tm4_gu2{}, tm4_dn2{};  // the same boxes left packed (4-bit in shared memory)
    // one-launch decode pass (T <= 8): router partial sums, partial sums of both products, counters
    int decode_sliced = 0;        // 1 = the one-launch pass runs sliced by intermediate channel (decode_sliced.cuh) where it can; measured no faster
    int decode_fused = 1;         // 1 = passes of at most decode_fused_tokens tokens run as one cooperative kernel
    int decode_max_tokens = 0;    // largest pass the one-launch kernel can serve on this handle (0 = not available)
    int decode_fused_tokens = 1;  // largest pass it serves by default: measured per pass at the gpt-oss-20b shapes, one launch vs
                                  // the multi-kernel path: T=1 36.5 vs 38.7 us, T=2 51 vs 49, T=8 129 vs 79 (more distinct experts per
                                  // CTA run: more rebuilds of the token-operand tiles, longer combine)
    int decode_stall_test = 0;    // test hook: the kernel's first wait expects one arrival too many and must time out
    long long decode_wait_limit = kWaitLimitCycles;
    int32_t *disp_blk_count = nullptr, *disp_blk_base = nullptr, *disp_tile_first = nullptr;  // many-CTA dispatch scratch
    unsigned* disp_done = nullptr;
    int dispatch_multi = 1;       // passes of more than 1024 entries: dispatch on one CTA per 1024 entries (0: one CTA)
    float *dec_router_part = nullptr, *dec_gu_part = nullptr, *dec_dn_part = nullptr;
    float* dec_y_part = nullptr;  // decode_sliced_kernel: [CTA][token][padded hidden] contributions to the output
    int dec_sliced_tokens = 0;    // largest pass decode_sliced_kernel can take (0: unavailable)
    unsigned* dec_counters = nullptr;
    int dec_gu_items_cap = 0, dec_counter_words = 0;
    int pair_ctas = 0;            // CTAs the paired kernel was last launched with (2 x resident clusters)
    // Decode tiles (16 / 32 tokens) on clusters of two CTAs with two-SM MMAs (tcgen05 cta_group::2): 0 never, 1 always,
    // 2 when the pass routes at most kPairMaxEntries entries.  Measured per pass at the gpt-oss shapes, single vs paired
    // (Zipf / uniform routing): T=8 58.8 vs 53.7 / 79.6 vs 72.5 us, T=16 72.7 vs 66.0 / 94.6 vs 87.8, T=64 108.7 vs 99.8 /
    // 116.4 vs 109.0, T=96 121.3 vs 114.4 / 119.5 vs 114.3, T=128 131.7 vs 126.1 / 124.3 vs 124.3, T=160 150.6 vs 147.7 /
    // 133.6 vs 137.2, T=224 175 vs 177.5 / 160 vs 168.
    int pair_mma = 2;
    int pair_prefill = 1;         // 128-token tiles on CTA pairs (two-SM MMAs, each CTA half of the token rows); 0 = one CTA per tile
    int pass_entries = 0;         // routed entries of the pass being launched
    int mxf4_prefill = 0;         // 128-token tiles: 1 = activations quantised to MXFP4, tcgen05.mma.kind::mxf4 (outside the accuracy contract)
    int mx4 = 0;                  // decode tiles: 1 = kind::mxf4 with e2m1 activation terms, 0 = kind::mxf8f6f4 with e4m3 terms
    // expert parallelism: source-side routing/dispatch over all experts, exchange buffers
    ncclComm_t comm = nullptr;
    int n_src = 0, n_cap = 0;     // entries this rank routes (max) / entries it can receive
    int32_t *s_idx = nullptr, *s_count = nullptr, *s_offset = nullptr, *s_perm = nullptr, *s_inv = nullptr;
    int32_t *all_counts_d = nullptr, *row_expert = nullptr, *host_pinned = nullptr;
    float *s_w = nullptr, *yrecv = nullptr, *yback = nullptr, *ones = nullptr;
    uint16_t *xsend = nullptr, *xrecv = nullptr;
    // exchanges by peer stores: the peers' xrecv / yrecv mapped through CUDA IPC
    int ep_peer = 0;                                // 1 = both exchanges are this library's own stores into peer memory
    uint16_t* peer_x[kMaxPeerRanks] = {};
    float* peer_y[kMaxPeerRanks] = {};
    bool peer_mapped[kMaxPeerRanks] = {};
    int32_t *ep_bar_src = nullptr, *ep_bar_dst = nullptr;
    cudaEvent_t ep_ev[6] = {};
    bool ep_timed = false;
    int ep_last_recv = 0;
    int ep_subpasses = 0;              // exchanges the last expert-parallel call needed (1 unless a rank's capacity was exceeded)
    std::vector<int32_t> ep_caps;      // receive capacity (rows) of every rank, gathered by ep_init
    // replay cache: a forward with the same arguments is captured once into a CUDA graph
    struct CachedGraph {
        const void *hidden, *bias, *out, *idx, *w;
        int T, seen, launches;
        cudaGraphExec_t exec;
    };
    std::vector<CachedGraph> graphs;
    int use_graphs = 1;
    // per-stage profiling: 5 events per forward
    bool profiling = false;
    std::vector<cudaEvent_t> events;
    size_t events_used = 0;
    // staging for the host-buffer entry point
    uint16_t* st_hidden = nullptr;
    float *st_out = nullptr, *st_bias = nullptr;
    // second staging set, copy streams and events of the pipelined host-batches call (created on first use)
    uint16_t* st_hidden2 = nullptr;
    float* st_out2 = nullptr;
    cudaStream_t s_in = nullptr, s_out = nullptr;
    cudaEvent_t ev_in[2] = {}, ev_comp[2] = {}, ev_out[2] = {};
};

namespace {

void drop_graphs(neon_moe_handle* h) {
    for (auto& g : h->graphs)
        if (g.exec) cudaGraphExecDestroy(g.exec);
    h->graphs.clear();
}

int fail(neon_moe_handle* h, int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (h) h->err = buf; else g_create_error = buf;
    return code;
}

#define CU(h, call)                                                                          \
    do {                                                                                     \
        cudaError_t e_ = (call);                                                             \
        if (e_ != cudaSuccess)                                                               \
            return fail(h, NEON_MOE_ECUDA, "%s failed: %s", #call, cudaGetErrorString(e_)); \
    } while (0)

// With the sync_debug option: wait for the kernel just launched and name it if it failed.
#define DBG_SYNC(h, st, what)                                                                        \
    do {                                                                                             \
        if ((h)->sync_debug) {                                                                       \
            cudaError_t e_ = cudaStreamSynchronize(st);                                              \
            if (e_ == cudaSuccess) e_ = cudaGetLastError();                                          \
            if (e_ != cudaSuccess) return fail(h, NEON_MOE_ECUDA, "%s: %s", what, cudaGetErrorString(e_)); \
        }                                                                                            \
    } while (0)

// Kernel launch with the programmatic-dependent-launch attribute (when `pdl`): the kernel may be
// scheduled while its predecessor in the stream drains; the kernels call pdl_wait() before they
// touch the predecessor's output.
template <typename... KArgs, typename... Args>
void launch_k(bool pdl, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
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
    cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

template <typename T>
int dev_alloc(neon_moe_handle* h, T** p, size_t count) {
    CU(h, cudaMalloc(reinterpret_cast<void**>(p), count * sizeof(T) + 16));
    return NEON_MOE_OK;
}

void free_all(neon_moe_handle* h) {
    void* ptrs[] = {h->router_w, h->router_b, h->gu_bias, h->dn_bias, h->gu_wq, h->dn_wq, h->gu_sq, h->dn_sq,
                    h->idx, h->count, h->offset, h->perm, h->inv, h->route_w, h->y, h->a_hi, h->a_lo,
                    h->status, h->st_hidden, h->st_out, h->st_bias, h->st_hidden2, h->st_out2, h->gu_wt, h->gu_sfa, h->dn_wt, h->dn_sfa,
                    h->x_act, h->a_act, h->x_scale, h->x_amax, h->a_f32, h->tile_expert, h->tile_row0, h->tile_rows,
                    h->n_tiles, h->row_tile, h->s_idx, h->s_count, h->s_offset, h->s_perm, h->s_inv, h->all_counts_d,
                    h->row_expert, h->s_w, h->yrecv, h->yback, h->ones, h->xsend, h->xrecv,
                    h->disp_blk_count, h->disp_blk_base, h->disp_tile_first, h->disp_done,
                    h->dec_router_part, h->dec_gu_part, h->dec_dn_part, h->dec_y_part, h->dec_counters, h->ep_bar_src, h->ep_bar_dst};
    for (void* p : ptrs)
        if (p) cudaFree(p);
    for (int r = 0; r < kMaxPeerRanks; ++r)
        if (h->peer_mapped[r]) {
            cudaIpcCloseMemHandle(h->peer_x[r]);
            cudaIpcCloseMemHandle(h->peer_y[r]);
        }
    if (h->host_pinned) cudaFreeHost(h->host_pinned);
    for (cudaEvent_t ev : h->ep_ev)
        if (ev) cudaEventDestroy(ev);
    if (h->comm && nccl_api().ok) nccl_api().CommDestroy(h->comm);
    for (auto& g : h->graphs)
        if (g.exec) cudaGraphExecDestroy(g.exec);
    if (h->own_stream) cudaStreamDestroy(h->own_stream);
    if (h->s_in) cudaStreamDestroy(h->s_in);
    if (h->s_out) cudaStreamDestroy(h->s_out);
    for (int b = 0; b < 2; ++b)
        for (cudaEvent_t e : {h->ev_in[b], h->ev_comp[b], h->ev_out[b]})
            if (e) cudaEventDestroy(e);
    for (cudaEvent_t ev : h->events) cudaEventDestroy(ev);
}

constexpr size_t kMaxProfiledForwards = 4096;
constexpr int kMaxDevicesAttr = 64;

// Records the next profiling event on `st` (no-op unless profiling is on and room is left).
void mark(neon_moe_handle* h, cudaStream_t st, bool active) {
    if (!active) return;
    if (h->events_used == h->events.size()) {
        cudaEvent_t ev;
        if (cudaEventCreate(&ev) != cudaSuccess) return;
        h->events.push_back(ev);
    }
    cudaEventRecord(h->events[h->events_used++], st);
}

// Frees device buffers on scope exit (temporaries of the loaders, also on their error returns).
struct ScopedDeviceFree {
    void* p[2] = {nullptr, nullptr};
    ~ScopedDeviceFree() {
        for (void* q : p)
            if (q) cudaFree(q);
    }
};

void free_mma16(neon_moe_handle* h) {
    for (void** p : {(void**)&h->gu_wq, (void**)&h->dn_wq, (void**)&h->gu_sq, (void**)&h->dn_sq}) {
        if (*p) cudaFree(*p);
        *p = nullptr;
    }
}

// Builds the mma.sync kernels' weight layout from the tensor-core layout the handle holds (only
// "path" 1 and neon_moe_forward_static read it, so it is not built - and takes no memory - until
// one of them is asked for).  Allocates; scale bytes above 128 are refused here and only here.
int ensure_mma16(neon_moe_handle* h) {
    if (h->gu_wq) return NEON_MOE_OK;
    if (!h->gu_wt || !h->dn_wt) return fail(h, NEON_MOE_ESTATE, "no weights loaded");
    CU(h, cudaSetDevice(h->cfg.device));
    const int E = h->n_local, H = h->cfg.hidden, I = h->cfg.inter;
    struct Job { const uint8_t *wt, *sfa; int rows, K, gate_up; uint4** wq; uint32_t** sq; };
    const Job jobs[2] = {{h->gu_wt, h->gu_sfa, 2 * I, H, 1, &h->gu_wq, &h->gu_sq}, {h->dn_wt, h->dn_sfa, H, I, 0, &h->dn_wq, &h->dn_sq}};
    int* flag = h->status + 3;  // fourth word of the status block
    CU(h, cudaMemset(flag, 0, sizeof(int)));
    for (const Job& j : jobs) {
        const int tiles = j.rows / 16, nbp = j.K / 64;
        int rc = dev_alloc(h, j.wq, (size_t)E * tiles * nbp * 32);
        if (!rc) rc = dev_alloc(h, j.sq, (size_t)E * tiles * nbp * 8);
        if (rc) { free_mma16(h); return rc; }
        repack_mma16_from_tc_kernel<<<148 * 8, 256>>>(j.wt, j.sfa, E, j.rows, j.K, j.gate_up, *j.wq, *j.sq, flag);
        h->launches++;
    }
    int bad = 0;
    cudaError_t ce = cudaMemcpy(&bad, flag, sizeof(int), cudaMemcpyDeviceToHost);
    if (ce == cudaSuccess) ce = cudaGetLastError();
    if (ce != cudaSuccess) { free_mma16(h); return fail(h, NEON_MOE_ECUDA, "building the mma.sync weight layout failed: %s", cudaGetErrorString(ce)); }
    if (bad) {
        free_mma16(h);
        return fail(h, NEON_MOE_EINVAL, "the mma.sync kernels (path 1, neon_moe_forward_static) do not support MXFP4 scale bytes above 128 "
                                        "(scale > 2); the tensor-core path has no such limit");
    }
    return NEON_MOE_OK;
}

int copy_in(neon_moe_handle* h, uint16_t** dst, const void* src, size_t count, int on_device) {
    if (!*dst) {
        int rc = dev_alloc(h, dst, count);
        if (rc) return rc;
    }
    CU(h, cudaMemcpy(*dst, src, count * 2, on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice));
    return NEON_MOE_OK;
}


// ---- tensor-core path helpers -----------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

// 2-D map over packed 4-bit weight boxes: rows of 128 nibbles (64 B), box = 128 x 128, expanded
// by TMA to one byte per nibble (16 nibbles + 8 pad bytes per 16 B) with 128-byte swizzle.
int make_weight_map(neon_moe_handle* h, CUtensorMap* map, void* base, uint64_t n_rows, uint32_t box_rows, bool packed) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail(h, NEON_MOE_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {128, n_rows};
    cuuint64_t strides[1] = {64};
    cuuint32_t box[2] = {128, box_rows};
    cuuint32_t estr[2] = {1, 1};
    // packed: nibbles stay packed (64-byte rows, 64-byte swizzle) for kind::mxf4
    CUresult r = fn(map, packed ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN8B : CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 2, base, dims,
                    strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    packed ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(h, NEON_MOE_ECUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return NEON_MOE_OK;
}

// 2-D map over the scale atoms of the weight boxes (512 bytes each, as 128 32-bit words): box = one or two atoms.
int make_atom_map(neon_moe_handle* h, CUtensorMap* map, const void* base, uint64_t n_atoms, uint32_t box_atoms) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail(h, NEON_MOE_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {128, n_atoms};
    cuuint64_t strides[1] = {512};
    cuuint32_t box[2] = {128, box_atoms};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(h, NEON_MOE_ECUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return NEON_MOE_OK;
}

// Upload (when needed) and re-tile one MXFP4 matrix set into the "tc" format.
int load_matrix_tc(neon_moe_handle* h, const uint8_t* blocks, const uint8_t* scales, int rows, int K, int gate_up,
                   int on_device, uint8_t** wt, uint8_t** sfa, CUtensorMap* map, CUtensorMap* map2, CUtensorMap* map4,
                   CUtensorMap* map4_2) {
    const int E = h->n_local;
    const size_t nb = (size_t)E * rows * (K / 2), ns = (size_t)E * rows * (K / 32);
    const uint8_t *d_blocks = blocks, *d_scales = scales;
    ScopedDeviceFree tmp;
    if (!on_device) {
        CU(h, cudaMalloc(&tmp.p[0], nb));
        CU(h, cudaMalloc(&tmp.p[1], ns));
        CU(h, cudaMemcpy(tmp.p[0], blocks, nb, cudaMemcpyHostToDevice));
        CU(h, cudaMemcpy(tmp.p[1], scales, ns, cudaMemcpyHostToDevice));
        d_blocks = static_cast<const uint8_t*>(tmp.p[0]);
        d_scales = static_cast<const uint8_t*>(tmp.p[1]);
    }
    const int Kp = round_up_int(K, kChunkK), m_tiles = (rows + 127) / 128, n_chunks = Kp / kChunkK;
    if (!*wt) {
        int rc = dev_alloc(h, wt, (size_t)E * m_tiles * n_chunks * 8192);
        if (rc) return rc;
        rc = dev_alloc(h, sfa, (size_t)E * m_tiles * n_chunks * 512);
        if (rc) return rc;
    }
    repack_tc_kernel<<<148 * 8, 256>>>(d_blocks, d_scales, E, rows, K, gate_up, *wt, *sfa);
    h->launches++;
    CU(h, cudaGetLastError());
    CU(h, cudaDeviceSynchronize());
    const uint64_t nrows = (uint64_t)E * m_tiles * n_chunks * 128;
    int rc;
    if ((rc = make_weight_map(h, map, *wt, nrows, 128, false)) || (rc = make_weight_map(h, map2, *wt, nrows, 256, false)) ||
        (rc = make_weight_map(h, map4, *wt, nrows, 128, true)) || (rc = make_weight_map(h, map4_2, *wt, nrows, 256, true)))
        return rc;
    return NEON_MOE_OK;
}

// Token-tile size: small and mid-size batches use 32-token tiles (16 up to 16 tokens) with the
// activation terms stacked along N (one MMA per k-block reads the weight tile once); from 225 tokens
// on, 128-token tiles with the terms as successive MMAs (on CTA pairs).  Measured per pass at the gpt-oss
// shapes (32 vs 128-token tiles): T=96 116 vs 149 us, T=128 123 vs 149, T=192 143 vs 158, T=256 173 vs 163,
// T=320 218 vs 181, T=384 232 vs 191, T=512 306 vs 217, T=768 409 vs 259.  (With the one-CTA prefill kernel
// the crossing was at 385 tokens.)
constexpr int kSmallTileMaxTokens = 224;
int tile_tokens_for(int T) { return T <= 16 ? 16 : (T <= kSmallTileMaxTokens ? 32 : 128); }
int tile_tokens_for(const neon_moe_handle* h, int T) { return h->tile_override ? h->tile_override : tile_tokens_for(T); }

template <int BN, int TERMS, bool GATE_UP, bool STACK, int KC, bool MX4 = false>
int launch_gmm_one(neon_moe_handle* h, const CUtensorMap& tm1, const CUtensorMap& tm2, GmmParams p, cudaStream_t st) {
    using L = GmmSmem<BN, TERMS, STACK, KC, MX4>;
    static bool configured[kMaxDevicesAttr] = {};
    auto kern = gmm_bs_kernel<BN, TERMS, GATE_UP, STACK, KC, MX4>;
    if (!configured[h->cfg.device]) {
        CU(h, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::smem_bytes(L::kStages)));
        configured[h->cfg.device] = true;
    }
    int stages = L::kStages, ctas = h->n_sms;
    if (h->ctas_per_sm == 2) {  // two half-size CTAs per SM when at least two stages fit in half the shared memory
        const int half = (110 * 1024 - 2048) / L::kStage;
        if (half >= 2 && L::tmem_cols(half) <= 256) {
            stages = std::min(stages, half);
            ctas = 2 * h->n_sms;
        }
    }
    if (h->max_stages > 0) stages = std::max(2, std::min(stages, h->max_stages));
    p.stages = stages;
    p.tmem_cols = L::tmem_cols(stages);
    launch_k(h->pdl != 0, kern, dim3(ctas), dim3(192), (size_t)L::smem_bytes(stages), st, KC == 2 ? tm2 : tm1, tm1, p);
    h->launches++;
    return NEON_MOE_OK;
}

// The paired kernel for decode tiles (gmm_pair_sm100.cuh): clusters of two CTAs, grid = an even number of CTAs.
template <int BN, int TERMS, bool GATE_UP>
int launch_gmm_pair(neon_moe_handle* h, const CUtensorMap& tm1, const CUtensorMap& tm2, GmmParams p, cudaStream_t st) {
    using L = PairSmem<BN, TERMS>;
    static bool configured[kMaxDevicesAttr] = {};
    auto kern = gmm_pair_kernel<BN, TERMS, GATE_UP>;
    CUtensorMap ts1, ts2;  // scale atoms, fetched by TMA so that the peer's copies can report to the leader's barrier
    const uint64_t n_atoms = (uint64_t)h->n_local * p.m_tiles * p.n_chunks;
    int rc;
    if ((rc = make_atom_map(h, &ts1, p.sfa, n_atoms, 1)) || (rc = make_atom_map(h, &ts2, p.sfa, n_atoms, 2))) return rc;
    if (!configured[h->cfg.device]) {
        CU(h, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::smem_bytes(L::kStages)));
        configured[h->cfg.device] = true;
    }
    int stages = L::kStages;
    if (h->max_stages > 0) stages = std::max(2, std::min(stages, h->max_stages));
    p.stages = stages;
    p.tmem_cols = L::tmem_cols(stages);
    // The kernel is persistent: a pair that cannot be resident with the others would run after them and double the
    // time.  Pairs need two SMs of one TPC, so fewer than n_sms / 2 may fit: ask the runtime how many do.
    static int max_pairs[kMaxDevicesAttr] = {};
    if (!max_pairs[h->cfg.device]) {
        cudaLaunchConfig_t q{};
        q.gridDim = dim3(h->n_sms & ~1);
        q.blockDim = dim3(192);
        q.dynamicSmemBytes = (size_t)L::smem_bytes(L::kStages);
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &q) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            n = h->n_sms / 2;
        }
        max_pairs[h->cfg.device] = n;
    }
    const int pairs = std::min(max_pairs[h->cfg.device], h->n_sms / 2);
    launch_k(h->pdl != 0, kern, dim3(2 * pairs), dim3(192), (size_t)L::smem_bytes(stages), st, tm2, tm1, ts2, ts1, p);
    h->launches++;
    h->pair_ctas = 2 * pairs;
    return NEON_MOE_OK;
}

// 128-token (prefill) tiles on CTA pairs (gmm_pair_prefill_sm100.cuh).
template <int TERMS, bool GATE_UP>
int launch_gmm_pair_prefill(neon_moe_handle* h, const CUtensorMap& tm1, GmmParams p, cudaStream_t st) {
    using L = PairPrefillSmem<TERMS>;
    static bool configured[kMaxDevicesAttr] = {};
    auto kern = gmm_pair_prefill_kernel<TERMS, GATE_UP>;
    CUtensorMap ts1;  // scale atoms, fetched by TMA so that the peer's copies can report to the leader's barrier
    int rc = make_atom_map(h, &ts1, p.sfa, (uint64_t)h->n_local * p.m_tiles * p.n_chunks, 1);
    if (rc) return rc;
    if (!configured[h->cfg.device]) {
        CU(h, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::smem_bytes(L::kStages)));
        configured[h->cfg.device] = true;
    }
    int stages = L::kStages;
    if (h->max_stages > 0) stages = std::max(2, std::min(stages, h->max_stages));
    p.stages = stages;
    p.tmem_cols = L::tmem_cols(stages);
    static int max_pairs[kMaxDevicesAttr] = {};
    if (!max_pairs[h->cfg.device]) {  // pairs need two SMs of one TPC: ask the runtime how many clusters can be resident
        cudaLaunchConfig_t q{};
        q.gridDim = dim3(h->n_sms & ~1);
        q.blockDim = dim3(192);
        q.dynamicSmemBytes = (size_t)L::smem_bytes(L::kStages);
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &q) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            n = h->n_sms / 2;
        }
        max_pairs[h->cfg.device] = n;
    }
    const int pairs = std::min(max_pairs[h->cfg.device], h->n_sms / 2);
    launch_k(h->pdl != 0, kern, dim3(2 * pairs), dim3(192), (size_t)L::smem_bytes(stages), st, tm1, ts1, p);
    h->launches++;
    h->pair_ctas = 2 * pairs;
    return NEON_MOE_OK;
}

// e4m3 terms of the fp32 SwiGLU output fed to the down product of 128-token (prefill) tiles.  Each
// term carries ~4 significant bits.  On the paired kernel the product is bound by tensor-core work, which
// is proportional to the term count: three terms measured 0.44 ms against 0.57 ms with four at T=4096, with
// max-abs 2.2e-3 / mean-rel 1.5e-5 against the oracle (four terms: 1.2e-3 / 6.6e-6; the contract is 2e-2 /
// 5e-3).  The decode tiles keep four: they are bound by the weight stream, not by tensor work.
constexpr int kDownTermsPrefill = 3;
constexpr int kDecodeSmemBytes = 227 * 1024;  // everything an SM has: what the token-operand tiles leave goes to weight stages
constexpr int kPairMaxEntries = 128 * 4;  // passes of up to 128 tokens at top-4 take the paired kernel
constexpr int kMx4Terms = 6;  // e2m1 terms per activation value on the packed 4-bit path

template <int TERMS, bool GATE_UP>
int launch_gmm(neon_moe_handle* h, int tile_tokens, const CUtensorMap& tm1, const CUtensorMap& tm2, const GmmParams& p,
               cudaStream_t st) {
    if (tile_tokens <= 32 && h->mx4) {  // packed 4-bit operands, kMx4Terms e2m1 terms per activation
        const CUtensorMap& q1 = GATE_UP ? h->tm4_gu : h->tm4_dn;
        const CUtensorMap& q2 = GATE_UP ? h->tm4_gu2 : h->tm4_dn2;
        if (tile_tokens == 16) return launch_gmm_one<16, kMx4Terms, GATE_UP, true, 2, true>(h, q1, q2, p, st);
        return launch_gmm_one<32, kMx4Terms, GATE_UP, true, 2, true>(h, q1, q2, p, st);
    }
    if constexpr (TERMS % 2 == 0) {  // the paired decode kernel splits the stacked terms between its two CTAs
        if (tile_tokens <= 32 && (h->pair_mma == 1 || (h->pair_mma == 2 && h->pass_entries <= kPairMaxEntries))) {
            if (tile_tokens == 16) return launch_gmm_pair<16, TERMS, GATE_UP>(h, tm1, tm2, p, st);
            return launch_gmm_pair<32, TERMS, GATE_UP>(h, tm1, tm2, p, st);
        }
    }
    if (tile_tokens == 16) return launch_gmm_one<16, TERMS, GATE_UP, true, 2>(h, tm1, tm2, p, st);
    if (tile_tokens == 32) return launch_gmm_one<32, TERMS, GATE_UP, true, 2>(h, tm1, tm2, p, st);
    if (h->mxf4_prefill)  // MXFP4-quantised activations, both operands packed 4-bit, two chunks per stage
        return launch_gmm_one<128, 1, GATE_UP, false, 2, true>(h, GATE_UP ? h->tm4_gu : h->tm4_dn, GATE_UP ? h->tm4_gu2 : h->tm4_dn2, p, st);
    if (h->pair_prefill) return launch_gmm_pair_prefill<TERMS, GATE_UP>(h, tm1, p, st);
    return launch_gmm_one<128, TERMS, GATE_UP, false, 1>(h, tm1, tm2, p, st);
}

template <int TERMS, bool FROM_BF16>
void launch_split(neon_moe_handle* h, int tile_tokens, const TileList& tl, const void* src, int K, int n, int top_k,
                  const float* amax, float amax_const, uint8_t* act, float* row_scale, cudaStream_t st) {
    const int n_chunks = round_up_int(K, kChunkK) / kChunkK;
    if (tile_tokens > 32 && h->mxf4_prefill)
        launch_k(h->pdl != 0, quant_rows_mxfp4_kernel<FROM_BF16>, dim3((n * n_chunks + 7) / 8), dim3(256), 0, st, src, h->perm, top_k, K, n,
                 tl.row_tile, tl.row0, act);
    else if (tile_tokens <= 32 && h->mx4)
        launch_k(h->pdl != 0, split_rows_fp4_kernel<kMx4Terms, FROM_BF16>, dim3((n * n_chunks + 7) / 8), dim3(256), 0, st, src,
                 h->perm, top_k, K, n, tl.row_tile, tl.row0, tl.rows, tile_tokens, amax, amax_const, act, row_scale);
    else if (tile_tokens <= 32)
        launch_k(h->pdl != 0, split_rows_stacked_kernel<TERMS, FROM_BF16>, dim3((n * n_chunks + 7) / 8), dim3(256), 0, st, src,
                 h->perm, top_k, K, n, tl.row_tile, tl.row0, tl.rows, tile_tokens, amax, amax_const, act, row_scale);
    else
        launch_k(h->pdl != 0, split_rows_kernel<TERMS, FROM_BF16, false>,
                 dim3((n * ((n_chunks + kSplitChunksPerWarp - 1) / kSplitChunksPerWarp) + 7) / 8), dim3(256), 0, st, src,
                 h->perm, top_k, K, n, tl.row_tile, tl.row0, tl.rows, tile_tokens, act);
    h->launches++;
}

template <bool GATE_UP>
void launch_expert(neon_moe_handle* h, const ExpertParams& p, int T, cudaStream_t st) {
    constexpr int WARPS = 4;
    dim3 grid((p.tiles + WARPS - 1) / WARPS, h->n_local), block(32 * WARPS);
    if (T <= 8) expert_mma_kernel<1, GATE_UP, WARPS><<<grid, block, 0, st>>>(p);
    else if (T <= 16) expert_mma_kernel<2, GATE_UP, WARPS><<<grid, block, 0, st>>>(p);
    else if (T <= 32) expert_mma_kernel<4, GATE_UP, WARPS><<<grid, block, 0, st>>>(p);
    else expert_mma_kernel<8, GATE_UP, WARPS><<<grid, block, 0, st>>>(p);
    h->launches++;
}

}  // namespace

extern "C" {

const char* neon_moe_version(void) { return "neon_moe 0.1 (sm_100a)"; }

int neon_moe_mma_rate(int device, int kind, int n, int chunks, double* ms, int64_t* cycles) {
    if (!ms || !cycles || kind < 0 || kind > 3 || n < 16 || n > 256 || n % 16 || chunks < 1 || chunks > (1 << 20))
        return NEON_MOE_EINVAL;
    int n_dev = 0, sms = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || device < 0 || device >= n_dev || cudaSetDevice(device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) {
        cudaGetLastError();
        return NEON_MOE_ECUDA;
    }
    const size_t smem = 16384 + 32768 + 512 + 1024;
    MmaRateOut* d_out = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    int rc = NEON_MOE_ECUDA;
    MmaRateOut host{};
    float elapsed = 0.f;
    if (cudaMalloc(&d_out, sizeof(MmaRateOut)) != cudaSuccess || cudaMemset(d_out, 0, sizeof(MmaRateOut)) != cudaSuccess ||
        cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess ||
        cudaFuncSetAttribute(mma_rate_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
        cudaFuncSetAttribute(mma_rate_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        goto out;
    for (int rep = 0; rep < 2; ++rep) {  // the first launch warms up
        cudaEventRecord(e0, nullptr);
        if (kind & 1) mma_rate_kernel<true><<<sms, 128, smem>>>(n, chunks, kind >> 1, d_out);
        else mma_rate_kernel<false><<<sms, 128, smem>>>(n, chunks, kind >> 1, d_out);
        cudaEventRecord(e1, nullptr);
        if (cudaEventSynchronize(e1) != cudaSuccess || cudaGetLastError() != cudaSuccess) goto out;
    }
    if (cudaEventElapsedTime(&elapsed, e0, e1) != cudaSuccess ||
        cudaMemcpy(&host, d_out, sizeof host, cudaMemcpyDeviceToHost) != cudaSuccess)
        goto out;
    *ms = elapsed;
    *cycles = host.cycles;
    rc = host.status ? NEON_MOE_EDEVICE : NEON_MOE_OK;
out:
    cudaGetLastError();
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    cudaFree(d_out);
    return rc;
}

int neon_moe_tma_rate(int device, int packed, int stages, int64_t buffer_bytes, int loads, double* ms, int64_t* cycles) {
    if (!ms || !cycles || stages < 1 || stages > (packed ? 8 : 6) || buffer_bytes < (1 << 20) || buffer_bytes > (int64_t(8) << 30) || loads < 1 ||
        loads > (1 << 22))
        return NEON_MOE_EINVAL;
    int n_dev = 0, sms = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || device < 0 || device >= n_dev || cudaSetDevice(device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) {
        cudaGetLastError();
        return NEON_MOE_ECUDA;
    }
    const int n_pairs = (int)(buffer_bytes / 16384);
    const int stage_bytes = packed ? 16384 : 32768;
    const size_t smem = (size_t)stages * stage_bytes + 1024;
    uint8_t* buf = nullptr;
    TmaRateOut* d_out = nullptr;
    TmaRateOut host{};
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    CUtensorMap tm;
    float elapsed = 0.f;
    int rc = NEON_MOE_ECUDA;
    if (cudaMalloc(&buf, (size_t)n_pairs * 16384) != cudaSuccess || cudaMemset(buf, 0x22, (size_t)n_pairs * 16384) != cudaSuccess ||
        cudaMalloc(&d_out, sizeof(TmaRateOut)) != cudaSuccess || cudaMemset(d_out, 0, sizeof(TmaRateOut)) != cudaSuccess ||
        cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess ||
        cudaFuncSetAttribute(tma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
        make_weight_map(nullptr, &tm, buf, (uint64_t)n_pairs * 256, 256, packed != 0) != NEON_MOE_OK)
        goto out;
    for (int rep = 0; rep < 2; ++rep) {  // the first launch warms up (and brings a small buffer into L2)
        cudaEventRecord(e0, nullptr);
        // both maps report a box pair's 16 KB of global memory to the barrier (the expanding one writes 32 KB of shared memory)
        tma_rate_kernel<<<sms, 32, smem>>>(tm, n_pairs, loads, stages, 16384u, stage_bytes, d_out);
        cudaEventRecord(e1, nullptr);
        if (cudaEventSynchronize(e1) != cudaSuccess || cudaGetLastError() != cudaSuccess) goto out;
    }
    if (cudaEventElapsedTime(&elapsed, e0, e1) != cudaSuccess ||
        cudaMemcpy(&host, d_out, sizeof host, cudaMemcpyDeviceToHost) != cudaSuccess)
        goto out;
    *ms = elapsed;
    *cycles = host.cycles;
    rc = host.status ? NEON_MOE_EDEVICE : NEON_MOE_OK;
out:
    cudaGetLastError();
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    cudaFree(d_out);
    cudaFree(buf);
    return rc;
}

int neon_moe_mma_pair_probe(int device, int n, int chunks, float* d32, uint32_t* tmem_addr2, int64_t* cycles) {
    if (!d32 || !tmem_addr2 || !cycles || n < 32 || n > 64 || n % 32 || chunks < 1 || chunks > (1 << 16)) return NEON_MOE_EINVAL;  // 128 columns of tensor memory: accumulator + scale atoms
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || device < 0 || device >= n_dev || cudaSetDevice(device) != cudaSuccess) {
        cudaGetLastError();
        return NEON_MOE_ECUDA;
    }
    const size_t smem = 16384 + 16384 + 512 + 1024;
    MmaPairOut* d_out = nullptr;
    MmaPairOut host{};
    int rc = NEON_MOE_ECUDA;
    if (cudaMalloc(&d_out, sizeof(MmaPairOut)) != cudaSuccess || cudaMemset(d_out, 0, sizeof(MmaPairOut)) != cudaSuccess ||
        cudaFuncSetAttribute(mma_pair_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(d_out);
        return rc;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2);       // one CTA pair
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, mma_pair_probe_kernel, n, chunks, d_out) == cudaSuccess && cudaDeviceSynchronize() == cudaSuccess &&
        cudaMemcpy(&host, d_out, sizeof host, cudaMemcpyDeviceToHost) == cudaSuccess) {
        memcpy(d32, host.d, sizeof host.d);
        tmem_addr2[0] = host.tmem_addr[0];
        tmem_addr2[1] = host.tmem_addr[1];
        *cycles = host.cycles;
        rc = host.status ? NEON_MOE_EDEVICE : NEON_MOE_OK;
    }
    cudaGetLastError();
    cudaFree(d_out);
    return rc;
}

const char* neon_moe_last_error(const neon_moe_handle* h) { return h ? h->err.c_str() : g_create_error.c_str(); }

int64_t neon_moe_launch_count(const neon_moe_handle* h) { return h ? h->launches : 0; }

int neon_moe_pair_ctas(const neon_moe_handle* h) { return h ? h->pair_ctas : 0; }

int neon_moe_create(const neon_moe_config* cfg, neon_moe_handle** out) {
    if (!cfg || !out) return fail(nullptr, NEON_MOE_EINVAL, "null argument");
    *out = nullptr;
    if (cfg->hidden <= 0 || cfg->hidden % 64 || cfg->inter <= 0 || cfg->inter % 64)
        return fail(nullptr, NEON_MOE_EINVAL, "hidden and inter must be positive multiples of 64");
    if (cfg->n_experts <= 0 || cfg->n_experts > kMaxExperts || cfg->top_k <= 0 || cfg->top_k > kMaxTopK ||
        cfg->top_k > cfg->n_experts)
        return fail(nullptr, NEON_MOE_EINVAL, "need 1 <= top_k <= min(8, n_experts) and n_experts <= 256");
    if (cfg->ep_size <= 0 || cfg->ep_rank < 0 || cfg->ep_rank >= cfg->ep_size || cfg->n_experts % cfg->ep_size)
        return fail(nullptr, NEON_MOE_EINVAL, "bad expert-parallel rank/size");
    if (cfg->max_tokens <= 0) return fail(nullptr, NEON_MOE_EINVAL, "max_tokens must be positive");
    if (!(cfg->swiglu_limit > 0.f) || !(cfg->swiglu_limit < 1e15f))
        return fail(nullptr, NEON_MOE_EINVAL, "swiglu_limit must be positive and finite");
    int ndev = 0;
    cudaError_t ce = cudaGetDeviceCount(&ndev);
    if (ce != cudaSuccess || ndev == 0)
        return fail(nullptr, NEON_MOE_ECUDA, "no CUDA device: %s", cudaGetErrorString(ce));
    if (cfg->device < 0 || cfg->device >= ndev) return fail(nullptr, NEON_MOE_EINVAL, "bad device ordinal");
    neon_moe_handle* h = new (std::nothrow) neon_moe_handle;
    if (!h) return fail(nullptr, NEON_MOE_EINVAL, "out of host memory");
    h->cfg = *cfg;
    h->n_local = cfg->n_experts / cfg->ep_size;
    h->e_lo = cfg->ep_rank * h->n_local;
    auto bail = [&](int rc) {
        g_create_error = h->err;
        free_all(h);
        delete h;
        return rc;
    };
    if (cudaSetDevice(cfg->device) != cudaSuccess) return bail(fail(h, NEON_MOE_ECUDA, "cudaSetDevice failed"));
    // entries the local expert pass may see: this rank's own when alone; with expert parallelism
    // up to twice the per-rank average (all ranks route max_tokens tokens), beyond which a pass fails
    h->n_src = cfg->max_tokens * cfg->top_k;
    h->n_cap = cfg->ep_size > 1 ? 2 * h->n_src : h->n_src;
    const size_t n = (size_t)h->n_cap;
    int rc = 0;
    if ((rc = dev_alloc(h, &h->idx, n)) || (rc = dev_alloc(h, &h->route_w, n)) ||
        (rc = dev_alloc(h, &h->count, (size_t)h->n_local)) || (rc = dev_alloc(h, &h->offset, (size_t)h->n_local + 1)) ||
        (rc = dev_alloc(h, &h->perm, n)) || (rc = dev_alloc(h, &h->inv, n)) ||
        (rc = dev_alloc(h, &h->a_hi, n * cfg->inter)) || (rc = dev_alloc(h, &h->a_lo, n * cfg->inter)) ||
        (rc = dev_alloc(h, &h->y, n * cfg->hidden)) || (rc = dev_alloc(h, &h->status, (size_t)4)) ||
        (rc = dev_alloc(h, &h->st_hidden, (size_t)cfg->max_tokens * cfg->hidden)) ||
        (rc = dev_alloc(h, &h->st_out, (size_t)cfg->max_tokens * cfg->hidden)) ||
        (rc = dev_alloc(h, &h->st_bias, (size_t)cfg->n_experts)))
        return bail(rc);
    {
        cudaDeviceProp prop;
        if (cudaGetDeviceProperties(&prop, cfg->device) != cudaSuccess)
            return bail(fail(h, NEON_MOE_ECUDA, "cudaGetDeviceProperties failed"));
        h->n_sms = prop.multiProcessorCount;
        if (prop.major != 10) h->path = 1;  // tcgen05 needs sm_100
    }
    h->kp_h = round_up_int(cfg->hidden, kChunkK);
    h->kp_i = round_up_int(cfg->inter, kChunkK);
    h->tile_cap = h->n_local + (int)(n / 16) + 2;
    const size_t nch_h = h->kp_h / kChunkK, nch_i = h->kp_i / kChunkK;
    size_t x_bytes = 0, a_bytes = 0;  // worst case over the three token-tile sizes
    for (int tt : {16, 32, 128}) {
        const size_t tiles = (size_t)h->n_local + n / tt + 1;
        x_bytes = std::max(x_bytes, tiles * nch_h * act_block_bytes(2, tt, tt <= 32));
        a_bytes = std::max(a_bytes, tiles * nch_i * act_block_bytes(4, tt, tt <= 32));
        if (tt <= 32) {
            x_bytes = std::max(x_bytes, tiles * nch_h * act4_block_bytes(kMx4Terms, tt));
            a_bytes = std::max(a_bytes, tiles * nch_i * act4_block_bytes(kMx4Terms, tt));
        }
    }
    if ((rc = dev_alloc(h, &h->x_act, x_bytes)) || (rc = dev_alloc(h, &h->a_act, a_bytes)) ||
        (rc = dev_alloc(h, &h->x_scale, n)) || (rc = dev_alloc(h, &h->x_amax, n)) ||
        (rc = dev_alloc(h, &h->a_f32, n * cfg->inter)) || (rc = dev_alloc(h, &h->tile_expert, (size_t)h->tile_cap)) ||
        (rc = dev_alloc(h, &h->tile_row0, (size_t)h->tile_cap)) || (rc = dev_alloc(h, &h->tile_rows, (size_t)h->tile_cap)) ||
        (rc = dev_alloc(h, &h->n_tiles, (size_t)4)) || (rc = dev_alloc(h, &h->row_tile, n)))
        return bail(rc);
    {   // the many-CTA dispatch of prefill-sized passes: per-chunk expert counts and write positions
        // (sized for all experts: the sender's sort of expert parallelism runs over the global expert ids)
        const size_t blocks = (std::max(n, (size_t)cfg->max_tokens * cfg->top_k) + 1023) / 1024;
        if ((rc = dev_alloc(h, &h->disp_blk_count, blocks * cfg->n_experts)) || (rc = dev_alloc(h, &h->disp_blk_base, blocks * cfg->n_experts)) ||
            (rc = dev_alloc(h, &h->disp_tile_first, (size_t)cfg->n_experts + 1)) || (rc = dev_alloc(h, &h->disp_done, (size_t)4)))
            return bail(rc);
        if (cudaMemset(h->disp_done, 0, 16) != cudaSuccess) return bail(fail(h, NEON_MOE_ECUDA, "cudaMemset failed"));
    }
    // one-launch decode pass: needs sm_100, one GPU holding all experts, at most 32 (token, slot) entries
    if (h->path == 2 && cfg->ep_size == 1 && cfg->n_experts <= h->n_sms && cfg->top_k <= kDecMaxEntries &&
        h->kp_h / kChunkK <= kDecCacheChunks && h->kp_i / kChunkK <= kDecCacheChunks) {
        const int t_dec = std::min({cfg->max_tokens, kDecMaxTok, kDecMaxEntries / cfg->top_k});
        const int exp_max = std::min(cfg->n_experts, t_dec * cfg->top_k);
        const int gu_tiles = 2 * cfg->inter / 128, dn_tiles = (cfg->hidden + 127) / 128;
        h->dec_gu_items_cap = exp_max * gu_tiles;
        h->dec_counter_words = 4 + 256 + 4 * h->dec_gu_items_cap + dn_tiles;
        if ((rc = dev_alloc(h, &h->dec_router_part, (size_t)kDecMaxTok * cfg->n_experts * kDecMaxSlices)) ||
            (rc = dev_alloc(h, &h->dec_gu_part, (size_t)h->dec_gu_items_cap * kDecParts * 1024)) ||
            (rc = dev_alloc(h, &h->dec_dn_part, (size_t)exp_max * dn_tiles * kDecParts * 1024)) ||
            (rc = dev_alloc(h, &h->dec_counters, (size_t)h->dec_counter_words)))
            return bail(rc);
        if (cudaMemset(h->dec_router_part, 0, (size_t)kDecMaxTok * cfg->n_experts * kDecMaxSlices * 4) != cudaSuccess ||
            cudaMemset(h->dec_counters, 0, (size_t)h->dec_counter_words * 4) != cudaSuccess)
            return bail(fail(h, NEON_MOE_ECUDA, "cudaMemset failed"));
        int coop = 0;
        cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, cfg->device);
        h->decode_max_tokens = coop ? t_dec : 0;
        // the channel-sliced variant: T <= 4, hidden a multiple of 4, at least 3 weight stages next to the output accumulator
        int t2 = std::min(t_dec, kDec2MaxTok);
        while (t2 > 0 && dec2_stages(t2, dn_tiles, kDecodeSmemBytes) < 3) --t2;
        if (coop && t2 > 0 && cfg->hidden % 4 == 0 && cfg->inter % 64 == 0) {
            if ((rc = dev_alloc(h, &h->dec_y_part, (size_t)h->n_sms * t2 * dn_tiles * 128))) return bail(rc);
            h->dec_sliced_tokens = t2;
        }
    }
    if (cfg->ep_size > 1) {
        const size_t ns = (size_t)h->n_src, E = (size_t)cfg->n_experts, Hh = (size_t)cfg->hidden;
        if ((rc = dev_alloc(h, &h->s_idx, ns)) || (rc = dev_alloc(h, &h->s_w, ns)) || (rc = dev_alloc(h, &h->s_count, E)) ||
            (rc = dev_alloc(h, &h->s_offset, E + 1)) || (rc = dev_alloc(h, &h->s_perm, ns)) ||
            (rc = dev_alloc(h, &h->s_inv, ns)) || (rc = dev_alloc(h, &h->all_counts_d, E * cfg->ep_size)) ||
            (rc = dev_alloc(h, &h->row_expert, n)) || (rc = dev_alloc(h, &h->ones, n)) ||
            (rc = dev_alloc(h, &h->xsend, ns * Hh)) || (rc = dev_alloc(h, &h->xrecv, n * Hh)) ||
            (rc = dev_alloc(h, &h->yrecv, ns * Hh)) || (rc = dev_alloc(h, &h->yback, n * Hh)) ||
            (rc = dev_alloc(h, &h->ep_bar_src, (size_t)4)) || (rc = dev_alloc(h, &h->ep_bar_dst, (size_t)cfg->ep_size + 4)))
            return bail(rc);
        if (cudaMallocHost(&h->host_pinned, (E * cfg->ep_size + n) * sizeof(int32_t)) != cudaSuccess)
            return bail(fail(h, NEON_MOE_ECUDA, "cudaMallocHost failed"));
        fill_ones_kernel<<<(unsigned)((n + 255) / 256), 256>>>(h->ones, (int)n);
        for (cudaEvent_t& ev : h->ep_ev)
            if (cudaEventCreate(&ev) != cudaSuccess) return bail(fail(h, NEON_MOE_ECUDA, "cudaEventCreate failed"));
    }
    if (cudaMemset(h->status, 0, 16) != cudaSuccess) return bail(fail(h, NEON_MOE_ECUDA, "cudaMemset failed"));
    h->route_done = reinterpret_cast<unsigned*>(h->status + 2);  // third word of the zeroed status block
    if (cudaStreamCreateWithFlags(&h->own_stream, cudaStreamNonBlocking) != cudaSuccess)
        return bail(fail(h, NEON_MOE_ECUDA, "cudaStreamCreate failed"));
    *out = h;
    return NEON_MOE_OK;
}

int neon_moe_destroy(neon_moe_handle* h) {
    if (!h) return NEON_MOE_EINVAL;
    cudaSetDevice(h->cfg.device);
    cudaDeviceSynchronize();
    free_all(h);
    delete h;
    return NEON_MOE_OK;
}

int neon_moe_set_weights(neon_moe_handle* h, const void* router_w, const void* router_b,
                         const uint8_t* gu_blocks, const uint8_t* gu_scales, const void* gu_bias,
                         const uint8_t* dn_blocks, const uint8_t* dn_scales, const void* dn_bias, int on_device) {
    if (!h) return NEON_MOE_EINVAL;
    if (!router_w || !router_b || !gu_blocks || !gu_scales || !gu_bias || !dn_blocks || !dn_scales || !dn_bias)
        return fail(h, NEON_MOE_EINVAL, "null weight pointer");
    CU(h, cudaSetDevice(h->cfg.device));
    CU(h, cudaDeviceSynchronize());
    const int H = h->cfg.hidden, I = h->cfg.inter, E = h->cfg.n_experts, EL = h->n_local;
    h->has_weights = false;
    drop_graphs(h);
    int rc;
    if ((rc = copy_in(h, &h->router_w, router_w, (size_t)E * H, on_device))) return rc;
    if ((rc = copy_in(h, &h->router_b, router_b, (size_t)E, on_device))) return rc;
    if ((rc = copy_in(h, &h->gu_bias, gu_bias, (size_t)EL * 2 * I, on_device))) return rc;
    if ((rc = copy_in(h, &h->dn_bias, dn_bias, (size_t)EL * H, on_device))) return rc;
    free_mma16(h);  // the mma.sync layout of the previous weights, if it was built
    if ((rc = load_matrix_tc(h, gu_blocks, gu_scales, 2 * I, H, 1, on_device, &h->gu_wt, &h->gu_sfa, &h->tm_gu, &h->tm_gu2, &h->tm4_gu, &h->tm4_gu2))) return rc;
    if ((rc = load_matrix_tc(h, dn_blocks, dn_scales, H, I, 0, on_device, &h->dn_wt, &h->dn_sfa, &h->tm_dn, &h->tm_dn2, &h->tm4_dn, &h->tm4_dn2))) return rc;
    CU(h, cudaDeviceSynchronize());
    if (h->path == 1 && (rc = ensure_mma16(h))) return rc;  // a handle already on the mma.sync kernels keeps working
    h->has_weights = true;
    return NEON_MOE_OK;
}

// Dispatch + expert products + combine for n = rows * k_eff entries: entry i uses activation
// row i / k_eff of `hidden` and expert idx[i] - e_lo; `weighted_out` gets, per row, the sum of
// its k_eff slots' down outputs, each multiplied by route_w[i].  Used by the single-GPU pass
// (rows = tokens, k_eff = top_k) and by the expert-parallel local pass (rows = received
// rows, k_eff = 1, route_w = 1).
static int experts_core(neon_moe_handle* h, const void* hidden, int rows, int k_eff, const int32_t* idx, int e_lo,
                        const float* route_w, const float* hidden_amax, float* out, cudaStream_t st, bool prof,
                        bool dispatched = false, const PeerRows<float>* peer = nullptr) {
    const int H = h->cfg.hidden, I = h->cfg.inter, EL = h->n_local;
    const int n = rows * k_eff;
    DispatchArrays d{h->count, h->offset, h->perm, h->inv};
    if (h->path == 2) {
        const int tt = tile_tokens_for(h, rows), tt_dn = tt;  // one tile list serves both products
        TileList tl{h->tile_expert, h->tile_row0, h->tile_rows, h->n_tiles, h->row_tile};
        const bool stacked = tt <= 32;
        if (dispatched) {
            // the router launch already produced the dispatch arrays and the tile list
        } else if (n <= 1024)
            launch_k(h->pdl != 0, dispatch_tiles_small_kernel, dim3(1), dim3(1024), (size_t)(32 * EL) * sizeof(int), st, idx, n,
                     e_lo, EL, d, tt, tl);
        else if (h->dispatch_multi) {
            const DispatchScratch sc{h->disp_blk_count, h->disp_blk_base, h->disp_tile_first, h->disp_done};
            const dim3 grid((n + 1023) / 1024);
            launch_k(h->pdl != 0, dispatch_count_kernel, grid, dim3(1024), (size_t)(32 * EL) * sizeof(int), st, idx, n, e_lo, EL, d, tt, tl, sc);
            launch_k(h->pdl != 0, dispatch_place_kernel, grid, dim3(1024), (size_t)(32 * EL) * sizeof(int), st, idx, n, e_lo, EL, d, tt, tl, sc);
            h->launches++;
        } else
            launch_k(h->pdl != 0, dispatch_tiles_kernel, dim3(1), dim3(1024), (size_t)(33 * EL) * sizeof(int), st, idx, n, e_lo,
                     EL, d, tt, tl);
        if (!dispatched) h->launches++;
        DBG_SYNC(h, st, "dispatch_tiles_kernel");
        const int nch_h = h->kp_h / kChunkK, nch_i = h->kp_i / kChunkK;
        if (stacked && !hidden_amax) {  // no producer kernel measured the rows: do it here
            launch_k(h->pdl != 0, row_amax_kernel<true>, dim3((rows + 7) / 8), dim3(256), 0, st, hidden, H, rows, h->x_amax);
            h->launches++;
            hidden_amax = h->x_amax;
        }
        launch_split<2, true>(h, tt, tl, hidden, H, n, k_eff, hidden_amax, 0.f, h->x_act, h->x_scale, st);
        DBG_SYNC(h, st, "split_rows (hidden)");
        GmmParams g{};
        h->pass_entries = n;
        g.a_tx_bytes = h->a_tx_bytes;
#ifdef NEON_MOE_INSTRUMENT
        g.trace = h->trace_which == 2 ? nullptr : h->trace;
#endif
        g.a_out = h->a_f32; g.inter = I; g.limit = h->cfg.swiglu_limit; g.alpha = h->cfg.swiglu_alpha;
        g.perm = h->perm; g.route_w = route_w; g.y = h->y; g.hidden = H; g.status = h->status;
        // gate_up: rows 2I, K = H
        g.tile_expert = tl.expert; g.tile_row0 = tl.row0; g.tile_rows = tl.rows; g.n_tiles = tl.n_tiles;
        g.sfa = h->gu_sfa; g.act = h->x_act; g.row_scale = h->x_scale; g.bias = h->gu_bias;
        g.m_tiles = 2 * I / 128; g.n_chunks = nch_h; g.rows_total = 2 * I;
        mark(h, st, prof);
        int rc = launch_gmm<2, true>(h, tt, h->tm_gu, h->tm_gu2, g, st);
        if (rc) return rc;
        DBG_SYNC(h, st, "gmm_bs_kernel gate_up");
        mark(h, st, prof);
        // |SwiGLU| <= limit * (limit + 1): a fixed bound replaces the row maximum
        const float a_bound = h->cfg.swiglu_limit * (h->cfg.swiglu_limit + 1.f);
        if (tt_dn > 32)
            launch_split<kDownTermsPrefill, false>(h, tt_dn, tl, h->a_f32, I, n, k_eff, nullptr, a_bound, h->a_act, nullptr, st);
        else
            launch_split<4, false>(h, tt_dn, tl, h->a_f32, I, n, k_eff, nullptr, a_bound, h->a_act, nullptr, st);
        const bool mx4_dn = tt_dn <= 32 && h->mx4;
        DBG_SYNC(h, st, "split_rows (activation)");
        // down: rows H, K = I
        g.tile_expert = tl.expert; g.tile_row0 = tl.row0; g.tile_rows = tl.rows; g.n_tiles = tl.n_tiles;
        g.sfa = h->dn_sfa; g.act = h->a_act; g.row_scale = nullptr; g.bias = h->dn_bias;
        {   // the scale split_rows derives from the bound: 2^(floor(log2 bound) - 7), same clamps
            uint32_t bits; memcpy(&bits, &a_bound, 4);
            int sb = std::min(std::max((int)((bits >> 23) & 0xffu) - 7, 4 * 4 + 1), 250);
            bits = (uint32_t)sb << 23; memcpy(&g.row_scale_const, &bits, 4);
            if (mx4_dn) g.row_scale_const = a_bound * (1.f / 6.f);  // split_rows_fp4_kernel's first-term scale
        }
        g.m_tiles = (H + 127) / 128; g.n_chunks = nch_i; g.rows_total = H;
        if (peer) g.peer = *peer;  // the epilogue writes every row straight into its token owner's buffer
#ifdef NEON_MOE_INSTRUMENT
        g.trace = h->trace_which == 1 ? nullptr : h->trace;
#endif
        rc = tt_dn > 32 ? launch_gmm<kDownTermsPrefill, false>(h, tt_dn, h->tm_dn, h->tm_dn2, g, st)
                        : launch_gmm<4, false>(h, tt_dn, h->tm_dn, h->tm_dn2, g, st);
        if (rc) return rc;
        DBG_SYNC(h, st, "gmm_bs_kernel down");
        mark(h, st, prof);
    } else {
        dispatch_kernel<<<1, 1024, (size_t)(33 * EL) * sizeof(int), st>>>(idx, n, e_lo, EL, d);
        h->launches++;
        ExpertParams p{};
        p.offset = h->offset;
        p.perm = h->perm;
        p.top_k = k_eff;
        p.x = static_cast<const uint16_t*>(hidden);
        p.a_hi = h->a_hi;
        p.a_lo = h->a_lo;
        p.limit = h->cfg.swiglu_limit;
        p.alpha = h->cfg.swiglu_alpha;
        p.route_w = route_w;
        p.y = h->y;
        // gate_up: rows 2I, K = H
        p.wq = h->gu_wq; p.sq = h->gu_sq; p.bias = h->gu_bias;
        p.rows = 2 * I; p.K = H; p.tiles = 2 * I / 16; p.nbp = H / 64;
        mark(h, st, prof);
        launch_expert<true>(h, p, rows, st);
        mark(h, st, prof);
        // down: rows H, K = I
        p.wq = h->dn_wq; p.sq = h->dn_sq; p.bias = h->dn_bias;
        p.rows = H; p.K = I; p.tiles = H / 16; p.nbp = I / 64;
        launch_expert<false>(h, p, rows, st);
        mark(h, st, prof);
    }
    if (peer && h->path == 2) return NEON_MOE_OK;  // nothing to gather: the rows are where they belong
    dim3 cgrid((H / 4 + 127) / 128, rows);
    if (h->path == 2)
        launch_k(h->pdl != 0, combine_main_kernel, cgrid, dim3(128), 0, st, (const float*)h->y, (const int32_t*)h->inv, rows, H,
                 k_eff, out);
    else
        combine_kernel<<<cgrid, 128, 0, st>>>(h->y, h->inv, rows, H, k_eff, out);
    h->launches++;
    mark(h, st, prof);
    return NEON_MOE_OK;
}

// Shared memory of decode_fused_kernel: the stage ring, barriers, routing tables and logits (+ alignment slack).

// The whole pass as one cooperative launch (decode_fused.cuh).  The caller has checked T.
static int launch_decode_fused(neon_moe_handle* h, const void* hidden, int T, const float* logit_bias, float* out, cudaStream_t st) {
    static bool configured[kMaxDevicesAttr] = {};
    if (!configured[h->cfg.device]) {
        CU(h, cudaFuncSetAttribute(decode_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecodeSmemBytes));
        configured[h->cfg.device] = true;
    }
    const int H = h->cfg.hidden, I = h->cfg.inter, E = h->cfg.n_experts;
    DecodeParams p{};
    p.x = static_cast<const uint16_t*>(hidden); p.wr = h->router_w; p.br = h->router_b; p.logit_bias = logit_bias;
    p.T = T; p.H = H; p.I = I; p.E = E; p.k = h->cfg.top_k;
    p.limit = h->cfg.swiglu_limit; p.alpha = h->cfg.swiglu_alpha;
    p.gu_sfa = h->gu_sfa; p.dn_sfa = h->dn_sfa; p.gu_bias = h->gu_bias; p.dn_bias = h->dn_bias;
    p.gu_m_tiles = 2 * I / 128; p.dn_m_tiles = (H + 127) / 128; p.nch_h = h->kp_h / kChunkK; p.nch_i = h->kp_i / kChunkK;
    const int grid = h->n_sms;
    p.n_slices = std::max(1, std::min(kDecMaxSlices, grid * kDecRouterWarps / E));  // (expert, slice) units for the 3 router warps of every CTA
    p.rows_dn = T <= 4 ? 4 : 8;
    p.stages = dec_stages(p.rows_dn, kDecodeSmemBytes);
    p.a_tx_bytes = h->a_tx_bytes;
    p.router_part = h->dec_router_part; p.gu_part = h->dec_gu_part; p.dn_part = h->dec_dn_part;
    p.counters = h->dec_counters; p.gu_items_cap = h->dec_gu_items_cap;
    p.router_expected_extra = h->decode_stall_test ? 1u : 0u;
    p.wait_limit = h->decode_wait_limit;
    p.status = h->status; p.out = out; p.idx = h->idx; p.route_w = h->route_w;
    p.d = DispatchArrays{h->count, h->offset, h->perm, h->inv};
#ifdef NEON_MOE_INSTRUMENT
    p.trace = h->trace;
#endif
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kDecThreads);
    cfg.dynamicSmemBytes = kDecodeSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;  // all CTAs resident at once: they wait on one another's counters
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CU(h, cudaLaunchKernelEx(&cfg, decode_fused_kernel, h->tm_gu, h->tm_gu2, h->tm_dn, h->tm_dn2, p));
    h->launches++;
    return NEON_MOE_OK;
}

// The same pass sliced by intermediate channel (decode_sliced.cuh): T <= kDec2MaxTok.
static int launch_decode_sliced(neon_moe_handle* h, const void* hidden, int T, const float* logit_bias, float* out, cudaStream_t st) {
    static bool configured[kMaxDevicesAttr] = {};
    if (!configured[h->cfg.device]) {
        CU(h, cudaFuncSetAttribute(decode_sliced_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecodeSmemBytes));
        configured[h->cfg.device] = true;
    }
    const int H = h->cfg.hidden, I = h->cfg.inter, E = h->cfg.n_experts;
    DecodeParams p{};
    p.x = static_cast<const uint16_t*>(hidden); p.wr = h->router_w; p.br = h->router_b; p.logit_bias = logit_bias;
    p.T = T; p.H = H; p.I = I; p.E = E; p.k = h->cfg.top_k;
    p.limit = h->cfg.swiglu_limit; p.alpha = h->cfg.swiglu_alpha;
    p.gu_sfa = h->gu_sfa; p.dn_sfa = h->dn_sfa; p.gu_bias = h->gu_bias; p.dn_bias = h->dn_bias;
    p.gu_m_tiles = 2 * I / 128; p.dn_m_tiles = (H + 127) / 128; p.nch_h = h->kp_h / kChunkK; p.nch_i = h->kp_i / kChunkK;
    const int grid = h->n_sms;
    p.n_slices = std::max(1, std::min(kDecMaxSlices, grid * kDecRouterWarps / E));
    p.rows_dn = 4;
    p.stages = dec2_stages(T, p.dn_m_tiles, kDecodeSmemBytes);
    p.a_tx_bytes = h->a_tx_bytes;
    p.router_part = h->dec_router_part; p.gu_part = nullptr; p.dn_part = h->dec_y_part;
    p.counters = h->dec_counters; p.gu_items_cap = h->dec_gu_items_cap;
    p.router_expected_extra = h->decode_stall_test ? 1u : 0u;
    p.wait_limit = h->decode_wait_limit;
    p.status = h->status; p.out = out; p.idx = h->idx; p.route_w = h->route_w;
    p.d = DispatchArrays{h->count, h->offset, h->perm, h->inv};
#ifdef NEON_MOE_INSTRUMENT
    p.trace = h->trace;
#endif
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kDecThreads);
    cfg.dynamicSmemBytes = kDecodeSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;  // all CTAs resident at once: they meet at a grid-wide barrier
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CU(h, cudaLaunchKernelEx(&cfg, decode_sliced_kernel, h->tm_gu, h->tm_gu2, h->tm_dn, p));
    h->launches++;
    return NEON_MOE_OK;
}

static void launch_router(neon_moe_handle* h, const void* hidden, int T, const float* logit_bias, int32_t* idx, float* w,
                          float* tok_amax, cudaStream_t st) {
    const int H = h->cfg.hidden, E = h->cfg.n_experts, k = h->cfg.top_k;
    if (h->path == 2 && T > h->router_wide_max && h->router_mma && (E == 32 || E == 128) && H % 32 == 0) {
        // tensor-core router, 16 tokens per CTA: no token maxima (128-token tiles scale per block)
        const size_t smem = (size_t)4 * 16 * E * sizeof(float);
        if (E == 32)
            launch_k(h->pdl != 0, router_topk_mma_kernel<4>, dim3((T + 15) / 16), dim3(128), smem, st,
                     static_cast<const uint16_t*>(hidden), (const uint16_t*)h->router_w, (const uint16_t*)h->router_b, logit_bias, T,
                     H, k, idx, w);
        else
            launch_k(h->pdl != 0, router_topk_mma_kernel<16>, dim3((T + 15) / 16), dim3(128), smem, st,
                     static_cast<const uint16_t*>(hidden), (const uint16_t*)h->router_w, (const uint16_t*)h->router_b, logit_bias, T,
                     H, k, idx, w);
    } else if (h->path == 2 && T > h->router_wide_max) {  // token-blocked router: no token maxima either
        const size_t smem = (size_t)8 * H * 2 + (size_t)8 * E * sizeof(float);
        static bool configured[kMaxDevicesAttr] = {};
        if (!configured[h->cfg.device]) {
            cudaFuncSetAttribute(router_topk_block8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
            configured[h->cfg.device] = true;
        }
        launch_k(h->pdl != 0, router_topk_block8_kernel, dim3((T + 7) / 8), dim3(1024), smem, st,
                 static_cast<const uint16_t*>(hidden), (const uint16_t*)h->router_w, (const uint16_t*)h->router_b, logit_bias, T, H,
                 E, k, idx, w);
    } else if (h->path == 2)
        launch_k(h->pdl != 0, router_topk_wide_kernel, dim3(T), dim3(1024), H * 2 + E * sizeof(float), st,
                 static_cast<const uint16_t*>(hidden), (const uint16_t*)h->router_w, (const uint16_t*)h->router_b, logit_bias, T, H,
                 E, k, idx, w, tok_amax);
    else
        router_topk_kernel<256><<<T, 256, (H + E) * sizeof(float), st>>>(
            static_cast<const uint16_t*>(hidden), h->router_w, h->router_b, logit_bias, T, H, E, k, idx, w);
    h->launches++;
}

static int forward_eager(neon_moe_handle* h, const void* hidden, int T, const float* logit_bias, float* out,
                         int32_t* topk_idx, float* topk_w, cudaStream_t st);

int neon_moe_forward(neon_moe_handle* h, const void* hidden, int T, const float* logit_bias, float* out,
                     int32_t* topk_idx, float* topk_w, void* cuda_stream) {
    if (!h) return NEON_MOE_EINVAL;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    // Small passes are launch-bound: the second time the same arguments come in, the launch
    // sequence is captured into a CUDA graph (on the handle's own stream) and replayed from then
    // on.  Not while profiling or debugging, and not inside a caller's own stream capture.
    const bool cacheable = h->use_graphs && h->has_weights && h->cfg.ep_size == 1 && T > 0 && T <= h->graph_max_tokens && hidden && out &&
                           !h->profiling && !h->sync_debug && !h->trace;
    if (!cacheable) return forward_eager(h, hidden, T, logit_bias, out, topk_idx, topk_w, st);
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) {
        cudaGetLastError();
        return forward_eager(h, hidden, T, logit_bias, out, topk_idx, topk_w, st);
    }
    neon_moe_handle::CachedGraph* hit = nullptr;
    for (auto& g : h->graphs)
        if (g.hidden == hidden && g.T == T && g.bias == logit_bias && g.out == out && g.idx == topk_idx && g.w == topk_w) {
            hit = &g;
            break;
        }
    if (!hit) {
        if (h->graphs.size() >= 64) drop_graphs(h);
        h->graphs.push_back({hidden, logit_bias, out, topk_idx, topk_w, T, 0, 0, nullptr});
        hit = &h->graphs.back();
    }
    if (!hit->exec) {
        if (hit->seen++ == 0) return forward_eager(h, hidden, T, logit_bias, out, topk_idx, topk_w, st);
        CU(h, cudaSetDevice(h->cfg.device));
        const int64_t before = h->launches;
        CU(h, cudaStreamBeginCapture(h->own_stream, cudaStreamCaptureModeThreadLocal));
        int rc = forward_eager(h, hidden, T, logit_bias, out, topk_idx, topk_w, h->own_stream);
        cudaGraph_t graph = nullptr;
        cudaError_t ce = cudaStreamEndCapture(h->own_stream, &graph);
        hit->launches = (int)(h->launches - before);
        h->launches = before;
        if (rc || ce != cudaSuccess || !graph) {
            if (graph) cudaGraphDestroy(graph);
            cudaGetLastError();
            h->use_graphs = 0;  // capture is not available here: stay eager
            return forward_eager(h, hidden, T, logit_bias, out, topk_idx, topk_w, st);
        }
        ce = cudaGraphInstantiate(&hit->exec, graph, 0);
        cudaGraphDestroy(graph);
        if (ce != cudaSuccess) {
            hit->exec = nullptr;
            h->use_graphs = 0;
            return forward_eager(h, hidden, T, logit_bias, out, topk_idx, topk_w, st);
        }
    }
    CU(h, cudaSetDevice(h->cfg.device));
    CU(h, cudaGraphLaunch(hit->exec, st));
    h->launches += hit->launches;
    h->last_stream = st;
    h->last_n = T * h->cfg.top_k;
    return NEON_MOE_OK;
}

static int forward_eager(neon_moe_handle* h, const void* hidden, int T, const float* logit_bias, float* out,
                         int32_t* topk_idx, float* topk_w, cudaStream_t st) {
    if (!h->has_weights) return fail(h, NEON_MOE_ESTATE, "forward before set_weights");
    if (h->cfg.ep_size != 1) return fail(h, NEON_MOE_ESTATE, "forward needs ep_size == 1; use neon_moe_forward_ep");
    if (T < 0 || T > h->cfg.max_tokens) return fail(h, NEON_MOE_EINVAL, "T=%d outside [0, max_tokens=%d]", T, h->cfg.max_tokens);
    if (T == 0) { h->last_n = 0; return NEON_MOE_OK; }
    if (!hidden || !out) return fail(h, NEON_MOE_EINVAL, "null hidden/out");
    CU(h, cudaSetDevice(h->cfg.device));
    const int k = h->cfg.top_k, n = T * k;
    const bool prof = h->profiling && h->events_used + 5 <= 5 * kMaxProfiledForwards;
    if (h->path == 2 && h->decode_fused && T <= std::min(h->decode_max_tokens, h->decode_fused_tokens) && !prof && h->tile_override == 0 && !h->mx4 && !h->fuse_dispatch) {
        int rc = (h->decode_sliced && T <= h->dec_sliced_tokens) ? launch_decode_sliced(h, hidden, T, logit_bias, out, st)
                                                                  : launch_decode_fused(h, hidden, T, logit_bias, out, st);
        if (rc) return rc;
        if (topk_idx) CU(h, cudaMemcpyAsync(topk_idx, h->idx, (size_t)n * 4, cudaMemcpyDeviceToDevice, st));
        if (topk_w) CU(h, cudaMemcpyAsync(topk_w, h->route_w, (size_t)n * 4, cudaMemcpyDeviceToDevice, st));
        h->last_stream = st;
        h->last_n = n;
        return NEON_MOE_OK;
    }
    mark(h, st, prof);
    // decode passes on the main path: the last router CTA also runs the dispatch
    const bool fused = h->path == 2 && h->fuse_dispatch && T <= 64 && n <= 1024 && h->n_local == h->cfg.n_experts;
    if (fused) {
        const int H = h->cfg.hidden, E = h->cfg.n_experts;
        const size_t smem = std::max((size_t)H * 2 + E * sizeof(float), (size_t)32 * E * sizeof(int));
        DispatchArrays d{h->count, h->offset, h->perm, h->inv};
        TileList tl{h->tile_expert, h->tile_row0, h->tile_rows, h->n_tiles, h->row_tile};
        launch_k(h->pdl != 0, router_dispatch_kernel, dim3(T), dim3(1024), smem, st, static_cast<const uint16_t*>(hidden),
                 (const uint16_t*)h->router_w, (const uint16_t*)h->router_b, logit_bias, T, H, E, k, h->idx, h->route_w, h->x_amax,
                 h->route_done, d, tile_tokens_for(h, T), tl);
        h->launches++;
    } else {
        launch_router(h, hidden, T, logit_bias, h->idx, h->route_w, h->x_amax, st);
    }
    // the token maxima come from the decode routers only (the token-blocked router does not produce them)
    int rc = experts_core(h, hidden, T, k, h->idx, 0, h->route_w, (h->path == 2 && T <= h->router_wide_max) ? h->x_amax : nullptr, out, st, prof,
                          fused);
    if (rc) return rc;
    if (topk_idx) CU(h, cudaMemcpyAsync(topk_idx, h->idx, (size_t)n * 4, cudaMemcpyDeviceToDevice, st));
    if (topk_w) CU(h, cudaMemcpyAsync(topk_w, h->route_w, (size_t)n * 4, cudaMemcpyDeviceToDevice, st));
    CU(h, cudaGetLastError());
    h->last_stream = st;
    h->last_n = n;
    return NEON_MOE_OK;
}

// ---- expert parallelism --------------------------------------------------------------------
#define NC(h, call)                                                                                  \
    do {                                                                                             \
        ncclResult_t r_ = (call);                                                                    \
        if (r_ != ncclSuccess)                                                                       \
            return fail(h, NEON_MOE_ENCCL, "%s failed: %s", #call, nccl_api().GetErrorString(r_)); \
    } while (0)

int neon_moe_ep_unique_id(void* id128) {
    if (!id128) return NEON_MOE_EINVAL;
    if (!nccl_api().ok) return fail(nullptr, NEON_MOE_ENCCL, "libnccl.so.2 could not be loaded");
    ncclUniqueId id;
    NC(nullptr, nccl_api().GetUniqueId(&id));
    memcpy(id128, id.internal, NCCL_UNIQUE_ID_BYTES);
    return NEON_MOE_OK;
}

int neon_moe_ep_init(neon_moe_handle* h, const void* id128) {
    if (!h || !id128) return NEON_MOE_EINVAL;
    if (h->cfg.ep_size < 2) return fail(h, NEON_MOE_ESTATE, "ep_init needs ep_size >= 2");
    if (!nccl_api().ok) return fail(h, NEON_MOE_ENCCL, "libnccl.so.2 could not be loaded");
    CU(h, cudaSetDevice(h->cfg.device));
    ncclUniqueId id;
    memcpy(id.internal, id128, NCCL_UNIQUE_ID_BYTES);
    NC(h, nccl_api().CommInitRank(&h->comm, h->cfg.ep_size, id, h->cfg.ep_rank));
    // every rank learns every rank's receive capacity, so that the overflow verdict of a pass is
    // the same everywhere (ranks may have been created with different max_tokens)
    const int G = h->cfg.ep_size;
    CU(h, cudaMemcpy(h->s_count, &h->n_cap, sizeof(int32_t), cudaMemcpyHostToDevice));
    NC(h, nccl_api().AllGather(h->s_count, h->all_counts_d, 1, ncclInt32, h->comm, h->own_stream));
    h->ep_caps.assign((size_t)G, 0);
    CU(h, cudaMemcpyAsync(h->ep_caps.data(), h->all_counts_d, (size_t)G * 4, cudaMemcpyDeviceToHost, h->own_stream));
    CU(h, cudaStreamSynchronize(h->own_stream));
    return NEON_MOE_OK;
}

int neon_moe_ep_peer_export(neon_moe_handle* h, void* handles128) {
    if (!h || !handles128) return NEON_MOE_EINVAL;
    if (h->cfg.ep_size < 2 || !h->xrecv || !h->yrecv) return fail(h, NEON_MOE_ESTATE, "peer export needs an expert-parallel handle");
    CU(h, cudaSetDevice(h->cfg.device));
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t hx, hy;
    CU(h, cudaIpcGetMemHandle(&hx, h->xrecv));
    CU(h, cudaIpcGetMemHandle(&hy, h->yrecv));
    memcpy(handles128, &hx, 64);
    memcpy(static_cast<char*>(handles128) + 64, &hy, 64);
    return NEON_MOE_OK;
}

int neon_moe_ep_peer_import(neon_moe_handle* h, const void* all_handles) {
    if (!h || !all_handles) return NEON_MOE_EINVAL;
    const int G = h->cfg.ep_size, me = h->cfg.ep_rank;
    if (G < 2 || G > kMaxPeerRanks) return fail(h, NEON_MOE_EINVAL, "peer stores serve 2..%d ranks", kMaxPeerRanks);
    CU(h, cudaSetDevice(h->cfg.device));
    for (int r = 0; r < G; ++r) {
        if (r == me) {
            h->peer_x[r] = h->xrecv;
            h->peer_y[r] = h->yrecv;
            continue;
        }
        if (h->peer_mapped[r]) continue;
        cudaIpcMemHandle_t hx, hy;
        memcpy(&hx, static_cast<const char*>(all_handles) + (size_t)r * 128, 64);
        memcpy(&hy, static_cast<const char*>(all_handles) + (size_t)r * 128 + 64, 64);
        void *px = nullptr, *py = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&px, hx, cudaIpcMemLazyEnablePeerAccess);
        if (e == cudaSuccess) e = cudaIpcOpenMemHandle(&py, hy, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            if (px) cudaIpcCloseMemHandle(px);
            cudaGetLastError();
            return fail(h, NEON_MOE_ECUDA, "mapping rank %d's buffers failed: %s", r, cudaGetErrorString(e));
        }
        h->peer_x[r] = static_cast<uint16_t*>(px);
        h->peer_y[r] = static_cast<float*>(py);
        h->peer_mapped[r] = true;
    }
    return NEON_MOE_OK;
}

int neon_moe_ep_plan(const int32_t* all_counts, int ep_size, int n_experts, int rank, int32_t* send_rows,
                     int32_t* send_off, int32_t* recv_rows, int32_t* recv_off, int32_t* row_expert, int row_expert_cap,
                     int* n_recv) {
    if (!all_counts || !send_rows || !send_off || !recv_rows || !recv_off || !n_recv || ep_size <= 0 || n_experts <= 0 ||
        n_experts % ep_size || rank < 0 || rank >= ep_size)
        return NEON_MOE_EINVAL;
    *n_recv = ep_plan(all_counts, ep_size, n_experts, rank, send_rows, send_off, recv_rows, recv_off, row_expert, row_expert_cap);
    return *n_recv < 0 ? NEON_MOE_EINVAL : NEON_MOE_OK;
}

int neon_moe_ep_overflow(const int32_t* all_counts, int ep_size, int n_experts, const int32_t* caps, int* first_rank) {
    if (!all_counts || !caps || !first_rank || ep_size <= 0 || n_experts <= 0 || n_experts % ep_size) return NEON_MOE_EINVAL;
    *first_rank = ep_first_overflow(all_counts, ep_size, n_experts, caps);
    return NEON_MOE_OK;
}

// NCCL call inside an open group: on failure the group is closed before the error is returned,
// so the communicator is not left with a half-built group.
#define NCG(h, call)                                                                                 \
    do {                                                                                             \
        ncclResult_t r_ = (call);                                                                    \
        if (r_ != ncclSuccess) {                                                                     \
            nccl_api().GroupEnd();                                                                   \
            return fail(h, NEON_MOE_ENCCL, "%s failed: %s", #call, nccl_api().GetErrorString(r_)); \
        }                                                                                            \
    } while (0)

// One exchange + local expert pass + exchange back over `T` of this rank's tokens.  When the
// gathered histograms show that some rank would receive more rows than it has room for, EVERY
// rank sees that from the same data and the token range is cut in two halves that run as passes
// of their own (each rank halves its own range; the verdict is collective, so the ranks stay in
// step).  Only when no rank has more than one token left does the call fail - on every rank.
static int ep_pass(neon_moe_handle* h, const uint16_t* hidden, int T, const float* logit_bias, float* out,
                   int32_t* topk_idx, float* topk_w, cudaStream_t st, int depth) {
    NcclApi& nc = nccl_api();
    const int H = h->cfg.hidden, E = h->cfg.n_experts, k = h->cfg.top_k, G = h->cfg.ep_size, me = h->cfg.ep_rank;
    const int n = T * k;
    // 1. route own tokens, sort entries by global expert (= by destination rank, then expert), pack rows
    CU(h, cudaEventRecord(h->ep_ev[0], st));
    DispatchArrays sd{h->s_count, h->s_offset, h->s_perm, h->s_inv};
    if (T > 0) launch_router(h, hidden, T, logit_bias, h->s_idx, h->s_w, nullptr, st);
    if (n > 1024 && h->dispatch_multi && h->path == 2) {  // the sort alone (no tile list), one CTA per 1024 entries
        const DispatchScratch sc{h->disp_blk_count, h->disp_blk_base, h->disp_tile_first, h->disp_done};
        const TileList none{};
        const dim3 grid((n + 1023) / 1024);
        launch_k(false, dispatch_count_kernel, grid, dim3(1024), (size_t)(32 * E) * sizeof(int), st, (const int32_t*)h->s_idx, n, 0, E, sd, 0, none, sc);
        launch_k(false, dispatch_place_kernel, grid, dim3(1024), (size_t)(32 * E) * sizeof(int), st, (const int32_t*)h->s_idx, n, 0, E, sd, 0, none, sc);
        h->launches += 2;
    } else {
        dispatch_kernel<<<1, 1024, (size_t)(33 * E) * sizeof(int), st>>>(h->s_idx, n, 0, E, sd);
        h->launches++;
    }
    // 2. every rank learns every histogram; sizes are needed on the host to post the exchange
    NC(h, nc.AllGather(h->s_count, h->all_counts_d, (size_t)E, ncclInt32, h->comm, st));
    int32_t* all_counts = h->host_pinned;
    int32_t* row_expert_h = h->host_pinned + (size_t)E * G;
    CU(h, cudaMemcpyAsync(all_counts, h->all_counts_d, (size_t)E * G * 4, cudaMemcpyDeviceToHost, st));
    if (n > 0 && !(h->ep_peer && h->path == 2)) {  // runs while the histograms travel (the peer-store exchange needs no packed copy)
        pack_rows_kernel<<<n, 128, 0, st>>>(hidden, h->s_perm, k, H, n, h->xsend);
        h->launches++;
    }
    CU(h, cudaEventRecord(h->ep_ev[1], st));
    CU(h, cudaStreamSynchronize(st));
    const int over = ep_first_overflow(all_counts, G, E, h->ep_caps.data());
    if (over >= 0) {
        long long most = 0;  // entries of the rank with the most tokens in this pass
        for (int r = 0; r < G; ++r) {
            long long nr = 0;
            for (int e = 0; e < E; ++e) nr += all_counts[(size_t)r * E + e];
            most = std::max(most, nr);
        }
        if (most <= k || depth >= 16)
            return fail(h, NEON_MOE_EINVAL, "rank %d would receive more than its %d rows even from single-token passes", over,
                        (int)h->ep_caps[over]);
        const int T0 = T / 2;  // every rank halves its own range; a rank with T <= 1 runs an empty first half
        int rc = ep_pass(h, hidden, T0, logit_bias, out, topk_idx, topk_w, st, depth + 1);
        if (rc) return rc;
        return ep_pass(h, hidden + (size_t)T0 * H, T - T0, logit_bias, out + (size_t)T0 * H, topk_idx ? topk_idx + (size_t)T0 * k : nullptr,
                       topk_w ? topk_w + (size_t)T0 * k : nullptr, st, depth + 1);
    }
    int32_t send_rows[64], send_off[64], recv_rows[64], recv_off[64];
    const int R = ep_plan(all_counts, G, E, me, send_rows, send_off, recv_rows, recv_off, row_expert_h, h->n_cap);
    if (R < 0) return fail(h, NEON_MOE_EINVAL, "exchange plan disagrees with the capacity verdict");  // cannot happen: same data
    h->ep_last_recv = R;
    h->ep_subpasses++;
    if (R > 0) CU(h, cudaMemcpyAsync(h->row_expert, row_expert_h, (size_t)R * 4, cudaMemcpyHostToDevice, st));
    const bool peer = h->ep_peer && h->path == 2 && G <= kMaxPeerRanks;
    // a collective with nothing to move: when it has run on this rank, every rank's work enqueued before it has finished
    auto rank_barrier = [&]() -> int {
        NC(h, nc.AllGather(h->ep_bar_src, h->ep_bar_dst, 1, ncclInt32, h->comm, st));
        return NEON_MOE_OK;
    };
    if (peer) {
        // 3'. token rows straight into the expert owners' receive buffers (this library's own stores over NVLink)
        int32_t disp_off[kMaxPeerRanks], ret_off[kMaxPeerRanks];
        ep_peer_offsets(all_counts, G, E, me, disp_off, ret_off);
        PeerRows<uint16_t> tx{};
        PeerRows<float> ty{};
        tx.n_ranks = ty.n_ranks = G;
        for (int r = 0; r < G; ++r) {
            tx.row_off[r] = send_off[r]; tx.dst_off[r] = disp_off[r]; tx.base[r] = h->peer_x[r];
            ty.row_off[r] = recv_off[r]; ty.dst_off[r] = ret_off[r]; ty.base[r] = h->peer_y[r];
        }
        tx.row_off[G] = n;
        ty.row_off[G] = R;
        if (n > 0) {
            scatter_rows_kernel<<<std::min(n, 8 * h->n_sms), 256, 0, st>>>(hidden, h->s_perm, k, H, n, tx);
            h->launches++;
        }
        int rc = rank_barrier();  // every rank's rows have landed before anyone multiplies
        if (rc) return rc;
        CU(h, cudaEventRecord(h->ep_ev[2], st));
        // 4'. local experts; the down product's epilogue writes every output row into its token owner's yrecv
        if (R > 0) {
            rc = experts_core(h, h->xrecv, R, 1, h->row_expert, 0, h->ones, nullptr, h->yback, st, false, false, &ty);
            if (rc) return rc;
        }
        CU(h, cudaEventRecord(h->ep_ev[3], st));
        rc = rank_barrier();      // every rank's products are done: all rows of my tokens are in yrecv
        if (rc) return rc;
        CU(h, cudaEventRecord(h->ep_ev[4], st));
    } else {
    // 3. token rows to the owners of their experts
    NC(h, nc.GroupStart());
    for (int r = 0; r < G; ++r) {
        if (send_rows[r]) NCG(h, nc.Send(h->xsend + (size_t)send_off[r] * H, (size_t)send_rows[r] * H, ncclBfloat16, r, h->comm, st));
        if (recv_rows[r]) NCG(h, nc.Recv(h->xrecv + (size_t)recv_off[r] * H, (size_t)recv_rows[r] * H, ncclBfloat16, r, h->comm, st));
    }
    NC(h, nc.GroupEnd());
    CU(h, cudaEventRecord(h->ep_ev[2], st));
    // 4. local experts on the received rows (one slot per row, unit weight); yback is in receive order
    if (R > 0) {
        int rc = experts_core(h, h->xrecv, R, 1, h->row_expert, 0, h->ones, nullptr, h->yback, st, false);
        if (rc) return rc;
    }
    CU(h, cudaEventRecord(h->ep_ev[3], st));
    // 5. outputs back to the token owners, in the order the rows were sent
    NC(h, nc.GroupStart());
    for (int r = 0; r < G; ++r) {
        if (recv_rows[r]) NCG(h, nc.Send(h->yback + (size_t)recv_off[r] * H, (size_t)recv_rows[r] * H, ncclFloat32, r, h->comm, st));
        if (send_rows[r]) NCG(h, nc.Recv(h->yrecv + (size_t)send_off[r] * H, (size_t)send_rows[r] * H, ncclFloat32, r, h->comm, st));
    }
    NC(h, nc.GroupEnd());
    CU(h, cudaEventRecord(h->ep_ev[4], st));
    }
    // 6. routing-weighted sum of each token's slots, fixed slot order
    if (T > 0) {
        dim3 cgrid((H / 4 + 127) / 128, T);
        combine_weighted_kernel<<<cgrid, 128, 0, st>>>(h->yrecv, h->s_inv, h->s_w, T, H, k, out);
        h->launches++;
    }
    CU(h, cudaEventRecord(h->ep_ev[5], st));
    h->ep_timed = true;
    if (topk_idx && n) CU(h, cudaMemcpyAsync(topk_idx, h->s_idx, (size_t)n * 4, cudaMemcpyDeviceToDevice, st));
    if (topk_w && n) CU(h, cudaMemcpyAsync(topk_w, h->s_w, (size_t)n * 4, cudaMemcpyDeviceToDevice, st));
    CU(h, cudaGetLastError());
    h->last_stream = st;
    h->last_n = R;
    return NEON_MOE_OK;
}

int neon_moe_forward_ep(neon_moe_handle* h, const void* hidden, int T, const float* logit_bias, float* out,
                        int32_t* topk_idx, float* topk_w, void* cuda_stream) {
    if (!h) return NEON_MOE_EINVAL;
    if (!h->has_weights) return fail(h, NEON_MOE_ESTATE, "forward_ep before set_weights");
    if (!h->comm) return fail(h, NEON_MOE_ESTATE, "forward_ep before ep_init");
    if (h->cfg.ep_size > 64) return fail(h, NEON_MOE_EINVAL, "ep_size above 64");
    if (T < 0 || T > h->cfg.max_tokens) return fail(h, NEON_MOE_EINVAL, "T=%d outside [0, max_tokens=%d]", T, h->cfg.max_tokens);
    if (T > 0 && (!hidden || !out)) return fail(h, NEON_MOE_EINVAL, "null hidden/out");
    CU(h, cudaSetDevice(h->cfg.device));
    h->ep_subpasses = 0;
    return ep_pass(h, static_cast<const uint16_t*>(hidden), T, logit_bias, out, topk_idx, topk_w, static_cast<cudaStream_t>(cuda_stream), 0);
}

int neon_moe_ep_subpasses(const neon_moe_handle* h) { return h ? h->ep_subpasses : 0; }

int neon_moe_ep_times(neon_moe_handle* h, double* ms5, int* rows_received) {
    if (!h || !ms5) return NEON_MOE_EINVAL;
    if (!h->ep_timed) return fail(h, NEON_MOE_ESTATE, "no expert-parallel pass has run");
    CU(h, cudaSetDevice(h->cfg.device));
    CU(h, cudaEventSynchronize(h->ep_ev[5]));
    for (int i = 0; i < 5; ++i) {
        float t = 0.f;
        CU(h, cudaEventElapsedTime(&t, h->ep_ev[i], h->ep_ev[i + 1]));
        ms5[i] = t;
    }
    if (rows_received) *rows_received = h->ep_last_recv;
    return NEON_MOE_OK;
}

int neon_moe_forward_host(neon_moe_handle* h, const void* hidden, int T, const float* logit_bias, float* out,
                          int32_t* topk_idx, float* topk_w) {
    if (!h) return NEON_MOE_EINVAL;
    if (T < 0 || T > h->cfg.max_tokens) return fail(h, NEON_MOE_EINVAL, "T=%d outside [0, max_tokens=%d]", T, h->cfg.max_tokens);
    if (T == 0) return NEON_MOE_OK;
    if (!hidden || !out) return fail(h, NEON_MOE_EINVAL, "null hidden/out");
    CU(h, cudaSetDevice(h->cfg.device));
    cudaStream_t st = h->own_stream;
    const size_t nh = (size_t)T * h->cfg.hidden;
    CU(h, cudaMemcpyAsync(h->st_hidden, hidden, nh * 2, cudaMemcpyHostToDevice, st));
    if (logit_bias)
        CU(h, cudaMemcpyAsync(h->st_bias, logit_bias, (size_t)h->cfg.n_experts * 4, cudaMemcpyHostToDevice, st));
    int rc = neon_moe_forward(h, h->st_hidden, T, logit_bias ? h->st_bias : nullptr, h->st_out, nullptr, nullptr, st);
    if (rc) return rc;
    CU(h, cudaMemcpyAsync(out, h->st_out, nh * 4, cudaMemcpyDeviceToHost, st));
    const size_t n = (size_t)T * h->cfg.top_k;
    if (topk_idx) CU(h, cudaMemcpyAsync(topk_idx, h->idx, n * 4, cudaMemcpyDeviceToHost, st));
    if (topk_w) CU(h, cudaMemcpyAsync(topk_w, h->route_w, n * 4, cudaMemcpyDeviceToHost, st));
    CU(h, cudaStreamSynchronize(st));
    return NEON_MOE_OK;
}

int neon_moe_forward_host_batches(neon_moe_handle* h, const void* const* hidden, int n_batches, int T,
                                  const float* logit_bias, float* const* out) {
    if (!h) return NEON_MOE_EINVAL;
    if (T < 0 || T > h->cfg.max_tokens) return fail(h, NEON_MOE_EINVAL, "T=%d outside [0, max_tokens=%d]", T, h->cfg.max_tokens);
    if (n_batches < 0) return fail(h, NEON_MOE_EINVAL, "negative batch count");
    if (T == 0 || n_batches == 0) return NEON_MOE_OK;
    if (!hidden || !out) return fail(h, NEON_MOE_EINVAL, "null hidden/out");
    for (int i = 0; i < n_batches; ++i)
        if (!hidden[i] || !out[i]) return fail(h, NEON_MOE_EINVAL, "null buffer of batch %d", i);
    CU(h, cudaSetDevice(h->cfg.device));
    if (!h->s_in) {  // first use: second staging set, two copy streams, events
        int rc;
        if ((rc = dev_alloc(h, &h->st_hidden2, (size_t)h->cfg.max_tokens * h->cfg.hidden)) ||
            (rc = dev_alloc(h, &h->st_out2, (size_t)h->cfg.max_tokens * h->cfg.hidden)))
            return rc;
        CU(h, cudaStreamCreateWithFlags(&h->s_in, cudaStreamNonBlocking));
        CU(h, cudaStreamCreateWithFlags(&h->s_out, cudaStreamNonBlocking));
        for (int b = 0; b < 2; ++b) {
            CU(h, cudaEventCreateWithFlags(&h->ev_in[b], cudaEventDisableTiming));
            CU(h, cudaEventCreateWithFlags(&h->ev_comp[b], cudaEventDisableTiming));
            CU(h, cudaEventCreateWithFlags(&h->ev_out[b], cudaEventDisableTiming));
        }
    }
    cudaStream_t sc = h->own_stream;
    const size_t nh = (size_t)T * h->cfg.hidden;
    if (logit_bias) {
        CU(h, cudaMemcpyAsync(h->st_bias, logit_bias, (size_t)h->cfg.n_experts * 4, cudaMemcpyHostToDevice, sc));
        CU(h, cudaStreamSynchronize(sc));
    }
    uint16_t* in_buf[2] = {h->st_hidden, h->st_hidden2};
    float* out_buf[2] = {h->st_out, h->st_out2};
    for (int i = 0; i < n_batches; ++i) {
        const int b = i & 1;
        // upload batch i while batch i-1 computes; its staging buffer is free once batch i-2 has computed
        if (i >= 2) CU(h, cudaStreamWaitEvent(h->s_in, h->ev_comp[b], 0));
        CU(h, cudaMemcpyAsync(in_buf[b], hidden[i], nh * 2, cudaMemcpyHostToDevice, h->s_in));
        CU(h, cudaEventRecord(h->ev_in[b], h->s_in));
        CU(h, cudaStreamWaitEvent(sc, h->ev_in[b], 0));
        if (i >= 2) CU(h, cudaStreamWaitEvent(sc, h->ev_out[b], 0));  // batch i-2's result has left the output buffer
        int rc = h->cfg.ep_size > 1 ? neon_moe_forward_ep(h, in_buf[b], T, logit_bias ? h->st_bias : nullptr, out_buf[b], nullptr, nullptr, sc)
                                    : neon_moe_forward(h, in_buf[b], T, logit_bias ? h->st_bias : nullptr, out_buf[b], nullptr, nullptr, sc);
        if (rc) return rc;
        CU(h, cudaEventRecord(h->ev_comp[b], sc));
        CU(h, cudaStreamWaitEvent(h->s_out, h->ev_comp[b], 0));
        CU(h, cudaMemcpyAsync(out[i], out_buf[b], nh * 4, cudaMemcpyDeviceToHost, h->s_out));
        CU(h, cudaEventRecord(h->ev_out[b], h->s_out));
    }
    CU(h, cudaStreamSynchronize(h->s_out));
    CU(h, cudaStreamSynchronize(sc));
    return NEON_MOE_OK;
}

int neon_moe_read_dispatch(neon_moe_handle* h, int32_t* count, int32_t* offset, int32_t* perm, int32_t* inv,
                           int* n_entries) {
    if (!h) return NEON_MOE_EINVAL;
    CU(h, cudaSetDevice(h->cfg.device));
    CU(h, cudaStreamSynchronize(h->last_stream));
    const int EL = h->n_local, n = h->last_n;
    if (n_entries) *n_entries = n;
    if (n == 0) return NEON_MOE_OK;
    if (count) CU(h, cudaMemcpy(count, h->count, (size_t)EL * 4, cudaMemcpyDeviceToHost));
    if (offset) CU(h, cudaMemcpy(offset, h->offset, (size_t)(EL + 1) * 4, cudaMemcpyDeviceToHost));
    if (perm) CU(h, cudaMemcpy(perm, h->perm, (size_t)n * 4, cudaMemcpyDeviceToHost));
    if (inv) CU(h, cudaMemcpy(inv, h->inv, (size_t)n * 4, cudaMemcpyDeviceToHost));
    return NEON_MOE_OK;
}

int neon_moe_set_option(neon_moe_handle* h, const char* name, int64_t value) {
    if (!h || !name) return NEON_MOE_EINVAL;
    drop_graphs(h);
    if (!strcmp(name, "path")) {
        if (value != 1 && value != 2) return fail(h, NEON_MOE_EINVAL, "path must be 1 (mma.sync) or 2 (tcgen05)");
        if (value == 1 && h->has_weights) {
            int rc = ensure_mma16(h);
            if (rc) return rc;
        }
        h->path = (int)value;
    } else if (!strcmp(name, "mma16_layout")) {
        if (value) {
            if (!h->has_weights) return fail(h, NEON_MOE_ESTATE, "mma16_layout before set_weights");
            int rc = ensure_mma16(h);
            if (rc) return rc;
        } else if (h->path != 1) {
            CU(h, cudaSetDevice(h->cfg.device));
            CU(h, cudaDeviceSynchronize());
            free_mma16(h);
        }
#ifdef NEON_MOE_INSTRUMENT
    } else if (!strcmp(name, "a_tx_bytes")) {
        h->a_tx_bytes = (uint32_t)value;
    } else if (!strcmp(name, "trace_ptr")) {
        h->trace = reinterpret_cast<long long*>(value);
    } else if (!strcmp(name, "trace_which")) {
        h->trace_which = (int)value;
    } else if (!strcmp(name, "sync_debug")) {
        h->sync_debug = (int)value;
    } else if (!strcmp(name, "max_stages")) {
        h->max_stages = (int)value;
#endif
    } else if (!strcmp(name, "ctas_per_sm")) {
        h->ctas_per_sm = (int)value;
    } else if (!strcmp(name, "n_ctas")) {
        h->n_sms = (int)value;
    } else if (!strcmp(name, "pdl")) {
        h->pdl = (int)value;
    } else if (!strcmp(name, "fuse_dispatch")) {
        h->fuse_dispatch = (int)value;
    } else if (!strcmp(name, "tile_tokens")) {
        if (value != 0 && value != 16 && value != 32 && value != 128) return fail(h, NEON_MOE_EINVAL, "tile_tokens must be 0, 16, 32 or 128");
        h->tile_override = (int)value;
    } else if (!strcmp(name, "router_wide_max")) {
        h->router_wide_max = (int)value;
    } else if (!strcmp(name, "router_mma")) {
        h->router_mma = (int)value;
    } else if (!strcmp(name, "graph_max_tokens")) {
        h->graph_max_tokens = (int)value;
        drop_graphs(h);
    } else if (!strcmp(name, "ep_peer")) {
        if (value) {
            for (int r = 0; r < h->cfg.ep_size && r < kMaxPeerRanks; ++r)
                if (!h->peer_x[r]) return fail(h, NEON_MOE_ESTATE, "ep_peer before neon_moe_ep_peer_import");
            if (h->cfg.ep_size > kMaxPeerRanks) return fail(h, NEON_MOE_EINVAL, "peer stores serve at most %d ranks", kMaxPeerRanks);
        }
        h->ep_peer = value != 0;
    } else if (!strcmp(name, "decode_fused")) {
        h->decode_fused = (int)value;
    } else if (!strcmp(name, "decode_sliced")) {
        h->decode_sliced = (int)value;
    } else if (!strcmp(name, "decode_fused_tokens")) {
        if (value < 0 || value > kDecMaxTok) return fail(h, NEON_MOE_EINVAL, "decode_fused_tokens must lie in [0, %d]", kDecMaxTok);
        h->decode_fused_tokens = (int)value;
    } else if (!strcmp(name, "decode_stall_test")) {
        h->decode_stall_test = (int)value;
    } else if (!strcmp(name, "decode_wait_limit")) {
        if (value < 1000) return fail(h, NEON_MOE_EINVAL, "decode_wait_limit is in SM clocks, at least 1000");
        h->decode_wait_limit = (long long)value;
    } else if (!strcmp(name, "pair_mma")) {
        if (value < 0 || value > 2) return fail(h, NEON_MOE_EINVAL, "pair_mma is 0 (never), 1 (always) or 2 (small passes)");
        h->pair_mma = (int)value;
    } else if (!strcmp(name, "dispatch_multi")) {
        h->dispatch_multi = value != 0;
    } else if (!strcmp(name, "pair_prefill")) {
        h->pair_prefill = value != 0;
    } else if (!strcmp(name, "mxf4_prefill")) {
        h->mxf4_prefill = (int)value;
    } else if (!strcmp(name, "mx4")) {
        h->mx4 = (int)value;
    } else if (!strcmp(name, "use_graphs")) {
        h->use_graphs = (int)value;
    } else {
        return fail(h, NEON_MOE_EINVAL, "unknown option '%s'", name);
    }
    return NEON_MOE_OK;
}

int neon_moe_profile(neon_moe_handle* h, int enable) {
    if (!h) return NEON_MOE_EINVAL;
    h->profiling = enable != 0;
    return NEON_MOE_OK;
}

int neon_moe_read_profile(neon_moe_handle* h, double* ms, int* n_forwards) {
    if (!h || !ms || !n_forwards) return NEON_MOE_EINVAL;
    CU(h, cudaSetDevice(h->cfg.device));
    CU(h, cudaStreamSynchronize(h->last_stream));
    for (int i = 0; i < 4; ++i) ms[i] = 0.0;
    const size_t nf = h->events_used / 5;
    for (size_t f = 0; f < nf; ++f)
        for (int i = 0; i < 4; ++i) {
            float t = 0.f;
            CU(h, cudaEventElapsedTime(&t, h->events[5 * f + i], h->events[5 * f + i + 1]));
            ms[i] += t;
        }
    *n_forwards = (int)nf;
    h->events_used = 0;
    return NEON_MOE_OK;
}

// ---- weight files ----------------------------------------------------------------------------
// Layout of a weight file (all integers little-endian):
//   neon_moe_file_header (64 bytes), n_sections x neon_moe_file_section (32 bytes), then the
//   sections' bytes, each starting on a 256-byte boundary.
//   layout 0 "raw": sections router_w, router_b, gu_blocks, gu_scales, gu_bias, dn_blocks,
//     dn_scales, dn_bias exactly as neon_moe_set_weights takes them (re-tiled on the GPU at load);
//   layout 1 "tiled": router_w, router_b, gu_bias, dn_bias as above and gu_tiles, gu_sfa, dn_tiles,
//     dn_sfa = the tensor-core layout byte for byte as it sits in HBM (box-contiguous nibbles and
//     512-byte scale atoms), so loading is a straight copy.
namespace {
struct FileSection { char name[16]; uint64_t offset, bytes; };
struct FileHeader {
    char magic[8];
    uint32_t version, layout;
    int32_t hidden, inter, n_experts, expert_lo, n_local, top_k;
    uint32_t n_sections, reserved[5];
};
static_assert(sizeof(FileHeader) == 64 && sizeof(FileSection) == 32, "file structs");
constexpr char kFileMagic[8] = {'N', 'M', 'O', 'E', 'W', '1', 0, 0};

const FileSection* find_section(const std::vector<FileSection>& secs, const char* name) {
    for (const auto& sec : secs)
        if (!strncmp(sec.name, name, sizeof sec.name)) return &sec;
    return nullptr;
}
}  // namespace

int neon_moe_save_weights(neon_moe_handle* h, const char* path) {
    if (!h || !path) return NEON_MOE_EINVAL;
    if (!h->has_weights || !h->gu_wt) return fail(h, NEON_MOE_ESTATE, "save_weights before set_weights");
    CU(h, cudaSetDevice(h->cfg.device));
    CU(h, cudaDeviceSynchronize());
    const size_t H = h->cfg.hidden, I = h->cfg.inter, E = h->cfg.n_experts, EL = h->n_local;
    const size_t mt_gu = (2 * I + 127) / 128, mt_dn = (H + 127) / 128, nch_h = h->kp_h / kChunkK, nch_i = h->kp_i / kChunkK;
    struct Item { const char* name; const void* dev; size_t bytes; };
    const Item items[] = {{"router_w", h->router_w, E * H * 2},       {"router_b", h->router_b, E * 2},
                          {"gu_bias", h->gu_bias, EL * 2 * I * 2},    {"dn_bias", h->dn_bias, EL * H * 2},
                          {"gu_tiles", h->gu_wt, EL * mt_gu * nch_h * 8192}, {"gu_sfa", h->gu_sfa, EL * mt_gu * nch_h * 512},
                          {"dn_tiles", h->dn_wt, EL * mt_dn * nch_i * 8192}, {"dn_sfa", h->dn_sfa, EL * mt_dn * nch_i * 512}};
    const uint32_t ns = sizeof items / sizeof items[0];
    FileHeader hd{};
    memcpy(hd.magic, kFileMagic, 8);
    hd.version = 1; hd.layout = 1;
    hd.hidden = (int)H; hd.inter = (int)I; hd.n_experts = (int)E; hd.expert_lo = h->e_lo; hd.n_local = (int)EL; hd.top_k = h->cfg.top_k;
    hd.n_sections = ns;
    std::vector<FileSection> secs(ns);
    uint64_t off = (sizeof hd + ns * sizeof(FileSection) + 255) & ~uint64_t(255);
    for (uint32_t i = 0; i < ns; ++i) {
        memset(&secs[i], 0, sizeof secs[i]);
        strncpy(secs[i].name, items[i].name, sizeof secs[i].name - 1);
        secs[i].offset = off;
        secs[i].bytes = items[i].bytes;
        off = (off + items[i].bytes + 255) & ~uint64_t(255);
    }
    FILE* f = fopen(path, "wb");
    if (!f) return fail(h, NEON_MOE_EINVAL, "cannot open '%s' for writing", path);
    bool ok = fwrite(&hd, sizeof hd, 1, f) == 1 && fwrite(secs.data(), sizeof(FileSection), ns, f) == ns;
    std::vector<unsigned char> buf;
    for (uint32_t i = 0; ok && i < ns; ++i) {
        buf.resize(items[i].bytes);
        if (cudaMemcpy(buf.data(), items[i].dev, items[i].bytes, cudaMemcpyDeviceToHost) != cudaSuccess) { ok = false; break; }
        ok = fseek(f, (long)secs[i].offset, SEEK_SET) == 0 && fwrite(buf.data(), 1, items[i].bytes, f) == items[i].bytes;
    }
    if (ok && ns && secs[ns - 1].offset + secs[ns - 1].bytes < off)  // zero padding up to the aligned end
        ok = fseek(f, (long)off - 1, SEEK_SET) == 0 && fputc(0, f) != EOF;
    ok = (fclose(f) == 0) && ok;
    cudaGetLastError();
    if (!ok) return fail(h, NEON_MOE_ECUDA, "writing '%s' failed", path);
    return NEON_MOE_OK;
}

int neon_moe_load_weights_file(neon_moe_handle* h, const char* path) {
    if (!h || !path) return NEON_MOE_EINVAL;
    FILE* f = fopen(path, "rb");
    if (!f) return fail(h, NEON_MOE_EINVAL, "cannot open '%s'", path);
    struct Closer { FILE* f; ~Closer() { fclose(f); } } closer{f};
    FileHeader hd{};
    if (fread(&hd, sizeof hd, 1, f) != 1 || memcmp(hd.magic, kFileMagic, 8) != 0 || hd.version != 1)
        return fail(h, NEON_MOE_EINVAL, "'%s' is not a version-1 weight file", path);
    if (hd.hidden != h->cfg.hidden || hd.inter != h->cfg.inter || hd.n_experts != h->cfg.n_experts || hd.top_k != h->cfg.top_k ||
        hd.n_local != h->n_local || hd.expert_lo != h->e_lo)
        return fail(h, NEON_MOE_EINVAL, "'%s' holds H=%d I=%d E=%d experts [%d,%d) top_k=%d; the handle expects H=%d I=%d E=%d [%d,%d) k=%d",
                    path, hd.hidden, hd.inter, hd.n_experts, hd.expert_lo, hd.expert_lo + hd.n_local, hd.top_k, h->cfg.hidden,
                    h->cfg.inter, h->cfg.n_experts, h->e_lo, h->e_lo + h->n_local, h->cfg.top_k);
    if (hd.layout > 1 || hd.n_sections == 0 || hd.n_sections > 64) return fail(h, NEON_MOE_EINVAL, "'%s': bad layout or section count", path);
    std::vector<FileSection> secs(hd.n_sections);
    if (fread(secs.data(), sizeof(FileSection), hd.n_sections, f) != hd.n_sections) return fail(h, NEON_MOE_EINVAL, "'%s' is truncated", path);
    if (fseek(f, 0, SEEK_END) != 0) return fail(h, NEON_MOE_EINVAL, "'%s': seek failed", path);
    const uint64_t file_bytes = (uint64_t)ftell(f);
    const size_t H = h->cfg.hidden, I = h->cfg.inter, E = h->cfg.n_experts, EL = h->n_local;
    const size_t mt_gu = (2 * I + 127) / 128, mt_dn = (H + 127) / 128, nch_h = h->kp_h / kChunkK, nch_i = h->kp_i / kChunkK;
    std::vector<std::vector<unsigned char>> data;
    auto read_section = [&](const char* name, size_t expect, const unsigned char** out) -> int {
        const FileSection* sec = find_section(secs, name);
        if (!sec) return fail(h, NEON_MOE_EINVAL, "'%s' has no section '%s'", path, name);
        if (sec->bytes != expect) return fail(h, NEON_MOE_EINVAL, "'%s': section '%s' holds %llu bytes, %zu expected", path, name,
                                              (unsigned long long)sec->bytes, expect);
        if (sec->offset + sec->bytes > file_bytes) return fail(h, NEON_MOE_EINVAL, "'%s' is truncated inside section '%s'", path, name);
        data.emplace_back(expect);
        if (fseek(f, (long)sec->offset, SEEK_SET) != 0 || fread(data.back().data(), 1, expect, f) != expect)
            return fail(h, NEON_MOE_EINVAL, "'%s': reading section '%s' failed", path, name);
        *out = data.back().data();
        return NEON_MOE_OK;
    };
    int rc;
    const unsigned char *rw, *rb, *gub, *dnb;
    if ((rc = read_section("router_w", E * H * 2, &rw)) || (rc = read_section("router_b", E * 2, &rb)) ||
        (rc = read_section("gu_bias", EL * 2 * I * 2, &gub)) || (rc = read_section("dn_bias", EL * H * 2, &dnb)))
        return rc;
    if (hd.layout == 0) {
        const unsigned char *g1, *g2, *d1, *d2;
        if ((rc = read_section("gu_blocks", EL * 2 * I * (H / 2), &g1)) || (rc = read_section("gu_scales", EL * 2 * I * (H / 32), &g2)) ||
            (rc = read_section("dn_blocks", EL * H * (I / 2), &d1)) || (rc = read_section("dn_scales", EL * H * (I / 32), &d2)))
            return rc;
        return neon_moe_set_weights(h, rw, rb, g1, g2, gub, d1, d2, dnb, 0);
    }
    // tiled: straight copies into the tensor-core buffers; the mma.sync layout is not in the file
    const unsigned char *gt, *gs, *dt, *ds;
    if ((rc = read_section("gu_tiles", EL * mt_gu * nch_h * 8192, &gt)) || (rc = read_section("gu_sfa", EL * mt_gu * nch_h * 512, &gs)) ||
        (rc = read_section("dn_tiles", EL * mt_dn * nch_i * 8192, &dt)) || (rc = read_section("dn_sfa", EL * mt_dn * nch_i * 512, &ds)))
        return rc;
    CU(h, cudaSetDevice(h->cfg.device));
    CU(h, cudaDeviceSynchronize());
    h->has_weights = false;
    drop_graphs(h);
    if ((rc = copy_in(h, &h->router_w, rw, E * H, 0)) || (rc = copy_in(h, &h->router_b, rb, E, 0)) ||
        (rc = copy_in(h, &h->gu_bias, gub, EL * 2 * I, 0)) || (rc = copy_in(h, &h->dn_bias, dnb, EL * H, 0)))
        return rc;
    struct Tiled { uint8_t** dst; const unsigned char* src; size_t bytes; };
    const Tiled tiled[] = {{&h->gu_wt, gt, EL * mt_gu * nch_h * 8192}, {&h->gu_sfa, gs, EL * mt_gu * nch_h * 512},
                           {&h->dn_wt, dt, EL * mt_dn * nch_i * 8192}, {&h->dn_sfa, ds, EL * mt_dn * nch_i * 512}};
    for (const auto& t : tiled) {
        if (!*t.dst && (rc = dev_alloc(h, t.dst, t.bytes))) return rc;
        CU(h, cudaMemcpy(*t.dst, t.src, t.bytes, cudaMemcpyHostToDevice));
    }
    const uint64_t rows_gu = (uint64_t)EL * mt_gu * nch_h * 128, rows_dn = (uint64_t)EL * mt_dn * nch_i * 128;
    if ((rc = make_weight_map(h, &h->tm_gu, h->gu_wt, rows_gu, 128, false)) || (rc = make_weight_map(h, &h->tm_gu2, h->gu_wt, rows_gu, 256, false)) ||
        (rc = make_weight_map(h, &h->tm4_gu, h->gu_wt, rows_gu, 128, true)) || (rc = make_weight_map(h, &h->tm4_gu2, h->gu_wt, rows_gu, 256, true)) ||
        (rc = make_weight_map(h, &h->tm_dn, h->dn_wt, rows_dn, 128, false)) || (rc = make_weight_map(h, &h->tm_dn2, h->dn_wt, rows_dn, 256, false)) ||
        (rc = make_weight_map(h, &h->tm4_dn, h->dn_wt, rows_dn, 128, true)) || (rc = make_weight_map(h, &h->tm4_dn2, h->dn_wt, rows_dn, 256, true)))
        return rc;
    // the mma.sync kernels' layout is rebuilt from these tiles when "path" 1 or "mma16_layout" asks for it
    free_mma16(h);
    h->path = 2;
    h->has_weights = true;
    return NEON_MOE_OK;
}

int neon_moe_status(neon_moe_handle* h, int* word) {
    if (!h || !word) return NEON_MOE_EINVAL;
    CU(h, cudaSetDevice(h->cfg.device));
    CU(h, cudaStreamSynchronize(h->last_stream));
    CU(h, cudaMemcpy(word, h->status, sizeof(int), cudaMemcpyDeviceToHost));
    CU(h, cudaMemset(h->status, 0, sizeof(int)));
    // a pass that gave up on a wait leaves the one-launch kernel's counters mid-way: start them afresh
    if (*word && h->dec_counters) CU(h, cudaMemset(h->dec_counters, 0, (size_t)h->dec_counter_words * 4));
    return *word ? NEON_MOE_EDEVICE : NEON_MOE_OK;
}

}  // extern "C"

// =======================================================================================
// Allocation-free variant of the layer pass.
//
// neon_moe_forward keeps its intermediates (routing, dispatch arrays, the SwiGLU
// activations and the per-slot down rows) in workspaces that neon_moe_create obtained from
// cudaMalloc, sized by max_tokens.  The variant below keeps the same intermediates in one
// fixed array that is part of the loaded library image, so a pass needs no allocation that
// belongs to the calling thread or handle.
// =======================================================================================
namespace {

constexpr size_t kStaticScratchBytes = 2u << 20;  // 2 MiB, held by every GPU that loads the library
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::atomic<void*> g_static_scratch_addr[kMaxDevices];  // device address of g_static_scratch, per device (zero-initialised)

// Makes `dev` current for the scope and puts the caller's device back afterwards.
struct ScopedDevice {
    int prev = -1;
    cudaError_t err;
    explicit ScopedDevice(int dev) {
        err = cudaGetDevice(&prev);
        if (err == cudaSuccess && prev != dev) err = cudaSetDevice(dev);
        else if (err == cudaSuccess) prev = -1;  // nothing to restore
    }
    ~ScopedDevice() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

}  // namespace

extern "C" int neon_moe_forward_static(const neon_moe_handle* h, const void* hidden, int T,
                                       const float* logit_bias, float* out, int32_t* topk_idx, float* topk_w,
                                       void* cuda_stream) {
    if (!h) return fail(nullptr, NEON_MOE_EINVAL, "null handle");
    if (!h->has_weights) return fail(nullptr, NEON_MOE_ESTATE, "forward_static before set_weights");
    if (!h->gu_wq)
        return fail(nullptr, NEON_MOE_ESTATE, "forward_static reads the mma.sync weight layout, which is built on request: call "
                                              "neon_moe_set_option(h, \"mma16_layout\", 1) once at set-up, where allocating is allowed");
    if (h->cfg.ep_size != 1) return fail(nullptr, NEON_MOE_ESTATE, "forward_static needs ep_size == 1");
    if (T < 0) return fail(nullptr, NEON_MOE_EINVAL, "negative T");
    if (T == 0) return NEON_MOE_OK;
    if (!hidden || !out) return fail(nullptr, NEON_MOE_EINVAL, "null hidden/out");
    const int H = h->cfg.hidden, I = h->cfg.inter, E = h->cfg.n_experts, k = h->cfg.top_k;
    const size_t n = (size_t)T * k;
    // carve the scratch: every piece starts on a 256-byte boundary
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off = align256(off + bytes); return o; };
    const size_t o_idx = take(n * 4), o_rw = take(n * 4), o_count = take((size_t)E * 4),
                 o_offset = take((size_t)(E + 1) * 4), o_perm = take(n * 4), o_inv = take(n * 4),
                 o_ahi = take(n * I * 2), o_alo = take(n * I * 2), o_y = take(n * H * 4);
    if (off > kStaticScratchBytes)
        return fail(nullptr, NEON_MOE_EINVAL,
                    "forward_static: T=%d needs %zu bytes of scratch, the built-in array holds %zu; "
                    "use neon_moe_forward for larger batches", T, off, kStaticScratchBytes);
    const int dev = h->cfg.device;
    if (dev < 0 || dev >= kMaxDevices) return fail(nullptr, NEON_MOE_EINVAL, "device ordinal beyond %d", kMaxDevices);
    ScopedDevice on_dev(dev);  // the caller's current device is restored on return
    cudaError_t ce = on_dev.err;
    if (ce != cudaSuccess) return fail(nullptr, NEON_MOE_ECUDA, "cudaSetDevice failed: %s", cudaGetErrorString(ce));
    void* scratch = g_static_scratch_addr[dev].load(std::memory_order_acquire);
    if (!scratch) {
        // The array's name is only a host-side stand-in; kernels need its device address,
        // looked up once per device with that device current.  Two threads racing here both
        // obtain the same address, so the plain store is enough.
        ce = cudaGetSymbolAddress(&scratch, g_static_scratch);
        if (ce != cudaSuccess || !scratch)
            return fail(nullptr, NEON_MOE_ECUDA, "cudaGetSymbolAddress failed: %s", cudaGetErrorString(ce));
        g_static_scratch_addr[dev].store(scratch, std::memory_order_release);
    }
    unsigned char* base = static_cast<unsigned char*>(scratch);
    int32_t* s_idx = reinterpret_cast<int32_t*>(base + o_idx);
    float* s_rw = reinterpret_cast<float*>(base + o_rw);
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);

    router_topk_kernel<256><<<T, 256, (H + E) * sizeof(float), st>>>(
        static_cast<const uint16_t*>(hidden), h->router_w, h->router_b, logit_bias, T, H, E, k, s_idx, s_rw);
    DispatchArrays d{reinterpret_cast<int32_t*>(base + o_count), reinterpret_cast<int32_t*>(base + o_offset),
                     reinterpret_cast<int32_t*>(base + o_perm), reinterpret_cast<int32_t*>(base + o_inv)};
    dispatch_kernel<<<1, 1024, (size_t)(33 * E) * sizeof(int), st>>>(s_idx, (int)n, 0, E, d);

    ExpertParams p{};
    p.offset = d.offset;
    p.perm = d.perm;
    p.top_k = k;
    p.x = static_cast<const uint16_t*>(hidden);
    p.a_hi = reinterpret_cast<uint16_t*>(base + o_ahi);
    p.a_lo = reinterpret_cast<uint16_t*>(base + o_alo);
    p.limit = h->cfg.swiglu_limit;
    p.alpha = h->cfg.swiglu_alpha;
    p.route_w = s_rw;
    p.y = reinterpret_cast<float*>(base + o_y);
    constexpr int WARPS = 4;
    const dim3 block(32 * WARPS);
    p.wq = h->gu_wq; p.sq = h->gu_sq; p.bias = h->gu_bias;
    p.rows = 2 * I; p.K = H; p.tiles = 2 * I / 16; p.nbp = H / 64;
    {
        dim3 grid((p.tiles + WARPS - 1) / WARPS, E);
        if (T <= 8) expert_mma_kernel<1, true, WARPS><<<grid, block, 0, st>>>(p);
        else if (T <= 16) expert_mma_kernel<2, true, WARPS><<<grid, block, 0, st>>>(p);
        else if (T <= 32) expert_mma_kernel<4, true, WARPS><<<grid, block, 0, st>>>(p);
        else expert_mma_kernel<8, true, WARPS><<<grid, block, 0, st>>>(p);
    }
    p.wq = h->dn_wq; p.sq = h->dn_sq; p.bias = h->dn_bias;
    p.rows = H; p.K = I; p.tiles = H / 16; p.nbp = I / 64;
    {
        dim3 grid((p.tiles + WARPS - 1) / WARPS, E);
        if (T <= 8) expert_mma_kernel<1, false, WARPS><<<grid, block, 0, st>>>(p);
        else if (T <= 16) expert_mma_kernel<2, false, WARPS><<<grid, block, 0, st>>>(p);
        else if (T <= 32) expert_mma_kernel<4, false, WARPS><<<grid, block, 0, st>>>(p);
        else expert_mma_kernel<8, false, WARPS><<<grid, block, 0, st>>>(p);
    }
    dim3 cgrid((H / 4 + 127) / 128, T);
    combine_kernel<<<cgrid, 128, 0, st>>>(p.y, d.inv, T, H, k, out);
    if (topk_idx) {
        ce = cudaMemcpyAsync(topk_idx, s_idx, n * 4, cudaMemcpyDeviceToDevice, st);
        if (ce != cudaSuccess) return fail(nullptr, NEON_MOE_ECUDA, "copy of topk_idx failed: %s", cudaGetErrorString(ce));
    }
    if (topk_w) {
        ce = cudaMemcpyAsync(topk_w, s_rw, n * 4, cudaMemcpyDeviceToDevice, st);
        if (ce != cudaSuccess) return fail(nullptr, NEON_MOE_ECUDA, "copy of topk_w failed: %s", cudaGetErrorString(ce));
    }
    ce = cudaGetLastError();
    if (ce != cudaSuccess) return fail(nullptr, NEON_MOE_ECUDA, "launch failed: %s", cudaGetErrorString(ce));
    return NEON_MOE_OK;
}
