/*
 * neon_moe.h - C ABI of libneon_moe.so: a gpt-oss-shaped mixture-of-experts layer
 * (router + top-k + softmax, dispatch, grouped MXFP4 expert products with clamped
 * SwiGLU and routing-weighted combine) as hand-written sm_100a CUDA kernels.
 *
 * Relation to the reference engine (paths inside the NeonEngine project).  The engine
 * has no MoE operator, FFI or plugin interface to bind; its compute workloads are
 * "system" classes that own their device buffers, record work into the caller's command
 * stream and expose results as buffer handles.  Every entry point below names the
 * engine convention it follows, which is what an engine-side `lve::MoeLayerSystem`
 * (include/lve_moe_layer_system.hpp) binds:
 *
 *   - construction owns all device buffers .... NeonEngine/src/water_physics.cpp:23-123
 *   - stream-ordered, non-blocking execution .. NeonEngine/src/water_physics.hpp:66
 *                                               NeonEngine/src/raytracing_system.hpp:79
 *   - explicit, rare host read-back ........... NeonEngine/src/water_app.cpp:601-612
 *   - failures surface as error values/strings  NeonEngine/src/lve_buffer.hpp:22-28,
 *     (thrown as std::runtime_error by the C++  NeonEngine/src/water_physics.cpp:617-620
 *     wrapper, never across this ABI)
 *
 * Conventions (this library's own; the engine defines none):
 *   bf16 tensors are raw 16-bit patterns.  MXFP4 blocks are uint8 [E, rows, cols/2], low
 *   nibble = even column, code bits s|e|e|m; scales are E8M0 uint8 [E, rows, cols/32]
 *   (value 2^(byte-127), bytes 2..254 supported).  gate_up rows interleave gate (even) and
 *   linear (odd).  out[t] = sum_s w[t,s] * (down_s + down_bias), slots summed in order
 *   s = 0..k-1; outputs are fp32.  Top-k ties go to the lower expert id.
 *
 * All functions return 0 on success or a NEON_MOE_E* code; none throws or aborts.
 * A handle serves one stream at a time and is not thread-safe; distinct handles are
 * independent (one per GPU for expert parallelism).
 */
#ifndef NEON_MOE_H
#define NEON_MOE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NEON_MOE_OK 0
#define NEON_MOE_EINVAL 1   /* bad argument or unsupported shape          */
#define NEON_MOE_ECUDA 2    /* a CUDA runtime call failed                 */
#define NEON_MOE_ESTATE 3   /* call out of order (e.g. no weights set)    */
#define NEON_MOE_EDEVICE 4  /* a kernel reported a bounded-wait failure   */
#define NEON_MOE_ENCCL 5    /* an NCCL call failed / NCCL not loadable    */

typedef struct neon_moe_handle neon_moe_handle;

/* Layer description.  Plays the part of the literal parameters the engine's systems take
 * in their constructors (NeonEngine/src/water_physics.cpp:23-40). */
typedef struct neon_moe_config {
    int hidden;          /* H, multiple of 64 (2880)                              */
    int inter;           /* I, multiple of 64 (2880)                              */
    int n_experts;       /* E, global expert count (32 | 128), <= 256            */
    int top_k;           /* k (4), <= 8                                           */
    float swiglu_limit;  /* 7.0                                                   */
    float swiglu_alpha;  /* 1.702                                                 */
    int max_tokens;      /* largest T of one forward call on this rank            */
    int ep_rank;         /* expert-parallel rank, 0 when ep_size == 1             */
    int ep_size;         /* ranks sharing the experts; n_experts % ep_size == 0   */
    int device;          /* CUDA device ordinal                                   */
} neon_moe_config;

/* Creates the layer on cfg->device and allocates its workspaces.
 * Follows: system constructors own their buffers, NeonEngine/src/water_physics.cpp:449-603. */
int neon_moe_create(const neon_moe_config* cfg, neon_moe_handle** out);

/* Copies (and re-tiles for the kernels) the weights; the caller may free its arrays
 * afterwards.  Expert tensors hold this rank's n_experts/ep_size experts; the router is
 * replicated.  on_device != 0: pointers are device memory on cfg->device.  Any E8M0 scale byte
 * is accepted.  Only the tensor-core layout is kept (4 bits + 1/32 byte per weight, padded to
 * 128); the second layout that "path" 1 and neon_moe_forward_static read is built from it when
 * option "mma16_layout" (or "path" 1) asks for it.
 * Follows: initial data handed to the constructor and uploaded once,
 * NeonEngine/src/water_physics.cpp:41-123 (staging upload of particle data). */
int neon_moe_set_weights(neon_moe_handle* h, const void* router_w_bf16, const void* router_b_bf16,
                         const uint8_t* gate_up_blocks, const uint8_t* gate_up_scales,
                         const void* gate_up_bias_bf16, const uint8_t* down_blocks,
                         const uint8_t* down_scales, const void* down_bias_bf16, int on_device);

/* Weight files (this library's own format; the engine serialises nothing).  A file is a 64-byte
 * header {magic "NMOEW1", version 1, layout, hidden, inter, n_experts, expert_lo, n_local, top_k,
 * n_sections}, a table of {name[16], offset, bytes} sections and the sections' bytes on 256-byte
 * boundaries.  Layout 0 ("raw") holds the eight tensors exactly as neon_moe_set_weights takes them
 * and is re-tiled on the GPU at load; layout 1 ("tiled") holds the tensor-core layout byte for byte
 * as it sits in HBM, so loading is a straight copy.
 * neon_moe_save_weights writes layout 1 from a handle that has weights; raw files are written by
 * the host (neonengine_b200/weight_file.py).  neon_moe_load_weights_file checks the header against
 * the handle's configuration and every section's size against the file before it touches the GPU.
 * Follows: model files read once at start-up, NeonEngine/src/lve_model.cpp:45-51 (createModelFromFile). */
int neon_moe_save_weights(neon_moe_handle* h, const char* path);
int neon_moe_load_weights_file(neon_moe_handle* h, const char* path);

/* One layer pass over T tokens, enqueued on `cuda_stream` (a cudaStream_t; NULL = default
 * stream).  All pointers are device memory: hidden bf16 [T,H]; logit_bias fp32 [E] or
 * NULL (added to the router logits); out fp32 [T,H]; topk_idx int32 [T,k] and topk_w
 * fp32 [T,k] may be NULL.  Returns after enqueueing.  ep_size must be 1.
 * Follows: RunSimulation(dt, frameInfo) recording dispatches into the caller's command
 * buffer, NeonEngine/src/water_physics.hpp:66 and .cpp:131,165-436. */
int neon_moe_forward(neon_moe_handle* h, const void* hidden_bf16, int T, const float* logit_bias,
                     float* out_f32, int32_t* topk_idx, float* topk_w, void* cuda_stream);

/* The same pass for callers that hold HOST memory: copies hidden (and logit_bias) to the
 * device, runs the layer, copies out (and idx/w when non-NULL) back and synchronises.
 * Follows: the explicit host read-back the engine does for its debug buffer,
 * NeonEngine/src/water_app.cpp:601-612. */
int neon_moe_forward_host(neon_moe_handle* h, const void* hidden_bf16, int T, const float* logit_bias,
                          float* out_f32, int32_t* topk_idx, float* topk_w);

/* A run of n_batches passes over HOST memory (T tokens each; hidden[i] bf16 [T,H] in, out[i] fp32
 * [T,H] out; the same optional logit_bias for all), pipelined: the upload of batch i+1 and the
 * download of batch i-1 overlap the layer pass of batch i on separate copy streams with two
 * staging sets, so with pinned host buffers the run proceeds at the device's pace.  Returns when
 * every result is in host memory.  Results equal n_batches calls of neon_moe_forward_host.
 * On an expert-parallel handle (after neon_moe_ep_init) every batch runs as neon_moe_forward_ep:
 * the call is then collective - every rank calls it with the same n_batches. */
int neon_moe_forward_host_batches(neon_moe_handle* h, const void* const* hidden_bf16, int n_batches, int T,
                                  const float* logit_bias, float* const* out_f32);

/* ---- Expert parallelism (n_experts sharded evenly over ep_size GPUs of one node) -----------
 * The engine is single-GPU (NeonEngine/src/lve_device.cpp:125-148 picks one device), so these
 * have no engine counterpart; they follow the same conventions as neon_moe_forward.
 *
 * neon_moe_ep_unique_id: rank 0 obtains a 128-byte NCCL id and hands it to the other ranks by
 * any host channel.  neon_moe_ep_init: every rank joins the communicator (collective call);
 * NCCL is loaded with dlopen at this point, single-GPU users never need it. */
int neon_moe_ep_unique_id(void* id128);
int neon_moe_ep_init(neon_moe_handle* h, const void* id128);

/* One pass over this rank's T tokens (collective: every rank calls it, T may differ per rank).
 * Router on own tokens, all-to-all-v of token rows (bf16) to the experts' owners over NVLink,
 * local grouped expert products, all-to-all-v of the outputs (fp32) back, routing-weighted
 * combine.  Arguments as neon_moe_forward.  The call synchronises the stream once in the
 * middle (the exchange sizes are needed on the host) and returns with the rest enqueued.
 * A rank has room for 2*max_tokens*top_k received rows (twice the average).  Whether a pass
 * fits is decided from the gathered histograms, which are the same on every rank, so all ranks
 * reach the same verdict before any row travels: when some rank would overflow, every rank
 * halves its token range and the halves run as passes of their own (skewed routing costs
 * extra exchanges, not a failure); only if single-token passes still overflow does the call
 * fail, with NEON_MOE_EINVAL on every rank alike. */
int neon_moe_forward_ep(neon_moe_handle* h, const void* hidden_bf16, int T, const float* logit_bias,
                        float* out_f32, int32_t* topk_idx, float* topk_w, void* cuda_stream);

/* Exchanges by this library's own stores over NVLink instead of NCCL send/receive.  Every rank exports 128
 * bytes (CUDA IPC handles of its two receive buffers), the application gathers them by any host channel
 * (ranks in rank order) and hands all of them to every rank's import, which maps the peers' buffers; when
 * EVERY rank has imported successfully, every rank sets option "ep_peer" to 1 (a collective decision: the
 * ranks must use the same exchange).  From then on neon_moe_forward_ep writes token rows straight into the
 * expert owners' receive buffers, and the down product's epilogue writes each output row straight into its
 * token owner's buffer while the product runs; NCCL only gathers the histograms and orders the ranks
 * (two barriers per pass).  Same results as the NCCL exchange.  One process per GPU, one node. */
int neon_moe_ep_peer_export(neon_moe_handle* h, void* handles128);
int neon_moe_ep_peer_import(neon_moe_handle* h, const void* all_handles /* ep_size x 128 bytes */);

/* Exchanges the last neon_moe_forward_ep call needed: 1, or more when it ran as split passes. */
int neon_moe_ep_subpasses(const neon_moe_handle* h);

/* Device times of the last expert-parallel pass, ms[5] = {route+dispatch+pack, counts +
 * dispatch all-to-all, local experts, combine all-to-all, combine}; rows received by this
 * rank in *rows_received (may be NULL).  Synchronises. */
int neon_moe_ep_times(neon_moe_handle* h, double* ms5, int* rows_received);

/* Host-only exchange plan from the gathered histograms all_counts[ep_size][n_experts]: rows this
 * rank sends to / receives from every peer with their offsets, and the local expert of each
 * received row (row_expert may be NULL).  Needs no GPU; used by neon_moe_forward_ep. */
int neon_moe_ep_plan(const int32_t* all_counts, int ep_size, int n_experts, int rank, int32_t* send_rows,
                     int32_t* send_off, int32_t* recv_rows, int32_t* recv_off, int32_t* row_expert,
                     int row_expert_cap, int* n_recv);

/* The collective capacity verdict neon_moe_forward_ep uses, host-only: *first_rank = the lowest
 * rank whose receive total under all_counts[ep_size][n_experts] exceeds caps[rank], or -1 when
 * every rank fits. */
int neon_moe_ep_overflow(const int32_t* all_counts, int ep_size, int n_experts, const int32_t* caps, int* first_rank);

/* The layer pass for callers that must not allocate device memory.  It has no counterpart
 * in the reference engine.
 *
 * Who needs it: code that is handed a finished layer (weights already on the GPU, set up by
 * some other component at start-up) but runs where cudaMalloc is off limits - a plugin that
 * lives inside a host application's fixed memory budget, a latency-critical decode loop that
 * may not take the allocator's lock or its implicit device synchronisation, or a second
 * thread that wants a pass while the handle's own workspaces are busy on another stream.
 * neon_moe_forward keeps its intermediates in workspaces that neon_moe_create took from
 * cudaMalloc; this variant keeps them in a 2 MiB array built into the library image (each
 * GPU that loads the library holds those 2 MiB until the process exits) and calls neither
 * cudaMalloc/cudaFree nor any allocating library routine.  `h` is only read: it supplies
 * the weights and the layer description.  It reads the mma.sync weight layout, which is built
 * on request: whoever sets the handle up calls neon_moe_set_option(h, "mma16_layout", 1) once
 * (that call allocates); without it this entry point fails with NEON_MOE_ESTATE.  The calling
 * thread's current device is the same after the call as before; the handle's device status
 * word is neither read nor cleared (these kernels have no bounded waits).
 *
 * Arguments are those of neon_moe_forward (all device pointers, stream-ordered).  Limit: the
 * intermediates of T tokens must fit the array - T*top_k*(4*inter + 4*hidden + 16) bytes plus
 * small tables, i.e. T <= 22 at hidden = inter = 2880, top_k = 4.  Larger T is rejected
 * with NEON_MOE_EINVAL and a message naming both sizes; nothing is launched then.
 *
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress);
 * make that first call before starting any stream capture.  All calls on a GPU share the
 * one array and it keeps the previous call's contents: every pass rewrites each table
 * entry it later reads, so nothing has to start at zero, but two calls whose kernels can
 * overlap on the GPU (different streams, no ordering between them) race on it - order them.
 * Errors are reported through neon_moe_last_error(NULL). */
int neon_moe_forward_static(const neon_moe_handle* h, const void* hidden_bf16, int T,
                            const float* logit_bias, float* out_f32, int32_t* topk_idx, float* topk_w,
                            void* cuda_stream);

/* Host copies of the dispatch arrays of the most recent forward on this handle
 * (synchronises the handle's last stream): count[E_local], offset[E_local+1],
 * perm[n] (sorted position -> entry t*k+s) and inv[n], n = *n_entries.  NULLs skipped.
 * Follows: getters handing out a system's buffers, NeonEngine/src/water_physics.hpp:68-92. */
int neon_moe_read_dispatch(neon_moe_handle* h, int32_t* count, int32_t* offset, int32_t* perm,
                           int32_t* inv, int* n_entries);

/* Reads (and clears) the device status word: non-zero when a kernel gave up on a bounded
 * wait.  Synchronises the handle's last stream. */
int neon_moe_status(neon_moe_handle* h, int* device_status_word);

/* Tuning / test switches.  "path": 2 (default on sm_100) = TMA + tcgen05 block-scaled
 * grouped GEMM, 1 = the mma.sync kernels (builds their weight layout on first use; that layout
 * cannot hold scale bytes above 128 and the switch fails with NEON_MOE_EINVAL then).
 * "mma16_layout": 1 builds that layout now (allocates ~the size of the expert weights again),
 * 0 frees it.  "use_graphs" (default 1): passes of up to 64
 * tokens are captured into a CUDA graph the second time the same arguments are seen and
 * replayed afterwards (the analogue of the engine re-submitting a recorded command buffer).
 * "mx4" (default 0): 1 runs decode-sized passes on tcgen05.mma.kind::mxf4 (weights stay packed
 * 4-bit in shared memory, activations as six e2m1 terms): ~5 % faster, errors ~40x larger (still
 * inside the 2e-2 / 5e-3 contract on random inputs, not on inputs whose errors add coherently).
 * "fuse_dispatch" (default 0): 1 = at decode-sized passes the router CTA that finishes last also
 * runs the dispatch, saving one launch (identical results; measured no faster than the separate
 * kernel under programmatic dependent launch, 0.1086 vs 0.1078 ms per 64-token pass).
 * "tile_tokens" (default 0 = by batch size: 16 up to 16 tokens, 32 up to 224, else 128): forces the
 * token-tile size of the grouped GEMMs (16 and 32 use the stacked-term kernels).
 * "router_wide_max" (default 384): passes of up to this many tokens run the router with one CTA per
 * token, which also produces the per-token maxima the 16/32-token tiles scale by; larger passes use
 * the router that shares each weight read between 8 tokens.  "graph_max_tokens" (default 64): the
 * largest pass that is replayed from a captured graph (measured gain above 64 tokens: ~1 us).
 * "router_mma" (default 1): passes above router_wide_max tokens compute the router logits on tensor
 * cores (mma.sync, 16 tokens per CTA; 32 or 128 experts); 0 = the CUDA-core router that shares each
 * weight read between 8 tokens.  Same routing; logits differ in summation order only.
 * "decode_fused" (default 1) / "decode_fused_tokens" (default 1, at most 8): passes of up to that many
 * tokens (and top_k * T <= 32) run as ONE cooperative kernel - router, both expert products, SwiGLU and
 * combine, no dispatch pass; its CTAs wait for one another with bounded waits (status word on a timeout).
 * Measured at the gpt-oss-20b shapes it wins for single-token passes and loses above, hence the default.
 * "decode_sliced" (default 0): 1 runs one-launch passes of up to 4 tokens on the variant that slices the layer by
 * intermediate channel (each CTA computes 128 channels of one expert through both products, one grid-wide
 * barrier, no partial sums between the products); measured no faster (T = 1: 36.3 vs 35.1-36.5 us).
 * "decode_wait_limit": SM clocks such a wait may take (default 4e8).  "decode_stall_test": 1 makes the
 * kernel's first wait expect a signal nobody sends, so that the bounded wait can be tested without
 * faulting the GPU.
 * "mxf4_prefill" (default 0): 1 runs passes of more than 224 tokens on tcgen05.mma.kind::mxf4 with the
 * activations quantised to MXFP4 (blocks of 32, E8M0 scale 2^(floor(log2 amax) - 2), nearest e2m1, ties to
 * even).  Four-bit activations put the result ~20 % (mean relative) away from the unquantised one - far
 * outside the 2e-2 / 5e-3 contract - so it is an option; it agrees with an oracle that applies the same
 * quantisation to accumulation noise.
 * "pair_mma" (default 2): decode-sized tiles (16 / 32 tokens) on clusters of two CTAs whose leader issues two-SM
 * MMAs (tcgen05 cta_group::2, 256 weight rows per instruction): 0 never, 1 always, 2 for passes that route at
 * most 512 entries (128 tokens at top-4), where it measured 3-9 % faster per pass; results are bit-identical to
 * the one-CTA kernel's.
 * "dispatch_multi" (default 1): passes of more than 1024 (token, slot) entries sort them on one CTA per 1024
 * entries (two launches) instead of one CTA for all; identical arrays.
 * "pair_prefill" (default 1): 128-token tiles (passes above 224 tokens) on clusters of two CTAs: two adjacent
 * weight tiles per pair, each CTA half of the token rows, M = 256 instructions; bit-identical to the one-CTA
 * kernel (0), measured 1.23 vs 1.36-1.40 ms per 4096-token pass.
 * "ep_peer" (default 0; expert-parallel handles, after neon_moe_ep_peer_import on every rank): 1 makes both
 * exchanges of neon_moe_forward_ep this library's own stores into the peers' buffers instead of NCCL
 * all-to-alls.  Every rank must set the same value.
 * "n_ctas", "ctas_per_sm": grid size of the grouped GEMMs (default: one CTA per SM).
 * Routing is deterministic for a given router kernel, but the three routers (one CTA per token,
 * tensor-core, and the one neon_moe_forward_static uses) add the 2880 products in different
 * orders; logits agree to ~1e-6, so two experts whose logits are closer than that may swap
 * between a pass of 384 and one of 385 tokens, or between forward and forward_static.  Exact
 * ties (equal logits) go to the lower expert id in every router.
 * Builds with -DNEON_MOE_INSTRUMENT add measurement aids ("trace_ptr", "trace_which",
 * "a_tx_bytes", "max_stages", "sync_debug"); the shipped library has none of them.
 * Follows: the literal knobs the engine's apps set before running a system,
 * NeonEngine/src/raytracing_app.cpp:605-631. */
int neon_moe_set_option(neon_moe_handle* h, const char* name, int64_t value);

/* Per-stage device timing.  enable != 0 makes every following forward record CUDA events
 * around its stages on the caller's stream; neon_moe_read_profile synchronises, adds the
 * elapsed times of all forwards since the last read into ms[4] = {router+dispatch, gate_up,
 * down, combine} (milliseconds), stores the number of forwards in *n_forwards and resets.
 * At most 4096 forwards are kept between reads.
 * Follows: the engine timing its own frames, NeonEngine/src/raytracing_app.cpp:648-656. */
int neon_moe_profile(neon_moe_handle* h, int enable);
int neon_moe_read_profile(neon_moe_handle* h, double* ms, int* n_forwards);

/* Number of kernel launches the handle has issued since creation (for launch accounting). */
int64_t neon_moe_launch_count(const neon_moe_handle* h);

/* CTAs the paired (two-SM MMA) kernel was last launched with: twice the number of CTA pairs the device can
 * hold at once (option "pair_mma"); 0 before its first launch. */
int neon_moe_pair_ctas(const neon_moe_handle* h);

/* Text of the last error on this handle (h == NULL: of this thread's last failed
 * neon_moe_create or neon_moe_forward_static).
 * Owned by the library; valid until the next call on the handle. */
const char* neon_moe_last_error(const neon_moe_handle* h);

/* Frees the layer.  Follows: RAII teardown of system-owned buffers,
 * NeonEngine/src/lve_buffer.cpp:49-53. */
int neon_moe_destroy(neon_moe_handle* h);

/* Library version string. */
const char* neon_moe_version(void);

/* Measures the issue rate of the block-scaled tensor-core instruction the grouped GEMM uses, with
 * the operands resident in shared memory (no global traffic): every SM issues `chunks` groups of
 * accumulating 128 x n MMAs (kind 0: tcgen05.mma.kind::mxf8f6f4, 4 instructions of K = 32 per group;
 * kind 1: kind::mxf4, 2 instructions of K = 64 per group) back to back; kinds 2 and 3 are kinds 0 and 1
 * with one scale-atom copy (tcgen05.cp) before every group, as the decode kernels issue them.
 * n: 16..256, multiple of 16.
 * ms receives the duration of the launch (CUDA events), cycles the SM clocks one SM needed from the
 * first issue to the completion of the last instruction.  Work per SM = chunks * 2 * 128 * n * 128
 * floating-point operations.  The measured ceiling of the prefill roofline (no library has one for
 * these instruction kinds); the engine has no counterpart. */
int neon_moe_mma_rate(int device, int kind, int n, int chunks, double* ms, int64_t* cycles);

/* Measures the rate at which one SM's TMA unit brings weight boxes into shared memory: every SM keeps `stages`
 * loads of two 128 x 128 four-bit boxes (16 KB of global memory) in flight, `loads` loads in all, with no
 * consumer.  packed 0: the expanding map the kind::mxf8f6f4 kernels use (one byte per nibble plus padding: 32 KB
 * land in shared memory; stages <= 6); packed 1: nibbles stay packed (kind::mxf4; stages <= 8).  The boxes come
 * from a buffer of buffer_bytes (>= 1 MiB) that the SMs walk round-robin: a few MiB stay in L2, several hundred
 * stream from HBM.  ms receives the launch duration, cycles the SM clocks CTA 0 needed.  Bytes per SM = loads *
 * 16384.  The engine has no counterpart. */
int neon_moe_tma_rate(int device, int packed, int stages, int64_t buffer_bytes, int loads, double* ms, int64_t* cycles);

/* Self-check of the two-SM form of the block-scaled tensor-core instruction (tcgen05 cta_group::2) that the
 * paired grouped GEMM uses: a cluster of two CTAs multiplies constant e4m3 operands held in shared memory
 * (CTA c: A = a_c, its half of the N operand = b_c; a = {1, 0.5}, b = {1, 2}) with `chunks` x 4 accumulating
 * 256 x n x 32 MMAs issued by the leader CTA.  d32 receives, per CTA, rows {0, 37, 100, 127} x columns
 * {0, n/2 - 1, n/2, n - 1} of that CTA's accumulator: chunks * 128 * a_c * b_(column half) when M = 256
 * splits by CTA and N is the concatenation of the two halves.  tmem_addr2: the tensor-memory base each CTA
 * got; cycles: SM clocks from first issue to completion.  n: 32 or 64.  No engine counterpart. */
int neon_moe_mma_pair_probe(int device, int n, int chunks, float* d32, uint32_t* tmem_addr2, int64_t* cycles);

#ifdef __cplusplus
}
#endif
#endif /* NEON_MOE_H */
