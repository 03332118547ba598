// One-launch layer pass for decode batches of at most 8 tokens (T * top_k <= 32).
//
// At these sizes the layer is a stream over the touched experts' weights (4 experts = 53 MB at
// T = 1) and every extra launch or grid-wide wait is a visible share of the pass, so the whole
// pass is ONE persistent cooperative kernel, one CTA per SM:
//
//   router     every (expert, K slice) dot product is computed once, by CTA expert + E * slice;
//              each CTA then adds the slices, picks the top k and builds the list of distinct
//              experts and their tokens itself (no dispatch pass: the experts are addressed
//              directly);
//   gate_up    the K chunks (128 columns of one 128-row weight tile) of all (expert, tile) items
//              form one flat sequence that is cut into equal runs, one per CTA, so that every SM
//              streams the same number of bytes whatever the number of items.  Weights go
//              HBM -> TMA -> shared memory -> tcgen05.mma.kind::mxf8f6f4.block_scale exactly as
//              in the grouped GEMM (gmm_sm100.cuh).  The token operand (two e4m3 terms of every
//              token's bf16 hidden state, stacked along N) is the same for every expert, so the
//              builder warps write its tiles, one per K chunk, into shared memory ONCE, while the
//              router runs; the MMAs read them in place.  A run that starts or ends inside an
//              item yields a partial sum; partial sums go to global memory
//              [item][part][8 tokens][128 rows] and a per-item counter tells consumers when all
//              parts are there;
//   down       same flat distribution; per expert in its run, a CTA's builders form the token
//              operand tiles from the gate_up partial sums (add the parts in order, bias, clamped
//              SwiGLU, four e4m3 terms) as soon as the gate_up tiles they need are complete, so no
//              grid-wide barrier separates the two products;
//   combine    the CTA that delivers the last partial sum of a 128-column output tile adds, per
//              token, the k slots in slot order (parts in order inside a slot): fixed order, no
//              float atomics.
//
// CTAs signal one another through words in global memory tied to the number of the pass (a
// counter CTA 0 advances at the end of every pass): the router shares are counted by a counter
// that is never reset (it must reach pass x shares), "part p of item i is written" is a flag
// equal to the pass number, the arrival counters of the output tiles wrap to zero by themselves.
// Nothing has to be reset between passes, and the host clears all of it when it reads a
// non-zero status word.  Every wait (mbarrier, flag) is bounded; on a timeout the CTA records a code in
// *status, every role leaves its loops and the kernel returns.
#pragma once
#include "gmm_sm100.cuh"

namespace neon {

constexpr int kDecMaxTok = 8;        // tokens per pass (token operand rows per term)
constexpr int kDecMaxEntries = 32;   // T * top_k
constexpr int kDecParts = 4;         // partial sums an item can have at most
constexpr int kDecStagesMax = 5;         // weight stages of TWO chunks (32 KB in shared memory = 16 KB of nibbles from HBM, + two 512 B scale atoms)
constexpr int kDecBuilderThreads = 384;  // 12 builder warps
constexpr int kDecThreads = 64 + 128 + kDecBuilderThreads;
constexpr int kDecCacheChunks = 24;      // K chunks of a product at most: one token-operand tile each
constexpr int kDecTailBytes = 12 * 1024; // barriers, routing tables, logits
constexpr int kDecMaxSlices = 16;       // K slices of a router dot product (one warp computes one slice of one expert)
constexpr int kDecRouterWarps = 3;      // warps 3..5 of every CTA compute router shares
// Token-operand tiles: gate_up = 2 terms x 8 token rows (2 KB); down = 4 terms x R rows, R = 4 when no
// expert can have more than 4 tokens (T <= 4: 2 KB tiles), else 8 (4 KB tiles).  What the tiles leave
// of the shared memory goes to weight stages: the stream from HBM needs ~2 us x 45 GB/s per SM in flight.
__host__ __device__ constexpr int dec_tile_bytes(int rows_dn) { return rows_dn == 8 ? 4096 : 2048; }
__host__ __device__ constexpr int dec_stages(int rows_dn, int smem_budget) {
    int n = (smem_budget - 1024 - kDecTailBytes - kDecCacheChunks * dec_tile_bytes(rows_dn)) / (32768 + 1024);
    return n > kDecStagesMax ? kDecStagesMax : n;
}

struct DecodeParams {
    const uint16_t *x, *wr, *br;
    const float* logit_bias;
    int T, H, I, E, k;
    float limit, alpha;
    const uint8_t *gu_sfa, *dn_sfa;
    const uint16_t *gu_bias, *dn_bias;
    int gu_m_tiles, dn_m_tiles, nch_h, nch_i;
    int n_slices;              // K slices of the router dot products
    int rows_dn;               // token rows per term of the down product's operand tiles: 4 or 8
    int stages;                // weight stages in use
    uint32_t a_tx_bytes;
    float* router_part;        // [T][E][16 slice slots]; slots >= n_slices are zero
    float* gu_part;            // [item][kDecParts][8 tokens][128 rows]
    float* dn_part;
    unsigned* counters;        // [0] pass number; [1] router shares written since set-up (never reset); [4+256 ..) flags
                               // [items][4 parts] "part written in pass n"; then dn_done[tiles] (arrival counters that wrap to zero)
    int gu_items_cap;          // start of dn_done = 4 + 256 + 4 * gu_items_cap
    unsigned router_expected_extra;  // 0; a test sets 1: the router wait then expects one share more than will ever arrive
    long long wait_limit;      // SM clocks a wait may take
    int* status;
    float* out;                // [T][H]
    int32_t* idx;              // [T][k]
    float* route_w;            // [T][k]
    DispatchArrays d;          // written by CTA 0 (same contents as the dispatch kernels produce)
#ifdef NEON_MOE_INSTRUMENT
    long long* trace;          // [CTA][16] globaltimer stamps of the phases (instrumented builds only)
#endif
};

#ifdef NEON_MOE_INSTRUMENT
__device__ __forceinline__ void dec_stamp(const DecodeParams& p, int slot) {
    if (p.trace) {
        long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t) : : "memory");
        p.trace[blockIdx.x * 16 + slot] = t;
    }
}
#define DEC_STAMP(slot) dec_stamp(p, slot)
#else
#define DEC_STAMP(slot)
#endif

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Bounded wait until *p >= target.  Returns false on timeout (code recorded) or when the CTA aborted.
__device__ __forceinline__ bool wait_counter(const unsigned* p, unsigned target, volatile int* abort_flag, int* status, int code,
                                             long long limit) {
    if (ld_acquire_u32(p) >= target) return true;
    const long long t0 = clock64();
    while (true) {
        for (int i = 0; i < 16; ++i)
            if (ld_acquire_u32(p) >= target) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > limit) {
            *abort_flag = 1;
            atomicCAS(status, 0, code);
            return false;
        }
    }
}

// Long wait on an mbarrier by a whole warp: lane 0 polls with a back-off (a warp that hammers
// try_wait for microseconds competes with the copy and tensor pipes for shared memory), the
// verdict is broadcast.  Same bound and abort protocol as sm100::mbar_wait.
__device__ __forceinline__ bool mbar_wait_quiet(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                                                long long limit, unsigned sleep_ns) {
    int ok = 0;
    if ((threadIdx.x & 31) == 0) {
        const long long t0 = clock64();
        while (true) {
            if (sm100::mbar_peek(bar, parity)) { ok = 1; break; }
            if (*abort_flag) break;
            if (clock64() - t0 > limit) {
                *abort_flag = 1;
                atomicCAS(status, 0, code);
                break;
            }
            if (sleep_ns) __nanosleep(sleep_ns);
        }
    }
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// Release-ordered increment of a counter another CTA polls with ld.acquire: the writes this thread made
// (and, through a preceding CTA barrier, the writes of its CTA) are visible to whoever sees the count.
__device__ __forceinline__ void red_release_add(unsigned* p, unsigned v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_u32(unsigned* p, unsigned v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Arrival counter that wraps to zero at `last`: returns the value before the increment.
__device__ __forceinline__ unsigned atom_acq_rel_inc(unsigned* p, unsigned last) {
    unsigned old;
    asm volatile("atom.acq_rel.gpu.global.inc.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(last) : "memory");
    return old;
}
__device__ __forceinline__ unsigned ld_relaxed_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }

// Bounded wait until the n (<= 4) flags at p all equal `want`.  The polls are relaxed loads, all in
// flight together (an acquire load would order each poll behind the one before it); one fence after
// the flags have been seen orders the reads of the data they guard.
__device__ __forceinline__ bool wait_flags(const unsigned* p, int n, unsigned want, volatile int* abort_flag, int* status, int code,
                                           long long limit) {
    const long long t0 = clock64();
    while (true) {
        unsigned f[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) f[i] = i < n ? ld_relaxed_u32(p + i) : want;
        if (f[0] == want && f[1] == want && f[2] == want && f[3] == want) {
            fence_acq_rel_gpu();
            return true;
        }
        if (*abort_flag) return false;
        if (clock64() - t0 > limit) {
            *abort_flag = 1;
            atomicCAS(status, 0, code);
            return false;
        }
    }
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// The flat chunk distribution of one product: item i = (expert slot, weight tile) owns chunks
// [i * n_chunks, (i + 1) * n_chunks); CTA c owns [c * q, (c + 1) * q).
struct DecPhase {
    int n_items, n_chunks, m_tiles, q, total;
    __device__ void init(int n_exp, int m_tiles_, int n_chunks_, int grid) {
        m_tiles = m_tiles_;
        n_chunks = n_chunks_;
        n_items = n_exp * m_tiles_;
        total = n_items * n_chunks_;
        q = max((total + grid - 1) / grid, (n_chunks_ + kDecParts - 2) / (kDecParts - 1));
    }
    __device__ int first_cta(int item) const { return (item * n_chunks) / q; }
    __device__ int parts(int item) const { return (item * n_chunks + n_chunks - 1) / q - first_cta(item) + 1; }
};

// e4m3 terms of sixteen consecutive K values of one token row with one power-of-two scale: term t =
// RN_e4m3(residual / 2^(sb - 4t - 127)).  Row j of term t is row t * 8 + j of the stacked token
// operand (128-byte-swizzled K-major rows of 128 bytes): 16-byte unit u sits at unit u ^ j.
template <int TERMS>
__device__ __forceinline__ void store_terms16(uint8_t* tile, int rows_per_term, int j, int u, float v[16], int sb) {
#pragma unroll
    for (int t = 0; t < TERMS; ++t) {
        const float inv = __uint_as_float((uint32_t)(254 - (sb - 4 * t)) << 23);
        const float scale = __uint_as_float((uint32_t)(sb - 4 * t) << 23);
        uint32_t w[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * x] * inv, v[4 * x + 1] * inv), __NV_SATFINITE, __NV_E4M3);
            const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * x + 2] * inv, v[4 * x + 3] * inv), __NV_SATFINITE, __NV_E4M3);
            w[x] = (uint32_t)lo | ((uint32_t)hi << 16);
            if (t + 1 < TERMS) {
                __half2_raw blo = __nv_cvt_fp8x2_to_halfraw2(lo, __NV_E4M3), bhi = __nv_cvt_fp8x2_to_halfraw2(hi, __NV_E4M3);
                const float2 flo = __half22float2(*reinterpret_cast<__half2*>(&blo)), fhi = __half22float2(*reinterpret_cast<__half2*>(&bhi));
                v[4 * x] -= flo.x * scale; v[4 * x + 1] -= flo.y * scale; v[4 * x + 2] -= fhi.x * scale; v[4 * x + 3] -= fhi.y * scale;
            }
        }
        const int n = t * rows_per_term + j;
        *reinterpret_cast<uint4*>(tile + (n >> 3) * 1024 + (n & 7) * 128 + ((u ^ (n & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

template <int TERMS>
__device__ __forceinline__ void store_zero16(uint8_t* tile, int rows_per_term, int j, int u) {
#pragma unroll
    for (int t = 0; t < TERMS; ++t) {
        const int n = t * rows_per_term + j;
        *reinterpret_cast<uint4*>(tile + (n >> 3) * 1024 + (n & 7) * 128 + ((u ^ (n & 7)) << 4)) = make_uint4(0, 0, 0, 0);
    }
}

// E8M0 byte of the first term's scale for a row whose largest magnitude is amax (same rule as
// split_rows_stacked_kernel): amax / scale lies in [128, 256), clamped so that every term's scale
// and its inverse stay normal numbers.
__device__ __forceinline__ int term_scale_byte(float amax, int terms) {
    const int ef = (int)((__float_as_uint(amax) >> 23) & 0xffu);
    return amax > 0.f ? min(max(ef - 7, 4 * terms + 1), 250) : 127;
}

// Top k of one token's logits (lgt[E] in shared memory), ties to the lower expert id, softmax over
// the selected logits; run by one warp.  Writes idx[k], w[k] (shared memory).
__device__ __forceinline__ void dec_topk_warp(const float* lgt, int E, int k, int lane, int* idx_out, float* w_out) {
    unsigned long long keys[kMaxExperts / 32];
#pragma unroll
    for (int j = 0; j < kMaxExperts / 32; ++j) {
        const int e = lane + 32 * j;
        keys[j] = (e < E) ? logit_key(lgt[e], e) : 0ull;
    }
    float sel[kMaxTopK];
    int seli[kMaxTopK];
#pragma unroll
    for (int s = 0; s < kMaxTopK; ++s) {
        if (s < k) {
            unsigned long long best = 0ull;
#pragma unroll
            for (int j = 0; j < kMaxExperts / 32; ++j) best = keys[j] > best ? keys[j] : best;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
                best = other > best ? other : best;
            }
            const int e = 0x7fffffff - (int)(uint32_t)(best & 0xffffffffull);
            seli[s] = e;
            sel[s] = lgt[e];
#pragma unroll
            for (int j = 0; j < kMaxExperts / 32; ++j)
                if (lane + 32 * j == e) keys[j] = 0ull;
        }
    }
    if (lane == 0) {
        const float m = sel[0];
        float den = 0.f, pr[kMaxTopK];
#pragma unroll
        for (int s = 0; s < kMaxTopK; ++s)
            if (s < k) {
                pr[s] = expf(sel[s] - m);
                den += pr[s];
            }
#pragma unroll
        for (int s = 0; s < kMaxTopK; ++s)
            if (s < k) {
                idx_out[s] = seli[s];
                w_out[s] = pr[s] / den;
            }
    }
}

// One share of the router: the dot products of one K slice of one expert's router row with every token, by one
// warp (one 16-byte load per lane and token); the share goes to router_part and is counted in *router_count.
__device__ __forceinline__ void dec_router_share(const DecodeParams& p, int unit, int lane, unsigned* router_count) {
    const int T = p.T, H = p.H, E = p.E;
    if (unit < E * p.n_slices) {
        const int nvec = H / 8;
        const int e = unit % E, sl = unit / E;
        const int vps = (nvec + p.n_slices - 1) / p.n_slices, v0 = sl * vps, v1 = min(nvec, v0 + vps);
        float acc[kDecMaxTok];
#pragma unroll
        for (int t = 0; t < kDecMaxTok; ++t) acc[t] = 0.f;
        const uint4* wrow = reinterpret_cast<const uint4*>(p.wr + (size_t)e * H);
        for (int vb = v0; vb < v1; vb += 32) {
            const int v = vb + lane;
            const uint4 wv = v < v1 ? __ldg(wrow + v) : make_uint4(0, 0, 0, 0);
            uint4 xv[kDecMaxTok];
#pragma unroll
            for (int t = 0; t < kDecMaxTok; ++t)
                xv[t] = (t < T && v < v1) ? __ldg(reinterpret_cast<const uint4*>(p.x + (size_t)t * H) + v) : make_uint4(0, 0, 0, 0);
            const uint32_t wa[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int t = 0; t < kDecMaxTok; ++t) {
                const uint32_t xa[4] = {xv[t].x, xv[t].y, xv[t].z, xv[t].w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[t] = fmaf(__uint_as_float(xa[j] << 16), __uint_as_float(wa[j] << 16), acc[t]);
                    acc[t] = fmaf(__uint_as_float(xa[j] & 0xffff0000u), __uint_as_float(wa[j] & 0xffff0000u), acc[t]);
                }
            }
        }
#pragma unroll
        for (int t = 0; t < kDecMaxTok; ++t) {
            if (t < T) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], o);
                if (lane == 0) __stcg(p.router_part + ((size_t)t * E + e) * kDecMaxSlices + sl, acc[t]);
            }
        }
        if (lane == 0) red_release_add(router_count, 1u);
        __syncwarp();
    }
}

// Builder warps (kDecBuilderThreads threads, bt = index among them): every token's largest magnitude, then the gate_up
// token-operand tiles of ALL tokens (two e4m3 terms, 8 token rows per term, one 2 KB tile of stride `TILE` per K chunk;
// the same for every expert).  Ends with the tiles written (the caller fences them for the async proxy).
__device__ __forceinline__ void dec_build_x_tiles(const DecodeParams& p, uint8_t* cache, int TILE, unsigned* s_amax, int bt, int lane) {
    const int T = p.T, H = p.H;
    const int nvec = H / 8;
    for (int t = 0; t < T; ++t) {
        unsigned m = 0u;
        const uint4* xr = reinterpret_cast<const uint4*>(p.x + (size_t)t * H);
        for (int v = bt; v < nvec; v += kDecBuilderThreads) {
            const uint4 xv = __ldg(xr + v);
            const uint32_t a[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) m = max(m, max(a[j] & 0x7fffu, (a[j] >> 16) & 0x7fffu));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0 && m) atomicMax(&s_amax[t], m);
    }
    named_bar_sync(2, kDecBuilderThreads);
    // real tasks (chunk c, token t < T, 16-byte unit u) spread evenly over the builder threads, then zero rows
    for (int task = bt; task < p.nch_h * T * 8; task += kDecBuilderThreads) {
        const int u = task & 7, t = (task >> 3) % T, c = (task >> 3) / T;
        uint8_t* tile = cache + c * TILE;
        const int kk = 128 * c + 16 * u;
        if (kk < H) {
            const uint4* src = reinterpret_cast<const uint4*>(p.x + (size_t)t * H + kk);
            const uint4 r0 = __ldg(src), r1 = __ldg(src + 1);
            const uint32_t raw[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
            float v[16];
#pragma unroll
            for (int x = 0; x < 8; ++x) {
                v[2 * x] = __uint_as_float(raw[x] << 16);
                v[2 * x + 1] = __uint_as_float(raw[x] & 0xffff0000u);
            }
            store_terms16<2>(tile, 8, t, u, v, term_scale_byte(__uint_as_float(s_amax[t] << 16), 2));
        } else {
            store_zero16<2>(tile, 8, t, u);
        }
    }
    for (int task = bt; task < p.nch_h * (8 - T) * 8; task += kDecBuilderThreads) {
        const int u = task & 7, t = T + (task >> 3) % (8 - T), c = (task >> 3) / (8 - T);
        store_zero16<2>(cache + c * TILE, 8, t, u);
    }
}

// Routing tables of a pass in shared memory.
struct DecTables {
    int* idx;        // [32] expert of every entry
    float* w;        // [32] routing weight of every entry
    int* ent_es;     // [32] expert slot of every entry
    int* ent_j;      // [32] row of the entry inside its expert
    int* exp;        // [32] expert id of every slot (ascending)
    int* ntok;       // [32] tokens of every slot
    int* tok;        // [32][8] token of every row
    float* lg;       // [8][E] logits
    int* misc;       // [0] number of distinct experts
};

// The four epilogue warps (q4 = 0..3, meeting at named barrier 1): wait until every router share of this pass has been
// counted, add the slices, top k and softmax per token, then the tables of distinct experts and their tokens.  CTA 0 also
// writes the routing and the dispatch permutation to global memory.  On a timeout the abort flag is set and the tables
// are left unwritten.
__device__ __forceinline__ void dec_route(const DecodeParams& p, const DecTables& tb, int q4, int lane, int cta, unsigned pass,
                                          unsigned* router_count, volatile int* abort_flag) {
    const int T = p.T, E = p.E, k = p.k, n_ent = T * k;
    int* const s_idx = tb.idx; float* const s_w = tb.w; int* const s_ent_es = tb.ent_es; int* const s_ent_j = tb.ent_j;
    int* const s_exp = tb.exp; int* const s_ntok = tb.ntok; int* const s_tok = tb.tok; float* const s_lg = tb.lg;
    int* const s_misc = tb.misc;
    {
        // the router counter is never reset: after this pass's n_router shares it stands at pass * n_router
        // (mod 2^32).  One lane per CTA polls it; the other warps wait at the named barrier.
        if (q4 == 0) {
            const unsigned target = pass * (unsigned)(E * p.n_slices) + p.router_expected_extra;
            if (lane == 0) {
                const long long t0 = clock64();
                while ((int)(ld_acquire_u32(router_count) - target) < 0) {
                    if (*abort_flag || clock64() - t0 > p.wait_limit) {
                        *abort_flag = 1;
                        atomicCAS(p.status, 0, 7);
                        break;
                    }
                }
            }
            __syncwarp();
        }
        named_bar_sync(1, 128);
        const int ok = !*abort_flag;
        if (ok) {
            for (int t = q4; t < T; t += 4) {  // logits, top k, softmax: every CTA, identically
                for (int e = lane; e < E; e += 32) {
                    // all sixteen slice slots in four loads (slots beyond n_slices stay zero from set-up), added in order
                    const float4* part = reinterpret_cast<const float4*>(p.router_part + ((size_t)t * E + e) * kDecMaxSlices);
                    const float4 a = __ldcg(part), b = __ldcg(part + 1), c = __ldcg(part + 2), d = __ldcg(part + 3);
                    float v = ((((((a.x + a.y) + a.z) + a.w) + b.x) + b.y) + b.z) + b.w;
                    v = (((((((v + c.x) + c.y) + c.z) + c.w) + d.x) + d.y) + d.z) + d.w;
                    v += bf16_bits_to_float(p.br[e]);
                    if (p.logit_bias) v += p.logit_bias[e];
                    s_lg[t * E + e] = v;
                }
                __syncwarp();
                dec_topk_warp(s_lg + t * E, E, k, lane, s_idx + t * k, s_w + t * k);
            }
        }
    }
    named_bar_sync(1, 128);
    if (q4 == 0 && lane == 0) DEC_STAMP(3);
    if (q4 == 0 && !*abort_flag) {
        // one entry (token, slot) per lane: slot of its expert among the distinct experts (ascending
        // id), its row among that expert's tokens (ascending token), its place in the sorted order
        const int e = lane < n_ent ? s_idx[lane] : -1 - lane;  // idle lanes get unique negative keys
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        const bool first = lane < n_ent && (__ffs(peers) - 1) == lane;
        const int j_row = __popc(peers & ((1u << lane) - 1u));
        int es = 0, pos = j_row;
        for (int o = 0; o < n_ent; ++o) {
            const int eo = __shfl_sync(0xffffffffu, e, o);
            const bool fo = __shfl_sync(0xffffffffu, (int)first, o) != 0;
            if (eo < e) {
                ++pos;
                if (fo) ++es;
            }
        }
        if (lane < n_ent) {
            s_ent_es[lane] = es;
            s_ent_j[lane] = j_row;
            s_tok[es * 8 + j_row] = lane / k;
            if (first) {
                s_exp[es] = e;
                s_ntok[es] = __popc(peers);
            }
            if (cta == 0) {
                p.idx[lane] = e;
                p.route_w[lane] = s_w[lane];
                p.d.perm[pos] = lane;
                p.d.inv[lane] = pos;
            }
        }
        const unsigned firsts = __ballot_sync(0xffffffffu, first);
        if (lane == 0) s_misc[0] = __popc(firsts);
    }
}

__global__ void __launch_bounds__(kDecThreads, 1)
decode_fused_kernel(const __grid_constant__ CUtensorMap tmGU, const __grid_constant__ CUtensorMap tmGU2,
                    const __grid_constant__ CUtensorMap tmDN, const __grid_constant__ CUtensorMap tmDN2, const DecodeParams p) {
    using namespace sm100;
    const int STAGES = p.stages;
    const int RD = p.rows_dn, TILE = dec_tile_bytes(RD);
    constexpr int ACC_COLS = 32;                // TMEM columns of one accumulator buffer (down: 4 terms x 8 tokens)
    constexpr int SF_UNIT = 2 * ACC_COLS;       // two atoms of unit scales for the token operand
    constexpr int SF_BASE = SF_UNIT + 8;        // weight scale atoms, 2 x 4 columns per stage
    constexpr uint32_t TMEM_COLS = 128;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* stages = smem;                                    // weight boxes, two chunks = 32 KB per stage
    uint8_t* cache = stages + STAGES * 32768;                  // token-operand tiles, one per K chunk
    uint8_t* sfa_ring = cache + kDecCacheChunks * TILE;        // weight scale atoms, 2 x 512 B per stage
    uint8_t* tail = sfa_ring + STAGES * 1024;
    uint64_t* full = reinterpret_cast<uint64_t*>(tail);
    uint64_t* empty = full + kDecStagesMax;
    uint64_t* acc_full = empty + kDecStagesMax;
    uint64_t* acc_empty = acc_full + 2;
    uint64_t* cache_full = acc_empty + 2;   // the builders have written the tiles of the next expert
    uint64_t* cache_free = cache_full + 1;  // every MMA that reads the current tiles has completed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(cache_free + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* s_misc = reinterpret_cast<int*>(tmem_slot + 2);              // [0] n_exp, [1] last-arriver flag, [2] exit flag
    volatile int* s_vote = reinterpret_cast<volatile int*>(tmem_slot + 6);  // [4] epilogue warps' verdicts on a wait
    uint32_t* unit_atom = reinterpret_cast<uint32_t*>(tail + 512);    // 512 B of E8M0 1.0
    int* s_idx = reinterpret_cast<int*>(tail + 1024);                 // [32] expert of every entry
    float* s_w = reinterpret_cast<float*>(s_idx + 32);                // [32] routing weight of every entry
    int* s_ent_es = reinterpret_cast<int*>(s_w + 32);                 // [32] expert slot of every entry
    int* s_ent_j = s_ent_es + 32;                                     // [32] row of the entry inside its expert
    int* s_exp = s_ent_j + 32;                                        // [32] expert id of every slot (ascending)
    int* s_ntok = s_exp + 32;                                         // [32] tokens of every slot
    int* s_tok = s_ntok + 32;                                         // [32][8] token of every row
    unsigned* s_amax = reinterpret_cast<unsigned*>(s_tok + 256);      // [8] largest |x| of each token (bf16 magnitude bits)
    float* s_lg = reinterpret_cast<float*>(s_amax + 8);               // [8][E] logits

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x, grid = gridDim.x;
    if (tid == 0) DEC_STAMP(0);
    const int T = p.T, H = p.H, E = p.E, k = p.k, n_ent = T * k;
    const unsigned pass = __ldcg(p.counters) + 1u;   // written by CTA 0 at the end of the previous pass
    unsigned* const router_count = p.counters + 1;
    unsigned* const gu_flag = p.counters + 4 + 256;
    unsigned* const dn_done = p.counters + 4 + 256 + 4 * p.gu_items_cap;

    // ---- router shares first, before anything else is set up: they need no shared memory, and every CTA waits for them.
    //      Unit u = (expert, K slice) is computed by warp 3 + u % 3 of CTA u / 3: one 16-byte load per lane and token.
    if (warp >= 3 && warp < 3 + kDecRouterWarps) {
        dec_router_share(p, cta * kDecRouterWarps + (warp - 3), lane, router_count);
        if (warp == 3 && lane == 0) DEC_STAMP(2);
    }

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);
        }
        mbar_init(cache_full, kDecBuilderThreads / 32);
        mbar_init(cache_free, 1);
        *abort_flag = 0;
        s_misc[0] = 0;
        fence_barrier_init();
        prefetch_tmap(&tmGU);
        prefetch_tmap(&tmGU2);
        prefetch_tmap(&tmDN);
        prefetch_tmap(&tmDN2);
    }
    if (tid < 128) unit_atom[tid] = 0x7f7f7f7fu;
    if (tid < 8) s_amax[tid] = 0u;
    fence_proxy_async();
    if (warp == 2) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (tid == 0) DEC_STAMP(1);

    if (warp >= 6) {
        // ---- builders, first job: token maxima, then the gate_up token-operand tiles of ALL tokens (the
        //      same for every expert), while the epilogue warps route
        const int bt = tid - 192;
        dec_build_x_tiles(p, cache, TILE, s_amax, bt, lane);
        fence_proxy_async();
        if (bt == 0) DEC_STAMP(9);
    } else if (warp >= 2) {
        // ---- epilogue warps, first job: the router --------------------------------------------------------
        const int q4 = warp - 2;
        const DecTables tb{s_idx, s_w, s_ent_es, s_ent_j, s_exp, s_ntok, s_tok, s_lg, s_misc};
        dec_route(p, tb, q4, lane, cta, pass, router_count, abort_flag);
    }
    __syncthreads();  // routing tables and the gate_up token-operand tiles are in shared memory
    if (tid == 0) DEC_STAMP(4);
    const int n_exp = s_misc[0];
    DecPhase gu, dn;
    gu.init(n_exp, p.gu_m_tiles, p.nch_h, grid);
    dn.init(n_exp, p.dn_m_tiles, p.nch_i, grid);
    const int gu_lo = min(cta * gu.q, gu.total), gu_hi = min(gu_lo + gu.q, gu.total);
    const int dn_lo = min(cta * dn.q, dn.total), dn_hi = min(dn_lo + dn.q, dn.total);
    const float a_bound = p.limit * (p.limit + 1.f);
    const int sb_dn = term_scale_byte(a_bound, 4);

    if (*abort_flag) {
        // nothing was started: fall through to the exit protocol
    } else if (warp == 0) {
        // ---- weight producer: per stage two K chunks = one 256 x 128 box (TMA, nibbles expanded to bytes) + their
        //      scale atoms; the odd last chunk of a run travels alone.  Divisions happen once per run of an item;
        //      stage, phase and box index are carried incrementally.
        int s = 0, par = 0;
        for (int phase = 0; phase < 2; ++phase) {
            const DecPhase& ph = phase ? dn : gu;
            const CUtensorMap* map1 = phase ? &tmDN : &tmGU;
            const CUtensorMap* map2 = phase ? &tmDN2 : &tmGU2;
            const uint8_t* sfa = phase ? p.dn_sfa : p.gu_sfa;
            const int lo = phase ? dn_lo : gu_lo, hi = phase ? dn_hi : gu_hi;
            for (int f = lo; f < hi;) {
                const int item = f / ph.n_chunks, c0 = f - item * ph.n_chunks;
                const int c1 = min(ph.n_chunks, c0 + (hi - f));
                const int es = item / ph.m_tiles, m = item - es * ph.m_tiles;
                uint32_t box = (uint32_t)((s_exp[es] * ph.m_tiles + m) * ph.n_chunks + c0);
                for (int left = c1 - c0; left > 0; left -= 2, box += 2) {
                    const int ok = mbar_wait(&empty[s], par ^ 1, abort_flag, p.status, 1, p.wait_limit);
                    if (!__all_sync(0xffffffffu, ok)) goto roles_done;
                    if (elect_one()) {
                        if (left >= 2) {
                            mbar_expect_tx(&full[s], 2 * (p.a_tx_bytes + 512));
                            tma_load_2d(stages + s * 32768, map2, &full[s], 0, (int)(box * 128));
                            bulk_load(sfa_ring + s * 1024, sfa + (size_t)box * 512, 1024, &full[s]);
                        } else {
                            mbar_expect_tx(&full[s], p.a_tx_bytes + 512);
                            tma_load_2d(stages + s * 32768, map1, &full[s], 0, (int)(box * 128));
                            bulk_load(sfa_ring + s * 1024, sfa + (size_t)box * 512, 512, &full[s]);
                        }
                    }
                    __syncwarp();
                    if (++s == STAGES) { s = 0; par ^= 1; }
                }
                f += c1 - c0;
            }
        }
        // every stage must have been released before the CTA may retire (late asynchronous arrives)
        for (int i = 0; i < STAGES; ++i) {
            const int ok = mbar_wait(&empty[s], par ^ 1, abort_flag, p.status, 6, p.wait_limit);
            if (!__all_sync(0xffffffffu, ok)) goto roles_done;
            if (++s == STAGES) { s = 0; par ^= 1; }
        }
    } else if (warp == 1) {
        // ---- MMA issuer -------------------------------------------------------------------------------
        if (elect_one()) {
            tc_copy_sf(tmem_base + SF_UNIT, make_sf_desc(smem_u32(unit_atom)));
            tc_copy_sf(tmem_base + SF_UNIT + 4, make_sf_desc(smem_u32(unit_atom)));
        }
        __syncwarp();
        const uint32_t stage_base = smem_u32(stages), cache_base = smem_u32(cache), sfa_base = smem_u32(sfa_ring);
        int s = 0, par = 0, seg = 0, frees = 0, fulls = 0, cur_es = -1;
        for (int phase = 0; phase < 2; ++phase) {
            const DecPhase& ph = phase ? dn : gu;
            const int lo = phase ? dn_lo : gu_lo, hi = phase ? dn_hi : gu_hi;
            const uint32_t idesc0 = make_idesc_bs(5, 0, phase ? (uint32_t)(4 * RD) : 16u, 0, 0);
            for (int f = lo; f < hi; ++seg) {
                const int item = f / ph.n_chunks, c0 = f - item * ph.n_chunks;
                const int c1 = min(ph.n_chunks, c0 + (hi - f));
                int ok;
                if (phase) {
                    const int es = item / ph.m_tiles;
                    if (es != cur_es) {  // the tiles of the next expert: release the current ones, wait for the builders
                        if (cur_es >= 0) {
                            if (elect_one()) tc_commit(cache_free);
                            __syncwarp();
                            ++frees;
                        }
                        ok = mbar_wait(cache_full, fulls & 1, abort_flag, p.status, 9, p.wait_limit);
                        if (!__all_sync(0xffffffffu, ok)) goto roles_done;
                        if (lane == 0 && fulls == 0) DEC_STAMP(15);
                        ++fulls;
                        cur_es = es;
                    }
                }
                const int b = seg & 1, apar = (seg >> 1) & 1;
                ok = mbar_wait(&acc_empty[b], apar ^ 1, abort_flag, p.status, 2, p.wait_limit);
                if (!__all_sync(0xffffffffu, ok)) goto roles_done;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + b * ACC_COLS;
                uint32_t b_tile = cache_base + c0 * TILE, first = 0;
                for (int left = c1 - c0; left > 0; left -= 2) {
                    ok = mbar_wait(&full[s], par, abort_flag, p.status, 3, p.wait_limit);
                    if (!__all_sync(0xffffffffu, ok)) goto roles_done;
                    if (lane == 0 && !phase && f == lo && first == 0) DEC_STAMP(11);
                    tc_fence_after();
                    if (elect_one()) {
                        const uint32_t st = stage_base + s * 32768, sf_tmem = tmem_base + SF_BASE + s * 8, sf_smem = sfa_base + s * 1024;
#pragma unroll
                        for (int kc = 0; kc < 2; ++kc) {
                            if (kc < left) {
                                tc_copy_sf(sf_tmem + 4 * kc, make_sf_desc(sf_smem + 512 * kc));
                                const uint64_t a_desc = make_sw128_desc(st + 16384 * kc), b_desc = make_sw128_desc(b_tile + kc * TILE);
#pragma unroll
                                for (int j = 0; j < 4; ++j)
                                    mma_mxf8f6f4(d_tmem, a_desc + 2 * j, b_desc + 2 * j, idesc0 + j * (1u << 29), sf_tmem + 4 * kc,
                                                 tmem_base + SF_UNIT, first | (uint32_t)(kc | j));
                            }
                        }
                        tc_commit(&empty[s]);
                    }
                    __syncwarp();
                    first = 1;
                    b_tile += 2 * TILE;
                    if (++s == STAGES) { s = 0; par ^= 1; }
                }
                if (elect_one()) tc_commit(&acc_full[b]);
                __syncwarp();
                f += c1 - c0;
            }
            if (!phase) {  // the gate_up tiles are no longer read once these MMAs have completed
                if (elect_one()) tc_commit(cache_free);
                __syncwarp();
                ++frees;
            }
            if (lane == 0) DEC_STAMP(5 + phase);
        }
        // the last arrive on cache_free must have landed before the CTA retires
        if (elect_one()) tc_commit(cache_free);
        __syncwarp();
        ++frees;
        {
            const int ok = mbar_wait(cache_free, (frees - 1) & 1, abort_flag, p.status, 10, p.wait_limit);
            if (!__all_sync(0xffffffffu, ok)) goto roles_done;
        }
    } else if (warp < 6) {
        // ---- epilogue: accumulator -> partial sum in global memory; last arriver of an output tile combines
        const int q = warp & 3;
        const int et = tid - 64;  // 0..127 among the epilogue threads
        int seg = 0;
        for (int phase = 0; phase < 2; ++phase) {
            const DecPhase& ph = phase ? dn : gu;
            const int lo = phase ? dn_lo : gu_lo, hi = phase ? dn_hi : gu_hi;
            float* part_base = phase ? p.dn_part : p.gu_part;
            for (int f = lo; f < hi; ++seg) {
                const int item = f / ph.n_chunks, c0 = f - item * ph.n_chunks;
                const int c1 = min(ph.n_chunks, c0 + (hi - f));
                const int es = item / ph.m_tiles, m = item - es * ph.m_tiles;
                const int part = cta - ph.first_cta(item);
                const int b = seg & 1, apar = (seg >> 1) & 1;
                {
                    // the four epilogue warps meet at named barriers below, so they must leave together: each
                    // posts its verdict on the wait, and all of them go on only if all four saw the accumulator
                    const int ok = (int)mbar_wait_quiet(&acc_full[b], apar, abort_flag, p.status, 4, p.wait_limit, 0);
                    if (lane == 0) s_vote[q] = ok;
                    named_bar_sync(1, 128);
                    if (!(s_vote[0] & s_vote[1] & s_vote[2] & s_vote[3])) goto roles_done;
                }
                tc_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + b * ACC_COLS;
                float v[8];
                tmem_ld8(taddr, v);
                if (phase && RD == 4) {
                    // four terms x four token rows in 16 columns: (term 0 | term 1), (term 2 | term 3)
                    float u[8];
                    tmem_ld8(taddr + 8, u);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        v[i] = fmaf(v[4 + i], 0.0625f, v[i]);
                        v[i] = fmaf(u[i], 0.00390625f, v[i]);
                        v[i] = fmaf(u[4 + i], 0.000244140625f, v[i]);
                        v[4 + i] = 0.f;
                    }
                } else {
                    float fct = 1.f;
                    const int terms = phase ? 4 : 2;
                    for (int t = 1; t < terms; ++t) {
                        fct *= 0.0625f;
                        float u[8];
                        tmem_ld8(taddr + 8 * t, u);
#pragma unroll
                        for (int i = 0; i < 8; ++i) v[i] = fmaf(u[i], fct, v[i]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[b]);
                // rows of the token operand: gate_up = token t (all tokens), down = the expert's j-th token
                const int nrow = phase ? s_ntok[es] : T;
                float* dst = part_base + ((size_t)item * kDecParts + part) * 1024 + 32 * q + lane;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (j < nrow) {
                        const int sb = phase ? sb_dn : term_scale_byte(__uint_as_float(s_amax[j] << 16), 2);
                        __stcg(dst + j * 128, v[j] * __uint_as_float((uint32_t)sb << 23));
                    }
                }
                named_bar_sync(1, 128);  // the 128 threads' stores precede the one release below
                if (!phase) {
                    if (et == 0) st_release_u32(gu_flag + 4 * item + part, pass);
                    if (et == 0) DEC_STAMP(10);
                } else {
                    if (et == 0) {
                        unsigned expected = 0;
                        for (int x = 0; x < n_exp; ++x) expected += (unsigned)dn.parts(x * dn.m_tiles + m);
                        s_misc[1] = (atom_acq_rel_inc(&dn_done[m], expected - 1u) == expected - 1u);
                    }
                    named_bar_sync(1, 128);
                    const bool last = s_misc[1] != 0;
                    named_bar_sync(1, 128);  // everybody has read the flag before the next segment rewrites it
                    if (last) {
                        // out[t, col] = sum over slots (in order) of w * (sum of parts (in order) + bias)
                        const int col = 128 * m + et;
                        if (col < H) {
                            for (int t = 0; t < T; ++t) {
                                // the k slots' parts, all loads in flight together (a chain of dependent L2 round trips otherwise)
                                float y[kMaxTopK][kDecParts], bias[kMaxTopK];
#pragma unroll
                                for (int s = 0; s < kMaxTopK; ++s) {
                                    bias[s] = 0.f;
#pragma unroll
                                    for (int pp = 0; pp < kDecParts; ++pp) y[s][pp] = 0.f;
                                    if (s < k) {
                                        const int ent = t * k + s, xs = s_ent_es[ent], jj = s_ent_j[ent];
                                        const int it = xs * dn.m_tiles + m, np = dn.parts(it);
                                        bias[s] = bf16_bits_to_float(p.dn_bias[(size_t)s_exp[xs] * H + col]);
#pragma unroll
                                        for (int pp = 0; pp < kDecParts; ++pp)
                                            if (pp < np) y[s][pp] = __ldcg(p.dn_part + ((size_t)it * kDecParts + pp) * 1024 + jj * 128 + et);
                                    }
                                }
                                float o = 0.f;
#pragma unroll
                                for (int s = 0; s < kMaxTopK; ++s)
                                    if (s < k) o += s_w[t * k + s] * ((((y[s][0] + y[s][1]) + y[s][2]) + y[s][3]) + bias[s]);
                                p.out[(size_t)t * H + col] = o;
                            }
                        }
                    }
                }
                f += c1 - c0;
            }
        }
    } else {
        // ---- builders, second job: per expert in this CTA's down run, the token-operand tiles from the
        //      gate_up partial sums (parts in order, bias, clamped SwiGLU, four e4m3 terms)
        const int bt = tid - 192;
        if (cta == 0) {  // histogram and offsets over all experts, as the dispatch kernels write them
            for (int e = bt; e <= E; e += kDecBuilderThreads) {
                int c = 0, below = 0;
                for (int i = 0; i < n_ent; ++i) {
                    c += s_idx[i] == e;
                    below += s_idx[i] < e;
                }
                if (e < E) p.d.count[e] = c;
                p.d.offset[e] = below;
            }
        }
        int epoch = 0;
        for (int f = dn_lo; f < dn_hi; ++epoch) {
            // the run of this expert: [f, f_end); the chunks it needs: those of its single item, or all
            const int es = (f / dn.n_chunks) / dn.m_tiles;
            const int f_exp_end = (es + 1) * dn.m_tiles * dn.n_chunks;
            const int f_end = min(dn_hi, f_exp_end);
            const int item0 = f / dn.n_chunks, item1 = (f_end - 1) / dn.n_chunks;
            int c_lo = 0, c_hi = dn.n_chunks;
            if (item0 == item1) {
                c_lo = f - item0 * dn.n_chunks;
                c_hi = f_end - item0 * dn.n_chunks;
            }
            // the tiles in place are still being read until the MMA warp says otherwise
            if (!mbar_wait_quiet(cache_free, epoch & 1, abort_flag, p.status, 5, p.wait_limit, 400)) goto roles_done;
            if (bt == 0 && epoch == 0) DEC_STAMP(12);
            const int ntok = s_ntok[es];
            // real tasks (chunk c, row j < ntok, 4 channels) spread evenly over the builder threads, then zero rows
            for (int task = bt; task < (c_hi - c_lo) * ntok * 32; task += kDecBuilderThreads) {
                const int w4 = task & 31, j = (task >> 5) % ntok, c = c_lo + (task >> 5) / ntok;
                const int u = w4 >> 2;                  // 16-byte unit of the row; this task fills 4 of its bytes per term
                uint8_t* tile = cache + c * TILE;
                const int ch0 = 128 * c + 4 * w4;       // first of this task's 4 channels
                const int gm = ch0 >> 6;                // gate_up tile holding them: gate row 32 * ((ch % 64) / 16) + ch % 16, linear row 16 further
                float v[4] = {0.f, 0.f, 0.f, 0.f};
                if (gm < gu.m_tiles && ch0 < p.I) {
                    const int gitem = es * gu.m_tiles + gm, np = gu.parts(gitem);
                    const uint4 braw = __ldg(reinterpret_cast<const uint4*>(p.gu_bias + (size_t)s_exp[es] * 2 * p.I + 2 * ch0));  // 4 (gate, linear) pairs
                    if (!wait_flags(gu_flag + 4 * gitem, np, pass, abort_flag, p.status, 8, p.wait_limit)) goto roles_done;
                    if (bt == 0 && epoch == 0) DEC_STAMP(13);
                    const int tok = s_tok[es * 8 + j];
                    const int row_g = 32 * ((ch0 & 63) >> 4) + (ch0 & 15);
                    float4 gs = make_float4(0.f, 0.f, 0.f, 0.f), ls = gs;
                    for (int pp = 0; pp < np; ++pp) {
                        const float* src = p.gu_part + ((size_t)gitem * kDecParts + pp) * 1024 + tok * 128 + row_g;
                        const float4 g4 = __ldcg(reinterpret_cast<const float4*>(src)), l4 = __ldcg(reinterpret_cast<const float4*>(src + 16));
                        gs.x += g4.x; gs.y += g4.y; gs.z += g4.z; gs.w += g4.w;
                        ls.x += l4.x; ls.y += l4.y; ls.z += l4.z; ls.w += l4.w;
                    }
                    const float gsum[4] = {gs.x, gs.y, gs.z, gs.w}, lsum[4] = {ls.x, ls.y, ls.z, ls.w};
                    const uint32_t bw[4] = {braw.x, braw.y, braw.z, braw.w};
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        const float gg = fminf(gsum[x] + __uint_as_float(bw[x] << 16), p.limit);
                        const float ll = fminf(fmaxf(lsum[x] + __uint_as_float(bw[x] & 0xffff0000u), -p.limit), p.limit);
                        v[x] = gg / (1.f + expf(-p.alpha * gg)) * (ll + 1.f);
                    }
                }
#pragma unroll
                for (int t = 0; t < 4; ++t) {  // four e4m3 terms, 4 bytes each
                    const float inv = __uint_as_float((uint32_t)(254 - (sb_dn - 4 * t)) << 23);
                    const float scale = __uint_as_float((uint32_t)(sb_dn - 4 * t) << 23);
                    const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[0] * inv, v[1] * inv), __NV_SATFINITE, __NV_E4M3);
                    const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[2] * inv, v[3] * inv), __NV_SATFINITE, __NV_E4M3);
                    const int n = t * RD + j;
                    *reinterpret_cast<uint32_t*>(tile + (n >> 3) * 1024 + (n & 7) * 128 + ((u ^ (n & 7)) << 4) + ((w4 & 3) << 2)) =
                        (uint32_t)lo | ((uint32_t)hi << 16);
                    if (t < 3) {
                        __half2_raw blo = __nv_cvt_fp8x2_to_halfraw2(lo, __NV_E4M3), bhi = __nv_cvt_fp8x2_to_halfraw2(hi, __NV_E4M3);
                        const float2 flo = __half22float2(*reinterpret_cast<__half2*>(&blo)), fhi = __half22float2(*reinterpret_cast<__half2*>(&bhi));
                        v[0] -= flo.x * scale; v[1] -= flo.y * scale; v[2] -= fhi.x * scale; v[3] -= fhi.y * scale;
                    }
                }
            }
            for (int task = bt; task < (c_hi - c_lo) * (RD - ntok) * 8; task += kDecBuilderThreads) {
                const int u = task & 7, j = ntok + (task >> 3) % (RD - ntok), c = c_lo + (task >> 3) / (RD - ntok);
                store_zero16<4>(cache + c * TILE, RD, j, u);
            }
            fence_proxy_async();
            __syncwarp();
            if (bt == 0 && epoch == 0) DEC_STAMP(14);
            if (lane == 0) mbar_arrive(cache_full);
            f = f_end;
        }
    }
roles_done:
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) DEC_STAMP(7);
    if (*abort_flag) {
        const long long t0 = clock64();  // copies that were already issued get time to land
        while (clock64() - t0 < 2000000ll) {}
    }
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
    // the next pass gets the next number (a pass that gave up advances it too: its flags then mean nothing)
    if (cta == 0 && tid == 0) __stcg(p.counters, pass);
    if (tid == 0) DEC_STAMP(8);
}

}  // namespace neon
