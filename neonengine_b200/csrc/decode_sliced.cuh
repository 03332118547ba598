// One-launch layer pass for the smallest decode batches (T <= 4), sliced by intermediate channel.
//
// decode_fused_kernel (decode_fused.cuh) cuts each product into equal runs of K chunks, which balances the
// stream perfectly but makes the down product of every CTA wait for gate_up results of many other CTAs: at
// T = 1 that wait (flags through global memory, partial sums re-read, tiles rebuilt) was measured at ~8 of
// the pass's 36 us.  This kernel cuts the layer the other way.  A unit is (expert, 128 intermediate
// channels): the CTA that owns it computes those channels' gate and linear rows over the whole hidden
// dimension (two 128-row gate_up weight tiles x all K chunks), applies bias, clamped SwiGLU and the routing
// weight in its own epilogue, writes the result as the token operand of the down product into its own shared
// memory, and at once multiplies it with the matching K chunk of every down weight tile.  Nothing a CTA
// needs after the routing comes from another CTA.  What is left is a sum: every CTA accumulates its units'
// contributions to out[T][H] in shared memory, writes them once, the grid meets at ONE barrier and every CTA
// adds a slice of the columns over all CTAs in CTA order (fixed order, no float atomics).
//
//   weights    the same tensor-core layout and tensor maps as everywhere else: 128 x 128 boxes, nibbles
//              expanded by TMA, scale atoms by bulk copies, tcgen05.mma.kind::mxf8f6f4.block_scale;
//   gate_up    token operand = two e4m3 terms of every token's hidden state (built once per pass while the
//              router runs, as in decode_fused_kernel), N = 16;
//   down       token operand = four e4m3 terms of w[token, expert] * SwiGLU, all T tokens as rows (zero
//              for tokens the expert does not serve), N = 16 (T <= 4);
//   units      T = 1: 4 experts x 23 chunks = 92 units on 92 of the 148 SMs, one each.
//
// Measured at the gpt-oss-20b shapes (one pass, replayed from a graph): T = 1 36.3 us against 35.1-36.5 us for
// decode_fused_kernel, T = 2 57.7 against 49.9, T = 4 83.0 against 74.7.  The wait between the two products is gone
// (the down MMAs start 1.5 us after the last gate_up MMA), but a unit is 69 weight boxes on one SM where the equal-run
// cut gives every SM 42: with four stages in flight an SM streams ~46 GB/s (its MMA warp waits for data 72 % of the
// gate_up phase), so 92 SMs draw 4.3 TB/s and the stream takes 16 us instead of 8.  Asking for the unit's boxes in L2
// ahead of the stage copies (cp.async.bulk.prefetch.L2, all at once) delayed the first copy by 4 us and changed
// nothing afterwards.  The kernel therefore stays an option (decode_sliced, default 0).
//
// Router, routing tables, pass counter and status protocol are decode_fused_kernel's (shared functions).
// Every wait is bounded; the epilogue warps, which meet at named barriers, agree on leaving by a vote.
#pragma once
#include "decode_fused.cuh"

namespace neon {

constexpr int kDec2MaxTok = 4;       // tokens per pass
constexpr int kDec2XTile = 2048;     // gate_up token-operand tile of one K chunk: 2 terms x 8 rows x 128 B
constexpr int kDec2ATile = 2048;     // down token-operand tile of the unit's chunk: 4 terms x 4 rows x 128 B
constexpr int kDec2DnSlots = 8;      // accumulators of the down product in flight (one per 128-row output tile)
constexpr uint32_t kDec2TmemCols = 256;
__host__ __device__ constexpr int dec2_y_bytes(int T, int dn_m_tiles) { return (T * dn_m_tiles * 128 * 4 + 1023) / 1024 * 1024; }
__host__ __device__ constexpr int dec2_stages(int T, int dn_m_tiles, int smem_budget) {
    int n = (smem_budget - 1024 - kDecTailBytes - kDecCacheChunks * kDec2XTile - kDec2ATile - dec2_y_bytes(T, dn_m_tiles)) / (32768 + 1024);
    return n > kDecStagesMax ? kDecStagesMax : n;
}

__global__ void __launch_bounds__(kDecThreads, 1)
decode_sliced_kernel(const __grid_constant__ CUtensorMap tmGU, const __grid_constant__ CUtensorMap tmGU2,
                     const __grid_constant__ CUtensorMap tmDN, const DecodeParams p) {
    using namespace sm100;
    const int STAGES = p.stages;
    constexpr int GU_COLS = 16;                       // one gate_up accumulator: 2 terms x 8 tokens
    constexpr int DN_COLS = 16;                       // one down accumulator: 4 terms x 4 tokens
    constexpr int DN_BASE = 2 * GU_COLS;              // two gate_up accumulators first
    constexpr int SF_UNIT = DN_BASE + kDec2DnSlots * DN_COLS;  // two atoms of unit scales for the token operands
    constexpr int SF_BASE = SF_UNIT + 8;              // weight scale atoms, 2 x 4 columns per stage
    static_assert(SF_BASE + kDecStagesMax * 8 <= (int)kDec2TmemCols, "tensor memory columns");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int HP = p.dn_m_tiles * 128;                         // padded output columns
    uint8_t* stages = smem;                                    // weight boxes, two per stage = 32 KB
    uint8_t* cache = stages + STAGES * 32768;                  // gate_up token-operand tiles, one per K chunk
    uint8_t* atile = cache + kDecCacheChunks * kDec2XTile;     // down token-operand tile of the current unit
    float* yacc = reinterpret_cast<float*>(atile + kDec2ATile);  // [T][HP] this CTA's contribution to the output
    uint8_t* sfa_ring = reinterpret_cast<uint8_t*>(yacc) + dec2_y_bytes(p.T, p.dn_m_tiles);  // weight scale atoms, 2 x 512 B per stage
    uint8_t* tail = sfa_ring + STAGES * 1024;
    uint64_t* full = reinterpret_cast<uint64_t*>(tail);
    uint64_t* empty = full + kDecStagesMax;
    uint64_t* gu_full = empty + kDecStagesMax;   // [2] a gate_up accumulator is complete
    uint64_t* a_full = gu_full + 2;              // the unit's down token operand is in shared memory
    uint64_t* dn_full = a_full + 1;              // [4] a down accumulator is complete
    uint64_t* dn_empty = dn_full + kDec2DnSlots; // [4] ... and has been read
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dn_empty + kDec2DnSlots);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* s_misc = reinterpret_cast<int*>(tmem_slot + 2);                     // [0] n_exp
    volatile int* s_vote = reinterpret_cast<volatile int*>(tmem_slot + 6);   // [2][4] epilogue warps' verdicts, alternating sets
    uint32_t* unit_atom = reinterpret_cast<uint32_t*>(tail + 512);    // 512 B of E8M0 1.0
    int* s_idx = reinterpret_cast<int*>(tail + 1024);
    float* s_w = reinterpret_cast<float*>(s_idx + 32);
    int* s_ent_es = reinterpret_cast<int*>(s_w + 32);
    int* s_ent_j = s_ent_es + 32;
    int* s_exp = s_ent_j + 32;
    int* s_ntok = s_exp + 32;
    int* s_tok = s_ntok + 32;
    unsigned* s_amax = reinterpret_cast<unsigned*>(s_tok + 256);
    float* s_lg = reinterpret_cast<float*>(s_amax + 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x, grid = gridDim.x;
    if (tid == 0) DEC_STAMP(0);
    const int T = p.T, H = p.H, k = p.k;
    const unsigned pass = __ldcg(p.counters) + 1u;   // written by CTA 0 at the end of the previous pass
    unsigned* const router_count = p.counters + 1;
    // the grid barrier counts arrivals in a counter that is never reset: after the n-th pass of THIS kernel it stands at
    // n x grid (the other one-launch kernel shares the pass number but not this barrier)
    unsigned* const grid_count = p.counters + 2;
    const unsigned sliced_pass = __ldcg(p.counters + 3) + 1u;

    if (warp >= 3 && warp < 3 + kDecRouterWarps) {
        dec_router_share(p, cta * kDecRouterWarps + (warp - 3), lane, router_count);
        if (warp == 3 && lane == 0) DEC_STAMP(2);
    }

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(&gu_full[0], 1);
        mbar_init(&gu_full[1], 1);
        mbar_init(a_full, 1);
        for (int b = 0; b < kDec2DnSlots; ++b) {
            mbar_init(&dn_full[b], 1);
            mbar_init(&dn_empty[b], 4);
        }
        *abort_flag = 0;
        s_misc[0] = 0;
        fence_barrier_init();
        prefetch_tmap(&tmGU);
        prefetch_tmap(&tmGU2);
        prefetch_tmap(&tmDN);
    }
    if (tid < 128) unit_atom[tid] = 0x7f7f7f7fu;
    if (tid < 8) s_amax[tid] = 0u;
    if (tid < 8) s_vote[tid] = 1;
    fence_proxy_async();
    if (warp == 2) tmem_alloc(tmem_slot, kDec2TmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (tid == 0) DEC_STAMP(1);

    if (warp >= 6) {
        // ---- builders: token maxima and the gate_up token-operand tiles; the output accumulator and the down
        //      tile start as zeros (rows of absent tokens stay zero for the whole pass)
        const int bt = tid - 192;
        dec_build_x_tiles(p, cache, kDec2XTile, s_amax, bt, lane);
        for (int i = bt; i < T * HP / 4; i += kDecBuilderThreads) reinterpret_cast<float4*>(yacc)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int i = bt; i < kDec2ATile / 16; i += kDecBuilderThreads) reinterpret_cast<uint4*>(atile)[i] = make_uint4(0, 0, 0, 0);
        fence_proxy_async();
        if (bt == 0) DEC_STAMP(9);
    } else if (warp >= 2) {
        const DecTables tb{s_idx, s_w, s_ent_es, s_ent_j, s_exp, s_ntok, s_tok, s_lg, s_misc};
        dec_route(p, tb, warp - 2, lane, cta, pass, router_count, abort_flag);
    }
    __syncthreads();  // routing tables, token-operand tiles and zeroed accumulators are in shared memory
    if (tid == 0) DEC_STAMP(4);
    const int n_exp = s_misc[0];
    const int n_units = n_exp * p.nch_i;   // unit u = (expert slot u / nch_i, down K chunk u % nch_i)
    const float a_bound = p.limit * (p.limit + 1.f);
    const int sb_dn = term_scale_byte(a_bound, 4);

    if (*abort_flag) {
        // nothing was started: fall through to the exit protocol
    } else if (warp == 0) {
        // ---- weight producer: per unit the gate_up tiles 2j and 2j + 1 over all K chunks (two chunks = one 256-row
        //      box per stage), then K chunk j of every down tile (two tiles per stage, one box each)
        int s = 0, par = 0;
        for (int u = cta; u < n_units; u += grid) {
            const int es = u / p.nch_i, j = u - es * p.nch_i, e = s_exp[es];
            const int n_mt = min(2, p.gu_m_tiles - 2 * j);
            for (int h = 0; h < n_mt; ++h) {
                uint32_t box = (uint32_t)((e * p.gu_m_tiles + 2 * j + h) * p.nch_h);
                for (int left = p.nch_h; left > 0; left -= 2, box += 2) {
                    const int ok = mbar_wait(&empty[s], par ^ 1, abort_flag, p.status, 1, p.wait_limit);
                    if (!__all_sync(0xffffffffu, ok)) goto roles_done;
                    if (elect_one()) {
                        if (left >= 2) {
                            mbar_expect_tx(&full[s], 2 * (p.a_tx_bytes + 512));
                            tma_load_2d(stages + s * 32768, &tmGU2, &full[s], 0, (int)(box * 128));
                            bulk_load(sfa_ring + s * 1024, p.gu_sfa + (size_t)box * 512, 1024, &full[s]);
                        } else {
                            mbar_expect_tx(&full[s], p.a_tx_bytes + 512);
                            tma_load_2d(stages + s * 32768, &tmGU, &full[s], 0, (int)(box * 128));
                            bulk_load(sfa_ring + s * 1024, p.gu_sfa + (size_t)box * 512, 512, &full[s]);
                        }
                    }
                    __syncwarp();
                    if (++s == STAGES) { s = 0; par ^= 1; }
                }
            }
            for (int m = 0; m < p.dn_m_tiles; m += 2) {
                const int nb = min(2, p.dn_m_tiles - m);
                const int ok = mbar_wait(&empty[s], par ^ 1, abort_flag, p.status, 1, p.wait_limit);
                if (!__all_sync(0xffffffffu, ok)) goto roles_done;
                if (elect_one()) {
                    mbar_expect_tx(&full[s], nb * (p.a_tx_bytes + 512));
                    for (int i = 0; i < nb; ++i) {
                        const uint32_t box = (uint32_t)((e * p.dn_m_tiles + m + i) * p.nch_i + j);
                        tma_load_2d(stages + s * 32768 + i * 16384, &tmDN, &full[s], 0, (int)(box * 128));
                        bulk_load(sfa_ring + s * 1024 + i * 512, p.dn_sfa + (size_t)box * 512, 512, &full[s]);
                    }
                }
                __syncwarp();
                if (++s == STAGES) { s = 0; par ^= 1; }
            }
        }
        for (int i = 0; i < STAGES; ++i) {  // late asynchronous arrives must land before the CTA retires
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
        const uint32_t idesc_gu = make_idesc_bs(5, 0, (uint32_t)GU_COLS, 0, 0), idesc_dn = make_idesc_bs(5, 0, (uint32_t)DN_COLS, 0, 0);
        const uint64_t a_tile_desc = make_sw128_desc(smem_u32(atile));
        int s = 0, par = 0, it = 0, n_dn = 0;
#ifdef NEON_MOE_INSTRUMENT
        long long wait_cyc = 0, wait_dn = 0, wait_slot = 0;
#endif
        for (int u = cta; u < n_units; u += grid, ++it) {
            const int es = u / p.nch_i, j = u - es * p.nch_i;
            const int n_mt = min(2, p.gu_m_tiles - 2 * j);
            // gate_up: accumulator h may be overwritten: its last reader (the previous unit's epilogue) finished before that
            // unit's down operand was announced, which this warp waited for before it issued that unit's down MMAs
            for (int h = 0; h < n_mt; ++h) {
                const uint32_t d_tmem = tmem_base + h * GU_COLS;
                uint32_t b_tile = cache_base, first = 0;
                for (int left = p.nch_h; left > 0; left -= 2) {
#ifdef NEON_MOE_INSTRUMENT
                    const long long tw0 = clock64();
#endif
                    const int ok = mbar_wait(&full[s], par, abort_flag, p.status, 3, p.wait_limit);
                    if (!__all_sync(0xffffffffu, ok)) goto roles_done;
#ifdef NEON_MOE_INSTRUMENT
                    wait_cyc += clock64() - tw0;
#endif
                    if (lane == 0 && it == 0 && h == 0 && first == 0) DEC_STAMP(11);
                    tc_fence_after();
                    if (elect_one()) {
                        const uint32_t st = stage_base + s * 32768, sf_tmem = tmem_base + SF_BASE + s * 8, sf_smem = sfa_base + s * 1024;
#pragma unroll
                        for (int kc = 0; kc < 2; ++kc) {
                            if (kc < left) {
                                tc_copy_sf(sf_tmem + 4 * kc, make_sf_desc(sf_smem + 512 * kc));
                                const uint64_t a_desc = make_sw128_desc(st + 16384 * kc), b_desc = make_sw128_desc(b_tile + kc * kDec2XTile);
#pragma unroll
                                for (int jj = 0; jj < 4; ++jj)
                                    mma_mxf8f6f4(d_tmem, a_desc + 2 * jj, b_desc + 2 * jj, idesc_gu + jj * (1u << 29), sf_tmem + 4 * kc,
                                                 tmem_base + SF_UNIT, first | (uint32_t)(kc | jj));
                            }
                        }
                        tc_commit(&empty[s]);
                    }
                    __syncwarp();
                    first = 1;
                    b_tile += 2 * kDec2XTile;
                    if (++s == STAGES) { s = 0; par ^= 1; }
                }
                if (elect_one()) tc_commit(&gu_full[h]);
                __syncwarp();
            }
            if (lane == 0 && it == 0) DEC_STAMP(5);
            // down: the unit's token operand comes from this CTA's own epilogue
            {
                const int ok = mbar_wait(a_full, it & 1, abort_flag, p.status, 9, p.wait_limit);
                if (!__all_sync(0xffffffffu, ok)) goto roles_done;
                if (lane == 0 && it == 0) DEC_STAMP(15);
            }
            for (int m = 0; m < p.dn_m_tiles; m += 2) {
                const int nb = min(2, p.dn_m_tiles - m);
#ifdef NEON_MOE_INSTRUMENT
                const long long tw0 = clock64();
#endif
                int ok = mbar_wait(&full[s], par, abort_flag, p.status, 3, p.wait_limit);
                if (!__all_sync(0xffffffffu, ok)) goto roles_done;
#ifdef NEON_MOE_INSTRUMENT
                wait_dn += clock64() - tw0;
#endif
                for (int i = 0; i < nb; ++i, ++n_dn) {
                    const int slot = n_dn & (kDec2DnSlots - 1), spar = (n_dn / kDec2DnSlots) & 1;
#ifdef NEON_MOE_INSTRUMENT
                    const long long tw1 = clock64();
#endif
                    ok = mbar_wait(&dn_empty[slot], spar ^ 1, abort_flag, p.status, 2, p.wait_limit);
                    if (!__all_sync(0xffffffffu, ok)) goto roles_done;
#ifdef NEON_MOE_INSTRUMENT
                    wait_slot += clock64() - tw1;
#endif
                    tc_fence_after();
                    if (elect_one()) {
                        const uint32_t st = stage_base + s * 32768 + i * 16384, sf_tmem = tmem_base + SF_BASE + s * 8 + 4 * i;
                        tc_copy_sf(sf_tmem, make_sf_desc(sfa_base + s * 1024 + 512 * i));
                        const uint64_t a_desc = make_sw128_desc(st);
                        const uint32_t d_tmem = tmem_base + DN_BASE + slot * DN_COLS;
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj)
                            mma_mxf8f6f4(d_tmem, a_desc + 2 * jj, a_tile_desc + 2 * jj, idesc_dn + jj * (1u << 29), sf_tmem, tmem_base + SF_UNIT,
                                         (uint32_t)jj);
                        tc_commit(&dn_full[slot]);
                    }
                    __syncwarp();
                }
                if (elect_one()) tc_commit(&empty[s]);
                __syncwarp();
                if (++s == STAGES) { s = 0; par ^= 1; }
            }
            if (lane == 0 && it == 0) DEC_STAMP(6);
        }
#ifdef NEON_MOE_INSTRUMENT
        if (lane == 0 && p.trace) {  // SM clocks this warp spent waiting: gate_up stages, down stages, down accumulators
            p.trace[blockIdx.x * 16 + 13] = wait_cyc;
            p.trace[blockIdx.x * 16 + 14] = wait_dn * 100000 + wait_slot;
        }
#endif
    } else if (warp < 6) {
        // ---- epilogue warps: gate_up accumulators -> down token operand; down accumulators -> output accumulator.
        //      A warp whose wait failed stops touching tensor memory but keeps meeting the others at the named barrier,
        //      where the verdicts are compared and all four leave together.
        const int q = warp & 3, et = tid - 64;
        bool alive = true;
        int it = 0, n_dn = 0, n_vote = 0;
        int n_gu[2] = {0, 0};  // completed uses of each gate_up accumulator (the last unit of an expert has one tile only)
        for (int u = cta; u < n_units; u += grid, ++it) {
            const int es = u / p.nch_i, j = u - es * p.nch_i, e = s_exp[es];
            const int n_mt = min(2, p.gu_m_tiles - 2 * j);
            float wte[kDec2MaxTok];   // routing weight of (token, this expert); zero when the token does not use the expert
#pragma unroll
            for (int t = 0; t < kDec2MaxTok; ++t) {
                wte[t] = 0.f;
                if (t < T)
                    for (int sl = 0; sl < k; ++sl)
                        if (s_idx[t * k + sl] == e) wte[t] = s_w[t * k + sl];
            }
            for (int h = 0; h < 2; ++h) {
                // rows 32 q + lane of the tile: lanes 0..15 hold the gate rows of channels 16 q + lane of the tile's 64,
                // lanes 16..31 the linear rows of the same channels
                float a[kDec2MaxTok] = {0.f, 0.f, 0.f, 0.f};
                if (h < n_mt) {
                    if (alive) alive = mbar_wait_quiet(&gu_full[h], n_gu[h] & 1, abort_flag, p.status, 4, p.wait_limit, 0);
                    ++n_gu[h];
                    if (alive) {
                        tc_fence_after();
                        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + h * GU_COLS;
                        float v0[8], v1[8];
                        tmem_ld8(taddr, v0);
                        tmem_ld8(taddr + 8, v1);
                        tc_fence_before();
                        const int ch = 64 * (2 * j + h) + 16 * q + (lane & 15);
                        const float bias = bf16_bits_to_float(p.gu_bias[(size_t)e * 2 * p.I + 2 * ch + (lane >> 4)]);
#pragma unroll
                        for (int t = 0; t < kDec2MaxTok; ++t) {
                            const int sb = term_scale_byte(__uint_as_float(s_amax[t] << 16), 2);
                            const float mine = fmaf(v1[t], 0.0625f, v0[t]) * __uint_as_float((uint32_t)sb << 23) + bias;
                            const float lin = __shfl_down_sync(0xffffffffu, mine, 16);
                            const float gg = fminf(mine, p.limit);
                            const float ll = fminf(fmaxf(lin, -p.limit), p.limit);
                            a[t] = (t < T && ch < p.I) ? gg / (1.f + expf(-p.alpha * gg)) * (ll + 1.f) * wte[t] : 0.f;
                        }
                    }
                }
                if (lane < 16) {
                    const int col = 64 * h + 16 * q + lane;  // byte of the 128-byte operand row
#pragma unroll
                    for (int t = 0; t < kDec2MaxTok; ++t) {
                        if (t < T) {
                            float v = a[t];
#pragma unroll
                            for (int term = 0; term < 4; ++term) {
                                const float inv = __uint_as_float((uint32_t)(254 - (sb_dn - 4 * term)) << 23);
                                const float scale = __uint_as_float((uint32_t)(sb_dn - 4 * term) << 23);
                                const __nv_fp8_storage_t b8 = __nv_cvt_float_to_fp8(v * inv, __NV_SATFINITE, __NV_E4M3);
                                const int n = term * 4 + t;
                                atile[(n >> 3) * 1024 + (n & 7) * 128 + (((col >> 4) ^ (n & 7)) << 4) + (col & 15)] = b8;
                                if (term < 3) {
                                    const __half_raw hr = __nv_cvt_fp8_to_halfraw(b8, __NV_E4M3);
                                    v -= __half2float(*reinterpret_cast<const __half*>(&hr)) * scale;
                                }
                            }
                        }
                    }
                }
            }
            fence_proxy_async();
            {
                volatile int* vote = s_vote + 4 * (n_vote & 1);
                ++n_vote;
                __syncwarp();
                if (lane == 0) vote[q] = alive ? 1 : 0;
                named_bar_sync(1, 128);
                if (!(vote[0] & vote[1] & vote[2] & vote[3])) goto roles_done;
            }
            if (et == 0) mbar_arrive(a_full);
            if (et == 0 && it == 0) DEC_STAMP(10);
            for (int m = 0; m < p.dn_m_tiles; ++m, ++n_dn) {
                const int slot = n_dn & (kDec2DnSlots - 1), spar = (n_dn / kDec2DnSlots) & 1;
                if (alive) alive = mbar_wait_quiet(&dn_full[slot], spar, abort_flag, p.status, 4, p.wait_limit, 0);
                if (!alive) continue;
                tc_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + DN_BASE + slot * DN_COLS;
                float v[8], w8[8];
                tmem_ld8(taddr, v);       // term 0 | term 1, four tokens each
                tmem_ld8(taddr + 8, w8);  // term 2 | term 3
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&dn_empty[slot]);
                const float sc = __uint_as_float((uint32_t)sb_dn << 23);
                float* yrow = yacc + 128 * m + 32 * q + lane;
#pragma unroll
                for (int t = 0; t < kDec2MaxTok; ++t) {
                    if (t < T) {
                        float y = fmaf(v[4 + t], 0.0625f, v[t]);
                        y = fmaf(w8[t], 0.00390625f, y);
                        y = fmaf(w8[4 + t], 0.000244140625f, y);
                        yrow[t * HP] += y * sc;
                    }
                }
            }
        }
    } else {
        // ---- builders, second job (CTA 0): histogram and offsets over all experts, as the dispatch kernels write them
        const int bt = tid - 192;
        if (cta == 0) {
            const int n_ent = T * k;
            for (int e = bt; e <= p.E; e += kDecBuilderThreads) {
                int c = 0, below = 0;
                for (int i = 0; i < n_ent; ++i) {
                    c += s_idx[i] == e;
                    below += s_idx[i] < e;
                }
                if (e < p.E) p.d.count[e] = c;
                p.d.offset[e] = below;
            }
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
        tmem_dealloc(tmem_base, kDec2TmemCols);
    }
    // ---- the sum over CTAs: contributions to global memory, one grid-wide barrier, every CTA adds a slice of the columns
    const int n_act = min(grid, n_units);   // CTAs that had a unit
    if (!*abort_flag) {
        if (cta < n_act)
            for (int i = tid; i < T * HP / 4; i += kDecThreads)
                __stcg(reinterpret_cast<float4*>(p.dn_part + (size_t)cta * T * HP) + i, reinterpret_cast<const float4*>(yacc)[i]);
        __syncthreads();
        if (tid == 0) {
            red_release_add(grid_count, 1u);
            const unsigned target = sliced_pass * (unsigned)grid;
            const long long t0 = clock64();
            while ((int)(ld_acquire_u32(grid_count) - target) < 0) {
                if (clock64() - t0 > p.wait_limit) {
                    *abort_flag = 1;
                    atomicCAS(p.status, 0, 12);
                    break;
                }
            }
        }
        __syncthreads();
    }
    if (tid == 0) DEC_STAMP(12);
    if (!*abort_flag) {
        // groups of four columns of one token, one per warp; lanes take the CTAs c = lane, lane + 32, ... in ascending
        // order, then a fixed tree over the lanes
        const int h4n = H / 4, n_groups = T * h4n;
        for (int g = cta * (kDecThreads / 32) + warp; g < n_groups; g += grid * (kDecThreads / 32)) {
            const int t = g / h4n, h4 = g - t * h4n;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int c = lane; c < n_act; c += 32) {
                const float4 v = __ldcg(reinterpret_cast<const float4*>(p.dn_part + ((size_t)c * T + t) * HP) + h4);
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                acc.x += __shfl_xor_sync(0xffffffffu, acc.x, o);
                acc.y += __shfl_xor_sync(0xffffffffu, acc.y, o);
                acc.z += __shfl_xor_sync(0xffffffffu, acc.z, o);
                acc.w += __shfl_xor_sync(0xffffffffu, acc.w, o);
            }
            if (lane == 0) {
                for (int sl = 0; sl < k; ++sl) {  // the down bias of every slot's expert, in slot order
                    const float wt = s_w[t * k + sl];
                    const uint2 braw = __ldg(reinterpret_cast<const uint2*>(p.dn_bias + (size_t)s_idx[t * k + sl] * H + 4 * h4));
                    acc.x = fmaf(wt, __uint_as_float(braw.x << 16), acc.x);
                    acc.y = fmaf(wt, __uint_as_float(braw.x & 0xffff0000u), acc.y);
                    acc.z = fmaf(wt, __uint_as_float(braw.y << 16), acc.z);
                    acc.w = fmaf(wt, __uint_as_float(braw.y & 0xffff0000u), acc.w);
                }
                *reinterpret_cast<float4*>(p.out + (size_t)t * H + 4 * h4) = acc;
            }
        }
    }
    // the next pass gets the next number (a pass that gave up advances it too: its counters then mean nothing and the
    // host clears them when it reads the status)
    if (cta == 0 && tid == 0) {
        __stcg(p.counters, pass);
        __stcg(p.counters + 3, sliced_pass);
    }
    if (tid == 0) DEC_STAMP(8);
}

}  // namespace neon
