// Grouped block-scaled expert GEMM for prefill tiles (128 tokens) on two-SM tensor-core instructions.
//
// The one-CTA prefill kernel (gmm_bs_kernel<128, TERMS, ..., STACK = false>) is bound by operand traffic from L2
// to the SMs: every 128 x 128 output tile fetches, per K chunk, 16 KB of weights and TERMS x 16 KB of token
// rows (e4m3 terms), and with four terms only two pipeline stages fit.  Here a cluster of two CTAs owns two
// adjacent weight tiles of one expert and ONE token tile: each CTA streams its own weight tile and HALF of
// the token rows, and the leader's elected thread issues tcgen05.mma.cta_group::2 (M = 256 split by CTA,
// N = all tokens of the tile, the N operand being the concatenation of the two CTAs' halves).  Per output
// element the token-row traffic halves, a stage shrinks from 49 / 81 KB to 34 / 51 KB (two / four terms), and
// six / four stages fit instead of four / two.
//
// Data formats, arithmetic and epilogues are those of the one-CTA kernel; results are bit-identical.  Every
// token row keeps its own per-32-block scales: each CTA copies the WHOLE scale header of the block (the scale
// atoms cover all 128 token rows and every CTA's tensor core needs all of them) and its half of the rows.
// Synchronisation is gmm_pair_kernel's (gmm_pair_sm100.cuh): weight copies of both CTAs report to the leader's
// stage barrier, the peer's token rows to a barrier of its own that its idle MMA warp forwards, completion is
// published to both CTAs by multicast commits, every wait is bounded.  No TMA load is multicast.
#pragma once
#include "gmm_pair_sm100.cuh"

namespace neon {

template <int TERMS>
struct PairPrefillSmem {
    static constexpr int kABytes = 16384;
    static constexpr int kHdr = act_header_bytes(TERMS);            // scale atoms of all 128 token rows, one per term
    static constexpr int kRowBytes = 8 * TERMS * 1024;              // this CTA's 64 token rows: 8 row groups x TERMS x 1 KB
    static constexpr int kStage = (kABytes + kHdr + kRowBytes + 512 + 1023) / 1024 * 1024;
    static constexpr int kSfCols = 4 * (1 + TERMS);                 // weight scales + one atom per term
    static constexpr int kAccCols = 128;
    static constexpr int kSfBase = 2 * kAccCols;
    static constexpr int kTail = 1024;
    static constexpr int kStagesFit = (225 * 1024 - kTail - 1024) / kStage;
    static constexpr int kStagesTmem = (512 - kSfBase) / kSfCols;
    static constexpr int kStages = kStagesFit < kStagesTmem ? (kStagesFit < 8 ? kStagesFit : 8) : kStagesTmem;
    static constexpr int smem_bytes(int stages) { return stages * kStage + kTail + 1024; }
    static constexpr int tmem_cols(int stages) {
        int need = kSfBase + stages * kSfCols, cols = 32;
        while (cols < need) cols *= 2;
        return cols;
    }
};

template <int TERMS, bool GATE_UP>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192)
gmm_pair_prefill_kernel(const __grid_constant__ CUtensorMap tmA1, const __grid_constant__ CUtensorMap tmS1, const GmmParams p) {
    using namespace sm100;
    using L = PairPrefillSmem<TERMS>;
    constexpr int BN_MAX = 128;
    constexpr size_t act_stride = (size_t)L::kHdr + (BN_MAX / 8) * TERMS * 1024;  // one chunk's whole block in global memory
    constexpr int STAGES_MAX = L::kStages;
    const int STAGES = p.stages;
    constexpr int SF_COLS = L::kSfCols, SF_BASE = L::kSfBase;
    constexpr int HDR_OFF = L::kABytes, ROW_OFF = HDR_OFF + L::kHdr, SFA_OFF = ROW_OFF + L::kRowBytes;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * L::kStage);
    uint64_t* empty = full + STAGES_MAX;
    uint64_t* peer_full = empty + STAGES_MAX;  // leader: the peer's token rows of the stage have landed; peer: its own barrier for them
    uint64_t* acc_full = peer_full + STAGES_MAX;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t crank = cluster_ctarank();
    const bool leader = crank == 0;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
            mbar_init(&peer_full[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 8);  // four epilogue warps of each CTA
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmA1);
        prefetch_tmap(&tmS1);
    }
    const uint32_t tmem_cols = (uint32_t)p.tmem_cols;
    if (warp == 2) tmem_alloc_pair(tmem_slot, tmem_cols);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers and tensor memory exist before anyone signals across
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int mp_tiles = (p.m_tiles + 1) / 2;            // pairs of weight tiles per expert (the last may be half empty)
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const uint32_t full_leader = mapa_shared(smem_u32(&full[0]), 0);
    pdl_wait();
    const int n_items = *p.n_tiles * mp_tiles;

    if (warp == 0) {
        // ---- producer (both CTAs): own weight tile and scales, the block's scale header, own half of the token rows
        int s = 0, ph = 0;
        for (int item = pair; item < n_items; item += n_pairs) {
            const int tile = item / mp_tiles, m = 2 * (item - tile * mp_tiles) + (int)crank;
            const int m_ld = min(m, p.m_tiles - 1);  // the absent second tile of an odd count: a duplicate load, never stored
            const int e = p.tile_expert[tile], rows = p.tile_rows[tile];
            const uint32_t n_mma = (uint32_t)max(16, round_up_int(rows, 16));
            const uint32_t half_bytes = (n_mma / 16) * TERMS * 1024;   // n_mma / 2 rows = n_mma / 16 row groups of all terms
            const uint32_t box = (uint32_t)((e * p.m_tiles + m_ld) * p.n_chunks);
            int box_row = (int)(box * 128);
            uint32_t atom = box;
            const uint8_t* blk = p.act + (size_t)tile * p.n_chunks * act_stride;
            for (int c = 0; c < p.n_chunks; ++c) {
                const int ok = mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 1, kWaitLimitCycles);
                if (!__all_sync(0xffffffffu, ok)) goto done;
                uint8_t* st = smem + s * L::kStage;
                if (elect_one()) {
                    uint64_t* rows_bar = leader ? &full[s] : &peer_full[s];
                    if (leader) {
                        mbar_expect_tx_only(&full[s], 2 * (p.a_tx_bytes + 512));   // both CTAs' weights and weight scales
                        tma_load_2d(st, &tmA1, &full[s], 0, box_row);
                        tma_load_2d(st + SFA_OFF, &tmS1, &full[s], 0, (int)atom);
                    } else {
                        tma_load_2d_pair(st, &tmA1, full_leader + s * 8, 0, box_row);
                        tma_load_2d_pair(st + SFA_OFF, &tmS1, full_leader + s * 8, 0, (int)atom);
                    }
                    mbar_expect_tx(rows_bar, L::kHdr + half_bytes);
                    bulk_load(st + HDR_OFF, blk, L::kHdr, rows_bar);
                    bulk_load(st + ROW_OFF, blk + L::kHdr + crank * half_bytes, half_bytes, rows_bar);
                }
                __syncwarp();
                box_row += 128;
                atom += 1;
                blk += act_stride;
                if (++s == STAGES) { s = 0; ph ^= 1; }
            }
        }
        for (int i = 0; i < STAGES; ++i) {  // late asynchronous arrives must land before the CTA retires
            const int ok = mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 6, kWaitLimitCycles);
            if (!__all_sync(0xffffffffu, ok)) goto done;
            if (++s == STAGES) { s = 0; ph ^= 1; }
        }
    } else if (warp == 1 && !leader) {
        // ---- peer CTA: forward every "token rows landed" to the leader --------------------------------------
        int s = 0, ph = 0;
        for (int item = pair; item < n_items; item += n_pairs) {
            for (int c = 0; c < p.n_chunks; ++c) {
                const int ok = mbar_wait(&peer_full[s], ph, abort_flag, p.status, 3, kWaitLimitCycles);
                if (!__all_sync(0xffffffffu, ok)) goto done;
                if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&peer_full[s]), 0));
                __syncwarp();
                if (++s == STAGES) { s = 0; ph ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ---- leader CTA: MMA issuer for the pair -----------------------------------------------------------
        int s = 0, ph = 0, iter = 0;
        const uint32_t smem_base = smem_u32(smem);
        constexpr uint32_t kIdescStep = (1u << 4) | (1u << 29);  // next scale id for both operands
        for (int item = pair; item < n_items; item += n_pairs, ++iter) {
            const int tile = item / mp_tiles, rows = p.tile_rows[tile];
            const uint32_t idesc0 = make_idesc_bs_m(5, 0, 256, (uint32_t)max(16, round_up_int(rows, 16)), 0, 0);
            const int b = iter & 1, aph = (iter >> 1) & 1;
            int ok = mbar_wait_cluster(&acc_empty[b], aph ^ 1, abort_flag, p.status, 2, kWaitLimitCycles);
            if (!__all_sync(0xffffffffu, ok)) goto done;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + b * L::kAccCols;
            uint32_t first = 0;
            for (int c = 0; c < p.n_chunks; ++c) {
                ok = mbar_wait(&full[s], ph, abort_flag, p.status, 3, kWaitLimitCycles);
                ok = ok && mbar_wait_cluster(&peer_full[s], ph, abort_flag, p.status, 11, kWaitLimitCycles);
                if (!__all_sync(0xffffffffu, ok)) goto done;
                tc_fence_after();
                if (elect_one()) {
                    const uint32_t st = smem_base + s * L::kStage;
                    const uint32_t sf_tmem = tmem_base + SF_BASE + s * SF_COLS;
                    tc_copy_sf_pair(sf_tmem, make_sf_desc(st + SFA_OFF));  // each CTA: its own weight tile's scales
#pragma unroll
                    for (int t = 0; t < TERMS; ++t) tc_copy_sf_pair(sf_tmem + 4 * (1 + t), make_sf_desc(st + HDR_OFF + 512 * t));
                    const uint64_t a_desc = make_sw128_desc(st);
#pragma unroll
                    for (int t = 0; t < TERMS; ++t) {
                        const uint64_t b_desc = make_sw128_desc(st + ROW_OFF + t * 1024, TERMS * 1024);
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            mma_mxf8f6f4_pair(d_tmem, a_desc + 2 * j, b_desc + 2 * j, idesc0 + j * kIdescStep, sf_tmem, sf_tmem + 4 * (1 + t),
                                              first | (uint32_t)(t | j));
                    }
                    tc_commit_pair(&empty[s], 3);  // the stage is free in both CTAs once these MMAs have completed
                }
                __syncwarp();
                first = 1;
                if (++s == STAGES) { s = 0; ph ^= 1; }
            }
            if (elect_one()) tc_commit_pair(&acc_full[b], 3);
            __syncwarp();
        }
    } else {
        // ---- epilogue (both CTAs): this CTA's 128 weight rows x all tokens of the tile ----------------------
        const int q = warp & 3;
        const uint32_t acc_empty_leader = mapa_shared(smem_u32(&acc_empty[0]), 0);
        int iter = 0;
        for (int item = pair; item < n_items; item += n_pairs, ++iter) {
            const int tile = item / mp_tiles, m = 2 * (item - tile * mp_tiles) + (int)crank;
            const int e = p.tile_expert[tile], row0 = p.tile_row0[tile], rows = p.tile_rows[tile];
            const int b = iter & 1, aph = (iter >> 1) & 1;
            const int npad = (rows + 7) & ~7;
            // GATE_UP: lanes 0..15 hold gate rows of channels ch, lanes 16..31 their linear rows
            const int ch = 64 * m + 16 * q + (lane & 15);
            const int row = 128 * m + 32 * q + lane;
            const bool valid = m < p.m_tiles && (GATE_UP ? true : row < p.rows_total);
            float bias = 0.f;
            if (valid) bias = bf16_bits_to_float(p.bias[(size_t)e * p.rows_total + (GATE_UP ? 2 * ch + (lane >> 4) : row)]);
            constexpr int NW = BN_MAX / 32;
            float tok_w[NW];
            float* tok_dst[NW];  // down product: where each token's output row goes
#pragma unroll
            for (int k = 0; k < NW; ++k) {
                const int tix = 32 * k + lane;
                tok_w[k] = 0.f;
                tok_dst[k] = nullptr;
                if (!GATE_UP && tix < rows) {
                    const int ent = p.perm[row0 + tix];
                    tok_w[k] = p.route_w[ent];
                    tok_dst[k] = p.peer.n_ranks ? peer_row(p.peer, ent, p.hidden) : p.y + (size_t)(row0 + tix) * p.hidden;
                }
            }
            // (all of the above is independent of the accumulator: fetched before the wait for it)
            if (!mbar_wait(&acc_full[b], aph, abort_flag, p.status, 4, kWaitLimitCycles)) goto done;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + b * L::kAccCols;
#pragma unroll
            for (int k = 0; k < NW; ++k) {
                const int jend = min(npad, 32 * (k + 1));
                for (int j8 = 32 * k; j8 < jend; j8 += 8) {
                    float v[8];
                    tmem_ld8(taddr + j8, v);
                    if (GATE_UP) {
                        // two tokens per step: lanes 0..15 (gate rows) finish token j, lanes 16..31 (linear rows) token j + 1,
                        // each half getting the other half's row of its token by one exchange
#pragma unroll
                        for (int i = 0; i < 8; i += 2) {
                            const float m0 = v[i] + bias, m1 = v[i + 1] + bias;
                            const float got = __shfl_xor_sync(0xffffffffu, lane < 16 ? m1 : m0, 16);
                            const float gate = lane < 16 ? m0 : got, lin = lane < 16 ? got : m1;
                            const int tix = j8 + i + (lane >> 4);
                            if (valid && tix < rows) {
                                const float g = fminf(gate, p.limit);
                                const float l = fminf(fmaxf(lin, -p.limit), p.limit);
                                p.a_out[(size_t)(row0 + tix) * p.inter + ch] = __fdividef(g, 1.f + __expf(-p.alpha * g)) * (l + 1.f);
                            }
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int tix = j8 + i;
                            const float mine = v[i] + bias;
                            const float wt = __shfl_sync(0xffffffffu, tok_w[k], tix & 31);
                            float* dst = reinterpret_cast<float*>(__shfl_sync(0xffffffffu, (unsigned long long)tok_dst[k], tix & 31));
                            if (valid && tix < rows) dst[row] = wt * mine;
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {  // the buffer goes back to the leader's MMA warp
                if (leader) mbar_arrive(&acc_empty[b]);
                else mbar_arrive_cluster(acc_empty_leader + b * 8);
            }
        }
        if (!GATE_UP && p.peer.n_ranks) {  // rows written into other GPUs' buffers: published before the kernel ends
            __syncwarp();
            if (lane == 0) __threadfence_system();
        }
    }
done:
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        const long long t0 = clock64();  // copies that were already issued get time to land
        while (clock64() - t0 < 2000000ll) {}
    }
    cluster_sync_all();  // neither CTA retires (or frees tensor memory) while its partner may still signal it or read its operands
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, tmem_cols);
    }
}

}  // namespace neon
