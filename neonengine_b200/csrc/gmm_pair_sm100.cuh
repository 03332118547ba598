// Grouped block-scaled expert GEMM for decode tiles on TWO-SM tensor-core instructions
// (tcgen05 cta_group::2): thread-block clusters of two CTAs, each CTA streaming its own 128-row weight
// tile (two adjacent tiles of one expert per pair) and HALF of the stacked token operand; the leader
// CTA's elected thread issues one 256 x N x 32 MMA where two single-SM kernels would issue two.
//
// Why: at decode sizes the grouped GEMM's steady state is bound by the one thread that issues the
// tcgen05 instructions (a constant ~630 clocks per two-chunk stage, of which the MMAs proper need
// ~380).  A pair spends the same issue time on twice the weight bytes, so the stream from HBM, not the
// issuing thread, sets the pace; and each SM fetches only half of the token operand from L2.
//
// Same data formats, same arithmetic and same epilogues as gmm_bs_kernel<..., STACK = true, KC = 2>
// (gmm_sm100.cuh); what differs is the synchronisation:
//   - the leader may issue a stage's MMAs when BOTH CTAs' copies have landed: weights and weight scales of
//     both CTAs report their bytes to the leader's stage barrier; the peer's token rows land on a barrier of
//     its own, and the peer's MMA warp, which issues nothing, forwards that as a second arrival on the leader's
//     stage barrier (remote arrive), so the leader waits for ONE barrier per stage;
//   - MMA completion frees the stage and publishes the accumulator in both CTAs at once
//     (tcgen05.commit ... multicast::cluster);
//   - the leader reuses an accumulator buffer when the epilogue warps of both CTAs have read it (the
//     peer's warps arrive remotely);
//   - tensor memory is allocated and freed by one warp of each CTA with the cta_group::2 forms; the
//     pair meets at a cluster barrier after set-up and before it retires.
// No TMA load is multicast: every CTA copies its own operands into its own shared memory.
// Every wait is bounded (status word, as in gmm_bs_kernel).
#pragma once
#include "gmm_sm100.cuh"
#include "mma_pair.cuh"

namespace neon {
namespace sm100 {

__device__ __forceinline__ uint32_t mapa_shared(uint32_t local_addr, uint32_t cta_rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(cta_rank));
    return r;
}
// Arrive on a barrier of another CTA of the cluster (address from mapa_shared).  The default semantics (release at CTA
// scope) on purpose: the cluster-scope release was measured at ~1500 clocks per arrive while TMA traffic is in flight
// (it drains the memory pipeline), which made the pair's stage period twice the single-CTA kernel's.  What the arrive
// orders is covered without it: operand bytes are written by TMA and observed complete through an mbarrier before the
// arrive, and accumulator reads are fenced with tcgen05.fence::before_thread_sync.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Wait variant for barriers that other CTAs of the cluster arrive on.
__device__ __forceinline__ bool mbar_test_cluster(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                                                  long long limit_cycles) {
    if (mbar_test_cluster(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        for (int i = 0; i < 64; ++i)
            if (mbar_test_cluster(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > limit_cycles) {
            *abort_flag = 1;
            atomicCAS(status, 0, code);
            return false;
        }
    }
}

// Tiled TMA load into THIS CTA's shared memory whose bytes are reported to a barrier that may live in the other CTA
// of the pair (cluster address from mapa_shared).  No multicast: one destination.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}

}  // namespace sm100

// Shared-memory layout of the paired kernel: as GmmSmem<..., STACK, KC = 2>, with half the token-operand rows per CTA.
template <int BN_MAX, int TERMS>
struct PairSmem {
    static constexpr int kABytes = 16384;
    static constexpr int kActBytes = (TERMS / 2) * BN_MAX * 128;   // this CTA's half of the stacked rows of one chunk
    static constexpr int kStage = (2 * (kABytes + kActBytes + 512) + 1023) / 1024 * 1024;
    static constexpr int kSfCols = 2 * 4;
    static constexpr int kAccCols = TERMS * BN_MAX;
    static constexpr int kSfBase = 2 * kAccCols + 8;
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

template <int BN_MAX, int TERMS, bool GATE_UP>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192)
gmm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmA1, const __grid_constant__ CUtensorMap tmS,
                const __grid_constant__ CUtensorMap tmS1, const GmmParams p) {
    using namespace sm100;
    static_assert(TERMS % 2 == 0 && BN_MAX <= 32, "the stacked terms split evenly between the two CTAs");
    using L = PairSmem<BN_MAX, TERMS>;
    constexpr size_t kFullActBytes = (size_t)TERMS * BN_MAX * 128;  // one chunk's whole block in global memory
    constexpr int KC = 2;
    constexpr int STAGES_MAX = L::kStages;
    const int STAGES = p.stages;
    constexpr int SF_COLS = L::kSfCols, SF_BASE = L::kSfBase, SF_UNIT = 2 * L::kAccCols;
    constexpr int ACT_OFF = KC * L::kABytes, SFA_OFF = ACT_OFF + KC * L::kActBytes;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * L::kStage);
    uint64_t* empty = full + STAGES_MAX;
    uint64_t* peer_full = empty + STAGES_MAX;  // peer CTA only: its token rows of the stage have landed (forwarded to the leader's stage barrier)
    uint64_t* acc_full = peer_full + STAGES_MAX;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    uint32_t* unit_atom = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(full) + 512);

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t crank = cluster_ctarank();
    const bool leader = crank == 0;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], leader ? 2 : 1);  // leader: its own producer's arrival + the peer's "token rows landed"
            mbar_init(&empty[s], 1);
            mbar_init(&peer_full[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 8);  // four epilogue warps of each CTA
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmA1);
    }
    if (threadIdx.x < 128) unit_atom[threadIdx.x] = 0x7f7f7f7fu;
    fence_proxy_async();
    const uint32_t tmem_cols = (uint32_t)p.tmem_cols;
    if (warp == 2) tmem_alloc_pair(tmem_slot, tmem_cols);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers, unit atoms and tensor memory exist before anyone signals across
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int mp_tiles = (p.m_tiles + 1) / 2;            // pairs of weight tiles per expert (the last may be half empty)
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    constexpr size_t act_stride = kFullActBytes;
    const uint32_t full_leader = mapa_shared(smem_u32(&full[0]), 0);  // the leader's stage barriers (this CTA's own for the leader)
    // Weight boxes and scale atoms of one stage.  They report to the LEADER's barrier from both CTAs (the long latency,
    // from HBM); the leader raises that barrier's byte count for both.
    auto load_weights = [&](int s, int kc, int box_row, uint32_t atom) {
        uint8_t* st = smem + s * L::kStage;
        if (leader) {
            mbar_expect_tx_only(&full[s], kc * (2 * (p.a_tx_bytes + 512)));
            tma_load_2d(st, kc == 2 ? &tmA : &tmA1, &full[s], 0, box_row);
            tma_load_2d(st + SFA_OFF, kc == 2 ? &tmS : &tmS1, &full[s], 0, (int)atom);
        } else {
            tma_load_2d_pair(st, kc == 2 ? &tmA : &tmA1, full_leader + s * 8, 0, box_row);
            tma_load_2d_pair(st + SFA_OFF, kc == 2 ? &tmS : &tmS1, full_leader + s * 8, 0, (int)atom);
        }
    };
    pdl_wait();
    const int n_items = *p.n_tiles * mp_tiles;

    if (warp == 0) {
        // ---- producer (both CTAs): own weight tile + own half of the stacked token rows -------------------
        int s = 0, ph = 0;
        for (int item = pair; item < n_items; item += n_pairs) {
            const int tile = item / mp_tiles, m = 2 * (item - tile * mp_tiles) + (int)crank;
            const int m_ld = min(m, p.m_tiles - 1);  // the absent second tile of an odd count: a duplicate load, never stored
            const int e = p.tile_expert[tile], rows = p.tile_rows[tile];
            const uint32_t half_bytes = (TERMS / 2) * ((rows + 7) >> 3) * 1024;  // N / 2 rows of 128 bytes
            const uint32_t box = (uint32_t)((e * p.m_tiles + m_ld) * p.n_chunks);
            int box_row = (int)(box * 128);
            uint32_t atom = box;  // row of the scale-atom tensor (one 512-byte atom per weight box)
            const uint8_t* act_src = p.act + (size_t)tile * p.n_chunks * act_stride + crank * half_bytes;
            for (int left = p.n_chunks; left > 0; left -= KC) {
                const int kc = left >= KC ? KC : 1;
                const int ok = mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 1, kWaitLimitCycles);
                if (!__all_sync(0xffffffffu, ok)) goto done;
                uint8_t* st = smem + s * L::kStage;
                if (elect_one()) {
                    load_weights(s, kc, box_row, atom);
                    // The token rows (from L2, early) report to a barrier of their own CTA; the leader's is the stage barrier,
                    // on which this is also the one arrival; the peer's warp 1 forwards its "rows landed" to the leader.
                    uint64_t* rows_bar = leader ? &full[s] : &peer_full[s];
                    mbar_expect_tx(rows_bar, kc * half_bytes);
                    for (int k = 0; k < kc; ++k) bulk_load(st + ACT_OFF + k * L::kActBytes, act_src + k * act_stride, half_bytes, rows_bar);
                }
                __syncwarp();
                box_row += KC * 128;
                atom += KC;
                act_src += KC * act_stride;
                if (++s == STAGES) { s = 0; ph ^= 1; }
            }
        }
        for (int i = 0; i < STAGES; ++i) {  // late asynchronous arrives must land before the CTA retires
            const int ok = mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 6, kWaitLimitCycles);
            if (!__all_sync(0xffffffffu, ok)) goto done;
            if (++s == STAGES) { s = 0; ph ^= 1; }
        }
    } else if (warp == 1 && !leader) {
        // ---- peer CTA: forward every "stage full" to the leader -----------------------------------------
        int s = 0, ph = 0;
        for (int item = pair; item < n_items; item += n_pairs) {
            for (int left = p.n_chunks; left > 0; left -= KC) {
                const int ok = mbar_wait(&peer_full[s], ph, abort_flag, p.status, 3, kWaitLimitCycles);  // own token rows landed
                if (!__all_sync(0xffffffffu, ok)) goto done;
                if (lane == 0) mbar_arrive_cluster(full_leader + s * 8);  // the second arrival of the leader's stage barrier
                __syncwarp();
                if (++s == STAGES) { s = 0; ph ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ---- leader CTA: MMA issuer for the pair -----------------------------------------------------------
        int s = 0, ph = 0, iter = 0;
#ifdef NEON_MOE_INSTRUMENT
        int ctr = 0;
#endif
        const uint32_t smem_base = smem_u32(smem);
        if (elect_one()) {
            tc_copy_sf_pair(tmem_base + SF_UNIT, make_sf_desc(smem_u32(unit_atom)));
            tc_copy_sf_pair(tmem_base + SF_UNIT + 4, make_sf_desc(smem_u32(unit_atom)));
        }
        __syncwarp();
        // the next item's row count is fetched one item ahead: a dependent global load at every item boundary cost
        // the issuing warp 400-1300 clocks per item (12 stages of ~600)
        int next_rows = pair < n_items ? p.tile_rows[pair / mp_tiles] : 0;
        for (int item = pair; item < n_items; item += n_pairs, ++iter) {
            const int rows = next_rows;
            if (item + n_pairs < n_items) next_rows = p.tile_rows[(item + n_pairs) / mp_tiles];
            const int npad = (rows + 7) & ~7;
            const uint32_t idesc0 = make_idesc_bs_m(5, 0, 256, (uint32_t)(TERMS * npad), 0, 0);
            const int b = iter & 1, aph = (iter >> 1) & 1;
            int ok = mbar_wait_cluster(&acc_empty[b], aph ^ 1, abort_flag, p.status, 2, kWaitLimitCycles);
            if (!__all_sync(0xffffffffu, ok)) goto done;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + b * L::kAccCols;
            uint32_t first = 0;
            for (int left = p.n_chunks; left > 0; left -= KC) {
#ifdef NEON_MOE_INSTRUMENT
                const bool tracing = p.trace && blockIdx.x == 0 && lane == 0 && ctr < 256;
                if (tracing) p.trace[ctr * 4] = clock64();
#endif
                ok = mbar_wait(&full[s], ph, abort_flag, p.status, 3, kWaitLimitCycles);
#ifdef NEON_MOE_INSTRUMENT
                if (tracing) p.trace[ctr * 4 + 1] = clock64();
#endif
                if (!__all_sync(0xffffffffu, ok)) goto done;
#ifdef NEON_MOE_INSTRUMENT
                if (tracing) p.trace[ctr * 4 + 2] = clock64();
#endif
                tc_fence_after();
                if (elect_one()) {
                    const uint32_t st = smem_base + s * L::kStage;
                    const uint32_t sf_stage = tmem_base + SF_BASE + s * SF_COLS;
#pragma unroll
                    for (int k = 0; k < KC; ++k) {
                        if (k < left) {
                            const uint32_t sf_tmem = sf_stage + k * (SF_COLS / KC);
                            tc_copy_sf_pair(sf_tmem, make_sf_desc(st + SFA_OFF + k * 512));  // each CTA: its own tile's scales
                            const uint64_t a_desc = make_sw128_desc(st + k * L::kABytes), b_desc = make_sw128_desc(st + ACT_OFF + k * L::kActBytes);
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                mma_mxf8f6f4_pair(d_tmem, a_desc + 2 * j, b_desc + 2 * j, idesc0 + j * (1u << 29), sf_tmem, tmem_base + SF_UNIT,
                                                  first | (uint32_t)(k | j));
                        }
                    }
                    tc_commit_pair(&empty[s], 3);  // the stage is free in both CTAs once these MMAs have completed
                }
                __syncwarp();
#ifdef NEON_MOE_INSTRUMENT
                if (tracing) p.trace[ctr * 4 + 3] = clock64();
                ++ctr;
#endif
                first = 1;
                if (++s == STAGES) { s = 0; ph ^= 1; }
            }
            if (elect_one()) tc_commit_pair(&acc_full[b], 3);
            __syncwarp();
        }
    } else {
        // ---- epilogue (both CTAs): this CTA's 128 rows of the pair's accumulator ---------------------------
        const int q = warp & 3;
        const uint32_t acc_empty_leader = mapa_shared(smem_u32(&acc_empty[0]), 0);
        int iter = 0;
        for (int item = pair; item < n_items; item += n_pairs, ++iter) {
            const int tile = item / mp_tiles, m = 2 * (item - tile * mp_tiles) + (int)crank;
            const int e = p.tile_expert[tile], row0 = p.tile_row0[tile], rows = p.tile_rows[tile];
            const int b = iter & 1, aph = (iter >> 1) & 1;
            // everything that does not depend on the accumulator is fetched BEFORE the wait for it (two rounds of
            // dependent global loads otherwise sit between "accumulator ready" and "buffer returned")
            const int npad = (rows + 7) & ~7;
            const int ch = 64 * m + 16 * q + (lane & 15);
            const int row = 128 * m + 32 * q + lane;
            const bool valid = m < p.m_tiles && (GATE_UP ? true : row < p.rows_total);
            float bias = 0.f;
            if (valid) bias = bf16_bits_to_float(p.bias[(size_t)e * p.rows_total + (GATE_UP ? 2 * ch + (lane >> 4) : row)]);
            float tok_scale = 0.f, tok_w = 0.f;
            float* tok_dst = nullptr;
            if (lane < rows) {
                tok_scale = p.row_scale ? p.row_scale[row0 + lane] : p.row_scale_const;
                if (!GATE_UP) {
                    const int ent = p.perm[row0 + lane];
                    tok_w = p.route_w[ent];
                    tok_dst = p.peer.n_ranks ? peer_row(p.peer, ent, p.hidden) : p.y + (size_t)(row0 + lane) * p.hidden;
                }
            }
            if (!mbar_wait(&acc_full[b], aph, abort_flag, p.status, 4, kWaitLimitCycles)) goto done;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + b * L::kAccCols;
            float vals[BN_MAX];
#pragma unroll
            for (int j8 = 0; j8 < BN_MAX; j8 += 8) {
                float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                if (j8 < npad) {
                    tmem_ld8(taddr + j8, v);
                    float f = 1.f;
#pragma unroll
                    for (int t = 1; t < TERMS; ++t) {
                        f *= 0.0625f;
                        float u[8];
                        tmem_ld8(taddr + t * npad + j8, u);
#pragma unroll
                        for (int i = 0; i < 8; ++i) v[i] = fmaf(u[i], f, v[i]);
                    }
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) vals[j8 + i] = v[i];
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {  // the buffer goes back to the leader's MMA warp
                if (leader) mbar_arrive(&acc_empty[b]);
                else mbar_arrive_cluster(acc_empty_leader + b * 8);
            }
#pragma unroll
            for (int j = 0; j < BN_MAX; ++j) {
                if (j < npad) {
                    const float sc = __shfl_sync(0xffffffffu, tok_scale, j);
                    const float mine = vals[j] * sc + bias;
                    if (GATE_UP) {
                        const float lin = __shfl_down_sync(0xffffffffu, mine, 16);
                        if (valid && lane < 16 && j < rows) {
                            const float g = fminf(mine, p.limit);
                            const float l = fminf(fmaxf(lin, -p.limit), p.limit);
                            p.a_out[(size_t)(row0 + j) * p.inter + ch] = g / (1.f + expf(-p.alpha * g)) * (l + 1.f);
                        }
                    } else {
                        const float wt = __shfl_sync(0xffffffffu, tok_w, j);
                        float* dst = reinterpret_cast<float*>(__shfl_sync(0xffffffffu, (unsigned long long)tok_dst, j));
                        if (valid && j < rows) dst[row] = wt * mine;
                    }
                }
            }
        }
        if (!GATE_UP && p.peer.n_ranks) {
            __syncwarp();
            if (lane == 0) __threadfence_system();
        }
    }
done:
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000ll) {}
    }
    cluster_sync_all();  // neither CTA retires (or frees tensor memory) while its partner may still signal it or read its operands
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, tmem_cols);
    }
}

}  // namespace neon
