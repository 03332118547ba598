// Two-SM block-scaled MMA (tcgen05 cta_group::2): a self-check of the instruction forms the paired
// grouped GEMM builds on, with operands generated in shared memory (no global traffic).  A cluster of
// two CTAs; each CTA holds its own 128 rows of A (e4m3, one constant per CTA) and its own half of the
// N operand (N / 2 rows, one constant per CTA); the leader CTA's elected thread issues
// `chunks` x 4 accumulating 256 x N x 32 MMAs and one commit that arrives on both CTAs' barriers.
// Every CTA then reads its half of the accumulator.  With A = a_c and B = b_c in CTA c the result must
// be D_c[row][col] = chunks * 128 * a_c * b_(col >= N / 2): the check that M = 256 splits by CTA and
// that the N operand is the concatenation of the two CTAs' halves.  All waits are bounded.
#pragma once
#include <cstdint>

#include "sm100_ptx.cuh"

namespace neon {
namespace sm100 {

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {  // one whole warp of EACH CTA of the pair
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Arrives once on the barrier at this shared-memory offset in every CTA of `cta_mask` when all tcgen05
// operations this thread issued so far have completed.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar, uint16_t cta_mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)),
                 "h"(cta_mask)
                 : "memory");
}
__device__ __forceinline__ void mma_mxf8f6f4_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem,
                                                  uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}
__device__ __forceinline__ void tc_copy_sf_pair(uint32_t tmem_dst, uint64_t smem_desc) {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_dst), "l"(smem_desc) : "memory");
}
// Block-scaled instruction descriptor with an explicit M (256 for a CTA pair).
__device__ __forceinline__ uint32_t make_idesc_bs_m(uint32_t a_fmt, uint32_t b_fmt, uint32_t m, uint32_t n, uint32_t sf_a, uint32_t sf_b) {
    return (sf_b << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | (1u << 23) | ((m >> 4) << 24) | (sf_a << 29);
}

}  // namespace sm100

struct MmaPairOut {
    float d[2][4][4];       // per CTA: rows {0, 37, 100, 127} x columns {0, N/2 - 1, N/2, N - 1}
    uint32_t tmem_addr[2];
    long long cycles;
    int status;
};

__global__ void __launch_bounds__(128, 1) mma_pair_probe_kernel(int n, int chunks, MmaPairOut* out) {
    using namespace sm100;
    extern __shared__ __align__(1024) uint8_t pair_smem[];
    __shared__ uint64_t done_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag, wait_status;
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(pair_smem) + 1023) & ~uintptr_t(1023));
    const uint32_t rank = cluster_ctarank();
    constexpr int kA = 0, kB = 16384, kSF = 16384 + 16384;  // A 128 x 128 B | B up to 128 rows x 128 B | unit scale atom
    const uint8_t a_byte = rank == 0 ? 0x38 : 0x30;  // e4m3 1.0 / 0.5
    const uint8_t b_byte = rank == 0 ? 0x38 : 0x40;  // e4m3 1.0 / 2.0
    for (int i = threadIdx.x; i < 16384 / 4; i += blockDim.x) {
        reinterpret_cast<uint32_t*>(base + kA)[i] = 0x01010101u * a_byte;
        reinterpret_cast<uint32_t*>(base + kB)[i] = 0x01010101u * b_byte;
    }
    for (int i = threadIdx.x; i < 128; i += blockDim.x) reinterpret_cast<uint32_t*>(base + kSF)[i] = 0x7f7f7f7fu;
    if (threadIdx.x == 0) {
        mbar_init(&done_bar, 1);
        abort_flag = 0;
        wait_status = 0;
        fence_barrier_init();
    }
    fence_proxy_async();
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0) tmem_alloc_pair(&tmem_slot, 128);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // both CTAs' operands, barriers and tensor memory are ready
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    long long t0 = 0;
    if (warp == 0 && rank == 0) {
        if (elect_one()) {
            const uint32_t sb = smem_u32(base);
            const uint32_t sf_a = tmem_base + 96, sf_b = tmem_base + 100;
            tc_copy_sf_pair(sf_a, make_sf_desc(sb + kSF));
            tc_copy_sf_pair(sf_b, make_sf_desc(sb + kSF));
            tc_copy_sf_pair(sf_b + 4, make_sf_desc(sb + kSF));
            const uint32_t idesc0 = make_idesc_bs_m(0, 0, 256, (uint32_t)n, 0, 0);
            const uint64_t a_desc = make_sw128_desc(sb + kA), b_desc = make_sw128_desc(sb + kB);
            t0 = clock64();
            for (int c = 0; c < chunks; ++c)
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    mma_mxf8f6f4_pair(tmem_base, a_desc + 2 * j, b_desc + 2 * j, idesc0, sf_a, sf_b, (uint32_t)(c | j));
            tc_commit_pair(&done_bar, 3);
        }
        __syncwarp();
    }
    const bool ok = mbar_wait(&done_bar, 0, &abort_flag, &wait_status, 1, 2000000000ll);
    const long long t1 = clock64();
    tc_fence_after();
    if (ok) {
        // warp w reads rows 32 w .. 32 w + 31 of this CTA's accumulator
        const int rows[4] = {0, 37, 100, 127}, cols[4] = {0, n / 2 - 1, n / 2, n - 1};
        for (int ci = 0; ci < 4; ++ci) {
            float v[8];
            tmem_ld8(tmem_base + ((uint32_t)(warp * 32) << 16) + (cols[ci] & ~7), v);
            for (int ri = 0; ri < 4; ++ri)
                if (rows[ri] / 32 == warp && rows[ri] % 32 == lane) out->d[rank][ri][ci] = v[cols[ci] & 7];
        }
    }
    if (threadIdx.x == 0) {
        out->tmem_addr[rank] = tmem_base;
        if (!ok) out->status = 1;
        if (rank == 0) out->cycles = t1 - t0;
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // nobody frees tensor memory the pair's MMAs may still touch
    if (warp == 0) tmem_dealloc_pair(tmem_base, 128);
}

}  // namespace neon
