// Issue-rate measurement of the block-scaled tensor-core instructions the grouped GEMM is built on:
// one CTA per SM, operands resident in shared memory (zero-filled tiles in the swizzled layouts the
// GEMM uses), one elected thread issuing `chunks` x 4 (kind::mxf8f6f4, K = 32 each) or `chunks` x 2
// (kind::mxf4, K = 64 each) accumulating MMAs of shape 128 x N back to back into one TMEM
// accumulator, then one commit and a bounded wait.  No global-memory traffic inside the timed
// span, so the figure is the ceiling the tensor pipe (with its shared-memory operand reads) sets for
// a kernel of this shape: the measured denominator of the prefill roofline.
#pragma once
#include <cstdint>

#include "sm100_ptx.cuh"

namespace neon {

struct MmaRateOut {
    long long cycles;   // SM clocks between the first issue and the completion of the last MMA (CTA 0)
    int status;         // non-zero: the bounded wait gave up
};

template <bool MX4>
__global__ void __launch_bounds__(128, 1) mma_rate_kernel(int n, int chunks, int sf_per_chunk, MmaRateOut* out) {
    using namespace sm100;
    extern __shared__ __align__(1024) uint8_t rate_smem[];
    __shared__ uint64_t done_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag, wait_status;
    // layout: A tile 128 rows x 128 B (16 KB), B tile 256 rows x 128 B (32 KB), one zero scale atom (512 B)
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(rate_smem) + 1023) & ~uintptr_t(1023));
    constexpr int kA = 0, kB = 16384, kSF = 16384 + 32768, kBytes = kSF + 512;
    for (int i = threadIdx.x; i < kBytes / 16; i += blockDim.x) reinterpret_cast<uint4*>(base)[i] = make_uint4(0, 0, 0, 0);
    if (threadIdx.x == 0) {
        mbar_init(&done_bar, 1);
        abort_flag = 0;
        wait_status = 0;
        fence_barrier_init();
    }
    fence_proxy_async();
    __syncthreads();
    const int warp = threadIdx.x >> 5;
    if (warp == 0) tmem_alloc(&tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    if (warp == 0) {
        const uint32_t sb = smem_u32(base);
        const uint32_t sf_a = tmem_base + 256, sf_b = tmem_base + 272;  // accumulator in columns 0..N-1
        long long t0 = 0;
        if (elect_one()) {
            // defined scale factors (all zero bytes = 2^-127) for A and, replicated, for every B row group
            tc_copy_sf(sf_a, make_sf_desc(sb + kSF));
            for (int g = 0; g < 8; ++g) tc_copy_sf(sf_b + 4 * g, make_sf_desc(sb + kSF));
            const uint32_t idesc0 = MX4 ? make_idesc_bs(1, 1, (uint32_t)n, 0, 0) : make_idesc_bs(5, 0, (uint32_t)n, 0, 0);
            t0 = clock64();
            if (MX4) {
                const uint64_t a4 = make_sw64_desc(sb + kA), b4 = make_sw64_desc(sb + kB);
                for (int c = 0; c < chunks; ++c) {
                    if (sf_per_chunk) tc_copy_sf(sf_a, make_sf_desc(sb + kSF));  // as the GEMMs do: one weight scale atom per K = 128
#pragma unroll
                    for (int j = 0; j < 2; ++j)
                        mma_mxf4(tmem_base, a4 + 2 * j, b4 + 2 * j, idesc0 + j * (2u << 29), sf_a, sf_b, (uint32_t)(c | j));
                }
            } else {
                const uint64_t a_desc = make_sw128_desc(sb + kA), b_desc = make_sw128_desc(sb + kB);
                for (int c = 0; c < chunks; ++c) {
                    if (sf_per_chunk) tc_copy_sf(sf_a, make_sf_desc(sb + kSF));
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        mma_mxf8f6f4(tmem_base, a_desc + 2 * j, b_desc + 2 * j, idesc0 + j * (1u << 29), sf_a, sf_b,
                                     (uint32_t)(c | j));
                }
            }
            tc_commit(&done_bar);
        }
        __syncwarp();
        const bool ok = mbar_wait(&done_bar, 0, &abort_flag, &wait_status, 1, 4000000000ll);
        const long long t1 = clock64();
        tc_fence_after();
        if (blockIdx.x == 0) {
            // the elected lane holds t0; the others hold 0: the maximum over the warp is the issue time
            long long start = t0;
            for (int o = 16; o > 0; o >>= 1) {
                const long long other = __shfl_xor_sync(0xffffffffu, start, o);
                start = other > start ? other : start;
            }
            if ((threadIdx.x & 31) == 0) {
                out->cycles = t1 - start;
                out->status = ok ? 0 : 1;
            }
        } else if (!ok && (threadIdx.x & 31) == 0) {
            out->status = 1;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, 512);
}

// Copy-rate measurement of the weight stream into one SM's shared memory: one CTA per SM, one thread keeps
// `stages` TMA loads of two weight boxes (256 rows x 128 four-bit columns = 16 KB in global memory) in flight,
// each into its own stage, and reissues a stage as soon as its copy has landed.  No consumer.  With the
// 16U4_ALIGN16B map the nibbles are expanded on the way (32 KB land in shared memory), with the packed map 16 KB.
// CTA b reads boxes b, b + grid, ... of a buffer of n_pairs box pairs, wrapping around: a small buffer stays in L2,
// a large one streams from HBM.
struct TmaRateOut {
    long long cycles;   // SM clocks CTA 0 needed for its `loads` copies
    int status;
};

__global__ void __launch_bounds__(32, 1) tma_rate_kernel(const __grid_constant__ CUtensorMap tm, int n_pairs, int loads, int stages,
                                                         uint32_t tx_bytes, int stage_bytes, TmaRateOut* out) {
    using namespace sm100;
    extern __shared__ __align__(1024) uint8_t rate_smem[];
    __shared__ uint64_t full[8];
    __shared__ int abort_flag, wait_status;
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(rate_smem) + 1023) & ~uintptr_t(1023));
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
        abort_flag = 0;
        wait_status = 0;
        fence_barrier_init();
        prefetch_tmap(&tm);
    }
    fence_proxy_async();
    __syncwarp();
    const long long t0 = clock64();
    bool ok = true;
    int pair = blockIdx.x % n_pairs;
    for (int i = 0; i < loads + stages && ok; ++i) {
        const int s = i % stages;
        if (i >= stages) ok = mbar_wait(&full[s], ((i / stages) - 1) & 1, &abort_flag, &wait_status, 1, 2000000000ll);  // the copy issued `stages` ago
        if (ok && i < loads && elect_one()) {
            mbar_expect_tx(&full[s], tx_bytes);
            tma_load_2d(base + (size_t)s * stage_bytes, &tm, &full[s], 0, pair * 256);
        }
        __syncwarp();
        pair += gridDim.x;
        while (pair >= n_pairs) pair -= n_pairs;
    }
    const long long t1 = clock64();
    if (threadIdx.x == 0) {
        if (blockIdx.x == 0) out->cycles = t1 - t0;
        if (!ok) out->status = 1;
    }
}

}  // namespace neon
