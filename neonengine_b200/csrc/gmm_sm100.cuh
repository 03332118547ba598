// Grouped block-scaled expert GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma with
// TMEM accumulators, plus the weight re-tiling, token-tile list and activation splitting
// kernels around it.
//
// Orientation ("swap-AB"): the 128 weight rows of an item are the M operand (one TMEM lane
// per row), the item's tokens are the N operand (16..128 columns).  Weights stay MXFP4 in HBM
// (4 bits + one E8M0 byte per 32); TMA expands the nibbles into the 8-bit containers that
// tcgen05.mma.kind::mxf8f6f4 reads, and the tensor core applies the E8M0 block scales, so no
// CUDA-core instruction touches a weight.  Activations are split into TERMS e4m3 terms with
// their own E8M0 block scales (bf16 = 2 terms exactly, fp32 SwiGLU output = 4 terms, error
// <= 2^-16 relative); each term is one more accumulating MMA.
#pragma once
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "moe_common.cuh"
#include "moe_kernels.cuh"
#include "sm100_ptx.cuh"
#include "ep.cuh"

namespace neon {

constexpr int kChunkK = 128;  // K elements per pipeline stage (one 128-byte swizzle row)

__host__ __device__ inline int round_up_int(int v, int m) { return (v + m - 1) / m * m; }

// ---------------------------------------------------------------------------------------
// "tc" weight format.  Nibbles are stored box by box: [E][m_tiles][n_chunks][128 rows][64 B],
// so the 128-row x 128-column box one TMA operation fetches is 8 KB of contiguous HBM.
// Kp = K rounded up to 128 and rows rounded up to 128 are padded with zero nibbles.
// gate_up rows are permuted so that TMEM lane quarter q of tile m holds 16 gate rows (lanes
// 0..15: channels 64m+16q+l) followed by their 16 linear rows (lanes 16..31): SwiGLU is then
// one warp shuffle away.  Scales: [E][m_tiles][n_chunks][512 B] atoms, byte
// (r%32)*16 + (r/32)*4 + kb for tile row r and k-block kb of the chunk - the layout that
// tcgen05.cp.32x128b.warpx4 turns into the TMEM scale-factor format.  Pads hold 127 (1.0).
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ int tc_source_row(int r, int gate_up) {
    if (!gate_up) return r;
    int m = r >> 7, q = (r >> 5) & 3, l = r & 31;
    int ch = 64 * m + 16 * q + (l & 15);
    return 2 * ch + (l >> 4);
}

__global__ void repack_tc_kernel(const uint8_t* __restrict__ blocks, const uint8_t* __restrict__ scales, int n_experts,
                                 int rows, int K, int gate_up, uint8_t* __restrict__ wt, uint8_t* __restrict__ sfa) {
    const int Kp = round_up_int(K, kChunkK);
    const int m_tiles = (rows + 127) / 128, n_chunks = Kp / kChunkK;
    const long long total = (long long)n_experts * m_tiles * n_chunks * 128 * 4;  // 16-byte units
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        int u = (int)(i & 3);
        int r = (int)((i >> 2) & 127);
        long long rr = i >> 9;
        int c = (int)(rr % n_chunks);
        rr /= n_chunks;
        int m = (int)(rr % m_tiles), e = (int)(rr / m_tiles);
        int row = 128 * m + r, byte0 = c * 64 + u * 16;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < rows && byte0 < K / 2)
            v = *reinterpret_cast<const uint4*>(blocks + ((size_t)e * rows + tc_source_row(row, gate_up)) * (K / 2) + byte0);
        reinterpret_cast<uint4*>(wt)[i] = v;
    }
    const long long total_sf = (long long)n_experts * m_tiles * n_chunks * 128;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total_sf;
         i += (long long)gridDim.x * blockDim.x) {
        int r = (int)(i % 128);
        long long rr = i / 128;
        int c = (int)(rr % n_chunks);
        rr /= n_chunks;
        int m = (int)(rr % m_tiles), e = (int)(rr / m_tiles);
        int row = 128 * m + r;
        uint32_t word = 0;
        for (int kb = 0; kb < 4; ++kb) {
            int blk = 4 * c + kb;
            uint32_t byte = 127;
            if (row < rows && blk < K / 32) byte = scales[((size_t)e * rows + tc_source_row(row, gate_up)) * (K / 32) + blk];
            word |= byte << (8 * kb);
        }
        *reinterpret_cast<uint32_t*>(sfa + (((size_t)e * m_tiles + m) * n_chunks + c) * 512 + (r & 31) * 16 + (r >> 5) * 4) = word;
    }
}

// Inverse of tc_source_row: the tile row that holds matrix row `row`.
__device__ __forceinline__ int tc_tile_row(int row, int gate_up) {
    if (!gate_up) return row;
    const int ch = row >> 1, half = row & 1;
    return 128 * (ch >> 6) + 32 * ((ch & 63) >> 4) + (ch & 15) + 16 * half;
}

// The mma16 layout (moe_common.cuh) rebuilt from the "tc" layout, so that the mma.sync kernels can
// be served from a handle that keeps only the tensor-core format (the caller's arrays are gone by
// then).  Same output as repack_mma16_kernel on the original tensors; *bad_scale is set when a scale
// byte exceeds 128, which the mma16 scale encoding cannot hold.
__global__ void repack_mma16_from_tc_kernel(const uint8_t* __restrict__ wt, const uint8_t* __restrict__ sfa, int n_experts,
                                            int rows, int K, int gate_up, uint4* __restrict__ wq, uint32_t* __restrict__ sq,
                                            int* bad_scale) {
    const int tiles = rows / 16, nbp = K / 64;
    const int Kp = round_up_int(K, kChunkK), m_tiles = (rows + 127) / 128, n_chunks = Kp / kChunkK;
    const long long total = (long long)n_experts * tiles * nbp * 32;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int lane = (int)(i % 32);
        long long r = i / 32;
        const int bp = (int)(r % nbp);
        r /= nbp;
        const int tl = (int)(r % tiles), e = (int)(r / tiles);
        const int g = lane >> 2, t = lane & 3;
        const int row_lo = gate_up ? 2 * (8 * tl + g) : 16 * tl + g;
        const int row_hi = gate_up ? row_lo + 1 : row_lo + 8;
        uint32_t words[4], sword = 0;
        for (int part = 0; part < 4; ++part) {
            const int row = (part & 1) ? row_hi : row_lo, blk = 2 * bp + (part >> 1);
            const int tr = tc_tile_row(row, gate_up), m = tr >> 7, rr = tr & 127;
            const int byte0 = blk * 16 + 4 * t, c = byte0 >> 6;
            const uint8_t* src = wt + ((((size_t)e * m_tiles + m) * n_chunks + c) * 128 + rr) * 64 + (byte0 & 63);
            uint32_t cds[8];
            for (int b = 0; b < 4; ++b) {
                cds[2 * b] = src[b] & 15u;
                cds[2 * b + 1] = src[b] >> 4;
            }
            words[part] = pack8(cds);
            if (t == 0) {
                const uint32_t byte = sfa[(((size_t)e * m_tiles + m) * n_chunks + (blk >> 2)) * 512 + (rr & 31) * 16 + (rr >> 5) * 4 + (blk & 3)];
                if (byte > 128u) *bad_scale = 1;
                sword |= ((byte + 126u) & 255u) << (8 * part);
            }
        }
        wq[i] = make_uint4(words[0], words[1], words[2], words[3]);
        if (t == 0) sq[(((size_t)e * tiles + tl) * nbp + bp) * 8 + g] = sword;
    }
}

// ---------------------------------------------------------------------------------------
// Token tiles: each expert's run of sorted rows is cut into tiles of at most `tile_tokens`
// rows.  One CTA; writes the tile list, *n_tiles and the tile of every sorted row.
// ---------------------------------------------------------------------------------------
struct TileList {
    int32_t* expert;    // [cap]
    int32_t* row0;      // [cap] first sorted row
    int32_t* rows;      // [cap] rows in the tile (1..tile_tokens)
    int32_t* n_tiles;   // [1]
    int32_t* row_tile;  // [n] tile of each sorted row
};

__global__ void __launch_bounds__(1024) build_tiles_kernel(const int32_t* __restrict__ offset, int n_local,
                                                           int tile_tokens, TileList tl) {
    __shared__ int s_first[kMaxExperts + 1];  // first tile index of each expert
    if (threadIdx.x == 0) {
        int nt = 0;
        for (int e = 0; e < n_local; ++e) {
            s_first[e] = nt;
            int lo = offset[e], hi = offset[e + 1];
            for (int r = lo; r < hi; r += tile_tokens) {
                tl.expert[nt] = e;
                tl.row0[nt] = r;
                tl.rows[nt] = min(tile_tokens, hi - r);
                ++nt;
            }
        }
        s_first[n_local] = nt;
        *tl.n_tiles = nt;
    }
    __syncthreads();
    for (int e = 0; e < n_local; ++e) {
        int lo = offset[e], hi = offset[e + 1];
        for (int r = lo + threadIdx.x; r < hi; r += blockDim.x) tl.row_tile[r] = s_first[e] + (r - lo) / tile_tokens;
    }
}

// Dispatch and token tiles in one launch (one CTA of 1024 threads): the stable counting sort
// of dispatch_block, then up to two tile lists (the gate_up and the down product may cut the
// same sorted rows into tiles of different sizes), one thread per expert.
__device__ void build_tile_list(const int32_t* __restrict__ idx, int n, int e_lo, int n_local, const DispatchArrays& d,
                                int tile_tokens, const TileList& tl, int* s_first) {
    const int tid = threadIdx.x;
    if (tid == 0) {
        int nt = 0;
        for (int e = 0; e < n_local; ++e) {
            s_first[e] = nt;
            nt += (d.count[e] + tile_tokens - 1) / tile_tokens;
        }
        s_first[n_local] = nt;
        *tl.n_tiles = nt;
    }
    __syncthreads();
    for (int e = tid; e < n_local; e += blockDim.x) {
        const int lo = d.offset[e], cnt = d.count[e];
        int t = s_first[e];
        for (int r = 0; r < cnt; r += tile_tokens, ++t) {
            tl.expert[t] = e;
            tl.row0[t] = lo + r;
            tl.rows[t] = min(tile_tokens, cnt - r);
        }
    }
    for (int i = tid; i < n; i += blockDim.x) {
        const int pos = d.inv[i];
        if (pos >= 0) {
            const int e = idx[i] - e_lo;
            tl.row_tile[pos] = s_first[e] + (pos - d.offset[e]) / tile_tokens;
        }
    }
    __syncthreads();
}

__global__ void __launch_bounds__(1024) dispatch_tiles_kernel(const int32_t* __restrict__ idx, int n, int e_lo, int n_local,
                                                              DispatchArrays d, int tile_tokens, TileList tl) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ int dsmem[];
    __shared__ int s_first[kMaxExperts + 1];
    dispatch_block(idx, n, e_lo, n_local, d, dsmem);
    __syncthreads();  // offsets and counts are in global memory, written by this CTA
    build_tile_list(idx, n, e_lo, n_local, d, tile_tokens, tl, s_first);
}

// The same result from many CTAs, for prefill-sized passes (one CTA needs ~110 us for 32 768 entries).  Two
// launches.  dispatch_count_kernel: CTA b counts the experts of entries [1024 b, 1024 b + 1024) into
// blk_count[b][e]; the CTA that finishes last turns the counts into everything that does not depend on single
// entries: count / offset per expert, the write position blk_base[b][e] of CTA b's first entry of expert e
// (offset[e] + the counts of the CTAs before it: the sort stays stable), the first tile of every expert and the
// tile list.  dispatch_place_kernel: every CTA ranks its entries again (same warp-match scheme) and writes perm,
// inv and the tile of every sorted row.
struct DispatchScratch {
    int32_t* blk_count;   // [blocks][n_local]
    int32_t* blk_base;    // [blocks][n_local]
    int32_t* tile_first;  // [n_local + 1]
    unsigned* done;       // [1] CTAs that have written their counts; left at zero
};

// Entry of thread tid of a 1024-entry chunk: its local expert (or -1), its rank among the entries of that expert
// in its warp, and - in wc[warp][e] - the number of such entries in the warps before it (after the barriers).
__device__ __forceinline__ void dispatch_rank_chunk(const int32_t* idx, int n, int e_lo, int n_local, int i, int* wc, int* cnt, int& e, int& rank) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int j = tid; j < 32 * n_local; j += 1024) wc[j] = 0;
    e = -1;
    if (i < n) {
        e = __ldcg(idx + i) - e_lo;
        if (e < 0 || e >= n_local) e = -1;
    }
    __syncthreads();
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    rank = __popc(peers & ((1u << lane) - 1u));
    if (e >= 0 && rank == 0) wc[warp * n_local + e] = __popc(peers);
    __syncthreads();
    for (int ee = tid; ee < n_local; ee += 1024) {
        int run = 0;
#pragma unroll 8
        for (int w = 0; w < 32; ++w) {
            const int c = wc[w * n_local + ee];
            wc[w * n_local + ee] = run;
            run += c;
        }
        cnt[ee] = run;
    }
    __syncthreads();
}

__global__ void __launch_bounds__(1024) dispatch_count_kernel(const int32_t* __restrict__ idx, int n, int e_lo, int n_local,
                                                              DispatchArrays d, int tile_tokens, TileList tl, DispatchScratch sc) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ int dsmem[];  // [32][n_local]
    __shared__ int cnt[kMaxExperts], off[kMaxExperts + 1], first[kMaxExperts + 1];
    __shared__ int s_last;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, b = blockIdx.x, nb = gridDim.x;
    int e, rank;
    dispatch_rank_chunk(idx, n, e_lo, n_local, b * 1024 + tid, dsmem, cnt, e, rank);
    for (int ee = tid; ee < n_local; ee += 1024) __stcg(sc.blk_count + (size_t)b * n_local + ee, cnt[ee]);
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(sc.done, 1u) == (unsigned)(nb - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const int tt = tile_tokens > 0 ? tile_tokens : 1;   // tile_tokens 0: the sort alone, no tile list (the sender's sort of expert parallelism)
    for (int ee = tid; ee < n_local; ee += 1024) {  // totals per expert
        int run = 0;
        for (int bb = 0; bb < nb; ++bb) run += __ldcg(sc.blk_count + (size_t)bb * n_local + ee);
        cnt[ee] = run;
    }
    __syncthreads();
    if (warp == 0) {  // exclusive scans of the counts and of the tile counts, 8 experts per lane
        int c[8], tsum = 0, csum = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int ee = lane * 8 + j;
            c[j] = ee < n_local ? cnt[ee] : 0;
            csum += c[j];
            tsum += (c[j] + tt - 1) / tt;
        }
        int cpre = csum, tpre = tsum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int a = __shfl_up_sync(0xffffffffu, cpre, o), t2 = __shfl_up_sync(0xffffffffu, tpre, o);
            if (lane >= o) { cpre += a; tpre += t2; }
        }
        int crun = cpre - csum, trun = tpre - tsum;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int ee = lane * 8 + j;
            if (ee < n_local) {
                off[ee] = crun;
                first[ee] = trun;
                d.count[ee] = c[j];
                d.offset[ee] = crun;
                sc.tile_first[ee] = trun;
            }
            crun += c[j];
            trun += (c[j] + tt - 1) / tt;
        }
        if (lane == 31) {
            off[n_local] = cpre;
            first[n_local] = tpre;
            d.offset[n_local] = cpre;
            sc.tile_first[n_local] = tpre;
            if (tile_tokens > 0) *tl.n_tiles = tpre;
        }
    }
    __syncthreads();
    for (int ee = tid; ee < n_local; ee += 1024) {
        int run = off[ee];
        for (int bb = 0; bb < nb; ++bb) {  // where every CTA's entries of this expert start
            sc.blk_base[(size_t)bb * n_local + ee] = run;
            run += __ldcg(sc.blk_count + (size_t)bb * n_local + ee);
        }
        if (tile_tokens > 0) {
            const int lo = off[ee], c = cnt[ee];
            int t = first[ee];
            for (int r = 0; r < c; r += tile_tokens, ++t) {
                tl.expert[t] = ee;
                tl.row0[t] = lo + r;
                tl.rows[t] = min(tile_tokens, c - r);
            }
        }
    }
    if (tid == 0) *sc.done = 0u;  // ready for the next pass
}

__global__ void __launch_bounds__(1024) dispatch_place_kernel(const int32_t* __restrict__ idx, int n, int e_lo, int n_local,
                                                              DispatchArrays d, int tile_tokens, TileList tl, DispatchScratch sc) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ int dsmem[];  // [32][n_local]
    __shared__ int cnt[kMaxExperts];
    const int tid = threadIdx.x, warp = tid >> 5, b = blockIdx.x, i = b * 1024 + tid;
    int e, rank;
    dispatch_rank_chunk(idx, n, e_lo, n_local, i, dsmem, cnt, e, rank);
    if (i < n) {
        if (e >= 0) {
            const int pos = sc.blk_base[(size_t)b * n_local + e] + dsmem[warp * n_local + e] + rank;
            d.perm[pos] = i;
            d.inv[i] = pos;
            if (tile_tokens > 0) tl.row_tile[pos] = sc.tile_first[e] + (pos - d.offset[e]) / tile_tokens;
        } else {
            d.inv[i] = -1;
        }
    }
}

// The same for at most 1024 entries (decode batches): one entry per thread, four barriers, all
// scans done by warps in shared memory.  Identical results to dispatch_tiles_kernel.
__device__ __forceinline__ void dispatch_tiles_small_body(const int32_t* idx, int n, int e_lo, int n_local, DispatchArrays d,
                                                          int tile_tokens, TileList tl, int* dsmem) {
    int* wc = dsmem;                // [32][n_local] entries of each expert per warp, then their prefix
    __shared__ int cnt[kMaxExperts], off[kMaxExperts + 1], first[kMaxExperts + 1];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int j = tid; j < 32 * n_local; j += 1024) wc[j] = 0;
    int e = -1;
    if (tid < n) {
        e = __ldcg(idx + tid) - e_lo;  // L2: the entries may have been written by other CTAs of this launch
        if (e < 0 || e >= n_local) e = -1;
    }
    __syncthreads();
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    if (e >= 0 && rank == 0) wc[warp * n_local + e] = __popc(peers);
    __syncthreads();
    for (int ee = tid; ee < n_local; ee += 1024) {
        int run = 0;
#pragma unroll 8
        for (int w = 0; w < 32; ++w) {
            int c = wc[w * n_local + ee];
            wc[w * n_local + ee] = run;
            run += c;
        }
        cnt[ee] = run;
    }
    __syncthreads();
    if (warp == 0) {  // exclusive scans of the counts and of the tile counts, 8 experts per lane
        int c[8], tsum = 0, csum = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            int ee = lane * 8 + j;
            c[j] = ee < n_local ? cnt[ee] : 0;
            csum += c[j];
            tsum += (c[j] + tile_tokens - 1) / tile_tokens;
        }
        int cpre = csum, tpre = tsum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int a = __shfl_up_sync(0xffffffffu, cpre, o), b = __shfl_up_sync(0xffffffffu, tpre, o);
            if (lane >= o) { cpre += a; tpre += b; }
        }
        int crun = cpre - csum, trun = tpre - tsum;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            int ee = lane * 8 + j;
            if (ee < n_local) {
                off[ee] = crun;
                first[ee] = trun;
                d.count[ee] = c[j];
                d.offset[ee] = crun;
            }
            crun += c[j];
            trun += (c[j] + tile_tokens - 1) / tile_tokens;
        }
        if (lane == 31) {
            off[n_local] = cpre;
            first[n_local] = tpre;
            d.offset[n_local] = cpre;
            *tl.n_tiles = tpre;
        }
    }
    __syncthreads();
    if (tid < n) {
        if (e >= 0) {
            const int pos = off[e] + wc[warp * n_local + e] + rank;
            d.perm[pos] = tid;
            d.inv[tid] = pos;
            tl.row_tile[pos] = first[e] + (pos - off[e]) / tile_tokens;
        } else {
            d.inv[tid] = -1;
        }
    }
    for (int ee = tid; ee < n_local; ee += 1024) {
        const int lo = off[ee], c = cnt[ee];
        int t = first[ee];
        for (int r = 0; r < c; r += tile_tokens, ++t) {
            tl.expert[t] = ee;
            tl.row0[t] = lo + r;
            tl.rows[t] = min(tile_tokens, c - r);
        }
    }
}

__global__ void __launch_bounds__(1024) dispatch_tiles_small_kernel(const int32_t* __restrict__ idx, int n, int e_lo,
                                                                    int n_local, DispatchArrays d, int tile_tokens,
                                                                    TileList tl) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ int dsmem[];
    dispatch_tiles_small_body(idx, n, e_lo, n_local, d, tile_tokens, tl, dsmem);
}

// Router and dispatch in one launch for decode batches (T * k <= 1024): one CTA of 1024 threads
// routes each token; the CTA that finishes last (a counter in global memory) then runs the
// dispatch + token-tile construction over all entries, so the pass needs no separate dispatch
// launch.  Results are identical to router_topk_wide_kernel followed by
// dispatch_tiles_small_kernel.  Dynamic shared memory: max(router need, 32 * n_local ints).
__global__ void __launch_bounds__(1024)
router_dispatch_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ wr, const uint16_t* __restrict__ br,
                       const float* __restrict__ logit_bias, int T, int H, int E, int k, int32_t* idx, float* __restrict__ w,
                       float* __restrict__ tok_amax, unsigned* done, DispatchArrays d, int tile_tokens, TileList tl) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char rsmem[];
    __shared__ int is_last;
    router_topk_wide_body(x, wr, br, logit_bias, T, H, E, k, idx, w, tok_amax, rsmem);
    __syncthreads();  // this token's entries are written
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned prev = atomicAdd(done, 1u);
        is_last = prev == gridDim.x - 1;
        if (is_last) *done = 0u;  // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    dispatch_tiles_small_body(idx, T * k, 0, E, d, tile_tokens, tl, reinterpret_cast<int*>(rsmem));
}

// ---------------------------------------------------------------------------------------
// Activation splitting.  One warp per (sorted row p, 128-wide K chunk); lane l owns 4
// elements.  Term t: per 32-block scale 2^(floor(log2 amax) - 7) (E8M0), value rounded to
// e4m3, remainder carried to the next term.
//
// Output: one block per (token tile, chunk), written as the exact shared-memory image the
// GEMM stage wants, so a single bulk copy brings in all terms and their scales:
//   [TERMS x 512 B scale atoms, padded to 1024 B][row group 0: term 0 | term 1 | ...][row group 1: ...] ...
// A row group is 8 rows x 128 B of one term in the 128-byte-swizzled K-major layout (the
// 16-byte unit u of row r sits at unit u ^ (r % 8)).  Block stride = act_block_bytes().
// FROM_BF16: source rows are bf16 hidden states gathered through perm (token = perm[p]/k);
// otherwise fp32 rows [p][K].
// ---------------------------------------------------------------------------------------
// Two block layouts.  Sequential (prefill, tile_tokens = 128): as above, one MMA per term.
// Stacked (decode, tile_tokens <= 32): the terms are stacked along N - B row t*npad + j is
// term t of tile row j, npad = rows rounded up to 8 - so one MMA covers all terms and reads
// the weight tile once; the block is just TERMS*npad rows x 128 B.  Stacked terms use one
// power-of-two scale per ROW (term t: row scale / 16^t) instead of per 32-block scales; it is
// applied by the GEMM epilogue when it adds the terms' columns, so the tensor core sees unit
// activation scales and no activation scale factor ever travels (split_rows_stacked_kernel).
// Bytes the scale atoms take at the head of a sequential block: TERMS x 512 B, rounded up to the
// 1024-byte alignment the 128-byte-swizzled row groups behind them need.
__host__ __device__ constexpr int act_header_bytes(int terms) { return (terms * 512 + 1023) / 1024 * 1024; }

__host__ __device__ inline size_t act_block_bytes(int terms, int tile_tokens, bool stacked) {
    if (stacked) return (size_t)terms * tile_tokens * 128;
    return (size_t)act_header_bytes(terms) + (size_t)(tile_tokens / 8) * terms * 1024;
}

// Chunks one warp of split_rows_kernel handles (all their loads are issued before any arithmetic).
constexpr int kSplitChunksPerWarp = 4;

template <int TERMS, bool FROM_BF16, bool STACK>
__global__ void __launch_bounds__(256) split_rows_kernel(const void* __restrict__ src, const int32_t* __restrict__ perm,
                                                         int top_k, int K, int n_rows, const int32_t* __restrict__ row_tile,
                                                         const int32_t* __restrict__ tile_row0,
                                                         const int32_t* __restrict__ tile_rows, int tile_tokens,
                                                         uint8_t* __restrict__ act) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int U = kSplitChunksPerWarp;
    const int Kp = round_up_int(K, kChunkK), n_chunks = Kp / kChunkK, groups = (n_chunks + U - 1) / U;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= n_rows * groups) return;
    const int p = warp / groups, c0 = (warp % groups) * U;
    float vv[U][4];
    {
        const uint16_t* row16 = nullptr;
        const float* row32 = nullptr;
        if (FROM_BF16) row16 = static_cast<const uint16_t*>(src) + (size_t)(perm[p] / top_k) * K;
        else row32 = static_cast<const float*>(src) + (size_t)p * K;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k0 = (c0 + u) * kChunkK + 4 * lane;
            vv[u][0] = vv[u][1] = vv[u][2] = vv[u][3] = 0.f;
            if (c0 + u < n_chunks && k0 < K) {
                if (FROM_BF16) {
                    const uint2 raw = *reinterpret_cast<const uint2*>(row16 + k0);
                    vv[u][0] = __uint_as_float(raw.x << 16);
                    vv[u][1] = __uint_as_float(raw.x & 0xffff0000u);
                    vv[u][2] = __uint_as_float(raw.y << 16);
                    vv[u][3] = __uint_as_float(raw.y & 0xffff0000u);
                } else {
                    const float4 raw = *reinterpret_cast<const float4*>(row32 + k0);
                    vv[u][0] = raw.x; vv[u][1] = raw.y; vv[u][2] = raw.z; vv[u][3] = raw.w;
                }
            }
        }
    }
    const int tile = row_tile[p], j = p - tile_row0[tile];
    const int npad = (tile_rows[tile] + 7) & ~7;
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int c = c0 + u;
        if (c >= n_chunks) break;
        float* v = vv[u];
        uint8_t* blk = act + ((size_t)tile * n_chunks + c) * act_block_bytes(TERMS, tile_tokens, STACK);
#pragma unroll
        for (int t = 0; t < TERMS; ++t) {
            float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
            int ef = (int)((__float_as_uint(amax) >> 23) & 0xffu);
            int sb = amax > 0.f ? max(ef - 7, 0) : 127;           // E8M0 byte: amax / scale in [128, 256)
            float inv = __uint_as_float((uint32_t)(254 - sb) << 23);
            float scale = sb > 0 ? __uint_as_float((uint32_t)sb << 23) : __uint_as_float(0x00400000u);
            __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[0] * inv, v[1] * inv), __NV_SATFINITE, __NV_E4M3);
            __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[2] * inv, v[3] * inv), __NV_SATFINITE, __NV_E4M3);
            // row of this term inside the block and the place of its scale word
            const int n = STACK ? t * npad + j : j;
            uint8_t* row_ptr = STACK ? blk + 1024 + (size_t)(n >> 3) * 1024
                                     : blk + act_header_bytes(TERMS) + ((size_t)(n >> 3) * TERMS + t) * 1024;
            *reinterpret_cast<uint32_t*>(row_ptr + (n & 7) * 128 + (((lane >> 2) ^ (n & 7)) << 4) + ((lane & 3) << 2)) =
                (uint32_t)lo | ((uint32_t)hi << 16);
            if (t + 1 < TERMS) {
                __half2_raw blo = __nv_cvt_fp8x2_to_halfraw2(lo, __NV_E4M3), bhi = __nv_cvt_fp8x2_to_halfraw2(hi, __NV_E4M3);
                float2 flo = __half22float2(*reinterpret_cast<__half2*>(&blo)), fhi = __half22float2(*reinterpret_cast<__half2*>(&bhi));
                v[0] -= flo.x * scale; v[1] -= flo.y * scale; v[2] -= fhi.x * scale; v[3] -= fhi.y * scale;
            }
            uint32_t w = (uint32_t)sb;
            w |= __shfl_sync(0xffffffffu, (uint32_t)sb, 8) << 8;
            w |= __shfl_sync(0xffffffffu, (uint32_t)sb, 16) << 16;
            w |= __shfl_sync(0xffffffffu, (uint32_t)sb, 24) << 24;
            if (lane == 0) *reinterpret_cast<uint32_t*>(blk + (STACK ? 0 : t * 512) + (n & 31) * 16 + (n >> 5) * 4) = w;
        }
    }
}

// Largest magnitude of every row (one warp per row, all loads issued before the reduction);
// used when no producer kernel has already computed it.
template <bool FROM_BF16>
__global__ void __launch_bounds__(256) row_amax_kernel(const void* __restrict__ src, int K, int n_rows,
                                                       float* __restrict__ amax_out) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (r >= n_rows) return;
    float m = 0.f;
    if (FROM_BF16) {
        const uint2* row = reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(src) + (size_t)r * K);
        for (int i = lane; i < K / 4; i += 32) {
            uint2 raw = row[i];
            m = fmaxf(m, fmaxf(fmaxf(fabsf(__uint_as_float(raw.x << 16)), fabsf(__uint_as_float(raw.x & 0xffff0000u))),
                               fmaxf(fabsf(__uint_as_float(raw.y << 16)), fabsf(__uint_as_float(raw.y & 0xffff0000u)))));
        }
    } else {
        const float4* row = reinterpret_cast<const float4*>(static_cast<const float*>(src) + (size_t)r * K);
        for (int i = lane; i < K / 4; i += 32) {
            float4 v = row[i];
            m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) amax_out[r] = m;
}

// Stacked-mode splitting: one warp per (sorted row p, 128-wide chunk), lane l owns 4 elements.
// The row's largest magnitude comes precomputed: amax_in[perm[p]/top_k] for gathered bf16 hidden
// rows (FROM_BF16), amax_in[p] otherwise; with amax_in == null every row uses the bound
// amax_const (the clamped SwiGLU output is bounded by limit*(limit+1), so the down product's
// input needs no measurement at all).  Term t is RN_e4m3(residual / (s / 16^t)) with
// s = 2^(floor(log2 amax) - 7); row_scale[p] = s.
template <int TERMS, bool FROM_BF16>
__global__ void __launch_bounds__(256) split_rows_stacked_kernel(const void* __restrict__ src, const int32_t* __restrict__ perm,
                                                                 int top_k, int K, int n_rows,
                                                                 const int32_t* __restrict__ row_tile,
                                                                 const int32_t* __restrict__ tile_row0,
                                                                 const int32_t* __restrict__ tile_rows, int tile_tokens,
                                                                 const float* __restrict__ amax_in, float amax_const,
                                                                 uint8_t* __restrict__ act, float* __restrict__ row_scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int Kp = round_up_int(K, kChunkK), n_chunks = Kp / kChunkK;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= n_rows * n_chunks) return;
    const int p = warp / n_chunks, c = warp - p * n_chunks;
    const int src_row = FROM_BF16 ? perm[p] / top_k : p;
    const int k0 = c * kChunkK + 4 * lane;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (k0 < K) {
        if (FROM_BF16) {
            uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(src) + (size_t)src_row * K + k0);
            v[0] = __uint_as_float(raw.x << 16);
            v[1] = __uint_as_float(raw.x & 0xffff0000u);
            v[2] = __uint_as_float(raw.y << 16);
            v[3] = __uint_as_float(raw.y & 0xffff0000u);
        } else {
            float4 raw = *reinterpret_cast<const float4*>(static_cast<const float*>(src) + (size_t)src_row * K + k0);
            v[0] = raw.x; v[1] = raw.y; v[2] = raw.z; v[3] = raw.w;
        }
    }
    const float amax = amax_in ? amax_in[src_row] : amax_const;
    // exponent field of the row scale, kept where every term's scale and its inverse stay normal
    const int ef = (int)((__float_as_uint(amax) >> 23) & 0xffu);
    const int sb = amax > 0.f ? min(max(ef - 7, 4 * TERMS + 1), 250) : 127;
    if (row_scale && lane == 0 && c == 0) row_scale[p] = __uint_as_float((uint32_t)sb << 23);
    const int tile = row_tile[p], j = p - tile_row0[tile];
    const int npad = (tile_rows[tile] + 7) & ~7;
    uint8_t* blk = act + ((size_t)tile * n_chunks + c) * act_block_bytes(TERMS, tile_tokens, true);
#pragma unroll
    for (int t = 0; t < TERMS; ++t) {
        const float inv = __uint_as_float((uint32_t)(254 - (sb - 4 * t)) << 23);
        const float scale = __uint_as_float((uint32_t)(sb - 4 * t) << 23);
        __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[0] * inv, v[1] * inv), __NV_SATFINITE, __NV_E4M3);
        __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[2] * inv, v[3] * inv), __NV_SATFINITE, __NV_E4M3);
        const int n = t * npad + j;
        *reinterpret_cast<uint32_t*>(blk + (size_t)(n >> 3) * 1024 + (n & 7) * 128 + (((lane >> 2) ^ (n & 7)) << 4) +
                                     ((lane & 3) << 2)) = (uint32_t)lo | ((uint32_t)hi << 16);
        if (t + 1 < TERMS) {
            __half2_raw blo = __nv_cvt_fp8x2_to_halfraw2(lo, __NV_E4M3), bhi = __nv_cvt_fp8x2_to_halfraw2(hi, __NV_E4M3);
            float2 flo = __half22float2(*reinterpret_cast<__half2*>(&blo)), fhi = __half22float2(*reinterpret_cast<__half2*>(&bhi));
            v[0] -= flo.x * scale; v[1] -= flo.y * scale; v[2] -= fhi.x * scale; v[3] -= fhi.y * scale;
        }
    }
}

// Packed-4-bit flavour of the stacked split, for tcgen05.mma.kind::mxf4 (both operands e2m1,
// weights straight from HBM without expansion).  An e2m1 term carries ~2.6 bits, so a value is
// written as TERMS terms with scales s, s/6, s/36, ... (s = amax/6; the residual of a term is
// at most one sixth of its scale's range); the scales are applied by the GEMM epilogue, so
// they need not be powers of two.  Rows are 64 bytes (128 codes, low nibble = even column)
// in the 64-byte-swizzled K-major layout: 16-byte unit u of row n sits at u ^ ((n >> 1) & 3).
// Block per (tile, chunk): TERMS*npad rows x 64 B.  row_scale[p] = s.
__host__ __device__ inline size_t act4_block_bytes(int terms, int tile_tokens) { return (size_t)terms * tile_tokens * 64; }

template <int TERMS, bool FROM_BF16>
__global__ void __launch_bounds__(256) split_rows_fp4_kernel(const void* __restrict__ src, const int32_t* __restrict__ perm,
                                                             int top_k, int K, int n_rows,
                                                             const int32_t* __restrict__ row_tile,
                                                             const int32_t* __restrict__ tile_row0,
                                                             const int32_t* __restrict__ tile_rows, int tile_tokens,
                                                             const float* __restrict__ amax_in, float amax_const,
                                                             uint8_t* __restrict__ act, float* __restrict__ row_scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int Kp = round_up_int(K, kChunkK), n_chunks = Kp / kChunkK;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= n_rows * n_chunks) return;
    const int p = warp / n_chunks, c = warp - p * n_chunks;
    const int src_row = FROM_BF16 ? perm[p] / top_k : p;
    const int k0 = c * kChunkK + 4 * lane;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (k0 < K) {
        if (FROM_BF16) {
            uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(src) + (size_t)src_row * K + k0);
            v[0] = __uint_as_float(raw.x << 16);
            v[1] = __uint_as_float(raw.x & 0xffff0000u);
            v[2] = __uint_as_float(raw.y << 16);
            v[3] = __uint_as_float(raw.y & 0xffff0000u);
        } else {
            float4 raw = *reinterpret_cast<const float4*>(static_cast<const float*>(src) + (size_t)src_row * K + k0);
            v[0] = raw.x; v[1] = raw.y; v[2] = raw.z; v[3] = raw.w;
        }
    }
    const float amax = amax_in ? amax_in[src_row] : amax_const;
    float scale = fmaxf(amax, 1e-30f) * (1.f / 6.f);
    if (row_scale && lane == 0 && c == 0) row_scale[p] = scale;
    const int tile = row_tile[p], j = p - tile_row0[tile];
    const int npad = (tile_rows[tile] + 7) & ~7;
    uint8_t* blk = act + ((size_t)tile * n_chunks + c) * act4_block_bytes(TERMS, tile_tokens);
#pragma unroll
    for (int t = 0; t < TERMS; ++t) {
        const float inv = 1.f / scale;
        __nv_fp4x2_storage_t lo = __nv_cvt_float2_to_fp4x2(make_float2(v[0] * inv, v[1] * inv), __NV_E2M1, cudaRoundNearest);
        __nv_fp4x2_storage_t hi = __nv_cvt_float2_to_fp4x2(make_float2(v[2] * inv, v[3] * inv), __NV_E2M1, cudaRoundNearest);
        const int n = t * npad + j;
        *reinterpret_cast<uint16_t*>(blk + (size_t)(n >> 3) * 512 + (n & 7) * 64 + ((((lane >> 3) ^ ((n >> 1) & 3))) << 4) +
                                     ((lane & 7) << 1)) = (uint16_t)((uint32_t)lo | ((uint32_t)hi << 8));
        if (t + 1 < TERMS) {
            __half2_raw blo = __nv_cvt_fp4x2_to_halfraw2(lo, __NV_E2M1), bhi = __nv_cvt_fp4x2_to_halfraw2(hi, __NV_E2M1);
            float2 flo = __half22float2(*reinterpret_cast<__half2*>(&blo)), fhi = __half22float2(*reinterpret_cast<__half2*>(&bhi));
            v[0] = fmaf(-flo.x, scale, v[0]); v[1] = fmaf(-flo.y, scale, v[1]);
            v[2] = fmaf(-fhi.x, scale, v[2]); v[3] = fmaf(-fhi.y, scale, v[3]);
            scale *= (1.f / 6.f);
        }
    }
}

// MXFP4 quantisation of activation rows for tcgen05.mma.kind::mxf4 at prefill (both operands 4-bit):
// per block of 32 along K the E8M0 scale is 2^(floor(log2 amax) - 2), so amax lands in [4, 8) and
// clips to 6; every value is rounded to the nearest e2m1 magnitude, ties to the even code.  One warp
// per (sorted row p, 128-wide chunk), lane l owns 4 elements.  Block per (token tile, chunk):
// [512 B scale atom: byte (n % 32) * 16 + (n / 32) * 4 + kb for tile row n, k-block kb]
// [16 row groups x 512 B: rows of 64 bytes (128 codes, low nibble = even column) in the
// 64-byte-swizzled K-major layout, 16-byte unit u of row n at u ^ ((n >> 1) & 3)].
constexpr int kQuant4BlockBytes = 512 + 128 * 64;

template <bool FROM_BF16>
__global__ void __launch_bounds__(256) quant_rows_mxfp4_kernel(const void* __restrict__ src, const int32_t* __restrict__ perm,
                                                               int top_k, int K, int n_rows, const int32_t* __restrict__ row_tile,
                                                               const int32_t* __restrict__ tile_row0, uint8_t* __restrict__ act) {
    pdl_launch_dependents();
    pdl_wait();
    const int Kp = round_up_int(K, kChunkK), n_chunks = Kp / kChunkK;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= n_rows * n_chunks) return;
    const int p = warp / n_chunks, c = warp - p * n_chunks;
    const int src_row = FROM_BF16 ? perm[p] / top_k : p;
    const int k0 = c * kChunkK + 4 * lane;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (k0 < K) {
        if (FROM_BF16) {
            const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(src) + (size_t)src_row * K + k0);
            v[0] = __uint_as_float(raw.x << 16);
            v[1] = __uint_as_float(raw.x & 0xffff0000u);
            v[2] = __uint_as_float(raw.y << 16);
            v[3] = __uint_as_float(raw.y & 0xffff0000u);
        } else {
            const float4 raw = *reinterpret_cast<const float4*>(static_cast<const float*>(src) + (size_t)src_row * K + k0);
            v[0] = raw.x; v[1] = raw.y; v[2] = raw.z; v[3] = raw.w;
        }
    }
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    const int ef = (int)((__float_as_uint(amax) >> 23) & 0xffu);
    const int sb = amax > 0.f ? min(max(ef - 2, 1), 254) : 127;       // E8M0 byte of the block scale
    const float inv = __uint_as_float((uint32_t)(254 - sb) << 23);     // 1 / scale, exact
    const __nv_fp4x2_storage_t lo = __nv_cvt_float2_to_fp4x2(make_float2(v[0] * inv, v[1] * inv), __NV_E2M1, cudaRoundNearest);
    const __nv_fp4x2_storage_t hi = __nv_cvt_float2_to_fp4x2(make_float2(v[2] * inv, v[3] * inv), __NV_E2M1, cudaRoundNearest);
    const int tile = row_tile[p], n = p - tile_row0[tile];
    uint8_t* blk = act + ((size_t)tile * n_chunks + c) * kQuant4BlockBytes;
    *reinterpret_cast<uint16_t*>(blk + 512 + (size_t)(n >> 3) * 512 + (n & 7) * 64 + (((lane >> 3) ^ ((n >> 1) & 3)) << 4) +
                                 ((lane & 7) << 1)) = (uint16_t)((uint32_t)lo | ((uint32_t)hi << 8));
    uint32_t w = (uint32_t)sb;
    w |= __shfl_sync(0xffffffffu, (uint32_t)sb, 8) << 8;
    w |= __shfl_sync(0xffffffffu, (uint32_t)sb, 16) << 16;
    w |= __shfl_sync(0xffffffffu, (uint32_t)sb, 24) << 24;
    if (lane == 0) *reinterpret_cast<uint32_t*>(blk + (n & 31) * 16 + (n >> 5) * 4) = w;
}

// ---------------------------------------------------------------------------------------
// The GEMM.  Persistent CTAs walk items = (token tile, 128-row weight tile), item index =
// blockIdx.x + i*gridDim.x, weight tile fastest so that concurrent CTAs share a token tile's
// activations in L2.  Six warps: 0 = TMA producer, 1 = MMA issuer, 2..5 = epilogue (TMEM
// lane quarter = warp % 4).
//
// A pipeline stage holds KC consecutive K chunks: KC weight boxes (one TMA operation; the
// boxes of an item are contiguous rows of the 2-D weight tensor), KC activation blocks (one
// bulk copy, they are contiguous too) and KC weight scale atoms (one bulk copy).  Each
// mbarrier round trip and each copy / tcgen05 issue costs a few hundred cycles of a single
// thread, so the per-stage fixed cost is spread over 2 x 8 KB of weights.
// Accumulators are double-buffered in TMEM so the epilogue of item i overlaps the MMAs of
// item i+1.  Every wait is bounded: on a timeout the CTA records a code in *status, all
// roles leave their loops, in-flight copies get time to land, TMEM is freed.
// ---------------------------------------------------------------------------------------
struct GmmParams {
    const uint8_t* sfa;    // [E][m_tiles][n_chunks][512]
    const uint8_t* act;    // [tile][n_chunks][act_block_bytes]
    const float* row_scale;  // stacked mode: power-of-two scale of each sorted row's first term, or null:
    float row_scale_const;   //   then every row uses this one
    const int32_t *tile_expert, *tile_row0, *tile_rows, *n_tiles;
    int m_tiles, n_chunks, rows_total;
    uint32_t a_tx_bytes;   // bytes one 128 x 128 4-bit box reports to its mbarrier
    int tmem_cols;         // TMEM columns to allocate (power of two)
    int stages;            // pipeline stages in use (<= GmmSmem::kStages)
#ifdef NEON_MOE_INSTRUMENT
    long long* trace;      // optional [2 roles][512 stages][2] clock stamps of CTA 0 (instrumented builds only)
#endif
    const uint16_t* bias;  // [E][rows_total], original row order
    // gate_up epilogue
    float* a_out;          // [n][inter] fp32
    int inter;
    float limit, alpha;
    // down epilogue
    const int32_t* perm;
    const float* route_w;
    float* y;              // [n][hidden] fp32, sorted order
    int hidden;
    int* status;
    // expert parallelism with peer stores: row perm[pos] of the received order goes straight into its token owner's
    // buffer (peer.n_ranks == 0: rows go to y)
    PeerRows<float> peer;
};

// MX4: packed 4-bit operands (kind::mxf4): a weight box is 8 KB in shared memory, rows are 64 B.
// Stacked: the activations are TERMS e2m1 terms with unit block scales (decode).  Not stacked
// (TERMS == 1): the activations are MXFP4-quantised, one scale atom + 64-byte rows per block.
template <int BN_MAX, int TERMS, bool STACK, int KC, bool MX4 = false>
struct GmmSmem {
    static_assert(!MX4 || STACK || TERMS == 1, "quantised 4-bit activations are a single term");
    static constexpr int kABytes = MX4 ? 8192 : 16384;  // one 128 x 128 weight box in shared memory
    static constexpr int kActBytes = MX4 ? (STACK ? TERMS * BN_MAX * 64 : 512 + BN_MAX * 64)
                                         : (STACK ? TERMS * BN_MAX * 128 : act_header_bytes(TERMS) + (BN_MAX / 8) * TERMS * 1024);
    static constexpr int kStage = (KC * (kABytes + kActBytes + 512) + 1023) / 1024 * 1024;
    static constexpr int kSfCols = KC * (STACK ? 4 : 4 * (1 + TERMS));  // TMEM columns of scales per stage
    static constexpr int kAccCols = STACK ? TERMS * BN_MAX : BN_MAX;    // TMEM columns of one accumulator buffer
    static constexpr int kSfBase = 2 * kAccCols + (STACK ? 8 : 0);  // stacked: two atoms (N up to 256) of unit scales first
    static constexpr int kTail = 1024;
    static constexpr int kBudget = 225 * 1024;
    static constexpr int kStagesFit = (kBudget - kTail - 1024) / kStage;
    static constexpr int kStagesTmem = (512 - kSfBase) / kSfCols;
    static constexpr int kStages = kStagesFit < kStagesTmem ? kStagesFit : kStagesTmem;
    static constexpr int smem_bytes(int stages) { return stages * kStage + kTail + 1024; }
    static constexpr int tmem_cols(int stages) {
        int need = kSfBase + stages * kSfCols, cols = 32;
        while (cols < need) cols *= 2;
        return cols;
    }
    static_assert(kStages >= 2, "at least two stages");
    static_assert(KC * kABytes % 1024 == 0 && kActBytes % 512 == 0, "alignment");
};

constexpr long long kWaitLimitCycles = 400000000ll;  // ~0.2 s at 2 GHz

template <int BN_MAX, int TERMS, bool GATE_UP, bool STACK, int KC, bool MX4>
__global__ void __launch_bounds__(192)
gmm_bs_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmA1, const GmmParams p) {
    using namespace sm100;
    using L = GmmSmem<BN_MAX, TERMS, STACK, KC, MX4>;
    constexpr int STAGES_MAX = L::kStages;
    const int STAGES = p.stages;
    constexpr int SF_COLS = L::kSfCols;
    constexpr int SF_BASE = L::kSfBase;
    constexpr int SF_UNIT = 2 * L::kAccCols;  // stacked mode: atom of unit activation scales
    constexpr int ACT_OFF = KC * L::kABytes, SFA_OFF = ACT_OFF + KC * L::kActBytes;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * L::kStage);  // barriers follow the stages in use
    uint64_t* empty = full + STAGES_MAX;
    uint64_t* acc_full = empty + STAGES_MAX;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmA1);
    }
    uint32_t* unit_atom = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(full) + 512);  // 512 B of E8M0 1.0
    if (STACK) {
        if (threadIdx.x < 128) unit_atom[threadIdx.x] = 0x7f7f7f7fu;
        fence_proxy_async();
    }
    const uint32_t tmem_cols = (uint32_t)p.tmem_cols;
    if (warp == 2) tmem_alloc(tmem_slot, tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();  // everything above touched only this CTA's shared memory and TMEM
    const int n_items = *p.n_tiles * p.m_tiles;
    constexpr size_t act_stride = L::kActBytes;

    if (warp == 0) {
        // Producer.  The warp stays converged so that copy operands live on the uniform
        // datapath; all lanes poll the barrier, one elected lane arms it and issues the
        // stage's three copies.  Stage index, phase and global addresses are carried
        // incrementally: every extra instruction in this loop costs ~10 cycles per stage.
        int s = 0, ph = 0;
#ifdef NEON_MOE_INSTRUMENT
        int tr = 0;
#endif
        // the next item's tile record is fetched one item ahead, off the critical path
        int next_e = 0, next_rows = 0;
        if ((int)blockIdx.x < n_items) {
            next_e = p.tile_expert[blockIdx.x / p.m_tiles];
            next_rows = p.tile_rows[blockIdx.x / p.m_tiles];
        }
        for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
            const int tile = item / p.m_tiles, m = item - tile * p.m_tiles;
            const int e = next_e, rows = next_rows;
            if (item + (int)gridDim.x < n_items) {
                const int nt = (item + (int)gridDim.x) / p.m_tiles;
                next_e = p.tile_expert[nt];
                next_rows = p.tile_rows[nt];
            }
            const uint32_t act_bytes = MX4 ? (STACK ? TERMS * ((rows + 7) >> 3) * 512 : 512 + ((rows + 7) >> 3) * 512)
                                           : STACK ? TERMS * ((rows + 7) >> 3) * 1024
                                                   : act_header_bytes(TERMS) + ((rows + 7) >> 3) * TERMS * 1024;
            const uint32_t box = (uint32_t)((e * p.m_tiles + m) * p.n_chunks);
            int box_row = (int)(box * 128);
            const uint8_t* sfa_src = p.sfa + (size_t)box * 512;
            const uint8_t* act_src = p.act + (size_t)tile * p.n_chunks * act_stride;
            const uint32_t tx_full = KC * (p.a_tx_bytes + 512) + (KC - 1) * (uint32_t)act_stride + act_bytes;
            for (int left = p.n_chunks; left > 0; left -= KC) {
                const bool whole = left >= KC;
                int ok = mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 1, kWaitLimitCycles);
                if (!__all_sync(0xffffffffu, ok)) goto done;
#ifdef NEON_MOE_INSTRUMENT
                if (p.trace && blockIdx.x == 0 && lane == 0 && tr < 512) p.trace[(0 * 512 + tr) * 2] = clock64();
#endif
                uint8_t* st = smem + s * L::kStage;
                if (elect_one()) {
                    if (whole) {
                        mbar_expect_tx(&full[s], tx_full);
                        tma_load_2d(st, &tmA, &full[s], 0, box_row);
                        bulk_load(st + SFA_OFF, sfa_src, KC * 512, &full[s]);
                        bulk_load(st + ACT_OFF, act_src, (KC - 1) * (uint32_t)act_stride + act_bytes, &full[s]);
                    } else {  // the odd last chunk of the item (KC == 2 only)
                        mbar_expect_tx(&full[s], p.a_tx_bytes + 512 + act_bytes);
                        tma_load_2d(st, &tmA1, &full[s], 0, box_row);
                        bulk_load(st + SFA_OFF, sfa_src, 512, &full[s]);
                        bulk_load(st + ACT_OFF, act_src, act_bytes, &full[s]);
                    }
                }
                __syncwarp();
#ifdef NEON_MOE_INSTRUMENT
                if (p.trace && blockIdx.x == 0 && lane == 0 && tr < 512) p.trace[(0 * 512 + tr) * 2 + 1] = clock64();
                ++tr;
#endif
                box_row += KC * 128;
                sfa_src += KC * 512;
                act_src += KC * act_stride;
                if (++s == STAGES) { s = 0; ph ^= 1; }
            }
        }
        // Tail: the MMA warps release a stage with an asynchronous arrive (tcgen05.commit) that
        // may land after the accumulator-ready arrive the epilogue waits for.  Wait until every
        // stage has been released, or a late arrive could hit shared memory that already
        // belongs to the next CTA on this SM.
        for (int i = 0; i < STAGES; ++i) {
            int ok = mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 6, kWaitLimitCycles);
            if (!__all_sync(0xffffffffu, ok)) goto done;
            if (++s == STAGES) { s = 0; ph ^= 1; }
        }
    } else if (warp == 1) {
        // MMA issuer.  Same shape as the producer: converged warp, all lanes poll, one elected
        // lane issues the tcgen05 instructions.
        {
            int s = 0, ph = 0, iter = 0;
#ifdef NEON_MOE_INSTRUMENT
            int ctr = 0;
#endif
            bool ready = false;  // the current stage's barrier was already seen complete
            const uint32_t smem_base = smem_u32(smem);
            if (STACK) {
                if (elect_one()) {  // rows 0..127 and 128..255 of the N operand
                    tc_copy_sf(tmem_base + SF_UNIT, make_sf_desc(smem_u32(unit_atom)));
                    tc_copy_sf(tmem_base + SF_UNIT + 4, make_sf_desc(smem_u32(unit_atom)));
                }
                __syncwarp();
            }
            int next_rows = (int)blockIdx.x < n_items ? p.tile_rows[blockIdx.x / p.m_tiles] : 0;
            for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++iter) {
                const int rows = next_rows;  // fetched one item ahead
                if (item + (int)gridDim.x < n_items) next_rows = p.tile_rows[(item + (int)gridDim.x) / p.m_tiles];
                const int npad = (rows + 7) & ~7;
                const uint32_t n_mma = STACK ? (uint32_t)(TERMS * npad) : (uint32_t)max(16, round_up_int(rows, 16));
                const uint32_t idesc0 = MX4 ? make_idesc_bs(1, 1, n_mma, 0, 0) : make_idesc_bs(5, 0, n_mma, 0, 0);
                constexpr uint32_t kIdescStep = (1u << 4) | (1u << 29);  // next scale id for A and B
                const int b = iter & 1, aph = (iter >> 1) & 1;
                int ok = mbar_wait(&acc_empty[b], aph ^ 1, abort_flag, p.status, 2, kWaitLimitCycles);
                if (!__all_sync(0xffffffffu, ok)) goto done;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + b * L::kAccCols;
                uint32_t first = 0;  // becomes non-zero after the item's first stage
                for (int left = p.n_chunks; left > 0; left -= KC) {
#ifdef NEON_MOE_INSTRUMENT
                    const bool tracing = p.trace && blockIdx.x == 0 && lane == 0 && ctr < 512;
                    if (tracing) p.trace[(1 * 512 + ctr) * 2] = clock64();  // about to wait for the stage's data
#endif
                    if (!ready) {
                        ok = mbar_wait(&full[s], ph, abort_flag, p.status, 3, kWaitLimitCycles);
                        if (!__all_sync(0xffffffffu, ok)) goto done;
                    }
#ifdef NEON_MOE_INSTRUMENT
                    if (tracing) p.trace[(1 * 512 + ctr) * 2 + 1] = clock64();  // data present
                    ++ctr;
#endif
                    tc_fence_after();
                    const uint32_t st = smem_base + s * L::kStage;
                    const uint32_t sf_stage = tmem_base + SF_BASE + s * SF_COLS;
                    // issues the copy of chunk k's weight scales and its MMAs (elected lane only)
                    auto issue_chunk = [&](int k) {
                        const uint32_t sf_tmem = sf_stage + k * (SF_COLS / KC);
                        const uint32_t act_smem = st + ACT_OFF + k * L::kActBytes;
                        tc_copy_sf(sf_tmem, make_sf_desc(st + SFA_OFF + k * 512));
                        if (MX4 && !STACK) {
                            // packed e2m1 x e2m1 with the activations' own block scales: K = 64 per instruction,
                            // two scales per row and instruction for both operands (scale ids 0 and 2)
                            tc_copy_sf(sf_tmem + 4, make_sf_desc(act_smem));
                            const uint64_t a4 = make_sw64_desc(st + k * L::kABytes), b4 = make_sw64_desc(act_smem + 512);
#pragma unroll
                            for (int j = 0; j < 2; ++j)
                                mma_mxf4(d_tmem, a4 + 2 * j, b4 + 2 * j, idesc0 + j * ((2u << 29) | (2u << 4)), sf_tmem, sf_tmem + 4,
                                         first | (uint32_t)(k | j));
                            return;
                        }
                        if (MX4) {
                            // packed e2m1 x e2m1, K = 64 per instruction, two weight scales each
                            // (scale ids 0 and 2); activation scales are the unit atom
                            const uint64_t a4 = make_sw64_desc(st + k * L::kABytes), b4 = make_sw64_desc(act_smem);
#pragma unroll
                            for (int j = 0; j < 2; ++j)
                                mma_mxf4(d_tmem, a4 + 2 * j, b4 + 2 * j, idesc0 + j * (2u << 29), sf_tmem, tmem_base + SF_UNIT,
                                         first | (uint32_t)(k | j));
                            return;
                        }
                        const uint64_t a_desc = make_sw128_desc(st + k * L::kABytes);
                        if (STACK) {
                            // activation scales are all 1.0 (scale id 0 of the unit atom); only A's id advances
                            const uint64_t b_desc = make_sw128_desc(act_smem);
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                mma_mxf8f6f4(d_tmem, a_desc + 2 * j, b_desc + 2 * j, idesc0 + j * (1u << 29), sf_tmem,
                                             tmem_base + SF_UNIT, first | (uint32_t)(k | j));
                        } else {
#pragma unroll
                            for (int t = 0; t < TERMS; ++t) tc_copy_sf(sf_tmem + 4 * (1 + t), make_sf_desc(act_smem + 512 * t));
#pragma unroll
                            for (int t = 0; t < TERMS; ++t) {
                                const uint64_t b_desc = make_sw128_desc(act_smem + act_header_bytes(TERMS) + t * 1024, TERMS * 1024);
#pragma unroll
                                for (int j = 0; j < 4; ++j)
                                    mma_mxf8f6f4(d_tmem, a_desc + 2 * j, b_desc + 2 * j, idesc0 + j * kIdescStep, sf_tmem,
                                                 sf_tmem + 4 * (1 + t), first | (uint32_t)(k | t | j));
                            }
                        }
                    };
                    if (elect_one()) issue_chunk(0);
                    __syncwarp();
                    // While those MMAs run, look whether the next stage has landed: the barrier
                    // round trip then overlaps tensor-pipe work instead of leaving the pipe idle.
                    {
                        const int sn = (s + 1 == STAGES) ? 0 : s + 1;
                        const int phn = (s + 1 == STAGES) ? ph ^ 1 : ph;
                        ready = __all_sync(0xffffffffu, (int)mbar_peek(&full[sn], phn));
                    }
                    if (elect_one()) {
                        if (KC == 2 && left > 1) issue_chunk(1);
                        tc_commit(&empty[s]);
                    }
                    __syncwarp();
                    first = 1;
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
                if (elect_one()) tc_commit(&acc_full[b]);
                __syncwarp();
            }
        }
    } else {
        const int q = warp & 3;
        int iter = 0;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++iter) {
            const int tile = item / p.m_tiles, m = item % p.m_tiles;
            const int e = p.tile_expert[tile], row0 = p.tile_row0[tile], rows = p.tile_rows[tile];
            const int b = iter & 1, aph = (iter >> 1) & 1;
            const int npad = (rows + 7) & ~7;
            // GATE_UP: lanes 0..15 hold gate rows of channels ch, lanes 16..31 their linear rows
            const int ch = 64 * m + 16 * q + (lane & 15);
            const int row = 128 * m + 32 * q + lane;
            const bool valid = GATE_UP ? true : row < p.rows_total;
            float bias = 0.f;
            if (GATE_UP) bias = bf16_bits_to_float(p.bias[(size_t)e * p.rows_total + 2 * ch + (lane >> 4)]);
            else if (valid) bias = bf16_bits_to_float(p.bias[(size_t)e * p.rows_total + row]);
            // Per-token factors are fetched once per item, one token per lane (32 at a time), and handed
            // round by shuffles: the store loop below then has no dependent global loads.
            constexpr int NW = (BN_MAX + 31) / 32;
            float tok_scale[NW], tok_w[NW];
            float* tok_dst[NW];  // down product: where each token's output row goes
#pragma unroll
            for (int k = 0; k < NW; ++k) {
                const int tix = 32 * k + lane;
                const bool in = tix < rows;
                tok_scale[k] = STACK ? (in ? (p.row_scale ? p.row_scale[row0 + tix] : p.row_scale_const) : 0.f) : 1.f;
                tok_w[k] = 0.f;
                tok_dst[k] = nullptr;
                if (!GATE_UP && in) {
                    const int ent = p.perm[row0 + tix];
                    tok_w[k] = p.route_w[ent];
                    tok_dst[k] = p.peer.n_ranks ? peer_row(p.peer, ent, p.hidden) : p.y + (size_t)(row0 + tix) * p.hidden;
                }
            }
            // everything above is independent of the accumulator and was fetched before the wait for it: the dependent
            // global loads no longer sit between "accumulator ready" and "buffer returned"
            if (!mbar_wait(&acc_full[b], aph, abort_flag, p.status, 4, kWaitLimitCycles)) goto done;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + b * L::kAccCols;
            // one token's value of this lane's row: bias, then SwiGLU (gate_up) or the routing weight (down)
            auto finish = [&](int tix, float acc, float w_tok, float* dst) {
                const int pos = row0 + tix;
                const float mine = acc + bias;
                if (GATE_UP) {
                    const float lin = __shfl_down_sync(0xffffffffu, mine, 16);
                    if (lane < 16 && tix < rows) {
                        const float g = fminf(mine, p.limit);
                        const float l = fminf(fmaxf(lin, -p.limit), p.limit);
                        p.a_out[(size_t)pos * p.inter + ch] = g / (1.f + expf(-p.alpha * g)) * (l + 1.f);
                    }
                } else if (valid && tix < rows) {
                    dst[row] = w_tok * mine;
                }
            };
            if (BN_MAX <= 32) {
                // decode tiles: pull the whole accumulator row into registers, hand the TMEM buffer back
                // to the MMA warp at once, and only then do the arithmetic and the global stores
                float vals[BN_MAX];
#pragma unroll
                for (int j8 = 0; j8 < BN_MAX; j8 += 8) {
                    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                    if (j8 < npad) {
                        tmem_ld8(taddr + j8, v);
                        if (STACK) {  // add the other terms' columns (term t carries 16^-t)
                            float f = 1.f;
#pragma unroll
                            for (int t = 1; t < TERMS; ++t) {
                                f *= MX4 ? (1.f / 6.f) : 0.0625f;
                                float u[8];
                                tmem_ld8(taddr + t * npad + j8, u);
#pragma unroll
                                for (int i = 0; i < 8; ++i) v[i] = fmaf(u[i], f, v[i]);
                            }
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) vals[j8 + i] = v[i];
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[b]);
#pragma unroll
                for (int j = 0; j < BN_MAX; ++j) {
                    if (j < npad) {  // uniform over the warp
                        const float sc = STACK ? __shfl_sync(0xffffffffu, tok_scale[0], j) : 1.f;
                        const float wt = GATE_UP ? 0.f : __shfl_sync(0xffffffffu, tok_w[0], j);
                        float* dst = GATE_UP ? nullptr : reinterpret_cast<float*>(__shfl_sync(0xffffffffu, (unsigned long long)tok_dst[0], j));
                        finish(j, STACK ? vals[j] * sc : vals[j], wt, dst);
                    }
                }
                continue;
            }
#pragma unroll
            for (int k = 0; k < NW; ++k) {
                const int jend = min(npad, 32 * (k + 1));
                for (int j8 = 32 * k; j8 < jend; j8 += 8) {
                    float v[8];
                    tmem_ld8(taddr + j8, v);
                    if (STACK) {
                        float f = 1.f;
#pragma unroll
                        for (int t = 1; t < TERMS; ++t) {
                            f *= MX4 ? (1.f / 6.f) : 0.0625f;
                            float u[8];
                            tmem_ld8(taddr + t * npad + j8, u);
#pragma unroll
                            for (int i = 0; i < 8; ++i) v[i] = fmaf(u[i], f, v[i]);
                        }
                    }
                    if (GATE_UP && !STACK) {
                        // two tokens per step: lanes 0..15 (gate rows) finish token j, lanes 16..31 (linear rows) token j + 1,
                        // each half getting the other half's row of its token by one exchange - all 32 lanes do SwiGLU work
#pragma unroll
                        for (int i = 0; i < 8; i += 2) {
                            const float m0 = v[i] + bias, m1 = v[i + 1] + bias;
                            const float got = __shfl_xor_sync(0xffffffffu, lane < 16 ? m1 : m0, 16);
                            const float gate = lane < 16 ? m0 : got, lin = lane < 16 ? got : m1;
                            const int tix = j8 + i + (lane >> 4);
                            if (tix < rows) {
                                const float g = fminf(gate, p.limit);
                                const float l = fminf(fmaxf(lin, -p.limit), p.limit);
                                p.a_out[(size_t)(row0 + tix) * p.inter + ch] = __fdividef(g, 1.f + __expf(-p.alpha * g)) * (l + 1.f);
                            }
                        }
                        continue;
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int tix = j8 + i, pos = row0 + tix;
                        const float sc = STACK ? __shfl_sync(0xffffffffu, tok_scale[k], tix & 31) : 1.f;
                        const float mine = (STACK ? v[i] * sc : v[i]) + bias;
                        if (GATE_UP) {
                            const float lin = __shfl_down_sync(0xffffffffu, mine, 16);
                            if (lane < 16 && tix < rows) {
                                const float g = fminf(mine, p.limit);
                                const float l = fminf(fmaxf(lin, -p.limit), p.limit);
                                p.a_out[(size_t)pos * p.inter + ch] = g / (1.f + expf(-p.alpha * g)) * (l + 1.f);
                            }
                        } else {
                            const float wt = __shfl_sync(0xffffffffu, tok_w[k], tix & 31);
                            float* dst = reinterpret_cast<float*>(__shfl_sync(0xffffffffu, (unsigned long long)tok_dst[k], tix & 31));
                            if (valid && tix < rows) dst[row] = wt * mine;
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[b]);
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
        // leave time for copies that were already issued to land before the CTA retires
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000ll) {}
    }
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc(tmem_base, tmem_cols);
    }
}

}  // namespace neon
