// Kernels of the gpt-oss-shaped decoder around the MoE layer (decode step, small batch):
// embedding gather, RMSNorm, bf16 GEMV for the attention projections and the unembedding,
// YaRN rotary embedding + KV-cache append, grouped-query attention over the cache with
// per-head sink logits and an optional sliding window, residual adds, argmax.
// All of them are HBM/L2 streaming work on CUDA cores; activations between them are fp32
// (residual stream, q, attention partials) or bf16 (normalised activations, K/V cache).
// Every kernel may be launched with programmatic stream serialization: it lets its successor
// start launching at once (pdl_launch_dependents) and waits for its predecessor's results
// (pdl_wait) before touching anything a predecessor writes; only loads of weights, which no
// kernel writes, are issued ahead of the wait.
#pragma once
#include "moe_common.cuh"

namespace neon {

constexpr int kDecMaxBatch = 8;

__device__ __forceinline__ uint16_t f32_to_bf16_rn(float f) { return __bfloat16_as_ushort(__float2bfloat16_rn(f)); }

// x[b, :] = embed[token[b], :] (bf16 -> fp32 residual stream).
// Token ids outside [0, vocab) are clamped into range rather than read out of bounds.
__global__ void embed_kernel(const uint16_t* __restrict__ embed, const int32_t* __restrict__ tokens, int H, int vocab,
                             float* __restrict__ x) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;
    const uint16_t* row = embed + (size_t)min(max(tokens[b], 0), vocab - 1) * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) x[(size_t)b * H + i] = bf16_bits_to_float(row[i]);
}

// x[b, :] += sum_i addend[i * add_stride + b * H + :] for i < n_add (x is written back when
// n_add > 0; the addends are added in order), then
// y[b, :] = bf16( x[b, :] * rsqrt(mean(x^2) + eps) * w[:] ).  One CTA of 1024 threads per token;
// a thread keeps its (at most one) 4-element vector in registers between the two phases, so the
// row is read once.  H % 4 == 0, H <= 4096.  The sum of squares is reduced in a fixed order.
__global__ void __launch_bounds__(1024) rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ addend, int n_add,
                                                       long long add_stride, const uint16_t* __restrict__ w, int H, float eps,
                                                       uint16_t* __restrict__ y) {
    __shared__ float part[32];
    const int b = blockIdx.x, tid = threadIdx.x;
    const bool have = tid * 4 < H;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    uint2 wv = make_uint2(0u, 0u);
    pdl_launch_dependents();
    if (have) wv = *reinterpret_cast<const uint2*>(w + tid * 4);
    pdl_wait();
    if (have) {
        float4* xr = reinterpret_cast<float4*>(x + (size_t)b * H) + tid;
        v = *xr;
        if (n_add > 0) {
            float4 a[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
                a[i] = i < n_add ? reinterpret_cast<const float4*>(addend + (size_t)i * add_stride + (size_t)b * H)[tid]
                                 : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int i = 0; i < 4; ++i) { v.x += a[i].x; v.y += a[i].y; v.z += a[i].z; v.w += a[i].w; }
            *xr = v;
        }
    }
    float s = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((tid & 31) == 0) part[tid >> 5] = s;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) tot += part[i];
    const float r = rsqrtf(tot / (float)H + eps);
    if (have) {
        const uint32_t lo = (uint32_t)f32_to_bf16_rn(v.x * r * __uint_as_float(wv.x << 16)) |
                            ((uint32_t)f32_to_bf16_rn(v.y * r * __uint_as_float(wv.x & 0xffff0000u)) << 16);
        const uint32_t hi = (uint32_t)f32_to_bf16_rn(v.z * r * __uint_as_float(wv.y << 16)) |
                            ((uint32_t)f32_to_bf16_rn(v.w * r * __uint_as_float(wv.y & 0xffff0000u)) << 16);
        *reinterpret_cast<uint2*>(y + (size_t)b * H + tid * 4) = make_uint2(lo, hi);
    }
}

// Padding (in bf16 elements) that makes a K-element activation row start 16 banks after the
// previous one, so that the eight rows a quarter-warp reads together never share a bank.
__host__ __device__ inline int gemv_row_pad(int K) { return ((16 - (K / 2) % 32 + 32) % 32) * 2; }

// out[b, r] (+)= sum_k W[r, k] * x[b, k] + bias[r] for b < B <= 8: a skinny GEMM whose N is the
// batch, on mma.sync m16n8k16 (bf16 in, fp32 accumulate).  W bf16 [rows, K] row-major is
// streamed from HBM exactly once; x bf16 [B, K] is staged in shared memory (missing batch rows
// are zero).  A CTA owns 16-row tiles; its 8 warps split K in interleaved 32-element blocks
// (together they read 512 contiguous bytes of each row) and their accumulators are summed
// through shared memory.  The sum over k does not depend on which mma slot a k lands in, so
// each thread feeds the 8 consecutive elements of one 16-byte load to two mma's and reads the
// matching 16 bytes of x: no shuffles, no scalar loads.  K % 32 == 0.
// accumulate != 0: out += result (residual add); otherwise out = result.
__global__ void __launch_bounds__(256, 2) gemv_mma_kernel(const uint16_t* __restrict__ W, const uint16_t* __restrict__ bias,
                                                          const uint16_t* __restrict__ x, int B, int rows, int K,
                                                          int accumulate, float* __restrict__ out) {
    extern __shared__ __align__(16) unsigned char gsm[];
    constexpr int U = 6;  // k-blocks per warp and batch; two batches are in flight
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int xstride = K + gemv_row_pad(K);  // elements
    uint16_t* xs = reinterpret_cast<uint16_t*>(gsm);
    float* red = reinterpret_cast<float*>(gsm + (size_t)8 * xstride * 2);  // [8 warps][128]
    const int nkb = K / 32, n_tiles = (rows + 15) / 16;

    auto load_batch = [&](uint4 (&wa)[U], uint4 (&wb)[U], const uint16_t* ra, const uint16_t* rb, int kb0) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int kb = kb0 + u * 8;
            if (kb < nkb) {
                wa[u] = ldg_stream(reinterpret_cast<const uint4*>(ra + kb * 32 + t * 8));
                wb[u] = ldg_stream(reinterpret_cast<const uint4*>(rb + kb * 32 + t * 8));
            } else {
                wa[u] = wb[u] = make_uint4(0, 0, 0, 0);
            }
        }
    };
    int tile = blockIdx.x;
    uint4 wa[U], wb[U];
    const uint16_t *ra = nullptr, *rb = nullptr;
    pdl_launch_dependents();
    if (tile < n_tiles) {  // first weights go in flight before the predecessor has even finished
        ra = W + (size_t)min(tile * 16 + g, rows - 1) * K;
        rb = W + (size_t)min(tile * 16 + g + 8, rows - 1) * K;
        load_batch(wa, wb, ra, rb, warp);
    }
    pdl_wait();
    {   // stage x: eight independent 16-byte loads per thread in flight, then the stores
        const int nvec = K / 8, total = 8 * nvec;
        for (int base = tid; base < total; base += 256 * 8) {
            uint4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = base + u * 256;
                v[u] = (i < total && i / nvec < B) ? reinterpret_cast<const uint4*>(x)[i] : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = base + u * 256;
                if (i < total) *reinterpret_cast<uint4*>(xs + (size_t)(i / nvec) * xstride + (i % nvec) * 8) = v[u];
            }
        }
    }
    __syncthreads();
    for (; tile < n_tiles; tile += gridDim.x) {
        float c[4] = {0.f, 0.f, 0.f, 0.f};
        for (int kb0 = warp; kb0 < nkb; kb0 += 8 * U) {
            uint4 na[U], nb[U];
            const int next = kb0 + 8 * U;
            if (next < nkb) load_batch(na, nb, ra, rb, next);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int kb = kb0 + u * 8;
                if (kb < nkb) {
                    const uint4 xv = *reinterpret_cast<const uint4*>(xs + (size_t)g * xstride + kb * 32 + t * 8);
                    const uint32_t a0[4] = {wa[u].x, wb[u].x, wa[u].y, wb[u].y};
                    const uint32_t a1[4] = {wa[u].z, wb[u].z, wa[u].w, wb[u].w};
                    mma_bf16_16816(c, a0, xv.x, xv.y);
                    mma_bf16_16816(c, a1, xv.z, xv.w);
                }
            }
            if (next < nkb) {
#pragma unroll
                for (int u = 0; u < U; ++u) { wa[u] = na[u]; wb[u] = nb[u]; }
            }
        }
        // next tile's first weights go in flight before the reduction
        const int this_tile = tile, nt = tile + gridDim.x;
        if (nt < n_tiles) {
            ra = W + (size_t)min(nt * 16 + g, rows - 1) * K;
            rb = W + (size_t)min(nt * 16 + g + 8, rows - 1) * K;
            load_batch(wa, wb, ra, rb, warp);
        }
        *reinterpret_cast<float4*>(red + warp * 128 + lane * 4) = make_float4(c[0], c[1], c[2], c[3]);
        __syncthreads();
        if (tid < 128) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) v += red[w * 128 + tid];
            const int l = tid >> 2, j = tid & 3;
            const int row = this_tile * 16 + (l >> 2) + (j >= 2 ? 8 : 0), n = (l & 3) * 2 + (j & 1);
            if (row < rows && n < B) {
                v += bias ? bf16_bits_to_float(bias[row]) : 0.f;
                float* dst = out + (size_t)n * rows + row;
                *dst = accumulate ? *dst + v : v;
            }
        }
        __syncthreads();
    }
}

constexpr int kGemvSplitU = 6;  // k-blocks per warp of gemv_mma_split_kernel (all loaded at once)

// The same product for matrices with few rows, cut along K over gridDim.y CTAs per 16-row tile
// so that enough CTAs exist to keep HBM busy: CTA (tile, ks) handles k-blocks
// [ks * nkb / KS, (ks + 1) * nkb / KS) (nkb = K / 32, at most 8 * kGemvSplitU of them), loads all
// of its weights up front (before it waits for its predecessor), reads the matching pieces of x
// straight from L2 into the mma B fragments, and writes the partial result parts[ks][b][r]; part
// 0 carries the bias.  The consumer adds
// the parts in order, which keeps the result independent of scheduling.
__global__ void __launch_bounds__(256, 3) gemv_mma_split_kernel(const uint16_t* __restrict__ W, const uint16_t* __restrict__ bias,
                                                                const uint16_t* __restrict__ x, int B, int rows, int K,
                                                                float* __restrict__ parts, long long part_stride) {
    __shared__ __align__(16) float red[8 * 128];  // [8 warps][128] accumulator fragments
    constexpr int U = kGemvSplitU;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int nkb = K / 32, KS = gridDim.y, ks = blockIdx.y, tile = blockIdx.x;
    const int kb_lo = ks * nkb / KS, kb_hi = (ks + 1) * nkb / KS;
    pdl_launch_dependents();
    const uint16_t* ra = W + (size_t)min(tile * 16 + g, rows - 1) * K;
    const uint16_t* rb = W + (size_t)min(tile * 16 + g + 8, rows - 1) * K;
    uint4 wa[U], wb[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int kb = kb_lo + warp + u * 8;
        if (kb < kb_hi) {
            wa[u] = ldg_stream(reinterpret_cast<const uint4*>(ra + kb * 32 + t * 8));
            wb[u] = ldg_stream(reinterpret_cast<const uint4*>(rb + kb * 32 + t * 8));
        } else {
            wa[u] = wb[u] = make_uint4(0, 0, 0, 0);
        }
    }
    pdl_wait();
    // the matching 16 bytes of x straight from L2 (row g = token g; rows past the batch are zero):
    // no shared-memory staging, no barrier before the mma's
    uint4 xv[U];
    const uint16_t* xr = x + (size_t)min(g, B - 1) * K;
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int kb = kb_lo + warp + u * 8;
        xv[u] = (kb < kb_hi && g < B) ? __ldcg(reinterpret_cast<const uint4*>(xr + kb * 32 + t * 8)) : make_uint4(0, 0, 0, 0);
    }
    float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const uint32_t a0[4] = {wa[u].x, wb[u].x, wa[u].y, wb[u].y};
        const uint32_t a1[4] = {wa[u].z, wb[u].z, wa[u].w, wb[u].w};
        mma_bf16_16816(c, a0, xv[u].x, xv[u].y);
        mma_bf16_16816(c, a1, xv[u].z, xv[u].w);
    }
    *reinterpret_cast<float4*>(red + warp * 128 + lane * 4) = make_float4(c[0], c[1], c[2], c[3]);
    __syncthreads();
    if (tid < 128) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) v += red[w * 128 + tid];
        const int l = tid >> 2, j = tid & 3;
        const int row = tile * 16 + (l >> 2) + (j >= 2 ? 8 : 0), n = (l & 3) * 2 + (j & 1);
        if (row < rows && n < B) {
            if (ks == 0 && bias) v += bf16_bits_to_float(bias[row]);
            parts[(size_t)ks * part_stride + (size_t)n * rows + row] = v;
        }
    }
}

// K/V cache of one layer, bf16.  Keys:   kcache[((b * nkv + h) * ctx + p) * 64 + d]  (positions of
// a head contiguous, one 128-byte row each).  Values are kept TRANSPOSED: vcache[((b * nkv + h) * 64
// + d) * ctx + p], so that eight consecutive positions of one dimension are one 16-byte load, which
// is what the tensor-core P.V product wants as its B operand.  ctx % 8 == 0.

// YaRN rotary embedding on q and k (rotate-half pairing: element i pairs with i + D/2) and
// append of k, v to the cache.  qkv fp32 [B, (nq + 2*nkv) * D]; cos/sin are computed from
// inv_freq[D/2] (fp32) and the token position; `mscale` multiplies cos and sin.  q is rotated
// in place; k (rotated) and v are written as bf16 at the token's cache position.
// qkv arrives as n_parts partial results of the K-split projection (part i at qkv + i *
// part_stride), which are added in order first; the rotated q lands in part 0.
// One CTA per (head or value head, sequence).
__global__ void __launch_bounds__(64) rope_cache_kernel(float* __restrict__ qkv, int n_parts, long long part_stride,
                                                        const float* __restrict__ inv_freq, const int32_t* __restrict__ pos,
                                                        int nq, int nkv, float mscale, int ctx, uint16_t* __restrict__ kcache,
                                                        uint16_t* __restrict__ vcache) {
    constexpr int D = 64, half = 32;
    const int head = blockIdx.x, b = blockIdx.y, j = threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    const int p = min(max(pos[b], 0), ctx - 1);  // positions outside the cache are clamped, never written out of bounds
    float* hrow = qkv + ((size_t)b * (nq + 2 * nkv) + head) * D;
    float mine = hrow[j];  // element j of the head, parts summed
    for (int i = 1; i < n_parts; ++i) mine += hrow[(size_t)i * part_stride + j];
    if (head >= nq + nkv) {  // value head: one element per dimension row of the transposed cache
        vcache[(((size_t)b * nkv + (head - nq - nkv)) * D + j) * ctx + p] = f32_to_bf16_rn(mine);
        return;
    }
    __shared__ float hv[D];  // the head's 64 summed elements (the branch above is uniform over the CTA)
    hv[j] = mine;
    __syncthreads();
    if (j >= half) return;
    float sn, cs;
    sincosf((float)p * inv_freq[j], &sn, &cs);
    sn *= mscale;
    cs *= mscale;
    const float a = hv[j], bb = hv[j + half];
    const float r0 = a * cs - bb * sn, r1 = bb * cs + a * sn;
    if (head < nq) {
        hrow[j] = r0;
        hrow[j + half] = r1;
    } else {
        uint16_t* dst = kcache + (((size_t)b * nkv + (head - nq)) * ctx + p) * D;
        dst[j] = f32_to_bf16_rn(r0);
        dst[j + half] = f32_to_bf16_rn(r1);
    }
}

// Key cache [batch][nkv][ctx][64] <- src [batch][n_pos][nkv][64] for positions < n_pos (16-byte vectors).
__global__ void k_load_kernel(const uint4* __restrict__ src, int batch, int n_pos, int nkv, int ctx, uint4* __restrict__ dst) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // over batch * n_pos * nkv * 8
    if (i >= (size_t)batch * n_pos * nkv * 8) return;
    const int v = (int)(i % 8), h = (int)((i / 8) % nkv);
    const size_t bp = i / 8 / nkv;
    const int p = (int)(bp % n_pos), b = (int)(bp / n_pos);
    dst[(((size_t)b * nkv + h) * ctx + p) * 8 + v] = src[i];
}

// Value cache [batch][nkv][64][ctx] <- src [batch][n_pos][nkv][64]: one thread per element,
// consecutive threads write consecutive positions.
__global__ void v_load_kernel(const uint16_t* __restrict__ src, int batch, int n_pos, int nkv, int ctx, uint16_t* __restrict__ dst) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // over batch * nkv * 64 * n_pos
    if (i >= (size_t)batch * nkv * 64 * n_pos) return;
    const int p = (int)(i % n_pos), d = (int)((i / n_pos) % 64);
    const size_t bh = i / n_pos / 64;
    const int h = (int)(bh % nkv), b = (int)(bh / nkv);
    dst[(((size_t)b * nkv + h) * 64 + d) * ctx + p] = src[(((size_t)b * n_pos + p) * nkv + h) * 64 + d];
}

constexpr int kAttnChunk = 256;  // cache positions per CTA of attn_partial_kernel

// fp32 pair -> bf16x2 "high" word and the bf16x2 of what is left (x ~= hi + lo to ~2^-17).
__device__ __forceinline__ void split_bf16x2(float x0, float x1, uint32_t& hi, uint32_t& lo) {
    const uint16_t h0 = f32_to_bf16_rn(x0), h1 = f32_to_bf16_rn(x1);
    hi = (uint32_t)h0 | ((uint32_t)h1 << 16);
    lo = (uint32_t)f32_to_bf16_rn(x0 - bf16_bits_to_float(h0)) | ((uint32_t)f32_to_bf16_rn(x1 - bf16_bits_to_float(h1)) << 16);
}

// Grouped-query attention of one new token per sequence over its cache, on mma.sync
// m16n8k16.  One CTA per (kv head, sequence, chunk of 256 positions); the G = nq/nkv <= 8
// query heads of the group are rows 0..G-1 of the 16-row tiles (the rest is zero), so every
// K/V byte is loaded once for all of them.  The range lo..p (lo = max(0, p - window + 1) when
// window > 0) is cut into chunks from lo rounded down to a multiple of 8; positions outside
// lo..p are masked.  Each CTA writes an unnormalised partial (chunk maximum m, sum l,
// accumulator) per head and attn_merge_kernel folds the chunks together with the head's sink
// logit, which enters the softmax denominator only.  Scores are q.k * scale.
// Warp w owns 32 positions.  Scores: four n-tiles of 8 positions, position = 4*n + tile, so
// that thread (g, t) ends up with the probabilities of positions 8t..8t+7 - exactly the k
// slots it feeds to the P.V mma's, whose B operand is one 16-byte load (8 positions of one
// dimension) from the transposed value cache.  The sums over dimensions / positions do not
// depend on the mma slot order, so each 16-byte load feeds two mma's.  q and the
// probabilities enter as hi + lo bf16 pairs (two mma's each), which keeps fp32-grade accuracy.
template <int G>
__global__ void __launch_bounds__(256, 3) attn_partial_kernel(const float* __restrict__ qkv, const uint16_t* __restrict__ kcache,
                                                              const uint16_t* __restrict__ vcache, const int32_t* __restrict__ pos,
                                                              int nq, int nkv, int ctx, int window, float scale, int splits,
                                                              float* __restrict__ part /* [B][nq][splits][66] */) {
    constexpr int D = 64;
    __shared__ float wm[8][8], wl[8][8];
    __shared__ __align__(16) float red[8][8][D];
    const int kvh = blockIdx.x, b = blockIdx.y, sp = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    pdl_launch_dependents();
    pdl_wait();
    const int p = min(max(pos[b], 0), ctx - 1);
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    const int s0 = (lo & ~7) + sp * kAttnChunk;
    float* dst = part + (((size_t)b * nq + kvh * G) * splits + sp) * (D + 2);
    if (s0 > p) {  // empty chunk (uniform over the CTA)
        for (int i = tid; i < G * (D + 2); i += 256) {
            const int gg = i / (D + 2), c = i % (D + 2);
            dst[(size_t)gg * splits * (D + 2) + c] = c == 0 ? -INFINITY : 0.f;
        }
        return;
    }
    const int wbase = s0 + warp * 32;  // first position of this warp (multiple of 8)
    const size_t head = (size_t)b * nkv + kvh;
    // keys: tile j, row n = g -> position wbase + 4g + j; two 16-byte halves of dims [8t, 8t+8) and [32+8t, ..)
    uint4 kr[4][2];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int kp = wbase + 4 * g + j;
        if (kp < ctx && wbase <= p) {
            const uint4* row = reinterpret_cast<const uint4*>(kcache + (head * ctx + kp) * D);
            kr[j][0] = __ldg(row + t);
            kr[j][1] = __ldg(row + 4 + t);
        } else {
            kr[j][0] = kr[j][1] = make_uint4(0, 0, 0, 0);
        }
    }
    // values: dimension tile dt, row n = g -> dimension 8*dt + g; positions wbase + 8t .. +7 in one load
    uint4 vr[8];
#pragma unroll
    for (int dt = 0; dt < 8; ++dt) {
        const int vp = wbase + 8 * t;
        vr[dt] = (vp < ctx && wbase <= p) ? __ldg(reinterpret_cast<const uint4*>(vcache + (head * D + dt * 8 + g) * ctx + vp))
                                          : make_uint4(0, 0, 0, 0);
    }
    // q of head g (rows >= G are zero), scaled, as hi/lo bf16 pairs in the same slot order as the key loads
    uint32_t qh[2][4], ql[2][4];
    {
        const float* qrow = qkv + (size_t)b * (nq + 2 * nkv) * D + (size_t)(kvh * G + min(g, G - 1)) * D;
        const float on = g < G ? scale : 0.f;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float4 u = *reinterpret_cast<const float4*>(qrow + i * 32 + t * 8);
            const float4 v = *reinterpret_cast<const float4*>(qrow + i * 32 + t * 8 + 4);
            split_bf16x2(u.x * on, u.y * on, qh[i][0], ql[i][0]);
            split_bf16x2(u.z * on, u.w * on, qh[i][1], ql[i][1]);
            split_bf16x2(v.x * on, v.y * on, qh[i][2], ql[i][2]);
            split_bf16x2(v.z * on, v.w * on, qh[i][3], ql[i][3]);
        }
    }
    // scores: c[j][0] = (head g, position 8t + j), c[j][1] = (head g, position 8t + 4 + j)
    float sc[4][2];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint32_t kw[4] = {kr[j][i].x, kr[j][i].y, kr[j][i].z, kr[j][i].w};
            const uint32_t ah0[4] = {qh[i][0], 0u, qh[i][1], 0u}, al0[4] = {ql[i][0], 0u, ql[i][1], 0u};
            const uint32_t ah1[4] = {qh[i][2], 0u, qh[i][3], 0u}, al1[4] = {ql[i][2], 0u, ql[i][3], 0u};
            mma_bf16_16816(c, ah0, kw[0], kw[1]);
            mma_bf16_16816(c, al0, kw[0], kw[1]);
            mma_bf16_16816(c, ah1, kw[2], kw[3]);
            mma_bf16_16816(c, al1, kw[2], kw[3]);
        }
        // C columns 2t, 2t+1 are rows n = 2t, 2t+1 of the tile: positions 4*(2t) + j and 4*(2t+1) + j
        const int p0 = wbase + 8 * t + j, p1 = p0 + 4;
        sc[j][0] = (p0 >= lo && p0 <= p) ? c[0] : -INFINITY;
        sc[j][1] = (p1 >= lo && p1 <= p) ? c[1] : -INFINITY;
    }
    // chunk maximum per head: over this thread's 8 positions, the 4 threads of a row, the 8 warps
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < 4; ++j) m = fmaxf(m, fmaxf(sc[j][0], sc[j][1]));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
    if (t == 0) wm[warp][g] = m;
    __syncthreads();
    m = wm[0][g];
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, wm[w][g]);
    // probabilities (0 where masked, and everywhere when the head saw no valid position)
    float pr[4][2], l = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        pr[j][0] = sc[j][0] == -INFINITY ? 0.f : __expf(sc[j][0] - m);
        pr[j][1] = sc[j][1] == -INFINITY ? 0.f : __expf(sc[j][1] - m);
        l += pr[j][0] + pr[j][1];
    }
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (t == 0) wl[warp][g] = l;
    // P as A operand: mma #0 covers positions 8t..8t+3 (a0 = +0,+1; a2 = +2,+3), mma #1 positions 8t+4..8t+7
    uint32_t ph[2][2], pl[2][2];
    split_bf16x2(pr[0][0], pr[1][0], ph[0][0], pl[0][0]);
    split_bf16x2(pr[2][0], pr[3][0], ph[0][1], pl[0][1]);
    split_bf16x2(pr[0][1], pr[1][1], ph[1][0], pl[1][0]);
    split_bf16x2(pr[2][1], pr[3][1], ph[1][1], pl[1][1]);
#pragma unroll
    for (int dt = 0; dt < 8; ++dt) {
        float c[4] = {0.f, 0.f, 0.f, 0.f};
        const uint32_t a0h[4] = {ph[0][0], 0u, ph[0][1], 0u}, a0l[4] = {pl[0][0], 0u, pl[0][1], 0u};
        const uint32_t a1h[4] = {ph[1][0], 0u, ph[1][1], 0u}, a1l[4] = {pl[1][0], 0u, pl[1][1], 0u};
        mma_bf16_16816(c, a0h, vr[dt].x, vr[dt].y);
        mma_bf16_16816(c, a0l, vr[dt].x, vr[dt].y);
        mma_bf16_16816(c, a1h, vr[dt].z, vr[dt].w);
        mma_bf16_16816(c, a1l, vr[dt].z, vr[dt].w);
        // c[0], c[1] = (head g, dimensions 8*dt + 2t, +1)
        *reinterpret_cast<float2*>(&red[warp][g][dt * 8 + 2 * t]) = make_float2(c[0], c[1]);
    }
    __syncthreads();
    for (int i = tid; i < G * D; i += 256) {
        const int gg = i / D, d = i % D;
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) acc += red[w][gg][d];
        float* o = dst + (size_t)gg * splits * (D + 2);
        o[2 + d] = acc;
        if (d == 0) {
            float ls = 0.f, mm = wm[0][gg];
#pragma unroll
            for (int w = 0; w < 8; ++w) { ls += wl[w][gg]; mm = fmaxf(mm, wm[w][gg]); }
            o[0] = mm;
            o[1] = ls;
        }
    }
}

// out[b, head*64 + d] = bf16( sum_splits acc*exp(m - M) / (sum_splits l*exp(m - M) + exp(sink - M)) ).
__global__ void attn_merge_kernel(const float* __restrict__ part, const uint16_t* __restrict__ sinks, int nq, int splits,
                                  uint16_t* __restrict__ out) {
    constexpr int D = 64;
    const int head = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    const float* src = part + ((size_t)b * nq + head) * splits * (D + 2);
    const float sink = bf16_bits_to_float(sinks[head]);
    float M = sink;
#pragma unroll 8
    for (int s = 0; s < splits; ++s) M = fmaxf(M, src[s * (D + 2)]);
    float den = __expf(sink - M), acc = 0.f;
#pragma unroll 8
    for (int s = 0; s < splits; ++s) {
        const float m = src[s * (D + 2)];
        const float c = m == -INFINITY ? 0.f : __expf(m - M);
        den += src[s * (D + 2) + 1] * c;
        acc += src[s * (D + 2) + 2 + d] * c;
    }
    out[((size_t)b * nq + head) * D + d] = f32_to_bf16_rn(acc / den);
}

// x += y (residual add of the MoE output), n elements.
__global__ void add_kernel(float* __restrict__ x, const float* __restrict__ y, int n) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += y[i];
}

// next[b] = argmax_v logits[b, v], lowest index among equals.
__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ logits, int V, int32_t* __restrict__ next) {
    __shared__ float sv[32];
    __shared__ int si[32];
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x, tid = threadIdx.x;
    const float* row = logits + (size_t)b * V;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = tid; i < V; i += 1024) {
        const float v = row[i];
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if ((tid & 31) == 0) { sv[tid >> 5] = best; si[tid >> 5] = bi; }
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < 32; ++w)
            if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
        next[b] = bi;
    }
}

}  // namespace neon
