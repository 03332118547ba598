// FLIP water step of the reference engine (NeonEngine/shaders/water_grid.comp, passes 0-8, in the
// dispatch order of NeonEngine/src/water_physics.cpp:164-430) as CUDA kernels behind the C ABI of
// include/neon_water.h.  This translation unit is compiled with -fmad=false: every kernel uses
// the shader's 32-bit float operations in the shader's order, so the results equal the CPU
// restatement bit for bit.  No CPU fallback exists.
//
// Redesign relative to the shader (results unchanged):
//  * pass 1 (all-pairs particle separation) runs one WARP per particle over shared-memory tiles
//    of positions: the 32 lanes test 32 neighbours at once and only the rare close ones are
//    applied one by one in ascending index, re-testing the later lanes with the moved position,
//    which is exactly the sequential loop's arithmetic at 32 neighbours per step;
//  * passes 2-4 (scatter with float compare-and-swap loops, then a normalising pass) become a
//    binned gather: count contributions per grid node (integer atomics), prefix-sum, fill,
//    then one thread per node sorts its few contributions by particle id and adds them in that
//    order - no float atomics, deterministic, and the normalisation (pass 3) happens in the same
//    kernel;
//  * one step is a CUDA graph.
#include "../../include/neon_water.h"

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>
#include <string>

namespace {

constexpr unsigned kFluid = 1u, kSolid = 2u;

struct WP {  // parameters every kernel takes by value
    int N, nx, ny, nz, C;
    float cs, orx, rd, damp, mass, dt;
    float bmin[3], bmax[3], g[3];
};

struct Stencil {
    int base[3];
    float frac[3];
};

__device__ __forceinline__ Stencil make_stencil(const WP& q, const float4& pos, float ox, float oy, float oz) {
    Stencil s;
    const float p[3] = {pos.x, pos.y, pos.z}, off[3] = {ox, oy, oz};
    const int dim[3] = {q.nx, q.ny, q.nz};
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        const float local = (p[a] - q.bmin[a]) / q.cs;
        const float l = local - off[a];
        s.base[a] = min(max((int)floorf(l), 0), dim[a] - 2);
        s.frac[a] = l - (float)s.base[a];
    }
    return s;
}

__device__ __forceinline__ float corner_weight(const Stencil& s, int ix, int iy, int iz) {
    return (ix == 0 ? (1.0f - s.frac[0]) : s.frac[0]) * (iy == 0 ? (1.0f - s.frac[1]) : s.frac[1]) *
           (iz == 0 ? (1.0f - s.frac[2]) : s.frac[2]);
}

__device__ __forceinline__ int corner_cell(const WP& q, const Stencil& s, int ix, int iy, int iz) {
    return (s.base[0] + ix) + (s.base[1] + iy) * q.nx + (s.base[2] + iz) * (q.nx * q.ny);
}

// staggering of grid g: 0 = u faces, 1 = v faces, 2 = w faces, 3 = cell centres (density)
__device__ __forceinline__ Stencil grid_stencil(const WP& q, const float4& pos, int g) {
    return make_stencil(q, pos, g == 0 ? 0.0f : 0.5f, g == 1 ? 0.0f : 0.5f, g == 2 ? 0.0f : 0.5f);
}

// ---- pass 0 (water_grid.comp:239-285) + reset of the gather's counters ------------------------
__global__ void k_grid_init(WP q, unsigned* flags, float* s, float* pa, float* pb, int* count, int* cursor, unsigned* bar) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx == 0) *bar = 0u;  // barrier counter of the fused Jacobi kernel
    if (idx >= q.C) return;
    const int gz = idx / (q.nx * q.ny), rem = idx - gz * (q.nx * q.ny), gy = rem / q.nx, gx = rem - gy * q.nx;
    const bool border = gx == 0 || gx == q.nx - 1 || gy == 0 || gy == q.ny - 1 || gz == 0 || gz == q.nz - 1;
    flags[idx] = border ? kSolid : 0u;
    s[idx] = border ? 0.0f : 1.0f;
    pa[idx] = 0.0f;
    pb[idx] = 0.0f;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        count[g * q.C + idx] = 0;
        cursor[g * q.C + idx] = 0;
    }
}

// ---- pass 1 (water_grid.comp:721-744) on a snapshot: src -> dst ---------------------------------
// Bounding boxes of the groups of 32 consecutive particles: box[g] = {lo.xyz, hi.xyz}.
struct Box { float lo[3], hi[3]; };

__device__ __forceinline__ void warp_box(float x, float y, float z, bool in, Box* out, int lane) {
    float lo[3] = {in ? x : INFINITY, in ? y : INFINITY, in ? z : INFINITY};
    float hi[3] = {in ? x : -INFINITY, in ? y : -INFINITY, in ? z : -INFINITY};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int a = 0; a < 3; ++a) {
            lo[a] = fminf(lo[a], __shfl_xor_sync(0xffffffffu, lo[a], o));
            hi[a] = fmaxf(hi[a], __shfl_xor_sync(0xffffffffu, hi[a], o));
        }
    if (lane == 0) {
#pragma unroll
        for (int a = 0; a < 3; ++a) { out->lo[a] = lo[a]; out->hi[a] = hi[a]; }
    }
}

__global__ void k_group_boxes(int N, const float4* __restrict__ pos, Box* boxes) {  // one warp per group
    const int g = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (g * 32 >= N) return;
    const int i = g * 32 + lane;
    const float4 v = i < N ? pos[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    warp_box(v.x, v.y, v.z, i < N, boxes + g, lane);
}

// One warp per particle, one CTA (32 warps) per group of 32 particles.  Lane k tests the particle
// against the box of group 32 * r + k: a group whose box is farther than the separation distance
// (with a 1e-4 relative safety margin, far above float rounding) cannot hold a close neighbour,
// so skipping it changes nothing.  The surviving groups are visited in ascending order; inside a
// group the 32 lanes test 32 neighbours at once and the close ones are applied one by one in
// ascending index, re-testing the later lanes with the moved position - the sequential loop's
// arithmetic.  Whenever the position moves, the boxes of the groups still ahead are tested again.
// The CTA finally writes the box of its own 32 moved particles for the next sub-step.
constexpr int kSepWarps = 32;
__global__ void __launch_bounds__(kSepWarps * 32) k_separate(WP q, const float4* __restrict__ src, const Box* __restrict__ boxes,
                                                             float4* __restrict__ dst, Box* __restrict__ boxes_out) {
    __shared__ float moved_pos[kSepWarps][3];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int i = blockIdx.x * kSepWarps + warp;
    const bool active = i < q.N;
    const int n_groups = (q.N + 31) / 32;
    const float min_dist = q.cs * 1.5f, min_dist2 = min_dist * min_dist;
    const float far2 = min_dist2 * 1.0001f;
    const float4 me = active ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    float px = me.x, py = me.y, pz = me.z;
    if (active) {
        for (int g0 = 0; g0 < n_groups; g0 += 32) {
            const int mine = g0 + lane;
            Box bx;
            if (mine < n_groups) bx = boxes[mine];
            else {
#pragma unroll
                for (int a = 0; a < 3; ++a) { bx.lo[a] = INFINITY; bx.hi[a] = -INFINITY; }
            }
            auto near_groups = [&](int from) {  // groups g0 + k, k >= from, whose box is within reach of the current position
                const float ex = fmaxf(fmaxf(bx.lo[0] - px, px - bx.hi[0]), 0.0f), ey = fmaxf(fmaxf(bx.lo[1] - py, py - bx.hi[1]), 0.0f),
                            ez = fmaxf(fmaxf(bx.lo[2] - pz, pz - bx.hi[2]), 0.0f);
                const bool near = lane >= from && !(ex * ex + ey * ey + ez * ez > far2);  // empty boxes are infinitely far
                return __ballot_sync(0xffffffffu, near);
            };
            unsigned groups = near_groups(0);
            while (groups) {
                const int k = __ffs(groups) - 1;
                groups &= groups - 1;
                const int j = (g0 + k) * 32 + lane;
                const bool valid = j < q.N && j != i;
                const float4 o = j < q.N ? src[j] : make_float4(0.f, 0.f, 0.f, 0.f);
                float dx = px - o.x, dy = py - o.y, dz = pz - o.z;
                float d2 = dx * dx + dy * dy + dz * dz;
                unsigned mask = __ballot_sync(0xffffffffu, valid && !(d2 >= min_dist2 || d2 == 0.0f));
                const bool moved = mask != 0u;
                while (mask) {
                    const int l = __ffs(mask) - 1;  // lowest close neighbour: apply it with the current position
                    const float ax = __shfl_sync(0xffffffffu, dx, l), ay = __shfl_sync(0xffffffffu, dy, l),
                                az = __shfl_sync(0xffffffffu, dz, l), a2 = __shfl_sync(0xffffffffu, d2, l);
                    const float d = sqrtf(a2);
                    const float f = 0.5f * (min_dist - d) / d;
                    px += ax * f;
                    py += ay * f;
                    pz += az * f;
                    // later neighbours see the moved position
                    dx = px - o.x; dy = py - o.y; dz = pz - o.z;
                    d2 = dx * dx + dy * dy + dz * dz;
                    mask = __ballot_sync(0xffffffffu, lane > l && valid && !(d2 >= min_dist2 || d2 == 0.0f));
                }
                if (moved) groups = near_groups(k + 1);
            }
        }
        if (lane == 0) dst[i] = make_float4(px, py, pz, me.w);
    }
    if (lane == 0) { moved_pos[warp][0] = px; moved_pos[warp][1] = py; moved_pos[warp][2] = pz; }
    __syncthreads();
    if (warp == 0) {
        const bool in = blockIdx.x * kSepWarps + lane < q.N;
        warp_box(moved_pos[lane][0], moved_pos[lane][1], moved_pos[lane][2], in, boxes_out + blockIdx.x, lane);
    }
}

// ---- passes 2-4 as a binned gather ------------------------------------------------------------------
// count[g * C + node] = particles that contribute to node of grid g (solid nodes take none)
template <bool FILL>
__global__ void k_p2g_bin(WP q, const float4* __restrict__ pos, const unsigned* __restrict__ flags, int* count,
                          const int* __restrict__ offset, int* cursor, int* entries) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;  // one thread per (particle, grid)
    if (t >= 4 * q.N) return;
    const int i = t >> 2, g = t & 3;
    const Stencil st = grid_stencil(q, pos[i], g);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const int node = corner_cell(q, st, c & 1, (c >> 1) & 1, c >> 2);
        if (flags[node] & kSolid) continue;
        const int idx = g * q.C + node;
        if (FILL) entries[offset[idx] + atomicAdd(&cursor[idx], 1)] = i * 8 + c;
        else atomicAdd(&count[idx], 1);
    }
}

// exclusive prefix sum of `n` ints in three kernels (1024 elements per block)
__global__ void __launch_bounds__(1024) k_scan_block(const int* __restrict__ in, int n, int* __restrict__ out, int* block_sums) {
    __shared__ int warp_sums[32];
    const int i = blockIdx.x * 1024 + threadIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int v = i < n ? in[i] : 0;
    int x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
    }
    if (lane == 31) warp_sums[warp] = x;
    __syncthreads();
    if (warp == 0) {
        int w = warp_sums[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int y = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += y;
        }
        warp_sums[lane] = w;
    }
    __syncthreads();
    const int before = warp ? warp_sums[warp - 1] : 0;
    if (i < n) out[i] = before + x - v;
    if (threadIdx.x == 1023) block_sums[blockIdx.x] = before + x;
}

__global__ void __launch_bounds__(1024) k_scan_sums(int* block_sums, int n_blocks) {  // one block, any n_blocks
    __shared__ int warp_sums[32];
    __shared__ int carry;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int base = 0; base < n_blocks; base += 1024) {
        const int i = base + threadIdx.x;
        const int v = i < n_blocks ? block_sums[i] : 0;
        int x = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int y = __shfl_up_sync(0xffffffffu, x, o);
            if (lane >= o) x += y;
        }
        if (lane == 31) warp_sums[warp] = x;
        __syncthreads();
        if (warp == 0) {
            int w = warp_sums[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int y = __shfl_up_sync(0xffffffffu, w, o);
                if (lane >= o) w += y;
            }
            warp_sums[lane] = w;
        }
        __syncthreads();
        const int before = carry + (warp ? warp_sums[warp - 1] : 0);
        if (i < n_blocks) block_sums[i] = before + x - v;
        __syncthreads();
        if (threadIdx.x == 1023) carry = before + x;
        __syncthreads();
    }
}

__global__ void k_scan_add(int* out, int n, const int* __restrict__ block_sums) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] += block_sums[i >> 10];
}

// One thread per (grid, node): sort the node's contributions by particle id, add them in that
// order (water_grid.comp:288-349 for g < 3, :695-720 for the density), normalise (:352-379).
__global__ void k_p2g_gather(WP q, const float4* __restrict__ pos, const float4* __restrict__ vel, const int* __restrict__ count,
                             const int* __restrict__ offset, int* entries, unsigned* flags, float* u, float* v, float* w,
                             float* pu, float* pv, float* pw, float* density) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= 4 * q.C) return;
    const int g = idx / q.C, node = idx - g * q.C;
    const int n = count[idx];
    int* e = entries + offset[idx];
    for (int a = 1; a < n; ++a) {  // insertion sort; n is a handful
        const int key = e[a];
        int b = a - 1;
        while (b >= 0 && e[b] > key) { e[b + 1] = e[b]; --b; }
        e[b + 1] = key;
    }
    float accum = 0.0f, weight = 0.0f;
    for (int a = 0; a < n; ++a) {
        const int pid = e[a] >> 3, c = e[a] & 7;
        const float4 p = pos[pid];
        const Stencil st = grid_stencil(q, p, g);
        const float wt = corner_weight(st, c & 1, (c >> 1) & 1, c >> 2);
        if (g == 3) {
            accum += wt * q.mass;
        } else {
            const float4 pv4 = vel[pid];
            const float comp = g == 0 ? pv4.x : (g == 1 ? pv4.y : pv4.z);
            accum += comp * wt;
            weight += wt;
        }
    }
    if (g == 3) {
        density[node] = accum;
        return;
    }
    if (n > 0) atomicOr(&flags[node], kFluid);
    const float eps = 1e-6f;
    const float val = weight > eps ? accum / weight : 0.0f;  // solid nodes received nothing: 0
    float* dst = g == 0 ? u : (g == 1 ? v : w);
    float* prev = g == 0 ? pu : (g == 1 ? pv : pw);
    dst[node] = val;
    prev[node] = val;
}

// ---- pass 5 (water_grid.comp:382-488) ----------------------------------------------------------------
__global__ void k_jacobi(WP q, const unsigned* __restrict__ flags, const float* __restrict__ s, const float* __restrict__ u,
                         const float* __restrict__ v, const float* __restrict__ w, const float* __restrict__ density,
                         const float* __restrict__ p_read, float* __restrict__ p_write) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= q.C) return;
    const int nx = q.nx, ny = q.ny, nz = q.nz;
    const int gz = idx / (nx * ny), rem = idx - gz * (nx * ny), gy = rem / nx, gx = rem - gy * nx;
    const float here = p_read[idx];
    if (gx == 0 || gx == nx - 1 || gy == 0 || gy == ny - 1 || gz == 0 || gz == nz - 1 || (flags[idx] & kFluid) == 0u) {
        p_write[idx] = here;
        return;
    }
    const int left = idx - 1, right = idx + 1, bottom = idx - nx, top = idx + nx, back = idx - nx * ny, front = idx + nx * ny;
    const float sx0 = s[left], sx1 = s[right], sy0 = s[bottom], sy1 = s[top], sz0 = s[back], sz1 = s[front];
    const float s_sum = sx0 + sx1 + sy0 + sy1 + sz0 + sz1;
    if (s_sum <= 1e-9f) {
        p_write[idx] = here;
        return;
    }
    const float sum_p = sx0 * p_read[left] + sx1 * p_read[right] + sy0 * p_read[bottom] + sy1 * p_read[top] +
                        sz0 * p_read[back] + sz1 * p_read[front];
    float div = ((u[right] - u[idx]) + (v[top] - v[idx]) + (w[front] - w[idx]));
    const float pd = density[idx];
    if (q.rd > 0.0f && pd > 0.0f) {
        const float compression = pd - q.rd;
        if (compression > 0.0f) div -= compression;
    }
    const float dt_safe = fmaxf(q.dt, 1e-6f), cs_safe = fmaxf(q.cs, 1e-6f), rd_safe = fmaxf(q.rd, 1e-6f);
    const float cp = rd_safe * cs_safe * cs_safe / dt_safe;
    const float div_safe = fminf(fmaxf(div, -1e6f), 1e6f);
    const float p_new = (sum_p - cp * div_safe) / fmaxf(s_sum, 1e-6f);
    p_write[idx] = here + q.orx * (p_new - here);
}

// All Jacobi iterations in ONE cooperative launch: every thread keeps the iteration-invariant
// terms of its (at most two) cells in registers - neighbour solidities, cp * div and the
// denominator, formed by the same float operations as k_jacobi - and an iteration is seven L2
// loads, one store and a grid-wide barrier.  Cells that only copy their pressure never leave
// the zero pass 0 gave both buffers, so they are not touched.  The barrier is a counter in
// global memory with a bounded spin: on a timeout the status word is set and every CTA leaves.
constexpr int kFusedThreads = 1024;
__global__ void __launch_bounds__(kFusedThreads, 1)
k_jacobi_fused(WP q, const unsigned* __restrict__ flags, const float* __restrict__ s, const float* __restrict__ u,
               const float* __restrict__ v, const float* __restrict__ w, const float* __restrict__ density, float* pa, float* pb,
               int iterations, unsigned* bar, int* status) {
    const int T = gridDim.x * kFusedThreads, t = blockIdx.x * kFusedThreads + threadIdx.x;
    const int nx = q.nx, ny = q.ny, nz = q.nz;
    int cell[2];
    bool upd[2];
    float B[2], D[2], sn[2][6];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int idx = t + k * T;
        cell[k] = idx;
        upd[k] = false;
        B[k] = 0.0f; D[k] = 1.0f;
#pragma unroll
        for (int a = 0; a < 6; ++a) sn[k][a] = 0.0f;
        if (idx >= q.C) continue;
        const int gz = idx / (nx * ny), rem = idx - gz * (nx * ny), gy = rem / nx, gx = rem - gy * nx;
        if (gx == 0 || gx == nx - 1 || gy == 0 || gy == ny - 1 || gz == 0 || gz == nz - 1 || (flags[idx] & kFluid) == 0u) continue;
        const int left = idx - 1, right = idx + 1, bottom = idx - nx, top = idx + nx, back = idx - nx * ny, front = idx + nx * ny;
        sn[k][0] = s[left]; sn[k][1] = s[right]; sn[k][2] = s[bottom]; sn[k][3] = s[top]; sn[k][4] = s[back]; sn[k][5] = s[front];
        const float s_sum = sn[k][0] + sn[k][1] + sn[k][2] + sn[k][3] + sn[k][4] + sn[k][5];
        if (s_sum <= 1e-9f) continue;
        float div = ((u[right] - u[idx]) + (v[top] - v[idx]) + (w[front] - w[idx]));
        const float pd = density[idx];
        if (q.rd > 0.0f && pd > 0.0f) {
            const float compression = pd - q.rd;
            if (compression > 0.0f) div -= compression;
        }
        const float dt_safe = fmaxf(q.dt, 1e-6f), cs_safe = fmaxf(q.cs, 1e-6f), rd_safe = fmaxf(q.rd, 1e-6f);
        const float cp = rd_safe * cs_safe * cs_safe / dt_safe;
        const float div_safe = fminf(fmaxf(div, -1e6f), 1e6f);
        B[k] = cp * div_safe;
        D[k] = fmaxf(s_sum, 1e-6f);
        upd[k] = true;
    }
    __shared__ int give_up;
    if (threadIdx.x == 0) give_up = 0;
    __syncthreads();
    for (int it = 0; it < iterations; ++it) {
        const float* p_read = (it % 2 == 0) ? pa : pb;
        float* p_write = (it % 2 == 0) ? pb : pa;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            if (!upd[k]) continue;
            const int idx = cell[k];
            const float here = __ldcg(p_read + idx);
            const float sum_p = sn[k][0] * __ldcg(p_read + idx - 1) + sn[k][1] * __ldcg(p_read + idx + 1) +
                                sn[k][2] * __ldcg(p_read + idx - nx) + sn[k][3] * __ldcg(p_read + idx + nx) +
                                sn[k][4] * __ldcg(p_read + idx - nx * ny) + sn[k][5] * __ldcg(p_read + idx + nx * ny);
            const float p_new = (sum_p - B[k]) / D[k];
            __stcg(p_write + idx, here + q.orx * (p_new - here));
        }
        if (it + 1 == iterations) break;
        // grid barrier number it + 1: all CTAs have added 1 when the counter reaches (it + 1) * gridDim.x
        __syncthreads();
        if (threadIdx.x == 0) {
            // arrive with release semantics (orders this CTA's stores, made visible to thread 0 by the
            // barrier above, before the count), then poll with acquire loads
            asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(bar) : "memory");
            const unsigned target = (unsigned)(it + 1) * gridDim.x;
            long long spins = 0;
            for (;;) {
                unsigned seen;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(bar) : "memory");
                if (seen >= target) break;
                if (++spins > 2000000ll || *reinterpret_cast<volatile int*>(status) != 0) {
                    atomicExch(status, 1);
                    give_up = 1;
                    break;
                }
            }
        }
        __syncthreads();
        if (give_up) return;
    }
}

// ---- pass 6 (water_grid.comp:491-560) ----------------------------------------------------------------
__global__ void k_pressure_apply(WP q, const unsigned* __restrict__ flags, const float* __restrict__ p, float* u, float* v,
                                 float* w) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= q.C) return;
    const int nx = q.nx, ny = q.ny, nz = q.nz;
    const int gz = idx / (nx * ny), rem = idx - gz * (nx * ny), gy = rem / nx, gx = rem - gy * nx;
    if (gx == 0 || gy == 0 || gz == 0 || gx >= nx - 1 || gy >= ny - 1 || gz >= nz - 1) return;
    if ((flags[idx] & kFluid) == 0u) return;
    const float inv_cp = q.dt / (q.rd * q.cs);
    const float p0 = p[idx];
    const int left = idx - 1, right = idx + 1, bot = idx - nx, top = idx + nx, back = idx - nx * ny, front = idx + nx * ny;
    u[idx] = (flags[left] & kSolid) ? 0.0f : u[idx] - (p0 - p[left]) * inv_cp;
    v[idx] = (flags[bot] & kSolid) ? 0.0f : v[idx] - (p0 - p[bot]) * inv_cp;
    w[idx] = (flags[back] & kSolid) ? 0.0f : w[idx] - (p0 - p[back]) * inv_cp;
    // faces of solid neighbours: those cells are border cells, whose own threads returned above
    if (flags[right] & kSolid) u[right] = 0.0f;
    if (flags[top] & kSolid) v[top] = 0.0f;
    if (flags[front] & kSolid) w[front] = 0.0f;
}

// ---- passes 7 and 8 (water_grid.comp:574-693), one thread per particle ----------------------------------
__global__ void k_g2p_integrate(WP q, const unsigned* __restrict__ flags, const float* __restrict__ u, const float* __restrict__ v,
                                const float* __restrict__ w, const float* __restrict__ pu, const float* __restrict__ pv,
                                const float* __restrict__ pw, float4* pos, float4* vel, Box* boxes) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if ((i & ~31) >= q.N) return;  // whole warp past the end
    // a partly filled last warp runs to the end with a clamped index (stores are predicated) so that
    // all 32 lanes reach the one box reduction below
    const bool in = i < q.N;
    const int ii = in ? i : q.N - 1;
    const float4 p = pos[ii];
    const float4 pv4 = vel[ii];
    const float old[3] = {pv4.x, pv4.y, pv4.z};
    float nv[3] = {pv4.x, pv4.y, pv4.z};
    const float flip = fminf(fmaxf(q.damp, 0.0f), 1.0f);
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        const float* grid = a == 0 ? u : (a == 1 ? v : w);
        const float* prev = a == 0 ? pu : (a == 1 ? pv : pw);
        const Stencil st = grid_stencil(q, p, a);
        float pic = 0.0f, fl = 0.0f, tw = 0.0f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const int ix = c & 1, iy = (c >> 1) & 1, iz = c >> 2;
            const float wt = corner_weight(st, ix, iy, iz);
            const int cell = corner_cell(q, st, ix, iy, iz);
            if (flags[cell] & kSolid) continue;
            const float val = grid[cell];
            pic += val * wt;
            fl += (val - prev[cell]) * wt;
            tw += wt;
        }
        if (tw > 0.01f) {
            pic /= tw;
            fl /= tw;
            nv[a] = (1.0f - flip) * pic + flip * (old[a] + fl);
        }
    }
    // pass 8
    const float restitution = 0.3f, friction = 0.9f, margin = q.cs;
    float np[3] = {p.x, p.y, p.z};
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        nv[a] = nv[a] + q.g[a] * q.dt;
        np[a] = np[a] + nv[a] * q.dt;
    }
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        const float lo = q.bmin[a] + margin, hi = q.bmax[a] - margin;
        const int b = (a + 1) % 3, c = (a + 2) % 3;
        if (np[a] < lo) { np[a] = lo; nv[a] = fabsf(nv[a]) * restitution; nv[b] *= friction; nv[c] *= friction; }
        if (np[a] > hi) { np[a] = hi; nv[a] = -fabsf(nv[a]) * restitution; nv[b] *= friction; nv[c] *= friction; }
    }
    if (in) {
        pos[i] = make_float4(np[0], np[1], np[2], 0.1f);
        vel[i] = make_float4(nv[0], nv[1], nv[2], pv4.w);
    }
    warp_box(np[0], np[1], np[2], in, boxes + (i >> 5), threadIdx.x & 31);  // the next step's first sub-step reads these
}

thread_local std::string g_water_create_error;

}  // namespace

struct neon_water_handle {
    neon_water_config cfg{};
    WP q{};
    std::string err;
    float4 *pos = nullptr, *pos_tmp = nullptr, *vel = nullptr;
    float *u = nullptr, *v = nullptr, *w = nullptr, *pu = nullptr, *pv = nullptr, *pw = nullptr, *s = nullptr, *pa = nullptr,
          *pb = nullptr, *density = nullptr;
    unsigned* flags = nullptr;
    int *count = nullptr, *offset = nullptr, *cursor = nullptr, *entries = nullptr, *block_sums = nullptr;
    Box *boxes = nullptr, *boxes_tmp = nullptr;  // bounding boxes of the particle groups of pos / pos_tmp
    unsigned* bar = nullptr;  // [0] grid-barrier counter, [1] status word (non-zero: a barrier wait gave up)
    int n_sms = 0, fused_jacobi = 1;
    const float* p_final = nullptr;
    int64_t launches = 0;
    int launches_per_step = 0;
    int use_graphs = 1;
    cudaStream_t own_stream = nullptr, last_stream = nullptr;
    cudaGraphExec_t graph = nullptr;
};

namespace {

int wfail(neon_water_handle* h, int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (h) h->err = buf; else g_water_create_error = buf;
    return code;
}

#define WCU(h, call)                                                                                       \
    do {                                                                                                   \
        cudaError_t e_ = (call);                                                                           \
        if (e_ != cudaSuccess) return wfail(h, NEON_MOE_ECUDA, "%s: %s", #call, cudaGetErrorString(e_)); \
    } while (0)

// the kernels of one step, in the reference's dispatch order; ev (optional) gets 5 event marks
int record_step(neon_water_handle* h, cudaStream_t st, cudaEvent_t* ev = nullptr) {
    const WP& q = h->q;
    const int cb = (q.C + 255) / 256, pb = (q.N + 255) / 256, n4 = 4 * q.C, sb = (n4 + 1023) / 1024;
    int n = 0;
    k_grid_init<<<cb, 256, 0, st>>>(q, h->flags, h->s, h->pa, h->pb, h->count, h->cursor, h->bar); ++n;
    if (ev) cudaEventRecord(ev[0], st);
    float4 *src = h->pos, *dst = h->pos_tmp;
    Box *bsrc = h->boxes, *bdst = h->boxes_tmp;
    for (int i = 0; i < h->cfg.collision_substeps; ++i) {
        k_separate<<<(q.N + kSepWarps - 1) / kSepWarps, kSepWarps * 32, 0, st>>>(q, src, bsrc, dst, bdst); ++n;
        float4* t = src; src = dst; dst = t;
        Box* bt = bsrc; bsrc = bdst; bdst = bt;
    }
    if (src != h->pos) WCU(h, cudaMemcpyAsync(h->pos, src, (size_t)q.N * sizeof(float4), cudaMemcpyDeviceToDevice, st));
    if (ev) cudaEventRecord(ev[1], st);
    k_p2g_bin<false><<<(4 * q.N + 255) / 256, 256, 0, st>>>(q, h->pos, h->flags, h->count, nullptr, nullptr, nullptr); ++n;
    k_scan_block<<<sb, 1024, 0, st>>>(h->count, n4, h->offset, h->block_sums); ++n;
    k_scan_sums<<<1, 1024, 0, st>>>(h->block_sums, sb); ++n;
    k_scan_add<<<(n4 + 255) / 256, 256, 0, st>>>(h->offset, n4, h->block_sums); ++n;
    k_p2g_bin<true><<<(4 * q.N + 255) / 256, 256, 0, st>>>(q, h->pos, h->flags, nullptr, h->offset, h->cursor, h->entries); ++n;
    k_p2g_gather<<<(n4 + 255) / 256, 256, 0, st>>>(q, h->pos, h->vel, h->count, h->offset, h->entries, h->flags, h->u, h->v, h->w,
                                                   h->pu, h->pv, h->pw, h->density); ++n;
    if (ev) cudaEventRecord(ev[2], st);
    const float* p_read = h->pa;
    const int iters = h->cfg.jacobi_iterations;
    if (h->fused_jacobi && iters > 1 && q.C <= 2 * h->n_sms * kFusedThreads) {
        // one cooperative launch (all CTAs co-resident, one per SM) instead of `iters` launches
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(h->n_sms);
        cfg.blockDim = dim3(kFusedThreads);
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeCooperative;
        attr[0].val.cooperative = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        WCU(h, cudaLaunchKernelEx(&cfg, k_jacobi_fused, q, (const unsigned*)h->flags, (const float*)h->s, (const float*)h->u,
                                  (const float*)h->v, (const float*)h->w, (const float*)h->density, h->pa, h->pb, iters, h->bar,
                                  reinterpret_cast<int*>(h->bar + 1)));
        ++n;
        p_read = ((iters - 1) % 2 == 0) ? h->pa : h->pb;
    } else {
        for (int it = 0; it < iters; ++it) {
            p_read = (it % 2 == 0) ? h->pa : h->pb;
            float* p_write = (it % 2 == 0) ? h->pb : h->pa;
            k_jacobi<<<cb, 256, 0, st>>>(q, h->flags, h->s, h->u, h->v, h->w, h->density, p_read, p_write); ++n;
        }
    }
    // the reference leaves the last iteration's descriptor set bound: passes 6-8 read what it read
    h->p_final = p_read;
    if (ev) cudaEventRecord(ev[3], st);
    k_pressure_apply<<<cb, 256, 0, st>>>(q, h->flags, p_read, h->u, h->v, h->w); ++n;
    k_g2p_integrate<<<pb, 256, 0, st>>>(q, h->flags, h->u, h->v, h->w, h->pu, h->pv, h->pw, h->pos, h->vel, h->boxes); ++n;
    if (ev) cudaEventRecord(ev[4], st);
    h->launches_per_step = n;
    WCU(h, cudaGetLastError());
    return NEON_MOE_OK;
}

}  // namespace

extern "C" {

const char* neon_water_last_error(const neon_water_handle* h) { return h ? h->err.c_str() : g_water_create_error.c_str(); }
int64_t neon_water_launch_count(const neon_water_handle* h) { return h ? h->launches : 0; }

int neon_water_destroy(neon_water_handle* h) {
    if (!h) return NEON_MOE_OK;
    cudaSetDevice(h->cfg.device);
    cudaDeviceSynchronize();
    if (h->graph) cudaGraphExecDestroy(h->graph);
    for (void* p : {(void*)h->pos, (void*)h->pos_tmp, (void*)h->vel, (void*)h->u, (void*)h->v, (void*)h->w, (void*)h->pu,
                    (void*)h->pv, (void*)h->pw, (void*)h->s, (void*)h->pa, (void*)h->pb, (void*)h->density, (void*)h->flags,
                    (void*)h->count, (void*)h->offset, (void*)h->cursor, (void*)h->entries, (void*)h->block_sums, (void*)h->bar, (void*)h->boxes, (void*)h->boxes_tmp})
        if (p) cudaFree(p);
    if (h->own_stream) cudaStreamDestroy(h->own_stream);
    cudaGetLastError();
    delete h;
    return NEON_MOE_OK;
}

int neon_water_create(const neon_water_config* cfg, const float* pos4, int on_device, neon_water_handle** out) {
    if (!cfg || !out) return wfail(nullptr, NEON_MOE_EINVAL, "null argument");
    *out = nullptr;
    const auto& c = *cfg;
    if (c.n_particles <= 0 || c.n_particles > (1 << 27)) return wfail(nullptr, NEON_MOE_EINVAL, "particle count %d out of range", c.n_particles);
    if (c.nx < 2 || c.ny < 2 || c.nz < 2 || (long long)c.nx * c.ny * c.nz > (1ll << 27))
        return wfail(nullptr, NEON_MOE_EINVAL, "grid %d x %d x %d out of range (at least 2 cells per axis)", c.nx, c.ny, c.nz);
    if (!(c.cell_size > 0.f) || !(c.dt > 0.f) || c.collision_substeps < 0 || c.jacobi_iterations < 0)
        return wfail(nullptr, NEON_MOE_EINVAL, "cell size and time step must be positive, loop counts non-negative");
    if (!pos4) return wfail(nullptr, NEON_MOE_EINVAL, "null start positions");
    if (cudaSetDevice(c.device) != cudaSuccess) {
        cudaGetLastError();
        return wfail(nullptr, NEON_MOE_ECUDA, "cudaSetDevice(%d) failed", c.device);
    }
    auto* h = new (std::nothrow) neon_water_handle;
    if (!h) return wfail(nullptr, NEON_MOE_ECUDA, "out of host memory");
    h->cfg = c;
    WP& q = h->q;
    q.N = c.n_particles; q.nx = c.nx; q.ny = c.ny; q.nz = c.nz; q.C = c.nx * c.ny * c.nz;
    q.cs = c.cell_size; q.orx = c.over_relaxation; q.rd = c.rest_density; q.damp = c.damping; q.mass = c.mass; q.dt = c.dt;
    for (int a = 0; a < 3; ++a) { q.bmin[a] = c.box_min[a]; q.bmax[a] = c.box_max[a]; q.g[a] = c.gravity[a]; }
    const size_t C = (size_t)q.C, N = (size_t)q.N;
    bool ok = true;
    auto alloc = [&](auto& ptr, size_t bytes) {
        if (ok && cudaMalloc(reinterpret_cast<void**>(&ptr), bytes) != cudaSuccess) ok = false;
        if (ok && cudaMemset(ptr, 0, bytes) != cudaSuccess) ok = false;
    };
    alloc(h->pos, N * 16); alloc(h->pos_tmp, N * 16); alloc(h->vel, N * 16);
    alloc(h->u, C * 4); alloc(h->v, C * 4); alloc(h->w, C * 4); alloc(h->pu, C * 4); alloc(h->pv, C * 4); alloc(h->pw, C * 4);
    alloc(h->s, C * 4); alloc(h->pa, C * 4); alloc(h->pb, C * 4); alloc(h->density, C * 4); alloc(h->flags, C * 4);
    alloc(h->count, 4 * C * 4); alloc(h->offset, 4 * C * 4); alloc(h->cursor, 4 * C * 4);
    alloc(h->entries, N * 32 * 4); alloc(h->block_sums, ((4 * C + 1023) / 1024 + 1) * 4); alloc(h->bar, 16);
    alloc(h->boxes, ((N + 31) / 32) * sizeof(Box)); alloc(h->boxes_tmp, ((N + 31) / 32) * sizeof(Box));
    if (ok && cudaDeviceGetAttribute(&h->n_sms, cudaDevAttrMultiProcessorCount, c.device) != cudaSuccess) ok = false;
    int coop = 0;
    if (ok && (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, c.device) != cudaSuccess || !coop)) h->fused_jacobi = 0;
    if (ok && cudaStreamCreateWithFlags(&h->own_stream, cudaStreamNonBlocking) != cudaSuccess) ok = false;
    if (!ok) {
        cudaGetLastError();
        neon_water_destroy(h);
        return wfail(nullptr, NEON_MOE_ECUDA, "device allocation failed");
    }
    h->p_final = h->pa;
    int rc = neon_water_set_particles(h, pos4, nullptr, on_device);
    if (rc) {
        g_water_create_error = h->err;
        neon_water_destroy(h);
        return rc;
    }
    *out = h;
    return NEON_MOE_OK;
}

int neon_water_set_particles(neon_water_handle* h, const float* pos4, const float* vel4, int on_device) {
    if (!h) return NEON_MOE_EINVAL;
    if (!pos4) return wfail(h, NEON_MOE_EINVAL, "null positions");
    WCU(h, cudaSetDevice(h->cfg.device));
    const size_t bytes = (size_t)h->q.N * 16;
    const cudaMemcpyKind kind = on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
    WCU(h, cudaDeviceSynchronize());
    WCU(h, cudaMemcpy(h->pos, pos4, bytes, kind));
    if (vel4) WCU(h, cudaMemcpy(h->vel, vel4, bytes, kind));
    else WCU(h, cudaMemset(h->vel, 0, bytes));
    k_group_boxes<<<(h->q.N + 255) / 256, 256>>>(h->q.N, h->pos, h->boxes);
    h->launches++;
    WCU(h, cudaDeviceSynchronize());
    return NEON_MOE_OK;
}

int neon_water_step(neon_water_handle* h, int n_steps, void* cuda_stream) {
    if (!h) return NEON_MOE_EINVAL;
    if (n_steps < 0) return wfail(h, NEON_MOE_EINVAL, "negative step count");
    WCU(h, cudaSetDevice(h->cfg.device));
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    h->last_stream = st;
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    const bool capturing = cudaStreamIsCapturing(st, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone;
    cudaGetLastError();
    if (h->use_graphs && !capturing && !h->graph) {
        WCU(h, cudaStreamBeginCapture(h->own_stream, cudaStreamCaptureModeThreadLocal));
        int rc = record_step(h, h->own_stream);
        cudaGraph_t graph = nullptr;
        cudaError_t ce = cudaStreamEndCapture(h->own_stream, &graph);
        if (!rc && ce == cudaSuccess && graph) ce = cudaGraphInstantiate(&h->graph, graph, 0);
        if (graph) cudaGraphDestroy(graph);
        if (rc || ce != cudaSuccess) {
            h->graph = nullptr;
            h->use_graphs = 0;  // capture is not available here: stay eager
            cudaGetLastError();
        }
    }
    for (int i = 0; i < n_steps; ++i) {
        if (h->use_graphs && !capturing && h->graph) {
            WCU(h, cudaGraphLaunch(h->graph, st));
        } else {
            int rc = record_step(h, st);
            if (rc) return rc;
        }
        h->launches += h->launches_per_step;
    }
    return NEON_MOE_OK;
}

int neon_water_step_host(neon_water_handle* h, float* pos4, float* vel4, int n_steps, void* cuda_stream) {
    if (!h) return NEON_MOE_EINVAL;
    if (!pos4 || !vel4) return wfail(h, NEON_MOE_EINVAL, "null particle arrays");
    WCU(h, cudaSetDevice(h->cfg.device));
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    const size_t bytes = (size_t)h->q.N * 16;
    WCU(h, cudaMemcpyAsync(h->pos, pos4, bytes, cudaMemcpyHostToDevice, st));
    WCU(h, cudaMemcpyAsync(h->vel, vel4, bytes, cudaMemcpyHostToDevice, st));
    k_group_boxes<<<(h->q.N + 255) / 256, 256, 0, st>>>(h->q.N, h->pos, h->boxes);
    h->launches++;
    int rc = neon_water_step(h, n_steps, st);
    if (rc) return rc;
    WCU(h, cudaMemcpyAsync(pos4, h->pos, bytes, cudaMemcpyDeviceToHost, st));
    WCU(h, cudaMemcpyAsync(vel4, h->vel, bytes, cudaMemcpyDeviceToHost, st));
    WCU(h, cudaStreamSynchronize(st));
    return NEON_MOE_OK;
}

int neon_water_particles_device(neon_water_handle* h, float** pos4, float** vel4) {
    if (!h) return NEON_MOE_EINVAL;
    if (pos4) *pos4 = reinterpret_cast<float*>(h->pos);
    if (vel4) *vel4 = reinterpret_cast<float*>(h->vel);
    return NEON_MOE_OK;
}

int neon_water_read_particles(neon_water_handle* h, float* pos4, float* vel4) {
    if (!h) return NEON_MOE_EINVAL;
    WCU(h, cudaSetDevice(h->cfg.device));
    WCU(h, cudaStreamSynchronize(h->last_stream));
    const size_t bytes = (size_t)h->q.N * 16;
    if (pos4) WCU(h, cudaMemcpy(pos4, h->pos, bytes, cudaMemcpyDeviceToHost));
    if (vel4) WCU(h, cudaMemcpy(vel4, h->vel, bytes, cudaMemcpyDeviceToHost));
    return NEON_MOE_OK;
}

int neon_water_read_grid(neon_water_handle* h, const char* name, void* dst, uint64_t bytes) {
    if (!h || !name || !dst) return NEON_MOE_EINVAL;
    const void* src = nullptr;
    if (!strcmp(name, "u")) src = h->u;
    else if (!strcmp(name, "v")) src = h->v;
    else if (!strcmp(name, "w")) src = h->w;
    else if (!strcmp(name, "pressure")) src = h->p_final;
    else if (!strcmp(name, "density")) src = h->density;
    else if (!strcmp(name, "flags")) src = h->flags;
    else return wfail(h, NEON_MOE_EINVAL, "unknown grid '%s'", name);
    if (bytes > (uint64_t)h->q.C * 4) return wfail(h, NEON_MOE_EINVAL, "'%s' holds %d bytes", name, h->q.C * 4);
    WCU(h, cudaSetDevice(h->cfg.device));
    WCU(h, cudaStreamSynchronize(h->last_stream));
    WCU(h, cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost));
    return NEON_MOE_OK;
}

int neon_water_status(neon_water_handle* h, int* word) {
    if (!h || !word) return NEON_MOE_EINVAL;
    WCU(h, cudaSetDevice(h->cfg.device));
    WCU(h, cudaStreamSynchronize(h->last_stream));
    WCU(h, cudaMemcpy(word, h->bar + 1, sizeof(int), cudaMemcpyDeviceToHost));
    WCU(h, cudaMemset(h->bar + 1, 0, sizeof(int)));
    return *word ? NEON_MOE_EDEVICE : NEON_MOE_OK;
}

int neon_water_profile_step(neon_water_handle* h, double* ms4, void* cuda_stream) {
    if (!h || !ms4) return NEON_MOE_EINVAL;
    WCU(h, cudaSetDevice(h->cfg.device));
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    h->last_stream = st;
    cudaEvent_t ev[5];
    for (auto& e : ev) WCU(h, cudaEventCreate(&e));
    int rc = record_step(h, st, ev);
    cudaError_t ce = cudaStreamSynchronize(st);
    if (!rc && ce == cudaSuccess) {
        for (int i = 0; i < 4; ++i) {
            float t = 0.f;
            cudaEventElapsedTime(&t, ev[i], ev[i + 1]);
            ms4[i] = t;
        }
        h->launches += h->launches_per_step;
    }
    for (auto& e : ev) cudaEventDestroy(e);
    if (rc) return rc;
    if (ce != cudaSuccess) return wfail(h, NEON_MOE_ECUDA, "profile step: %s", cudaGetErrorString(ce));
    return NEON_MOE_OK;
}

int neon_water_set_option(neon_water_handle* h, const char* name, int64_t value) {
    if (!h || !name) return NEON_MOE_EINVAL;
    if (!strcmp(name, "use_graphs")) {
        h->use_graphs = (int)value;
        if (!value && h->graph) { cudaGraphExecDestroy(h->graph); h->graph = nullptr; }
    } else if (!strcmp(name, "fused_jacobi")) {
        h->fused_jacobi = (int)value;
        if (h->graph) { cudaGraphExecDestroy(h->graph); h->graph = nullptr; }
    } else {
        return wfail(h, NEON_MOE_EINVAL, "unknown option '%s'", name);
    }
    return NEON_MOE_OK;
}

}  // extern "C"
