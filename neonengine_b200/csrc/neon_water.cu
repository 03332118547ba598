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
__global__ void k_grid_init(WP q, unsigned* flags, float* s, float* pa, float* pb, int* count, int* cursor) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
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
constexpr int kSepWarps = 32, kSepTile = 1024;
__global__ void __launch_bounds__(kSepWarps * 32) k_separate(WP q, const float4* __restrict__ src, float4* __restrict__ dst) {
    __shared__ float4 tile[kSepTile];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int i = blockIdx.x * kSepWarps + warp;
    const bool active = i < q.N;
    const float min_dist = q.cs * 1.5f, min_dist2 = min_dist * min_dist;
    float4 me = active ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    float px = me.x, py = me.y, pz = me.z;
    for (int t0 = 0; t0 < q.N; t0 += kSepTile) {
        __syncthreads();
        for (int k = threadIdx.x; k < kSepTile; k += kSepWarps * 32)
            tile[k] = t0 + k < q.N ? src[t0 + k] : make_float4(0.f, 0.f, 0.f, 0.f);
        __syncthreads();
        if (!active) continue;
        const int n_here = min(kSepTile, q.N - t0);
        for (int jj = 0; jj < n_here; jj += 32) {
            const int j = t0 + jj + lane;
            const bool valid = jj + lane < n_here && j != i;
            const float4 o = tile[jj + lane];
            float dx = px - o.x, dy = py - o.y, dz = pz - o.z;
            float d2 = dx * dx + dy * dy + dz * dz;
            unsigned mask = __ballot_sync(0xffffffffu, valid && !(d2 >= min_dist2 || d2 == 0.0f));
            while (mask) {
                const int l = __ffs(mask) - 1;  // lowest close neighbour: apply it with the current position
                const float bx = __shfl_sync(0xffffffffu, dx, l), by = __shfl_sync(0xffffffffu, dy, l),
                            bz = __shfl_sync(0xffffffffu, dz, l), b2 = __shfl_sync(0xffffffffu, d2, l);
                const float d = sqrtf(b2);
                const float f = 0.5f * (min_dist - d) / d;
                px += bx * f;
                py += by * f;
                pz += bz * f;
                // later neighbours see the moved position
                dx = px - o.x; dy = py - o.y; dz = pz - o.z;
                d2 = dx * dx + dy * dy + dz * dz;
                mask = __ballot_sync(0xffffffffu, lane > l && valid && !(d2 >= min_dist2 || d2 == 0.0f));
            }
        }
    }
    if (active && lane == 0) dst[i] = make_float4(px, py, pz, me.w);
}

// ---- passes 2-4 as a binned gather ------------------------------------------------------------------
// count[g * C + node] = particles that contribute to node of grid g (solid nodes take none)
template <bool FILL>
__global__ void k_p2g_bin(WP q, const float4* __restrict__ pos, const unsigned* __restrict__ flags, int* count,
                          const int* __restrict__ offset, int* cursor, int* entries) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= q.N) return;
    const float4 p = pos[i];
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        const Stencil st = grid_stencil(q, p, g);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const int node = corner_cell(q, st, c & 1, (c >> 1) & 1, c >> 2);
            if (flags[node] & kSolid) continue;
            const int idx = g * q.C + node;
            if (FILL) entries[offset[idx] + atomicAdd(&cursor[idx], 1)] = i * 8 + c;
            else atomicAdd(&count[idx], 1);
        }
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
                                const float* __restrict__ pw, float4* pos, float4* vel) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= q.N) return;
    const float4 p = pos[i];
    const float4 pv4 = vel[i];
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
    pos[i] = make_float4(np[0], np[1], np[2], 0.1f);
    vel[i] = make_float4(nv[0], nv[1], nv[2], pv4.w);
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

// the kernels of one step, in the reference's dispatch order
int record_step(neon_water_handle* h, cudaStream_t st) {
    const WP& q = h->q;
    const int cb = (q.C + 255) / 256, pb = (q.N + 255) / 256, n4 = 4 * q.C, sb = (n4 + 1023) / 1024;
    int n = 0;
    k_grid_init<<<cb, 256, 0, st>>>(q, h->flags, h->s, h->pa, h->pb, h->count, h->cursor); ++n;
    float4 *src = h->pos, *dst = h->pos_tmp;
    for (int i = 0; i < h->cfg.collision_substeps; ++i) {
        k_separate<<<(q.N + kSepWarps - 1) / kSepWarps, kSepWarps * 32, 0, st>>>(q, src, dst); ++n;
        float4* t = src; src = dst; dst = t;
    }
    if (src != h->pos) WCU(h, cudaMemcpyAsync(h->pos, src, (size_t)q.N * sizeof(float4), cudaMemcpyDeviceToDevice, st));
    k_p2g_bin<false><<<pb, 256, 0, st>>>(q, h->pos, h->flags, h->count, nullptr, nullptr, nullptr); ++n;
    k_scan_block<<<sb, 1024, 0, st>>>(h->count, n4, h->offset, h->block_sums); ++n;
    k_scan_sums<<<1, 1024, 0, st>>>(h->block_sums, sb); ++n;
    k_scan_add<<<(n4 + 255) / 256, 256, 0, st>>>(h->offset, n4, h->block_sums); ++n;
    k_p2g_bin<true><<<pb, 256, 0, st>>>(q, h->pos, h->flags, nullptr, h->offset, h->cursor, h->entries); ++n;
    k_p2g_gather<<<(n4 + 255) / 256, 256, 0, st>>>(q, h->pos, h->vel, h->count, h->offset, h->entries, h->flags, h->u, h->v, h->w,
                                                   h->pu, h->pv, h->pw, h->density); ++n;
    const float* p_read = h->pa;
    for (int it = 0; it < h->cfg.jacobi_iterations; ++it) {
        p_read = (it % 2 == 0) ? h->pa : h->pb;
        float* p_write = (it % 2 == 0) ? h->pb : h->pa;
        k_jacobi<<<cb, 256, 0, st>>>(q, h->flags, h->s, h->u, h->v, h->w, h->density, p_read, p_write); ++n;
    }
    // the reference leaves the last iteration's descriptor set bound: passes 6-8 read what it read
    h->p_final = p_read;
    k_pressure_apply<<<cb, 256, 0, st>>>(q, h->flags, p_read, h->u, h->v, h->w); ++n;
    k_g2p_integrate<<<pb, 256, 0, st>>>(q, h->flags, h->u, h->v, h->w, h->pu, h->pv, h->pw, h->pos, h->vel); ++n;
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
                    (void*)h->count, (void*)h->offset, (void*)h->cursor, (void*)h->entries, (void*)h->block_sums})
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
    alloc(h->entries, N * 32 * 4); alloc(h->block_sums, ((4 * C + 1023) / 1024 + 1) * 4);
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

int neon_water_set_option(neon_water_handle* h, const char* name, int64_t value) {
    if (!h || !name) return NEON_MOE_EINVAL;
    if (!strcmp(name, "use_graphs")) {
        h->use_graphs = (int)value;
        if (!value && h->graph) { cudaGraphExecDestroy(h->graph); h->graph = nullptr; }
    } else {
        return wfail(h, NEON_MOE_EINVAL, "unknown option '%s'", name);
    }
    return NEON_MOE_OK;
}

}  // extern "C"
