/*
 * water_oracle.c - CPU restatement of the reference engine's FLIP water step.
 *
 * TEST INFRASTRUCTURE ONLY: used by tests/, the smoke check and the CPU-baseline leg of the
 * benchmark; the product path never links or calls it.
 *
 * Restates, pass by pass and in the same floating-point operation order (32-bit floats, no
 * fused multiply-add: compile with -ffp-contract=off), the compute shader
 * NeonEngine/shaders/water_grid.comp and the dispatch sequence of
 * NeonEngine/src/water_physics.cpp:164-430:
 *   pass 0 grid init ............ water_grid.comp:239-285
 *   pass 1 particle separation .. water_grid.comp:721-744   (4 sub-steps, water_physics.cpp:240-259)
 *   pass 2 particles -> grid .... water_grid.comp:288-349
 *   pass 3 grid finalize ........ water_grid.comp:352-379
 *   pass 4 cell density ......... water_grid.comp:695-720
 *   pass 5 pressure Jacobi ...... water_grid.comp:382-488   (50 iterations, buffers swapped, water_physics.cpp:318-350)
 *   pass 6 pressure apply ....... water_grid.comp:491-560
 *   pass 7 grid -> particles .... water_grid.comp:574-662
 *   pass 8 integrate + walls .... water_grid.comp:663-693
 * Passes 6-8 run with the descriptor set of the LAST Jacobi iteration still bound
 * (water_physics.cpp:318-352 never rebinds), so with an even iteration count they read the
 * pressure of the last-but-one iteration; that is restated as is.  The shader's debug
 * buffer writes (water_grid.comp:455-485) and particle colours are not restated.
 *
 * Pinned: tests/test_water_oracle.py checks this file bit for bit against the reference
 * shader itself compiled for the CPU (oracle/water_ref_build.py -> oracle/_ref/libwater_ref.so)
 * and against tests/golden/water_small.npz, which that library produced.
 *
 * The shader has data races on a GPU; this file fixes their outcome two ways:
 *   collision_mode 0: invocations run one after the other in ascending id and pass 1 updates
 *       positions in place (what the serially executed reference shader does);
 *   collision_mode 1: pass 1 reads the positions as they were when the pass started and
 *       writes new ones (the order-independent form a parallel implementation can reproduce).
 * Float accumulations (passes 2 and 4) add in ascending particle id in both modes.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct water_params {
    int n_particles, nx, ny, nz;
    float cell_size, over_relaxation, rest_density, damping, mass, dt;
    float box_min[3], box_max[3], gravity[3];
    int collision_substeps, jacobi_iterations;
} water_params;

#define CELL_FLUID 1u
#define CELL_SOLID 2u

typedef struct {
    int base[3];
    float frac[3];
} stencil;

static int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* base cell and fractions of a particle for a grid staggered by (ox, oy, oz) cells */
static stencil make_stencil(const water_params* q, const float* pos, float ox, float oy, float oz) {
    stencil s;
    const float off[3] = {ox, oy, oz};
    const int dim[3] = {q->nx, q->ny, q->nz};
    for (int a = 0; a < 3; ++a) {
        const float local = (pos[a] - q->box_min[a]) / q->cell_size;
        const float l = local - off[a];
        s.base[a] = clampi((int)floorf(l), 0, dim[a] - 2);
        s.frac[a] = l - (float)s.base[a];
    }
    return s;
}

static float corner_weight(const stencil* s, int ix, int iy, int iz) {
    return (ix == 0 ? (1.0f - s->frac[0]) : s->frac[0]) * (iy == 0 ? (1.0f - s->frac[1]) : s->frac[1]) *
           (iz == 0 ? (1.0f - s->frac[2]) : s->frac[2]);
}

static int corner_cell(const water_params* q, const stencil* s, int ix, int iy, int iz) {
    return (s->base[0] + ix) + (s->base[1] + iy) * q->nx + (s->base[2] + iz) * (q->nx * q->ny);
}

int water_oracle_step(const water_params* q, float* pos4, float* vel4, int n_steps, int collision_mode, float* grid_u,
                      float* grid_v, float* grid_w, float* pressure, unsigned* flags_out, float* density_out) {
    const int N = q->n_particles, nx = q->nx, ny = q->ny, nz = q->nz, C = nx * ny * nz;
    float* mem = (float*)calloc((size_t)C * 14 + (size_t)N * 4, sizeof(float));
    unsigned* flags = (unsigned*)calloc((size_t)C, sizeof(unsigned));
    if (!mem || !flags) { free(mem); free(flags); return 1; }
    float *u = mem, *v = u + C, *w = v + C, *pu = w + C, *pv = pu + C, *pw = pv + C, *s = pw + C, *ua = s + C, *va = ua + C,
          *wa = va + C, *uw = wa + C, *vw = uw + C, *ww = vw + C, *den = ww + C, *snap = den + C;
    float* pa = (float*)calloc((size_t)C * 2, sizeof(float));
    float* pb = pa + C;
    const float* p_final = pa;
    const float dt = q->dt;
    for (int step = 0; step < n_steps; ++step) {
        /* pass 0 */
        for (int idx = 0; idx < C; ++idx) {
            const int gz = idx / (nx * ny), rem = idx - gz * (nx * ny), gy = rem / nx, gx = rem - gy * nx;
            const int border = gx == 0 || gx == nx - 1 || gy == 0 || gy == ny - 1 || gz == 0 || gz == nz - 1;
            flags[idx] = border ? CELL_SOLID : 0u;
            s[idx] = border ? 0.0f : 1.0f;
            u[idx] = v[idx] = w[idx] = ua[idx] = va[idx] = wa[idx] = uw[idx] = vw[idx] = ww[idx] = den[idx] = 0.0f;
            pa[idx] = pb[idx] = 0.0f;
        }
        /* pass 1 */
        {
            const float min_dist = q->cell_size * 1.5f, min_dist2 = min_dist * min_dist;
            for (int sub = 0; sub < q->collision_substeps; ++sub) {
                const float* src = pos4;
                if (collision_mode == 1) {
                    memcpy(snap, pos4, (size_t)N * 4 * sizeof(float));
                    src = snap;
                }
                for (int i = 0; i < N; ++i) {
                    float px = src[4 * i], py = src[4 * i + 1], pz = src[4 * i + 2];
                    for (int j = 0; j < N; ++j) {
                        if (j == i) continue;
                        const float dx = px - src[4 * j], dy = py - src[4 * j + 1], dz = pz - src[4 * j + 2];
                        const float d2 = dx * dx + dy * dy + dz * dz;
                        if (d2 >= min_dist2 || d2 == 0.0f) continue;
                        const float d = sqrtf(d2);
                        const float f = 0.5f * (min_dist - d) / d;
                        px += dx * f; py += dy * f; pz += dz * f;
                    }
                    pos4[4 * i] = px; pos4[4 * i + 1] = py; pos4[4 * i + 2] = pz;
                }
            }
        }
        /* pass 2 */
        for (int i = 0; i < N; ++i) {
            const float* pos = pos4 + 4 * i;
            const float* pvel = vel4 + 4 * i;
            const stencil su = make_stencil(q, pos, 0.0f, 0.5f, 0.5f), sv = make_stencil(q, pos, 0.5f, 0.0f, 0.5f),
                          sw = make_stencil(q, pos, 0.5f, 0.5f, 0.0f);
            for (int iz = 0; iz <= 1; ++iz)
                for (int iy = 0; iy <= 1; ++iy)
                    for (int ix = 0; ix <= 1; ++ix) {
                        const float wu = corner_weight(&su, ix, iy, iz);
                        const int cu = corner_cell(q, &su, ix, iy, iz);
                        if ((flags[cu] & CELL_SOLID) == 0u) { ua[cu] += pvel[0] * wu; uw[cu] += wu; flags[cu] |= CELL_FLUID; }
                        const float wv = corner_weight(&sv, ix, iy, iz);
                        const int cv = corner_cell(q, &sv, ix, iy, iz);
                        if ((flags[cv] & CELL_SOLID) == 0u) { va[cv] += pvel[1] * wv; vw[cv] += wv; flags[cv] |= CELL_FLUID; }
                        const float wz = corner_weight(&sw, ix, iy, iz);
                        const int cw = corner_cell(q, &sw, ix, iy, iz);
                        if ((flags[cw] & CELL_SOLID) == 0u) { wa[cw] += pvel[2] * wz; ww[cw] += wz; flags[cw] |= CELL_FLUID; }
                    }
        }
        /* pass 3 */
        for (int idx = 0; idx < C; ++idx) {
            if ((flags[idx] & CELL_SOLID) == 0u) {
                const float eps = 1e-6f;
                u[idx] = uw[idx] > eps ? ua[idx] / uw[idx] : 0.0f;
                v[idx] = vw[idx] > eps ? va[idx] / vw[idx] : 0.0f;
                w[idx] = ww[idx] > eps ? wa[idx] / ww[idx] : 0.0f;
            } else {
                u[idx] = v[idx] = w[idx] = 0.0f;
            }
            pu[idx] = u[idx]; pv[idx] = v[idx]; pw[idx] = w[idx];
        }
        /* pass 4 */
        for (int i = 0; i < N; ++i) {
            const stencil sc = make_stencil(q, pos4 + 4 * i, 0.5f, 0.5f, 0.5f);
            for (int iz = 0; iz <= 1; ++iz)
                for (int iy = 0; iy <= 1; ++iy)
                    for (int ix = 0; ix <= 1; ++ix) {
                        const int c = corner_cell(q, &sc, ix, iy, iz);
                        if ((flags[c] & CELL_SOLID) == 0u) den[c] += corner_weight(&sc, ix, iy, iz) * q->mass;
                    }
        }
        /* pass 5 */
        float *p_read = pa, *p_write = pb;
        {
            int ping = 1;
            for (int it = 0; it < q->jacobi_iterations; ++it) {
                p_read = ping ? pa : pb;
                p_write = ping ? pb : pa;
                for (int idx = 0; idx < C; ++idx) {
                    const int gz = idx / (nx * ny), rem = idx - gz * (nx * ny), gy = rem / nx, gx = rem - gy * nx;
                    if (gx == 0 || gx == nx - 1 || gy == 0 || gy == ny - 1 || gz == 0 || gz == nz - 1 ||
                        (flags[idx] & CELL_FLUID) == 0u) {
                        p_write[idx] = p_read[idx];
                        continue;
                    }
                    const int left = idx - 1, right = idx + 1, bottom = idx - nx, top = idx + nx, back = idx - nx * ny,
                              front = idx + nx * ny;
                    const float sx0 = s[left], sx1 = s[right], sy0 = s[bottom], sy1 = s[top], sz0 = s[back], sz1 = s[front];
                    const float s_sum = sx0 + sx1 + sy0 + sy1 + sz0 + sz1;
                    if (s_sum <= 1e-9f) { p_write[idx] = p_read[idx]; continue; }
                    const float sum_p = sx0 * p_read[left] + sx1 * p_read[right] + sy0 * p_read[bottom] + sy1 * p_read[top] +
                                        sz0 * p_read[back] + sz1 * p_read[front];
                    float div = ((u[right] - u[idx]) + (v[top] - v[idx]) + (w[front] - w[idx]));
                    const float pd = den[idx];
                    if (q->rest_density > 0.0f && pd > 0.0f) {
                        const float compression = pd - q->rest_density;
                        if (compression > 0.0f) div -= compression;
                    }
                    const float dt_safe = fmaxf(dt, 1e-6f), cs_safe = fmaxf(q->cell_size, 1e-6f),
                                rd_safe = fmaxf(q->rest_density, 1e-6f);
                    const float cp = rd_safe * cs_safe * cs_safe / dt_safe;
                    const float div_safe = fminf(fmaxf(div, -1e6f), 1e6f);
                    const float p_new = (sum_p - cp * div_safe) / fmaxf(s_sum, 1e-6f);
                    p_write[idx] = p_read[idx] + q->over_relaxation * (p_new - p_read[idx]);
                }
                ping = !ping;
            }
        }
        /* pass 6: reads what the last iteration READ (its set is still bound) */
        {
            const float inv_cp = dt / (q->rest_density * q->cell_size);
            for (int idx = 0; idx < C; ++idx) {
                const int gz = idx / (nx * ny), rem = idx - gz * (nx * ny), gy = rem / nx, gx = rem - gy * nx;
                if (gx == 0 || gy == 0 || gz == 0 || gx >= nx - 1 || gy >= ny - 1 || gz >= nz - 1) continue;
                if ((flags[idx] & CELL_FLUID) == 0u) continue;
                const float p0 = p_read[idx];
                const int left = idx - 1, right = idx + 1, bot = idx - nx, top = idx + nx, back = idx - nx * ny,
                          front = idx + nx * ny;
                u[idx] = (flags[left] & CELL_SOLID) ? 0.0f : u[idx] - (p0 - p_read[left]) * inv_cp;
                v[idx] = (flags[bot] & CELL_SOLID) ? 0.0f : v[idx] - (p0 - p_read[bot]) * inv_cp;
                w[idx] = (flags[back] & CELL_SOLID) ? 0.0f : w[idx] - (p0 - p_read[back]) * inv_cp;
                if (flags[right] & CELL_SOLID) u[right] = 0.0f;
                if (flags[top] & CELL_SOLID) v[top] = 0.0f;
                if (flags[front] & CELL_SOLID) w[front] = 0.0f;
            }
        }
        /* pass 7 */
        {
            const float flip = fminf(fmaxf(q->damping, 0.0f), 1.0f);
            const float* grid[3] = {u, v, w};
            const float* prev[3] = {pu, pv, pw};
            const float off[3][3] = {{0.0f, 0.5f, 0.5f}, {0.5f, 0.0f, 0.5f}, {0.5f, 0.5f, 0.0f}};
            for (int i = 0; i < N; ++i) {
                float* pvel = vel4 + 4 * i;
                float nv[3] = {pvel[0], pvel[1], pvel[2]};
                for (int a = 0; a < 3; ++a) {
                    const stencil st = make_stencil(q, pos4 + 4 * i, off[a][0], off[a][1], off[a][2]);
                    float pic = 0.0f, fl = 0.0f, tw = 0.0f;
                    for (int iz = 0; iz <= 1; ++iz)
                        for (int iy = 0; iy <= 1; ++iy)
                            for (int ix = 0; ix <= 1; ++ix) {
                                const float wt = corner_weight(&st, ix, iy, iz);
                                const int c = corner_cell(q, &st, ix, iy, iz);
                                if (flags[c] & CELL_SOLID) continue;
                                const float val = grid[a][c];
                                pic += val * wt;
                                fl += (val - prev[a][c]) * wt;
                                tw += wt;
                            }
                    if (tw > 0.01f) {
                        pic /= tw; fl /= tw;
                        nv[a] = (1.0f - flip) * pic + flip * (pvel[a] + fl);
                    }
                }
                pvel[0] = nv[0]; pvel[1] = nv[1]; pvel[2] = nv[2];
            }
        }
        /* pass 8 */
        {
            const float restitution = 0.3f, friction = 0.9f, margin = q->cell_size;
            for (int i = 0; i < N; ++i) {
                float* pos = pos4 + 4 * i;
                float* vel = vel4 + 4 * i;
                float nv[3], np[3];
                for (int a = 0; a < 3; ++a) {
                    nv[a] = vel[a] + q->gravity[a] * dt;
                    np[a] = pos[a] + nv[a] * dt;
                }
                for (int a = 0; a < 3; ++a) {
                    const float lo = q->box_min[a] + margin, hi = q->box_max[a] - margin;
                    const int b = (a + 1) % 3, c = (a + 2) % 3;
                    /* the shader names the two other axes in x, y, z order; multiplication by the
                       same factor commutes, so the pair order does not matter */
                    if (np[a] < lo) { np[a] = lo; nv[a] = fabsf(nv[a]) * restitution; nv[b] *= friction; nv[c] *= friction; }
                    if (np[a] > hi) { np[a] = hi; nv[a] = -fabsf(nv[a]) * restitution; nv[b] *= friction; nv[c] *= friction; }
                }
                pos[0] = np[0]; pos[1] = np[1]; pos[2] = np[2]; pos[3] = 0.1f;
                vel[0] = nv[0]; vel[1] = nv[1]; vel[2] = nv[2];
            }
        }
        p_final = p_read;
    }
    for (int i = 0; i < C; ++i) {
        if (grid_u) grid_u[i] = u[i];
        if (grid_v) grid_v[i] = v[i];
        if (grid_w) grid_w[i] = w[i];
        if (pressure) pressure[i] = p_final[i];
        if (flags_out) flags_out[i] = flags[i];
        if (density_out) density_out[i] = den[i];
    }
    free(mem); free(flags); free(pa);
    return 0;
}
