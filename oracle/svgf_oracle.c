/*
 * svgf_oracle.c - CPU restatement of the reference engine's denoiser: temporal accumulation
 * (NeonEngine/shaders/raytracing_pp.comp:35-247) and the edge-avoiding a-trous filter
 * (NeonEngine/shaders/raytracing_atrous.comp:59-160), scheduled per frame as
 * NeonEngine/src/raytracing_app.cpp:735-765 and NeonEngine/src/raytracing_rast.cpp:325-428 do.
 *
 * TEST INFRASTRUCTURE ONLY: the checker of the CUDA kernels, never the thing shipped or measured.
 * Pinned against the reference's own shaders compiled for the CPU (oracle/svgf_ref_build.py):
 * with serial = 1 this file reproduces them bit for bit (tests/test_svgf_oracle.py).
 *
 * The shaders as shipped begin with `return;` (the denoiser is switched off in the checkout);
 * this file restates the bodies behind that statement.
 *
 * serial = 1: pixels in ascending (y, x), the moments image updated in place, so a pixel sees the
 *             new moments of the pixels before it (the CPU-compiled shaders' behaviour);
 * serial = 0: every pass reads the moments image as it was when the pass started (the rule the
 *             CUDA kernels implement; on a GPU the shader's in-place update is a data race).
 *
 * Storage conversions and exp2 as in oracle/svgf_ref_build.py: rgba16f round to nearest even,
 * rgba8 = nearest-even(clamp(v, 0, 1) * 255) with NaN -> 0, exp2 = the fixed degree-7 polynomial.
 * Compile with -ffp-contract=off.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct { float x, y, z; } v3;

static float dot3(v3 a, v3 b) { return a.x * b.x + a.y * b.y + a.z * b.z; }
static float len3(v3 a) { return sqrtf(a.x * a.x + a.y * a.y + a.z * a.z); }
static v3 sub3(v3 a, v3 b) { v3 r = {a.x - b.x, a.y - b.y, a.z - b.z}; return r; }
static float fmax_glsl(float a, float b) { return a < b ? b : a; }
static float fmin_glsl(float a, float b) { return b < a ? b : a; }
static float mixf(float x, float y, float a) { return x * (1.0f - a) + y * a; }

static float exp2_poly(float x) {
    if (x != x) return x;
    if (x >= 128.0f) return INFINITY;
    if (!(x > -126.0f)) return 0.0f;
    const float n = nearbyintf(x), f = x - n;
    float p = 1.5252734e-5f;
    p = fmaf(p, f, 1.5403530e-4f);
    p = fmaf(p, f, 1.3333558e-3f);
    p = fmaf(p, f, 9.6181291e-3f);
    p = fmaf(p, f, 5.5504109e-2f);
    p = fmaf(p, f, 2.4022651e-1f);
    p = fmaf(p, f, 6.9314718e-1f);
    p = fmaf(p, f, 1.0f);
    const uint32_t bits = (uint32_t)((int)n + 127) << 23;
    float scale;
    memcpy(&scale, &bits, 4);
    return p * scale;
}

float svgf_oracle_exp2(float x) { return exp2_poly(x); }

static uint8_t to_unorm8(float v) {
    if (v != v) v = 0.0f;
    v = v < 0.0f ? 0.0f : (v > 1.0f ? 1.0f : v);
    return (uint8_t)nearbyintf(v * 255.0f);
}

static v3 load_rgb8(const uint8_t* im, int w, int x, int y) {
    const uint8_t* d = im + ((size_t)y * w + x) * 4;
    v3 r = {d[0] / 255.0f, d[1] / 255.0f, d[2] / 255.0f};
    return r;
}
static void store_rgb8(uint8_t* im, int w, int x, int y, v3 c) {
    uint8_t* d = im + ((size_t)y * w + x) * 4;
    d[0] = to_unorm8(c.x); d[1] = to_unorm8(c.y); d[2] = to_unorm8(c.z); d[3] = 255;
}
static v3 load_rgb16(const _Float16* im, int w, int x, int y) {
    const _Float16* d = im + ((size_t)y * w + x) * 4;
    v3 r = {(float)d[0], (float)d[1], (float)d[2]};
    return r;
}
static void store_rgba16(_Float16* im, int w, int x, int y, v3 c, float a) {
    _Float16* d = im + ((size_t)y * w + x) * 4;
    d[0] = (_Float16)c.x; d[1] = (_Float16)c.y; d[2] = (_Float16)c.z; d[3] = (_Float16)a;
}
static v3 load_xyz(const float* im, int w, int x, int y) {
    const float* d = im + ((size_t)y * w + x) * 4;
    v3 r = {d[0], d[1], d[2]};
    return r;
}

typedef struct {
    int w, h;
    const float *pos, *nrm, *bary, *mot;
} GBuffer;

/* raytracing_pp.comp:35-140 (LoadPreviousData): bilinear fetch of the history at the reprojected
 * position, each tap validated against the current pixel's surface. */
static int load_previous(const GBuffer* g, int px, int py, const _Float16* hist, const float* data_in, v3* prev_colour,
                         float* history_length, float prev_moments[2]) {
    const int w = g->w, h = g->h;
    prev_colour->x = prev_colour->y = prev_colour->z = 0.0f;
    *history_length = 0.0f;
    prev_moments[0] = prev_moments[1] = 0.0f;
    const v3 cur_pos = load_xyz(g->pos, w, px, py), cur_nrm = load_xyz(g->nrm, w, px, py), cur_bary = load_xyz(g->bary, w, px, py);
    const int cur_mesh = (int)roundf(g->nrm[((size_t)py * w + px) * 4 + 3]);
    if (dot3(cur_pos, cur_pos) < 1e-6f) return 0;
    const float mx = g->mot[((size_t)py * w + px) * 4], my = g->mot[((size_t)py * w + px) * 4 + 1];
    const float uvx = ((float)px + 0.5f) / (float)w, uvy = ((float)py + 0.5f) / (float)h;
    const float pux = uvx - mx, puy = uvy - my;
    if (pux < 0.0f || puy < 0.0f || pux > 1.0f || puy > 1.0f) return 0;
    const float ppx = pux * (float)w - 0.5f, ppy = puy * (float)h - 0.5f;
    const int bx = (int)floorf(ppx), by = (int)floorf(ppy);
    const float fx = ppx - floorf(ppx), fy = ppy - floorf(ppy);
    const float weights[4] = {(1.0f - fx) * (1.0f - fy), fx * (1.0f - fy), (1.0f - fx) * fy, fx * fy};
    const float dist = len3(cur_pos);
    const float pos_threshold = fmax_glsl(0.01f * dist, 0.005f);
    v3 acc_c = {0.0f, 0.0f, 0.0f};
    float acc_h = 0.0f, acc_m0 = 0.0f, acc_m1 = 0.0f, acc_w = 0.0f;
    for (int i = 0; i < 4; ++i) {
        const int tx = bx + (i & 1), ty = by + (i >> 1);
        if (tx < 0 || ty < 0 || tx >= w || ty >= h) continue;
        const v3 tap_pos = load_xyz(g->pos, w, tx, ty), tap_nrm = load_xyz(g->nrm, w, tx, ty), tap_bary = load_xyz(g->bary, w, tx, ty);
        const int tap_mesh = (int)roundf(g->nrm[((size_t)ty * w + tx) * 4 + 3]);
        if (dot3(tap_pos, tap_pos) < 1e-6f) continue;
        if (cur_mesh != tap_mesh) continue;
        const float cur_depth = len3(cur_pos), tap_depth = len3(tap_pos);
        if (fabsf(cur_depth - tap_depth) > 0.02f * cur_depth) continue;
        if (len3(sub3(cur_pos, tap_pos)) > pos_threshold) continue;
        if (dot3(cur_nrm, tap_nrm) < 0.9f) continue;
        if (len3(sub3(cur_bary, tap_bary)) > 0.2f) continue;
        const float wt = weights[i];
        const v3 hc = load_rgb16(hist, w, tx, ty);
        acc_c.x += hc.x * wt; acc_c.y += hc.y * wt; acc_c.z += hc.z * wt;
        const float* td = data_in + ((size_t)ty * w + tx) * 4;
        acc_h += td[0] * wt;
        acc_m0 += td[1] * wt;
        acc_m1 += td[2] * wt;
        acc_w += wt;
    }
    if (acc_w < 0.5f) return 0;
    const float inv = 1.0f / acc_w;
    prev_colour->x = acc_c.x * inv; prev_colour->y = acc_c.y * inv; prev_colour->z = acc_c.z * inv;
    *history_length = acc_h * inv;
    prev_moments[0] = acc_m0 * inv;
    prev_moments[1] = acc_m1 * inv;
    return 1;
}

/* raytracing_pp.comp:141-247 (main, mode 5): blends the new sample into the history. */
static void temporal_pass(const GBuffer* g, uint8_t* image, const _Float16* hist_prev, _Float16* hist_next, const float* data_in,
                          float* data_out) {
    const int w = g->w, h = g->h;
    for (int y = 0; y < h; ++y)
        for (int x = 0; x < w; ++x) {
            const v3 cur = load_rgb8(image, w, x, y);
            v3 prev;
            float hl, pm[2];
            const int ok = load_previous(g, x, y, hist_prev, data_in, &prev, &hl, pm);
            float alpha;
            if (ok) {
                hl = hl + 1.0f;
                alpha = 1.0f / hl;
                alpha = fmin_glsl(fmax_glsl(alpha, 0.0f), 1.0f);
            } else {
                alpha = 1.0f;
                hl = 1.0f;
            }
            const v3 bp = ok ? prev : cur;
            const v3 nc = {mixf(bp.x, cur.x, alpha), mixf(bp.y, cur.y, alpha), mixf(bp.z, cur.z, alpha)};
            float m0 = 0.2126f * cur.x + 0.7152f * cur.y + 0.0722f * cur.z;
            float m1 = m0 * m0;
            m0 = mixf(pm[0], m0, alpha);
            m1 = mixf(pm[1], m1, alpha);
            const float variance = fmax_glsl(0.0f, m1 - m0 * m0);
            store_rgba16(hist_next, w, x, y, nc, 1.0f);
            float* d = data_out + ((size_t)y * w + x) * 4;
            d[0] = hl; d[1] = m0; d[2] = m1; d[3] = variance;
            store_rgb8(image, w, x, y, nc);
        }
}

/* raytracing_atrous.comp:59-160 for iteration < 98: 5x5 taps `1 << iteration` pixels apart,
 * weighted by the B3 kernel, normal^128, depth and luminance; colour goes to the rgba8 image, the
 * filtered variance back into the moments image. */
static void atrous_pass(const GBuffer* g, int iteration, uint8_t* image, const _Float16* colour, const float* data_in, float* data_out) {
    static const float k1d[5] = {1.0f, 4.0f, 6.0f, 4.0f, 1.0f};
    const float inv256 = 1.0f / 256.0f, log2e = 1.4426950408889634f, eps = 1e-6f;
    const int w = g->w, h = g->h, step = 1 << iteration;
    const float step_f = (float)step;
    for (int y = 0; y < h; ++y)
        for (int x = 0; x < w; ++x) {
            const v3 c_pos = load_xyz(g->pos, w, x, y), c_nrm = load_xyz(g->nrm, w, x, y);
            const float* cd = data_in + ((size_t)y * w + x) * 4;
            const float cd0 = cd[0], cd1 = cd[1], cd2 = cd[2], cd3 = cd[3];
            float* od = data_out + ((size_t)y * w + x) * 4;
            if (dot3(c_pos, c_pos) < eps) {  /* no surface: colour passes through, moments untouched */
                store_rgb8(image, w, x, y, load_rgb16(colour, w, x, y));
                od[0] = cd0; od[1] = cd1; od[2] = cd2; od[3] = cd3;
                continue;
            }
            const float c_lum = cd1, c_var = fmax_glsl(cd3, 0.0f);
            const float inv_z = 1.0f / fmax_glsl(fabsf(c_pos.z) * step_f, eps);
            const float inv_l = 1.0f / fmax_glsl(1.0f * sqrtf(fmax_glsl(c_var, 1e-10f)), eps);
            v3 sum_c = {0.0f, 0.0f, 0.0f};
            float sum_w = 0.0f, sum_var = 0.0f, sum_wvar = 0.0f;
            for (int yy = -2; yy <= 2; ++yy)
                for (int xx = -2; xx <= 2; ++xx) {
                    int qx = x + xx * step, qy = y + yy * step;
                    qx = qx < 0 ? 0 : (qx > w - 1 ? w - 1 : qx);
                    qy = qy < 0 ? 0 : (qy > h - 1 ? h - 1 : qy);
                    const float wk = k1d[xx + 2] * k1d[yy + 2] * inv256;
                    if (wk == 0.0f) continue;
                    const v3 s_nrm = load_xyz(g->nrm, w, qx, qy);
                    float wn = fmax_glsl(dot3(c_nrm, s_nrm), 0.0f);
                    for (int r = 0; r < 7; ++r) wn *= wn;
                    if (wn <= eps) continue;
                    const v3 s_pos = load_xyz(g->pos, w, qx, qy);
                    const float* sd = data_in + ((size_t)qy * w + qx) * 4;
                    const v3 s_col = load_rgb16(colour, w, qx, qy);
                    const float s_lum = sd[1], s_var = fmax_glsl(sd[3], 0.0f);
                    const float dz = fabsf(c_pos.z - s_pos.z);
                    const float wd = exp2_poly(-dz * inv_z * log2e);
                    const float dl = fabsf(c_lum - s_lum);
                    const float wl = exp2_poly(-dl * inv_l * log2e);
                    const float wt = wk * wn * wd * wl;
                    sum_c.x += s_col.x * wt; sum_c.y += s_col.y * wt; sum_c.z += s_col.z * wt;
                    sum_w += wt;
                    const float w2 = wt * wt;
                    sum_var += s_var * w2;
                    sum_wvar += w2;
                }
            const float inv_w = 1.0f / fmax_glsl(sum_w, eps), inv_wv = 1.0f / fmax_glsl(sum_wvar, eps);
            const v3 fc = {sum_c.x * inv_w, sum_c.y * inv_w, sum_c.z * inv_w};
            store_rgb8(image, w, x, y, fc);
            od[0] = cd0; od[1] = cd1; od[2] = cd2; od[3] = sum_var * inv_wv;
        }
}

/* raytracing_atrous.comp:66-70 (iteration 98): the rgba8 image is copied into a history image. */
static void copy_pass(int w, int h, const uint8_t* image, _Float16* dst) {
    for (size_t i = 0; i < (size_t)w * h * 4; ++i) dst[i] = (_Float16)(image[i] / 255.0f);
}

/* One frame.  colour_a / colour_b: the two rgba16f history images; data: the rgba32f moments image
 * {history length, first moment, second moment, variance}; *ping_pong: RayTracingRast::pingPong. */
int svgf_oracle_frame(int w, int h, const float* position, const float* normal, const float* bary, const float* motion,
                      uint8_t* image, uint16_t* colour_a, uint16_t* colour_b, float* data, int* ping_pong, int atrous_iterations,
                      int serial) {
    const GBuffer g = {w, h, position, normal, bary, motion};
    const size_t n = (size_t)w * h * 4;
    float* scratch = serial ? NULL : (float*)malloc(n * sizeof(float));
    if (!serial && !scratch) return -1;
    _Float16 *a = (_Float16*)colour_a, *b = (_Float16*)colour_b;
    /* set 1 binds {5: a, 7: b}, set 2 binds {5: b, 7: a}; the temporal pass takes set 1 when the flag is set */
    _Float16* prev = *ping_pong ? a : b;
    _Float16* next = *ping_pong ? b : a;
    *ping_pong = !*ping_pong;
#define RUN(call_in_place, call_snapshot)                  \
    do {                                                   \
        if (serial) { call_in_place; }                     \
        else { call_snapshot; memcpy(data, scratch, n * sizeof(float)); } \
    } while (0)
    RUN(temporal_pass(&g, image, prev, next, data, data), temporal_pass(&g, image, prev, next, data, scratch));
    /* the a-trous passes start on the set whose binding 5 is the image the temporal pass wrote */
    for (int i = 0; i < atrous_iterations; ++i) {
        const _Float16* src = (i % 2 == 0) ? next : prev;
        RUN(atrous_pass(&g, i, image, src, data, data), atrous_pass(&g, i, image, src, data, scratch));
    }
    if (atrous_iterations % 2 == 0) RUN(atrous_pass(&g, 0, image, prev, data, data), atrous_pass(&g, 0, image, prev, data, scratch));
    copy_pass(w, h, image, prev);
#undef RUN
    free(scratch);
    return 0;
}
