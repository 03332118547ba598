/* CPU restatement of the reference engine's ray-traced frame, plain C.  TEST INFRASTRUCTURE: the
 * checker the CUDA path tracer is compared with; never on a product path.
 *
 * Follows NeonEngine/shaders/raygen.rgen:46-93 (PCG generator, jittered pinhole ray, rgba8 store),
 * closesthit.rchit:129-134 (generator), :136-140 (Schlick), :217-256 (cone sampling of a sphere light),
 * :259-594 (normal, emission, depth limit 3, diffuse/mirror blend with next-event estimation and a shadow
 * ray, textured and glass materials, the next ray as a tail call), miss.rmiss:21-27 (+0.1 x throughput),
 * shadow.rmiss:6-8.  The shaders' reservoir writes are left out (all rays write reservoir 0: raygen never
 * sets the index; nothing in the frame reads it).
 *
 * Pinned: oracle/_ref/libpt_ref.so is those four shaders themselves compiled for the CPU
 * (pt_ref_build.py); tests/test_pt_oracle.py requires this file's frames to equal its frames bit for bit
 * and keeps a committed fixture of its output for machines without the reference checkout.
 *
 * Conventions fixed where Vulkan leaves them open (same as include/neon_pt.h): front face = vertices
 * counter-clockwise from the ray origin; Moeller-Trumbore, tmin < t < tmax, equal t -> lower primitive;
 * normalize = v / sqrt(dot); fixed sin/cos polynomial on fused multiply-adds; pow(x,5) = x*x*x*x*x;
 * matrix x vector adds columns left to right; rgba8 = nearest-even(clamp * 255), NaN -> 0; textures
 * absent -> white.  Compile with -ffp-contract=off.  Traversal here is a brute-force-safe hierarchy of
 * its own (split by object median on x, y, z in turn): the closest hit does not depend on it. */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct { float x, y, z; } v3;
static v3 V(float x, float y, float z) { v3 r = {x, y, z}; return r; }
static v3 add(v3 a, v3 b) { return V(a.x + b.x, a.y + b.y, a.z + b.z); }
static v3 sub(v3 a, v3 b) { return V(a.x - b.x, a.y - b.y, a.z - b.z); }
static v3 mul(v3 a, v3 b) { return V(a.x * b.x, a.y * b.y, a.z * b.z); }
static v3 scl(v3 a, float s) { return V(a.x * s, a.y * s, a.z * s); }
static v3 dvs(v3 a, float s) { return V(a.x / s, a.y / s, a.z / s); }
static v3 neg(v3 a) { return V(-a.x, -a.y, -a.z); }
static float dot(v3 a, v3 b) { return a.x * b.x + a.y * b.y + a.z * b.z; }
static v3 cross(v3 a, v3 b) { return V(a.y * b.z - a.z * b.y, a.z * b.x - a.x * b.z, a.x * b.y - a.y * b.x); }
static float len(v3 a) { return sqrtf(dot(a, a)); }
static v3 nrm(v3 a) { return dvs(a, sqrtf(dot(a, a))); }
static v3 faceforward(v3 n, v3 i, v3 nref) { return dot(nref, i) < 0.0f ? n : neg(n); }
static v3 reflect(v3 i, v3 n) { return sub(i, scl(n, 2.0f * dot(n, i))); }
static v3 refract(v3 i, v3 n, float eta) {
    float d = dot(n, i), k = 1.0f - eta * eta * (1.0f - d * d);
    if (k < 0.0f) return V(0, 0, 0);
    return sub(scl(i, eta), scl(n, eta * d + sqrtf(k)));
}
static float mixf(float x, float y, float a) { return x * (1.0f - a) + y * a; }
static float clampf(float v, float lo, float hi) { return fminf(fmaxf(v, lo), hi); }

static void sincos_fixed(float x, float* sn, float* cs) {
    float kf = rintf(x * 0.636619747f);
    float r = fmaf(-kf, 1.57079625f, x);
    r = fmaf(-kf, 7.54978942e-08f, r);
    float s = r * r;
    float ps = fmaf(s, -1.95152959e-4f, 8.33216087e-3f);
    ps = fmaf(s, ps, -1.66666546e-1f);
    float sr = fmaf(r * s, ps, r);
    float pc = fmaf(s, 2.44331571e-5f, -1.38873163e-3f);
    pc = fmaf(s, pc, 4.16666457e-2f);
    float cr = fmaf(s * s, pc, fmaf(s, -0.5f, 1.0f));
    int q = (int)kf & 3;
    float a = (q & 1) ? cr : sr, b = (q & 1) ? sr : cr;
    *sn = (q & 2) ? -a : a;
    *cs = ((q + 1) & 2) ? -b : b;
}

static float rng(uint32_t* seed) {
    *seed = *seed * 747796405u + 2891336453u;
    uint32_t r = ((*seed >> ((*seed >> 28u) + 4u)) ^ *seed) * 277803737u;
    r = (r >> 22u) ^ r;
    return (float)r / 4294967296.0f; /* the shader's 4294967295.0 is this float */
}

typedef struct { float pos[4], normal[4], uv[4]; uint32_t material, pad[3]; } vertex;
typedef struct { float emission[4], albedo[4], position[4], misc[4]; } material;
typedef struct { float lo[3], hi[3]; int left, count; } node;

static const vertex* g_v;
static const uint32_t* g_i;
static const material* g_m;
static node* g_nodes;
static int g_n_nodes, *g_order, g_axis;
static unsigned long long g_rays;

static v3 vpos(int t, int c) { const float* p = g_v[g_i[3 * t + c]].pos; return V(p[0], p[1], p[2]); }
static float centroid(int t, int a) {
    return g_v[g_i[3 * t]].pos[a] + g_v[g_i[3 * t + 1]].pos[a] + g_v[g_i[3 * t + 2]].pos[a];
}
static int cmp_axis(const void* pa, const void* pb) {
    int a = *(const int*)pa, b = *(const int*)pb;
    float ka = centroid(a, g_axis), kb = centroid(b, g_axis);
    return ka < kb ? -1 : ka > kb ? 1 : (a < b ? -1 : a > b);
}
static void build(int nd, int first, int count, int depth) {
    node* n = &g_nodes[nd];
    for (int a = 0; a < 3; ++a) { n->lo[a] = INFINITY; n->hi[a] = -INFINITY; }
    for (int i = first; i < first + count; ++i)
        for (int c = 0; c < 3; ++c)
            for (int a = 0; a < 3; ++a) {
                float p = g_v[g_i[3 * g_order[i] + c]].pos[a];
                n->lo[a] = fminf(n->lo[a], p);
                n->hi[a] = fmaxf(n->hi[a], p);
            }
    for (int a = 0; a < 3; ++a) {
        float pad = 3e-5f * fmaxf(1.0f, fmaxf(fabsf(n->lo[a]), fabsf(n->hi[a])));
        n->lo[a] -= pad;
        n->hi[a] += pad;
    }
    if (count <= 3) { n->left = first; n->count = count; return; }
    g_axis = depth % 3;
    qsort(g_order + first, (size_t)count, sizeof(int), cmp_axis);
    int left = g_n_nodes, mid = count / 2;
    g_n_nodes += 2;
    n->left = left;
    n->count = 0;
    build(left, first, mid, depth + 1);
    build(left + 1, first + mid, count - mid, depth + 1);
}

static int tri_hit(int t, v3 o, v3 d, int cull, float tmin, float* tt, float* uu, float* vv) {
    v3 v0 = vpos(t, 0), e1 = sub(vpos(t, 1), v0), e2 = sub(vpos(t, 2), v0);
    v3 pv = cross(d, e2);
    float det = dot(e1, pv);
    if (cull ? !(det > 0.0f) : det == 0.0f) return 0;
    float inv = 1.0f / det;
    v3 tv = sub(o, v0);
    *uu = dot(tv, pv) * inv;
    if (!(*uu >= 0.0f && *uu <= 1.0f)) return 0;
    v3 qv = cross(tv, e1);
    *vv = dot(d, qv) * inv;
    if (!(*vv >= 0.0f && *uu + *vv <= 1.0f)) return 0;
    *tt = dot(e2, qv) * inv;
    return *tt > tmin;
}

typedef struct { float t, u, v; int prim; } hit;

static int trace(v3 o, v3 d, float tmin, float tmax, int cull, int any, hit* h) {
    ++g_rays;
    float inv[3] = {1.0f / d.x, 1.0f / d.y, 1.0f / d.z}, oo[3] = {o.x, o.y, o.z};
    int stack[128], sp = 0, found = 0, best_prim = 0x7fffffff;
    float best = tmax;
    stack[sp++] = 0;
    while (sp) {
        const node* n = &g_nodes[stack[--sp]];
        float lo = -INFINITY, hi = INFINITY;
        for (int a = 0; a < 3; ++a) {
            float t0 = (n->lo[a] - oo[a]) * inv[a], t1 = (n->hi[a] - oo[a]) * inv[a];
            lo = fmaxf(lo, fminf(t0, t1));
            hi = fminf(hi, fmaxf(t0, t1));
        }
        if (!(fmaxf(lo, tmin) <= fminf(hi, best))) continue;
        if (!n->count) { stack[sp++] = n->left; stack[sp++] = n->left + 1; continue; }
        for (int i = 0; i < n->count; ++i) {
            int t = g_order[n->left + i];
            float tt, uu, vv;
            if (!tri_hit(t, o, d, cull, tmin, &tt, &uu, &vv) || !(tt < tmax)) continue;
            if (tt < best || (tt == best && found && t < best_prim)) {
                best = tt; best_prim = t; found = 1;
                h->t = tt; h->u = uu; h->v = vv; h->prim = t;
                if (any) return 1;
            }
        }
    }
    return found;
}

static v3 sample_light(const material* l, v3 p, uint32_t* seed, v3* ldir, float* pdf) {
    v3 lpos = V(l->position[0], l->position[1], l->position[2]);
    float radius = l->position[3];
    float dist = len(sub(lpos, p));
    float sin2 = (radius * radius) / (dist * dist);
    float cos_max = sqrtf(fmaxf(0.0f, 1.0f - sin2));
    float r1 = rng(seed), r2 = rng(seed);
    float cos_t = 1.0f - r1 * (1.0f - cos_max);
    float sin_t = sqrtf(fmaxf(0.0f, 1.0f - cos_t * cos_t));
    float phi = 2.0f * 3.14159265f * r2;
    v3 to = nrm(sub(lpos, p));
    v3 tan = fabsf(to.x) > fabsf(to.y) ? nrm(V(-to.z, 0, to.x)) : nrm(V(0, to.z, -to.y));
    v3 bit = cross(to, tan);
    float sp, cp;
    sincos_fixed(phi, &sp, &cp);
    *ldir = nrm(add(add(scl(tan, sin_t * cp), scl(bit, sin_t * sp)), scl(to, cos_t)));
    *pdf = 1.0f / (2.0f * 3.14159265f * (1.0f - cos_max));
    return V(l->emission[0], l->emission[1], l->emission[2]);
}

static uint8_t unorm8(float v) {
    if (!(v == v)) return 0;
    return (uint8_t)rintf(fminf(fmaxf(v, 0.0f), 1.0f) * 255.0f);
}

static void matvec(const float* m, float x, float y, float z, float w, float* out) {
    for (int r = 0; r < 4; ++r) out[r] = ((m[r] * x + m[4 + r] * y) + m[8 + r] * z) + m[12 + r] * w;
}

unsigned long long pt_oracle_render(const void* vertices, int n_vertices, const uint32_t* indices, int n_indices, const void* materials,
                                    int n_materials, int n_lights, const float* inv_proj, const float* inv_view, float frame_id,
                                    int width, int height, uint8_t* image) {
    (void)n_vertices; (void)n_materials;
    g_v = (const vertex*)vertices;
    g_i = indices;
    g_m = (const material*)materials;
    int n_tri = n_indices / 3;
    g_order = (int*)malloc(sizeof(int) * (size_t)n_tri);
    g_nodes = (node*)malloc(sizeof(node) * (2 * (size_t)n_tri + 2));
    for (int i = 0; i < n_tri; ++i) g_order[i] = i;
    g_n_nodes = 1;
    build(0, 0, n_tri, 0);
    g_rays = 0;
    for (int py = 0; py < height; ++py)
        for (int px = 0; px < width; ++px) {
            float ux = ((float)px + 0.5f) / (float)width, uy = ((float)py + 0.5f) / (float)height;
            float o4[4], tg[4], d4[4];
            matvec(inv_view, 0, 0, 0, 1, o4);
            uint32_t seed = (uint32_t)((float)(px * 1973 + py * 9277) + frame_id * 26699.0f) | 1u;
            float r1 = rng(&seed), r2 = rng(&seed);
            float jx = (r1 - 0.5f) / (float)width, jy = (r2 - 0.5f) / (float)height;
            float dx = (ux + jx * 2.0f) * 2.0f - 1.0f, dy = (uy + jy * 2.0f) * 2.0f - 1.0f;
            matvec(inv_proj, dx, dy, 1, 1, tg);
            v3 tn = nrm(V(tg[0], tg[1], tg[2]));
            matvec(inv_view, tn.x, tn.y, tn.z, 0, d4);
            v3 origin = V(o4[0], o4[1], o4[2]), dir = V(d4[0], d4[1], d4[2]);
            v3 color = V(0, 0, 0), thr = V(1, 1, 1);
            uint32_t depth = 0, mat_type = 0;
            for (;;) {
                hit h;
                if (!trace(origin, dir, 0.001f, 10000.0f, 1, 0, &h)) { color = add(color, mul(thr, V(0.1f, 0.1f, 0.1f))); break; }
                float b0 = 1.0f - h.u - h.v;
                const vertex *v0 = &g_v[g_i[3 * h.prim]], *v1 = &g_v[g_i[3 * h.prim + 1]], *v2 = &g_v[g_i[3 * h.prim + 2]];
                v3 normal = nrm(add(add(scl(V(v0->normal[0], v0->normal[1], v0->normal[2]), b0), scl(V(v1->normal[0], v1->normal[1], v1->normal[2]), h.u)),
                                    scl(V(v2->normal[0], v2->normal[1], v2->normal[2]), h.v)));
                normal = faceforward(normal, dir, normal);
                const material* mat = &g_m[v0->material];
                v3 emission = V(mat->emission[0], mat->emission[1], mat->emission[2]);
                if (len(emission) > 0.0f) {
                    if (depth == 0u || mat_type == 1u) color = add(color, mul(thr, emission));
                    break;
                }
                if (depth >= 3u) break;
                if (depth > 2u) {
                    float q = fmaxf(0.05f, 1.0f - fmaxf(thr.x, fmaxf(thr.y, thr.z)));
                    if (rng(&seed) < q) break;
                    thr = dvs(thr, 1.0f - q);
                }
                ++depth;
                int type = (int)mat->misc[2];
                v3 new_dir = V(0, 0, 0), offset_pos = V(0, 0, 0);
                if (type == 0 || type == 2) {
                    normal = faceforward(normal, dir, normal);
                    offset_pos = add(add(origin, scl(dir, h.t)), scl(normal, 0.001f));
                    float q1 = rng(&seed), q2 = rng(&seed);
                    float r = sqrtf(q1), theta = 2.0f * 3.14159265f * q2;
                    v3 tan = fabsf(normal.x) > fabsf(normal.y) ? nrm(V(-normal.z, 0, normal.x)) : nrm(V(0, normal.z, -normal.y));
                    v3 bit = cross(normal, tan);
                    float st, ct;
                    sincos_fixed(theta, &st, &ct);
                    v3 diffuse = nrm(add(add(scl(tan, r * ct), scl(bit, r * st)), scl(normal, sqrtf(1.0f - q1))));
                    v3 specular = reflect(nrm(dir), normal);
                    float rough = clampf(mat->misc[0], 0.0f, 1.0f);
                    new_dir = nrm(V(mixf(specular.x, diffuse.x, rough), mixf(specular.y, diffuse.y, rough), mixf(specular.z, diffuse.z, rough)));
                    const material* light = &g_m[(int)(rng(&seed) * (float)n_lights)];
                    float pick = 1.0f / (float)n_lights, lpdf;
                    v3 ldir;
                    v3 Le = sample_light(light, offset_pos, &seed, &ldir, &lpdf);
                    float cos_t = dot(normal, ldir);
                    v3 albedo = type == 0 ? V(mat->albedo[0], mat->albedo[1], mat->albedo[2]) : V(1, 1, 1);
                    if (cos_t > 0.0f && lpdf > 0.0f) {
                        float sd = len(sub(V(light->position[0], light->position[1], light->position[2]), offset_pos)) - light->position[3] - 0.01f;
                        hit sh;
                        if (!trace(offset_pos, ldir, 0.001f, sd, 0, 1, &sh)) {
                            v3 brdf = scl(albedo, 0.3183098861837907f);
                            color = add(color, dvs(scl(mul(mul(thr, brdf), Le), cos_t), lpdf * pick));
                        }
                    }
                    thr = mul(thr, albedo);
                    mat_type = type == 0 ? 0u : 2u;
                } else if (type == 67) {
                    offset_pos = add(add(origin, scl(dir, h.t)), scl(normal, 0.001f));
                    v3 incoming = nrm(dir);
                    float cos_t = clampf(dot(neg(incoming), normal), 0.0f, 1.0f);
                    int entering = cos_t > 0.0f;
                    float ior = mat->misc[1], eta = entering ? (1.0f / ior) : ior;
                    v3 nn = entering ? normal : neg(normal);
                    float r0 = (1.0f - ior) / (1.0f + ior);
                    r0 = r0 * r0;
                    float m1 = 1.0f - cos_t;
                    float F = r0 + (1.0f - r0) * (m1 * m1 * m1 * m1 * m1);
                    if (rng(&seed) < F) new_dir = reflect(incoming, nn);
                    else {
                        new_dir = refract(incoming, nn, eta);
                        if (len(new_dir) < 0.001f) new_dir = reflect(incoming, nn);
                    }
                    mat_type = 1u;
                }
                origin = offset_pos;
                dir = new_dir;
            }
            uint8_t* out = image + ((size_t)py * width + px) * 4;
            out[0] = unorm8(color.x); out[1] = unorm8(color.y); out[2] = unorm8(color.z); out[3] = 255;
        }
    free(g_order);
    free(g_nodes);
    return g_rays;
}
