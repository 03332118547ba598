// The reference engine's ray-traced frame (raygen.rgen + closesthit.rchit + miss.rmiss + shadow.rmiss)
// as one CUDA kernel over a software bounding-volume hierarchy; C ABI in include/neon_pt.h.
// Compiled without fused multiply-add contraction: every float operation is the one the header's
// conventions name, so a CPU implementation of the same conventions gives the same bits.
#include "../../include/neon_pt.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>
#include <string>
#include <vector>

namespace {

thread_local std::string g_pt_create_error;

// ---- small vector vocabulary -----------------------------------------------------------------------
struct V3 {
    float x, y, z;
};
__host__ __device__ inline V3 v3(float x, float y, float z) { return V3{x, y, z}; }
__host__ __device__ inline V3 operator+(V3 a, V3 b) { return v3(a.x + b.x, a.y + b.y, a.z + b.z); }
__host__ __device__ inline V3 operator-(V3 a, V3 b) { return v3(a.x - b.x, a.y - b.y, a.z - b.z); }
__host__ __device__ inline V3 operator*(V3 a, V3 b) { return v3(a.x * b.x, a.y * b.y, a.z * b.z); }
__host__ __device__ inline V3 operator*(V3 a, float s) { return v3(a.x * s, a.y * s, a.z * s); }
__host__ __device__ inline V3 operator/(V3 a, float s) { return v3(a.x / s, a.y / s, a.z / s); }
__host__ __device__ inline V3 neg(V3 a) { return v3(-a.x, -a.y, -a.z); }
__host__ __device__ inline float dot3(V3 a, V3 b) { return a.x * b.x + a.y * b.y + a.z * b.z; }
__host__ __device__ inline V3 cross3(V3 a, V3 b) { return v3(a.y * b.z - a.z * b.y, a.z * b.x - a.x * b.z, a.x * b.y - a.y * b.x); }
__device__ inline float length3(V3 a) { return sqrtf(dot3(a, a)); }
__device__ inline V3 normalize3(V3 a) { return a / sqrtf(dot3(a, a)); }
__device__ inline V3 faceforward3(V3 n, V3 i, V3 nref) { return dot3(nref, i) < 0.f ? n : neg(n); }
__device__ inline V3 reflect3(V3 i, V3 n) { return i - n * (2.f * dot3(n, i)); }
__device__ inline V3 refract3(V3 i, V3 n, float eta) {
    const float d = dot3(n, i);
    const float k = 1.f - eta * eta * (1.f - d * d);
    if (k < 0.f) return v3(0.f, 0.f, 0.f);
    return i * eta - n * (eta * d + sqrtf(k));
}
__device__ inline float mixf(float x, float y, float a) { return x * (1.f - a) + y * a; }
__device__ inline V3 mix3(V3 x, V3 y, float a) { return v3(mixf(x.x, y.x, a), mixf(x.y, y.y, a), mixf(x.z, y.z, a)); }
__device__ inline float clampf(float v, float lo, float hi) { return fminf(fmaxf(v, lo), hi); }

// sin and cos by a two-step Cody-Waite reduction to [-pi/4, pi/4] and fixed polynomials evaluated with
// fused multiply-adds (each a single correctly rounded operation on every machine).
__device__ inline void sincos_fixed(float x, float* sn, float* cs) {
    const float kf = rintf(x * 0.636619747f);
    float r = fmaf(-kf, 1.57079625f, x);
    r = fmaf(-kf, 7.54978942e-08f, r);
    const float s = r * r;
    float ps = fmaf(s, -1.95152959e-4f, 8.33216087e-3f);
    ps = fmaf(s, ps, -1.66666546e-1f);
    const float sr = fmaf(r * s, ps, r);
    float pc = fmaf(s, 2.44331571e-5f, -1.38873163e-3f);
    pc = fmaf(s, pc, 4.16666457e-2f);
    const float cr = fmaf(s * s, pc, fmaf(s, -0.5f, 1.f));
    const int q = (int)kf & 3;
    const float a = (q & 1) ? cr : sr, b = (q & 1) ? sr : cr;
    *sn = (q & 2) ? -a : a;
    *cs = ((q + 1) & 2) ? -b : b;
}

// PCG step + output permutation of the shaders (raygen.rgen:46-51, closesthit.rchit:129-134).
__device__ inline float rng_next(uint32_t& seed) {
    seed = seed * 747796405u + 2891336453u;
    uint32_t result = ((seed >> ((seed >> 28u) + 4u)) ^ seed) * 277803737u;
    result = (result >> 22u) ^ result;
    return (float)result / 4294967296.0f;  // the shader's literal 4294967295.0 is this float
}

// ---- bounding-volume hierarchy -------------------------------------------------------------------------
struct BvhNode {
    float bmin[3];
    int left;   // inner node: index of the first child (second = left + 1); leaf: first triangle in the order array
    float bmax[3];
    int count;  // 0 = inner node, else number of triangles of the leaf
};

struct Tri {     // a triangle prepared for the intersection test
    float v0[3], e1[3], e2[3];
    int prim;    // primitive index in the caller's index buffer
};

struct Scene {
    const BvhNode* nodes;
    const Tri* tris;
    const neon_pt_vertex* verts;
    const uint32_t* indices;
    const neon_pt_material* mats;
    int n_lights;
};

struct Hit {
    float t, u, v;
    int prim;
};

// Moeller-Trumbore; front-facing = determinant > 0 for e1 = v1 - v0, e2 = v2 - v0 (counter-clockwise from the origin).
__device__ inline bool tri_hit(const Tri& tr, V3 o, V3 d, bool cull, float tmin, float* t, float* u, float* v) {
    const V3 e1 = v3(tr.e1[0], tr.e1[1], tr.e1[2]), e2 = v3(tr.e2[0], tr.e2[1], tr.e2[2]);
    const V3 pv = cross3(d, e2);
    const float det = dot3(e1, pv);
    if (cull ? !(det > 0.f) : det == 0.f) return false;
    const float inv = 1.f / det;
    const V3 tv = o - v3(tr.v0[0], tr.v0[1], tr.v0[2]);
    const float uu = dot3(tv, pv) * inv;
    if (!(uu >= 0.f && uu <= 1.f)) return false;
    const V3 qv = cross3(tv, e1);
    const float vv = dot3(d, qv) * inv;
    if (!(vv >= 0.f && uu + vv <= 1.f)) return false;
    const float tt = dot3(e2, qv) * inv;
    if (!(tt > tmin)) return false;
    *t = tt; *u = uu; *v = vv;
    return true;
}

__device__ inline bool box_hit(const BvhNode& n, V3 o, V3 inv, float tmin, float tmax) {
    float t0 = (n.bmin[0] - o.x) * inv.x, t1 = (n.bmax[0] - o.x) * inv.x;
    float lo = fminf(t0, t1), hi = fmaxf(t0, t1);
    t0 = (n.bmin[1] - o.y) * inv.y; t1 = (n.bmax[1] - o.y) * inv.y;
    lo = fmaxf(lo, fminf(t0, t1)); hi = fminf(hi, fmaxf(t0, t1));
    t0 = (n.bmin[2] - o.z) * inv.z; t1 = (n.bmax[2] - o.z) * inv.z;
    lo = fmaxf(lo, fminf(t0, t1)); hi = fminf(hi, fmaxf(t0, t1));
    return fmaxf(lo, tmin) <= fminf(hi, tmax);  // fmin/fmax drop the NaNs of 0 * inf: such a slab never rejects
}

constexpr int kStack = 48;

// Closest hit in (tmin, tmax), ties to the lower primitive index; any_hit: stop at the first hit.
__device__ inline bool trace(const Scene& sc, V3 o, V3 d, float tmin, float tmax, bool cull, bool any_hit, Hit* hit, int* status) {
    const V3 inv = v3(1.f / d.x, 1.f / d.y, 1.f / d.z);
    int stack[kStack], sp = 0;
    stack[sp++] = 0;
    float best = tmax;
    int best_prim = 0x7fffffff;
    bool found = false;
    while (sp) {
        const BvhNode n = sc.nodes[stack[--sp]];
        if (!box_hit(n, o, inv, tmin, best)) continue;
        if (n.count) {
            for (int i = 0; i < n.count; ++i) {
                const Tri& tr = sc.tris[n.left + i];
                float t, u, v;
                if (!tri_hit(tr, o, d, cull, tmin, &t, &u, &v)) continue;
                if (t < best || (t == best && found && tr.prim < best_prim)) {
                    if (!(t < tmax)) continue;
                    best = t; best_prim = tr.prim; found = true;
                    hit->t = t; hit->u = u; hit->v = v; hit->prim = tr.prim;
                    if (any_hit) return true;
                }
            }
        } else if (sp + 2 <= kStack) {
            stack[sp++] = n.left;
            stack[sp++] = n.left + 1;
        } else {
            atomicCAS(status, 0, 1);
        }
    }
    return found;
}

// Cone sampling of a sphere light (closesthit.rchit:217-256).
__device__ inline V3 sample_light(const neon_pt_material& light, V3 p, uint32_t& seed, V3* light_dir, float* pdf) {
    const V3 lpos = v3(light.position[0], light.position[1], light.position[2]);
    const float radius = light.position[3];
    const float dist = length3(lpos - p);
    const float sin2 = (radius * radius) / (dist * dist);
    const float cos_max = sqrtf(fmaxf(0.f, 1.f - sin2));
    const float r1 = rng_next(seed), r2 = rng_next(seed);
    const float cos_t = 1.f - r1 * (1.f - cos_max);
    const float sin_t = sqrtf(fmaxf(0.f, 1.f - cos_t * cos_t));
    const float phi = 2.f * 3.14159265f * r2;
    const V3 to = normalize3(lpos - p);
    const V3 tan = fabsf(to.x) > fabsf(to.y) ? normalize3(v3(-to.z, 0.f, to.x)) : normalize3(v3(0.f, to.z, -to.y));
    const V3 bit = cross3(to, tan);
    float sp, cp;
    sincos_fixed(phi, &sp, &cp);
    *light_dir = normalize3(tan * (sin_t * cp) + bit * (sin_t * sp) + to * cos_t);
    *pdf = 1.f / (2.f * 3.14159265f * (1.f - cos_max));
    return v3(light.emission[0], light.emission[1], light.emission[2]);
}

__device__ inline float fresnel_schlick(float cos_t, float eta) {
    float r0 = (1.f - eta) / (1.f + eta);
    r0 = r0 * r0;
    const float m = 1.f - cos_t;
    return r0 + (1.f - r0) * (m * m * m * m * m);
}

__device__ inline uint8_t to_unorm8(float v) {
    if (!(v == v)) return 0;
    return (uint8_t)rintf(fminf(fmaxf(v, 0.f), 1.f) * 255.f);
}

struct Camera {
    float inv_proj[16], inv_view[16];  // column-major
    float frame_id;
};

__device__ inline void mat_mul(const float* m, float x, float y, float z, float w, float out[4]) {
    for (int r = 0; r < 4; ++r) out[r] = ((m[r] * x + m[4 + r] * y) + m[8 + r] * z) + m[12 + r] * w;
}

constexpr int kMaxDepth = 3;  // closesthit.rchit:8

__global__ void __launch_bounds__(64) pt_frame_kernel(Scene sc, Camera cam, int width, int height, uint8_t* image,
                                                      unsigned long long* ray_counter, int* status) {
    // 8 x 8 pixel tiles: the rays of a warp stay close together
    const int tiles_x = (width + 7) / 8;
    const int tx = blockIdx.x % tiles_x, ty = blockIdx.x / tiles_x;
    const int px = tx * 8 + (threadIdx.x & 7), py = ty * 8 + (threadIdx.x >> 3);
    unsigned rays = 0;
    if (px < width && py < height) {
        // ---- ray generation (raygen.rgen:55-93) ----
        const float ux = ((float)px + 0.5f) / (float)width, uy = ((float)py + 0.5f) / (float)height;
        float o4[4];
        mat_mul(cam.inv_view, 0.f, 0.f, 0.f, 1.f, o4);
        uint32_t seed = (uint32_t)((float)(px * 1973 + py * 9277) + cam.frame_id * 26699.f) | 1u;
        const float r1 = rng_next(seed), r2 = rng_next(seed);
        const float jx = (r1 - 0.5f) / (float)width, jy = (r2 - 0.5f) / (float)height;
        const float dx = (ux + jx * 2.f) * 2.f - 1.f, dy = (uy + jy * 2.f) * 2.f - 1.f;
        float tg[4], dir4[4];
        mat_mul(cam.inv_proj, dx, dy, 1.f, 1.f, tg);
        const V3 tn = normalize3(v3(tg[0], tg[1], tg[2]));
        mat_mul(cam.inv_view, tn.x, tn.y, tn.z, 0.f, dir4);
        V3 origin = v3(o4[0], o4[1], o4[2]), dir = v3(dir4[0], dir4[1], dir4[2]);
        float tmax = 10000.f;
        // ---- the path: payload of the shaders ----
        V3 color = v3(0.f, 0.f, 0.f), thr = v3(1.f, 1.f, 1.f);
        float thr_w = 1.f;
        uint32_t depth = 0, mat_type = 0;   // payload.misc.y, misc.z (raygen.rgen does not set misc.z: zero here)
        while (true) {
            Hit h;
            ++rays;
            if (!trace(sc, origin, dir, 0.001f, tmax, true, false, &h, status)) {
                color = color + thr * v3(0.1f, 0.1f, 0.1f);  // miss.rmiss:25
                break;
            }
            // ---- closest hit (closesthit.rchit:259-594) ----
            const float b0 = 1.f - h.u - h.v, b1 = h.u, b2 = h.v;
            const neon_pt_vertex& v0 = sc.verts[sc.indices[3 * h.prim]];
            const neon_pt_vertex& v1 = sc.verts[sc.indices[3 * h.prim + 1]];
            const neon_pt_vertex& v2 = sc.verts[sc.indices[3 * h.prim + 2]];
            V3 normal = normalize3(v3(v0.normal[0], v0.normal[1], v0.normal[2]) * b0 + v3(v1.normal[0], v1.normal[1], v1.normal[2]) * b1 +
                                   v3(v2.normal[0], v2.normal[1], v2.normal[2]) * b2);
            normal = faceforward3(normal, dir, normal);
            const neon_pt_material& mat = sc.mats[v0.material];
            const V3 emission = v3(mat.emission[0], mat.emission[1], mat.emission[2]);
            if (length3(emission) > 0.f) {
                if (depth == 0u || mat_type == 1u) color = color + thr * emission;
                break;
            }
            if (depth >= (uint32_t)kMaxDepth) break;
            if (depth > 2u) {  // Russian roulette of the shader; unreachable below MAX_DEPTH = 3, kept for the same seed stream if that changes
                const float q = fmaxf(0.05f, 1.f - fmaxf(thr.x, fmaxf(thr.y, thr.z)));
                if (rng_next(seed) < q) break;
                thr = thr / (1.f - q);
                thr_w = thr_w / (1.f - q);
            }
            ++depth;
            const int type = (int)mat.misc[2];
            V3 new_dir = v3(0.f, 0.f, 0.f), offset_pos = v3(0.f, 0.f, 0.f);
            const float INV_PI = 0.3183098861837907f;
            if (type == 0 || type == 2) {
                normal = faceforward3(normal, dir, normal);
                const V3 world = origin + dir * h.t;
                offset_pos = world + normal * 0.001f;
                const float q1 = rng_next(seed), q2 = rng_next(seed);
                const float r = sqrtf(q1), theta = 2.f * 3.14159265f * q2;
                const V3 tan = fabsf(normal.x) > fabsf(normal.y) ? normalize3(v3(-normal.z, 0.f, normal.x)) : normalize3(v3(0.f, normal.z, -normal.y));
                const V3 bit = cross3(normal, tan);
                float st, ct;
                sincos_fixed(theta, &st, &ct);
                const V3 diffuse = normalize3(tan * (r * ct) + bit * (r * st) + normal * sqrtf(1.f - q1));
                const V3 specular = reflect3(normalize3(dir), normal);
                const float rough = clampf(mat.misc[0], 0.f, 1.f);
                new_dir = normalize3(mix3(specular, diffuse, rough));
                const neon_pt_material& light = sc.mats[(int)(rng_next(seed) * (float)sc.n_lights)];
                const float pick_pdf = 1.f / (float)sc.n_lights;
                V3 ldir;
                float lpdf;
                const V3 Le = sample_light(light, offset_pos, seed, &ldir, &lpdf);
                const float cos_t = dot3(normal, ldir);
                // the textured material reads its albedo from the (absent) texture array: a white texel stands in
                const V3 albedo = type == 0 ? v3(mat.albedo[0], mat.albedo[1], mat.albedo[2]) : v3(1.f, 1.f, 1.f);
                if (cos_t > 0.f && lpdf > 0.f) {
                    const float shadow_dist = length3(v3(light.position[0], light.position[1], light.position[2]) - offset_pos) - light.position[3] - 0.01f;
                    Hit sh;
                    ++rays;
                    if (!trace(sc, offset_pos, ldir, 0.001f, shadow_dist, false, true, &sh, status)) {
                        const V3 brdf = albedo * INV_PI;
                        color = color + ((thr * brdf) * Le * cos_t) / (lpdf * pick_pdf);
                    }
                }
                thr = thr * albedo;
                mat_type = type == 0 ? 0u : 2u;
            } else if (type == 67) {
                const V3 world = origin + dir * h.t;
                offset_pos = world + normal * 0.001f;
                const V3 incoming = normalize3(dir);
                const float cos_t = clampf(dot3(neg(incoming), normal), 0.f, 1.f);
                const bool entering = cos_t > 0.f;
                const float eta = entering ? (1.f / mat.misc[1]) : mat.misc[1];
                const V3 nn = entering ? normal : neg(normal);
                const float F = fresnel_schlick(cos_t, mat.misc[1]);
                if (rng_next(seed) < F) {
                    new_dir = reflect3(incoming, nn);
                } else {
                    new_dir = refract3(incoming, nn, eta);
                    if (length3(new_dir) < 0.001f) new_dir = reflect3(incoming, nn);
                }
                mat_type = 1u;
            }
            origin = offset_pos;
            dir = new_dir;
            tmax = 10000.f;
        }
        (void)thr_w;
        uint8_t* out = image + ((size_t)py * width + px) * 4;
        out[0] = to_unorm8(color.x);
        out[1] = to_unorm8(color.y);
        out[2] = to_unorm8(color.z);
        out[3] = 255;
    }
    // rays of the block -> one integer atomic
    __shared__ unsigned s_rays;
    if (threadIdx.x == 0) s_rays = 0;
    __syncthreads();
    for (int o = 16; o > 0; o >>= 1) rays += __shfl_xor_sync(0xffffffffu, rays, o);
    if ((threadIdx.x & 31) == 0) atomicAdd(&s_rays, rays);
    __syncthreads();
    if (threadIdx.x == 0) atomicAdd(ray_counter, (unsigned long long)s_rays);
}

// ---- host: hierarchy construction (median split of the longest centroid axis, leaves of at most 4) ----
struct Builder {
    std::vector<BvhNode> nodes;
    std::vector<int> order;
    std::vector<float> cmin, cmax, cen;  // per triangle: bounds and centroid (3 floats each)
    int max_depth = 0;

    void bounds(int first, int count, float* bmin, float* bmax) const {
        for (int a = 0; a < 3; ++a) { bmin[a] = INFINITY; bmax[a] = -INFINITY; }
        for (int i = first; i < first + count; ++i)
            for (int a = 0; a < 3; ++a) {
                bmin[a] = std::min(bmin[a], cmin[3 * order[i] + a]);
                bmax[a] = std::max(bmax[a], cmax[3 * order[i] + a]);
            }
    }
    void build(int node, int first, int count, int depth) {
        max_depth = std::max(max_depth, depth);
        float bmin[3], bmax[3];
        bounds(first, count, bmin, bmax);
        for (int a = 0; a < 3; ++a) {  // padded: the slab test must never lose a hit that lies on a face
            const float pad = 1e-5f * std::max(1.f, std::max(std::fabs(bmin[a]), std::fabs(bmax[a])));
            nodes[node].bmin[a] = bmin[a] - pad;
            nodes[node].bmax[a] = bmax[a] + pad;
        }
        if (count <= 4 || depth >= kStack - 4) {
            nodes[node].left = first;
            nodes[node].count = count;
            return;
        }
        float lo[3] = {INFINITY, INFINITY, INFINITY}, hi[3] = {-INFINITY, -INFINITY, -INFINITY};
        for (int i = first; i < first + count; ++i)
            for (int a = 0; a < 3; ++a) {
                lo[a] = std::min(lo[a], cen[3 * order[i] + a]);
                hi[a] = std::max(hi[a], cen[3 * order[i] + a]);
            }
        int axis = 0;
        if (hi[1] - lo[1] > hi[axis] - lo[axis]) axis = 1;
        if (hi[2] - lo[2] > hi[axis] - lo[axis]) axis = 2;
        const int mid = first + count / 2;
        std::nth_element(order.begin() + first, order.begin() + mid, order.begin() + first + count,
                         [&](int a, int b) { return cen[3 * a + axis] < cen[3 * b + axis] || (cen[3 * a + axis] == cen[3 * b + axis] && a < b); });
        const int left = (int)nodes.size();
        nodes.push_back(BvhNode{});
        nodes.push_back(BvhNode{});
        nodes[node].left = left;
        nodes[node].count = 0;
        build(left, first, mid - first, depth + 1);
        build(left + 1, mid, first + count - mid, depth + 1);
    }
};

}  // namespace

struct neon_pt_handle {
    neon_pt_config cfg{};
    std::string err;
    int64_t launches = 0;
    int n_nodes = 0, max_depth = 0;
    BvhNode* nodes = nullptr;
    Tri* tris = nullptr;
    neon_pt_vertex* verts = nullptr;
    uint32_t* indices = nullptr;
    neon_pt_material* mats = nullptr;
    unsigned long long* rays = nullptr;
    int* status = nullptr;
    uint8_t* st_image = nullptr;
    cudaStream_t own_stream = nullptr, last_stream = nullptr;
};

namespace {
int pt_fail(neon_pt_handle* h, int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (h) h->err = buf; else g_pt_create_error = buf;
    return code;
}
#define PCU(h, call)                                                                          \
    do {                                                                                      \
        cudaError_t e_ = (call);                                                              \
        if (e_ != cudaSuccess) return pt_fail(h, NEON_PT_ECUDA, "%s failed: %s", #call, cudaGetErrorString(e_)); \
    } while (0)

void pt_free(neon_pt_handle* h) {
    for (void* p : {(void*)h->nodes, (void*)h->tris, (void*)h->verts, (void*)h->indices, (void*)h->mats, (void*)h->rays, (void*)h->status,
                    (void*)h->st_image})
        if (p) cudaFree(p);
    if (h->own_stream) cudaStreamDestroy(h->own_stream);
}
}  // namespace

extern "C" {

const char* neon_pt_last_error(const neon_pt_handle* h) { return h ? h->err.c_str() : g_pt_create_error.c_str(); }
int64_t neon_pt_launch_count(const neon_pt_handle* h) { return h ? h->launches : 0; }

int neon_pt_create(const neon_pt_config* cfg, const neon_pt_vertex* vertices, int n_vertices, const uint32_t* indices, int n_indices,
                   const neon_pt_material* materials, int n_materials, neon_pt_handle** out) {
    if (!cfg || !vertices || !indices || !materials || !out) return pt_fail(nullptr, NEON_PT_EINVAL, "null argument");
    *out = nullptr;
    if (cfg->width <= 0 || cfg->height <= 0 || cfg->width > 16384 || cfg->height > 16384) return pt_fail(nullptr, NEON_PT_EINVAL, "bad image size");
    if (n_vertices <= 0 || n_indices <= 0 || n_indices % 3 || n_materials <= 0) return pt_fail(nullptr, NEON_PT_EINVAL, "bad scene sizes");
    if (cfg->n_lights <= 0 || cfg->n_lights > n_materials) return pt_fail(nullptr, NEON_PT_EINVAL, "n_lights must lie in [1, n_materials]");
    for (int i = 0; i < n_indices; ++i)
        if (indices[i] >= (uint32_t)n_vertices) return pt_fail(nullptr, NEON_PT_EINVAL, "index %d refers to vertex %u of %d", i, indices[i], n_vertices);
    for (int i = 0; i < n_vertices; ++i)
        if (vertices[i].material >= (uint32_t)n_materials) return pt_fail(nullptr, NEON_PT_EINVAL, "vertex %d refers to material %u of %d", i, vertices[i].material, n_materials);
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || cfg->device < 0 || cfg->device >= ndev) {
        cudaGetLastError();
        return pt_fail(nullptr, NEON_PT_ECUDA, "no such CUDA device");
    }
    neon_pt_handle* h = new (std::nothrow) neon_pt_handle;
    if (!h) return pt_fail(nullptr, NEON_PT_EINVAL, "out of host memory");
    h->cfg = *cfg;
    // triangles prepared for the test, hierarchy over their bounds
    const int n_tri = n_indices / 3;
    Builder b;
    b.order.resize(n_tri);
    b.cmin.resize(3 * (size_t)n_tri); b.cmax.resize(3 * (size_t)n_tri); b.cen.resize(3 * (size_t)n_tri);
    for (int t = 0; t < n_tri; ++t) {
        b.order[t] = t;
        for (int a = 0; a < 3; ++a) {
            const float p0 = vertices[indices[3 * t]].pos[a], p1 = vertices[indices[3 * t + 1]].pos[a], p2 = vertices[indices[3 * t + 2]].pos[a];
            b.cmin[3 * t + a] = std::min(p0, std::min(p1, p2));
            b.cmax[3 * t + a] = std::max(p0, std::max(p1, p2));
            b.cen[3 * t + a] = (p0 + p1 + p2) * (1.f / 3.f);
        }
    }
    b.nodes.reserve(2 * (size_t)n_tri);
    b.nodes.push_back(BvhNode{});
    b.build(0, 0, n_tri, 0);
    std::vector<Tri> tris(n_tri);
    for (int i = 0; i < n_tri; ++i) {
        const int t = b.order[i];
        const float *p0 = vertices[indices[3 * t]].pos, *p1 = vertices[indices[3 * t + 1]].pos, *p2 = vertices[indices[3 * t + 2]].pos;
        for (int a = 0; a < 3; ++a) {
            tris[i].v0[a] = p0[a];
            tris[i].e1[a] = p1[a] - p0[a];
            tris[i].e2[a] = p2[a] - p0[a];
        }
        tris[i].prim = t;
    }
    h->n_nodes = (int)b.nodes.size();
    h->max_depth = b.max_depth;
    auto bail = [&](int rc) {
        g_pt_create_error = h->err;
        pt_free(h);
        delete h;
        return rc;
    };
    auto upload = [&](auto** dst, const void* src, size_t bytes) -> int {
        if (cudaMalloc(reinterpret_cast<void**>(dst), bytes) != cudaSuccess || cudaMemcpy(*dst, src, bytes, cudaMemcpyHostToDevice) != cudaSuccess)
            return pt_fail(h, NEON_PT_ECUDA, "uploading the scene failed: %s", cudaGetErrorString(cudaGetLastError()));
        return NEON_PT_OK;
    };
    if (cudaSetDevice(cfg->device) != cudaSuccess) return bail(pt_fail(h, NEON_PT_ECUDA, "cudaSetDevice failed"));
    int rc;
    if ((rc = upload(&h->nodes, b.nodes.data(), b.nodes.size() * sizeof(BvhNode))) || (rc = upload(&h->tris, tris.data(), tris.size() * sizeof(Tri))) ||
        (rc = upload(&h->verts, vertices, (size_t)n_vertices * sizeof(neon_pt_vertex))) ||
        (rc = upload(&h->indices, indices, (size_t)n_indices * sizeof(uint32_t))) ||
        (rc = upload(&h->mats, materials, (size_t)n_materials * sizeof(neon_pt_material))))
        return bail(rc);
    if (cudaMalloc(&h->rays, 8) != cudaSuccess || cudaMalloc(&h->status, 4) != cudaSuccess || cudaMemset(h->rays, 0, 8) != cudaSuccess ||
        cudaMemset(h->status, 0, 4) != cudaSuccess || cudaMalloc(&h->st_image, (size_t)cfg->width * cfg->height * 4) != cudaSuccess ||
        cudaStreamCreateWithFlags(&h->own_stream, cudaStreamNonBlocking) != cudaSuccess)
        return bail(pt_fail(h, NEON_PT_ECUDA, "allocating the frame state failed"));
    *out = h;
    return NEON_PT_OK;
}

int neon_pt_render(neon_pt_handle* h, const float* inverse_projection, const float* inverse_view, float frame_id, uint8_t* image_rgba8,
                   void* cuda_stream) {
    if (!h) return NEON_PT_EINVAL;
    if (!inverse_projection || !inverse_view || !image_rgba8) return pt_fail(h, NEON_PT_EINVAL, "null argument");
    PCU(h, cudaSetDevice(h->cfg.device));
    Camera cam;
    memcpy(cam.inv_proj, inverse_projection, sizeof cam.inv_proj);
    memcpy(cam.inv_view, inverse_view, sizeof cam.inv_view);
    cam.frame_id = frame_id;
    Scene sc{h->nodes, h->tris, h->verts, h->indices, h->mats, h->cfg.n_lights};
    const int tiles = ((h->cfg.width + 7) / 8) * ((h->cfg.height + 7) / 8);
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    pt_frame_kernel<<<tiles, 64, 0, st>>>(sc, cam, h->cfg.width, h->cfg.height, image_rgba8, h->rays, h->status);
    h->launches++;
    PCU(h, cudaGetLastError());
    h->last_stream = st;
    return NEON_PT_OK;
}

int neon_pt_render_host(neon_pt_handle* h, const float* inverse_projection, const float* inverse_view, float frame_id, uint8_t* image_rgba8) {
    if (!h) return NEON_PT_EINVAL;
    if (!image_rgba8) return pt_fail(h, NEON_PT_EINVAL, "null image");
    int rc = neon_pt_render(h, inverse_projection, inverse_view, frame_id, h->st_image, h->own_stream);
    if (rc) return rc;
    PCU(h, cudaMemcpyAsync(image_rgba8, h->st_image, (size_t)h->cfg.width * h->cfg.height * 4, cudaMemcpyDeviceToHost, h->own_stream));
    PCU(h, cudaStreamSynchronize(h->own_stream));
    return NEON_PT_OK;
}

int neon_pt_rays(neon_pt_handle* h, uint64_t* rays) {
    if (!h || !rays) return NEON_PT_EINVAL;
    PCU(h, cudaSetDevice(h->cfg.device));
    PCU(h, cudaStreamSynchronize(h->last_stream));
    unsigned long long v = 0;
    PCU(h, cudaMemcpy(&v, h->rays, 8, cudaMemcpyDeviceToHost));
    PCU(h, cudaMemset(h->rays, 0, 8));
    *rays = v;
    return NEON_PT_OK;
}

int neon_pt_bvh_info(const neon_pt_handle* h, int* n_nodes, int* max_depth) {
    if (!h) return NEON_PT_EINVAL;
    if (n_nodes) *n_nodes = h->n_nodes;
    if (max_depth) *max_depth = h->max_depth;
    return NEON_PT_OK;
}

int neon_pt_status(neon_pt_handle* h, int* word) {
    if (!h || !word) return NEON_PT_EINVAL;
    PCU(h, cudaSetDevice(h->cfg.device));
    PCU(h, cudaStreamSynchronize(h->last_stream));
    PCU(h, cudaMemcpy(word, h->status, 4, cudaMemcpyDeviceToHost));
    PCU(h, cudaMemset(h->status, 0, 4));
    return *word ? NEON_PT_EDEVICE : NEON_PT_OK;
}

int neon_pt_destroy(neon_pt_handle* h) {
    if (!h) return NEON_PT_EINVAL;
    cudaSetDevice(h->cfg.device);
    cudaDeviceSynchronize();
    pt_free(h);
    delete h;
    return NEON_PT_OK;
}

}  // extern "C"
