// The reference engine's denoiser (NeonEngine/shaders/raytracing_pp.comp: temporal accumulation;
// NeonEngine/shaders/raytracing_atrous.comp: edge-avoiding a-trous filter) as CUDA kernels behind
// the C ABI of include/neon_svgf.h, scheduled per frame as NeonEngine/src/raytracing_app.cpp:735-765
// and NeonEngine/src/raytracing_rast.cpp:325-428 schedule the two shaders.  This translation unit is
// compiled with -fmad=false: every kernel uses the shaders' 32-bit float operations in the shaders'
// order (the only fused multiply-adds are the explicit ones of exp2_poly), so the results equal the
// CPU restatement bit for bit.  No CPU fallback exists.
//
// Redesign relative to the shaders (results unchanged):
//  * the moments image is double-buffered, so a pass never reads what it writes (the shaders update
//    it in place while neighbours read it);
//  * the copy of the storage image into the history image (the shaders' "iteration 98" dispatch) is
//    done by the last filter pass itself whenever that pass does not read the image being replaced
//    (always the case for an odd iteration count, the reference's 3);
//  * one frame is a CUDA graph.
#include "../../include/neon_svgf.h"

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>
#include <string>
#include <vector>

namespace {

__device__ __forceinline__ float dot3(float ax, float ay, float az, float bx, float by, float bz) { return ax * bx + ay * by + az * bz; }
__device__ __forceinline__ float len3(float x, float y, float z) { return sqrtf(x * x + y * y + z * z); }
__device__ __forceinline__ float max_glsl(float a, float b) { return a < b ? b : a; }
__device__ __forceinline__ float min_glsl(float a, float b) { return b < a ? b : a; }
__device__ __forceinline__ float mixf(float x, float y, float a) { return x * (1.0f - a) + y * a; }

// 2^x: nearest-integer split, degree-7 polynomial of 2^f on [-0.5, 0.5], exact scaling by 2^n.
// Inside (-126, 128) the nearest integer (ties to even) comes from adding and subtracting 1.5 * 2^23,
// whose sum also carries that integer in its low mantissa bits: two additions on the main pipes
// instead of a rounding and a conversion instruction, same values.
__device__ __forceinline__ float exp2_poly(float x) {
    if (!(x > -126.0f && x < 128.0f)) return x != x ? x : (x > 0.0f ? INFINITY : 0.0f);
    const float magic = 12582912.0f;
    const float shifted = x + magic;
    const float n = shifted - magic, f = x - n;
    float p = 1.5252734e-5f;
    p = fmaf(p, f, 1.5403530e-4f);
    p = fmaf(p, f, 1.3333558e-3f);
    p = fmaf(p, f, 9.6181291e-3f);
    p = fmaf(p, f, 5.5504109e-2f);
    p = fmaf(p, f, 2.4022651e-1f);
    p = fmaf(p, f, 6.9314718e-1f);
    p = fmaf(p, f, 1.0f);
    // (n + 127) << 23 with n = bits(shifted) - bits(magic)
    return p * __uint_as_float((__float_as_uint(shifted) - 0x4B400000u + 127u) << 23);
}

__device__ __forceinline__ unsigned to_unorm8(float v) {
    if (v != v) v = 0.0f;
    v = v < 0.0f ? 0.0f : (v > 1.0f ? 1.0f : v);
    return (unsigned)__float2int_rn(v * 255.0f);
}
__device__ __forceinline__ uchar4 pack_rgb8(float r, float g, float b) {
    return make_uchar4((unsigned char)to_unorm8(r), (unsigned char)to_unorm8(g), (unsigned char)to_unorm8(b), 255);
}
__device__ __forceinline__ float3 load_rgb16(const uint2* __restrict__ im, size_t i) {
    const uint2 v = __ldg(im + i);
    const __half2 lo = *reinterpret_cast<const __half2*>(&v.x), hi = *reinterpret_cast<const __half2*>(&v.y);
    return make_float3(__low2float(lo), __high2float(lo), __low2float(hi));
}
__device__ __forceinline__ uint2 pack_rgba16(float r, float g, float b, float a) {
    const __half2 lo = __halves2half2(__float2half_rn(r), __float2half_rn(g)), hi = __halves2half2(__float2half_rn(b), __float2half_rn(a));
    uint2 v;
    v.x = *reinterpret_cast<const unsigned*>(&lo);
    v.y = *reinterpret_cast<const unsigned*>(&hi);
    return v;
}

struct Frame {  // the caller's images of one frame
    const float4 *pos, *nrm, *bary, *mot;
    uchar4* image;
};

constexpr int kBlockX = 32, kBlockY = 8;

// ---- temporal accumulation (raytracing_pp.comp:35-247, display mode 5) ---------------------------
__global__ void __launch_bounds__(kBlockX* kBlockY) k_temporal(int w, int h, Frame fr, const uint2* __restrict__ hist_prev,
                                                               uint2* __restrict__ hist_next, const float4* __restrict__ data_in,
                                                               float4* __restrict__ data_out) {
    const int x = blockIdx.x * kBlockX + threadIdx.x, y = blockIdx.y * kBlockY + threadIdx.y;
    if (x >= w || y >= h) return;
    const size_t idx = (size_t)y * w + x;
    const uchar4 c8 = fr.image[idx];
    const float cr = c8.x / 255.0f, cg = c8.y / 255.0f, cb = c8.z / 255.0f;

    // LoadPreviousData (raytracing_pp.comp:35-140)
    float pr = 0.0f, pg = 0.0f, pb = 0.0f, hl = 0.0f, pm0 = 0.0f, pm1 = 0.0f;
    bool ok = false;
    const float4 cp = __ldg(fr.pos + idx), cn = __ldg(fr.nrm + idx);
    if (!(dot3(cp.x, cp.y, cp.z, cp.x, cp.y, cp.z) < 1e-6f)) {
        const float4 cbary = __ldg(fr.bary + idx), m = __ldg(fr.mot + idx);
        const int cur_mesh = (int)roundf(cn.w);
        const float uvx = ((float)x + 0.5f) / (float)w, uvy = ((float)y + 0.5f) / (float)h;
        const float pux = uvx - m.x, puy = uvy - m.y;
        if (!(pux < 0.0f || puy < 0.0f || pux > 1.0f || puy > 1.0f)) {
            const float ppx = pux * (float)w - 0.5f, ppy = puy * (float)h - 0.5f;
            const float flx = floorf(ppx), fly = floorf(ppy);
            const int bx = (int)flx, by = (int)fly;
            const float fx = ppx - flx, fy = ppy - fly;
            const float weights[4] = {(1.0f - fx) * (1.0f - fy), fx * (1.0f - fy), (1.0f - fx) * fy, fx * fy};
            const float dist = len3(cp.x, cp.y, cp.z);
            const float pos_threshold = max_glsl(0.01f * dist, 0.005f);
            float ar = 0.0f, ag = 0.0f, ab = 0.0f, ah = 0.0f, am0 = 0.0f, am1 = 0.0f, aw = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int tx = bx + (i & 1), ty = by + (i >> 1);
                if (tx < 0 || ty < 0 || tx >= w || ty >= h) continue;
                const size_t t = (size_t)ty * w + tx;
                const float4 tp = __ldg(fr.pos + t);
                if (dot3(tp.x, tp.y, tp.z, tp.x, tp.y, tp.z) < 1e-6f) continue;
                const float4 tn = __ldg(fr.nrm + t);
                if (cur_mesh != (int)roundf(tn.w)) continue;
                const float tap_depth = len3(tp.x, tp.y, tp.z);
                if (fabsf(dist - tap_depth) > 0.02f * dist) continue;
                if (len3(cp.x - tp.x, cp.y - tp.y, cp.z - tp.z) > pos_threshold) continue;
                if (dot3(cn.x, cn.y, cn.z, tn.x, tn.y, tn.z) < 0.9f) continue;
                const float4 tb = __ldg(fr.bary + t);
                if (len3(cbary.x - tb.x, cbary.y - tb.y, cbary.z - tb.z) > 0.2f) continue;
                const float wt = weights[i];
                const float3 hc = load_rgb16(hist_prev, t);
                ar += hc.x * wt; ag += hc.y * wt; ab += hc.z * wt;
                const float4 td = __ldg(data_in + t);
                ah += td.x * wt;
                am0 += td.y * wt;
                am1 += td.z * wt;
                aw += wt;
            }
            if (!(aw < 0.5f)) {
                const float inv = 1.0f / aw;
                pr = ar * inv; pg = ag * inv; pb = ab * inv;
                hl = ah * inv;
                pm0 = am0 * inv;
                pm1 = am1 * inv;
                ok = true;
            }
        }
    }
    float alpha;
    if (ok) {
        hl = hl + 1.0f;
        alpha = 1.0f / hl;
        alpha = min_glsl(max_glsl(alpha, 0.0f), 1.0f);
    } else {
        alpha = 1.0f;
        hl = 1.0f;
    }
    const float br = ok ? pr : cr, bg = ok ? pg : cg, bb = ok ? pb : cb;
    const float nr = mixf(br, cr, alpha), ng = mixf(bg, cg, alpha), nb = mixf(bb, cb, alpha);
    float m0 = 0.2126f * cr + 0.7152f * cg + 0.0722f * cb;
    float m1 = m0 * m0;
    m0 = mixf(pm0, m0, alpha);
    m1 = mixf(pm1, m1, alpha);
    const float variance = max_glsl(0.0f, m1 - m0 * m0);
    hist_next[idx] = pack_rgba16(nr, ng, nb, 1.0f);
    data_out[idx] = make_float4(hl, m0, m1, variance);
    fr.image[idx] = pack_rgb8(nr, ng, nb);
}

// ---- a-trous filter pass (raytracing_atrous.comp:59-160, iteration < 98) -------------------------
// copy_to != nullptr: the pass also stores its rgba8 result, converted back to floats, into that
// history image (the shaders' separate copy dispatch, raytracing_atrous.comp:66-70).
__global__ void __launch_bounds__(kBlockX* kBlockY) k_atrous(int w, int h, int step, Frame fr, const uint2* __restrict__ colour,
                                                             const float4* __restrict__ data_in, float4* __restrict__ data_out,
                                                             uint2* __restrict__ copy_to) {
    const int x = blockIdx.x * kBlockX + threadIdx.x, y = blockIdx.y * kBlockY + threadIdx.y;
    if (x >= w || y >= h) return;
    const size_t idx = (size_t)y * w + x;
    const float eps = 1e-6f, log2e = 1.4426950408889634f, inv256 = 1.0f / 256.0f;
    const float4 cp = __ldg(fr.pos + idx), cd = __ldg(data_in + idx);
    uchar4 result;
    float out_var = cd.w;
    if (dot3(cp.x, cp.y, cp.z, cp.x, cp.y, cp.z) < eps) {  // no surface: the colour passes through
        const float3 s = load_rgb16(colour, idx);
        result = pack_rgb8(s.x, s.y, s.z);
    } else {
        const float4 cn = __ldg(fr.nrm + idx);
        const float c_lum = cd.y, c_var = max_glsl(cd.w, 0.0f);
        const float step_f = (float)step;
        const float inv_z = 1.0f / max_glsl(fabsf(cp.z) * step_f, eps);
        const float inv_l = 1.0f / max_glsl(1.0f * sqrtf(max_glsl(c_var, 1e-10f)), eps);
        float sr = 0.0f, sg = 0.0f, sb = 0.0f, sum_w = 0.0f, sum_var = 0.0f, sum_wvar = 0.0f;
#pragma unroll
        for (int yy = -2; yy <= 2; ++yy) {
            const int qy = min(max(y + yy * step, 0), h - 1);
            const float ky = yy == 0 ? 6.0f : ((yy == 1 || yy == -1) ? 4.0f : 1.0f);
#pragma unroll
            for (int xx = -2; xx <= 2; ++xx) {
                const int qx = min(max(x + xx * step, 0), w - 1);
                const float kx = xx == 0 ? 6.0f : ((xx == 1 || xx == -1) ? 4.0f : 1.0f);
                const float wk = kx * ky * inv256;
                const size_t q = (size_t)qy * w + qx;
                const float4 sn = __ldg(fr.nrm + q);
                float wn = max_glsl(dot3(cn.x, cn.y, cn.z, sn.x, sn.y, sn.z), 0.0f);
                wn *= wn; wn *= wn; wn *= wn; wn *= wn; wn *= wn; wn *= wn; wn *= wn;
                if (wn <= eps) continue;
                const float s_pos_z = __ldg(&fr.pos[q].z);
                const float4 sd = __ldg(data_in + q);
                const float3 sc = load_rgb16(colour, q);
                const float s_var = max_glsl(sd.w, 0.0f);
                const float dz = fabsf(cp.z - s_pos_z);
                const float wd = exp2_poly(-dz * inv_z * log2e);
                const float dl = fabsf(c_lum - sd.y);
                const float wl = exp2_poly(-dl * inv_l * log2e);
                const float wt = wk * wn * wd * wl;
                sr += sc.x * wt; sg += sc.y * wt; sb += sc.z * wt;
                sum_w += wt;
                const float w2 = wt * wt;
                sum_var += s_var * w2;
                sum_wvar += w2;
            }
        }
        const float inv_w = 1.0f / max_glsl(sum_w, eps), inv_wv = 1.0f / max_glsl(sum_wvar, eps);
        result = pack_rgb8(sr * inv_w, sg * inv_w, sb * inv_w);
        out_var = sum_var * inv_wv;
    }
    fr.image[idx] = result;
    data_out[idx] = make_float4(cd.x, cd.y, cd.z, out_var);
    if (copy_to) copy_to[idx] = pack_rgba16(result.x / 255.0f, result.y / 255.0f, result.z / 255.0f, result.w / 255.0f);
}

// ---- copy pass (raytracing_atrous.comp:66-70, iteration 98) ---------------------------------------
__global__ void k_copy(size_t n, const uchar4* __restrict__ image, uint2* __restrict__ dst) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uchar4 c = image[i];
    dst[i] = pack_rgba16(c.x / 255.0f, c.y / 255.0f, c.z / 255.0f, c.w / 255.0f);
}

thread_local std::string g_svgf_create_error;

}  // namespace

struct neon_svgf_handle {
    neon_svgf_config cfg{};
    std::string err;
    uint2 *colour_a = nullptr, *colour_b = nullptr;  // rgba16f history images
    float4* data[2] = {nullptr, nullptr};            // moments: data[0] holds the state between frames
    int ping_pong = 0;
    float4* stage[4] = {nullptr, nullptr, nullptr, nullptr};  // device copies of host G-buffers (denoise_host)
    uchar4* stage_image = nullptr;
    int64_t launches = 0;
    int launches_per_frame = 0;
    int use_graphs = 1;
    cudaStream_t own_stream = nullptr, last_stream = nullptr;
    struct Cached {
        Frame fr;
        int ping_pong;
        cudaGraphExec_t exec;
    };
    std::vector<Cached> graphs;
};

namespace {

int sfail(neon_svgf_handle* h, int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (h) h->err = buf; else g_svgf_create_error = buf;
    return code;
}

#define SCU(h, call)                                                                                       \
    do {                                                                                                   \
        cudaError_t e_ = (call);                                                                           \
        if (e_ != cudaSuccess) return sfail(h, NEON_MOE_ECUDA, "%s: %s", #call, cudaGetErrorString(e_)); \
    } while (0)

void drop_graphs(neon_svgf_handle* h) {
    for (auto& g : h->graphs)
        if (g.exec) cudaGraphExecDestroy(g.exec);
    h->graphs.clear();
}

// the kernels of one frame in the reference's dispatch order; ev (optional) gets 3 event marks.
// ping_pong is the flag's value BEFORE the frame (RayTracingRast::renderCompute flips it).
int record_frame(neon_svgf_handle* h, const Frame& fr, int ping_pong, cudaStream_t st, cudaEvent_t* ev = nullptr) {
    const int w = h->cfg.width, ht = h->cfg.height, iters = h->cfg.atrous_iterations;
    const dim3 grid((w + kBlockX - 1) / kBlockX, (ht + kBlockY - 1) / kBlockY), block(kBlockX, kBlockY);
    // set 1 binds {5: colour_a, 7: colour_b}, set 2 the two swapped; the temporal pass takes set 1 when the flag is set
    uint2* prev = ping_pong ? h->colour_a : h->colour_b;
    uint2* next = ping_pong ? h->colour_b : h->colour_a;
    int n = 0, cur = 0;  // data[cur] is read, data[cur ^ 1] written
    if (ev) cudaEventRecord(ev[0], st);
    k_temporal<<<grid, block, 0, st>>>(w, ht, fr, prev, next, h->data[cur], h->data[cur ^ 1]); ++n;
    cur ^= 1;
    if (ev) cudaEventRecord(ev[1], st);
    // filter passes: even ones read the image the temporal pass wrote, odd ones the older one; the
    // even-count extra pass runs on the second set at step 1 (raytracing_rast.cpp:390-411)
    const int passes = iters + (iters % 2 == 0 ? 1 : 0);
    bool copied = false;
    for (int i = 0; i < passes; ++i) {
        const bool extra = i == iters;
        const uint2* src = extra ? prev : ((i % 2 == 0) ? next : prev);
        const bool last = i == passes - 1;
        uint2* copy_to = (last && src != prev) ? prev : nullptr;
        k_atrous<<<grid, block, 0, st>>>(w, ht, extra ? 1 : (1 << i), fr, src, h->data[cur], h->data[cur ^ 1], copy_to); ++n;
        cur ^= 1;
        copied = copy_to != nullptr;
    }
    if (!copied) {
        const size_t px = (size_t)w * ht;
        k_copy<<<(unsigned)((px + 255) / 256), 256, 0, st>>>(px, fr.image, prev); ++n;
    }
    if (cur != 0) {  // an odd number of passes: bring the moments back to data[0]
        if (cudaMemcpyAsync(h->data[0], h->data[1], (size_t)w * ht * sizeof(float4), cudaMemcpyDeviceToDevice, st) != cudaSuccess)
            return -1;
    }
    if (ev) cudaEventRecord(ev[2], st);
    h->launches_per_frame = n;
    return cudaGetLastError() == cudaSuccess ? n : -1;
}

int check_frame_args(neon_svgf_handle* h, const void* a, const void* b, const void* c, const void* d, const void* e) {
    if (!a || !b || !c || !d || !e) return sfail(h, NEON_MOE_EINVAL, "null image pointer");
    return 0;
}

}  // namespace

extern "C" {

int neon_svgf_create(const neon_svgf_config* cfg, neon_svgf_handle** out) {
    if (!cfg || !out) return NEON_MOE_EINVAL;
    *out = nullptr;
    if (cfg->width < 1 || cfg->height < 1 || (int64_t)cfg->width * cfg->height > (int64_t)1 << 28)
        return sfail(nullptr, NEON_MOE_EINVAL, "bad image size %d x %d", cfg->width, cfg->height);
    if (cfg->atrous_iterations < 0 || cfg->atrous_iterations > 16)
        return sfail(nullptr, NEON_MOE_EINVAL, "atrous_iterations=%d outside [0, 16]", cfg->atrous_iterations);
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || cfg->device < 0 || cfg->device >= n_dev) {
        cudaGetLastError();
        return sfail(nullptr, NEON_MOE_ECUDA, "no CUDA device %d", cfg->device);
    }
    neon_svgf_handle* h = new (std::nothrow) neon_svgf_handle;
    if (!h) return NEON_MOE_ECUDA;
    h->cfg = *cfg;
    const size_t px = (size_t)cfg->width * cfg->height;
    bool ok = cudaSetDevice(cfg->device) == cudaSuccess && cudaMalloc(&h->colour_a, px * 8) == cudaSuccess &&
              cudaMalloc(&h->colour_b, px * 8) == cudaSuccess && cudaMalloc(&h->data[0], px * 16) == cudaSuccess &&
              cudaMalloc(&h->data[1], px * 16) == cudaSuccess &&
              cudaStreamCreateWithFlags(&h->own_stream, cudaStreamNonBlocking) == cudaSuccess;
    ok = ok && cudaMemset(h->colour_a, 0, px * 8) == cudaSuccess && cudaMemset(h->colour_b, 0, px * 8) == cudaSuccess &&
         cudaMemset(h->data[0], 0, px * 16) == cudaSuccess && cudaMemset(h->data[1], 0, px * 16) == cudaSuccess;
    if (!ok) {
        const cudaError_t e = cudaGetLastError();
        neon_svgf_destroy(h);
        return sfail(nullptr, NEON_MOE_ECUDA, "device allocation failed: %s", cudaGetErrorString(e));
    }
    *out = h;
    return NEON_MOE_OK;
}

int neon_svgf_destroy(neon_svgf_handle* h) {
    if (!h) return NEON_MOE_OK;
    cudaSetDevice(h->cfg.device);
    if (h->last_stream) cudaStreamSynchronize(h->last_stream);
    drop_graphs(h);
    cudaFree(h->colour_a); cudaFree(h->colour_b); cudaFree(h->data[0]); cudaFree(h->data[1]);
    for (auto* p : h->stage) cudaFree(p);
    cudaFree(h->stage_image);
    if (h->own_stream) cudaStreamDestroy(h->own_stream);
    cudaGetLastError();
    delete h;
    return NEON_MOE_OK;
}

const char* neon_svgf_last_error(const neon_svgf_handle* h) { return h ? h->err.c_str() : g_svgf_create_error.c_str(); }

int neon_svgf_set_history(neon_svgf_handle* h, const uint16_t* colour_a, const uint16_t* colour_b, const float* moments,
                          int ping_pong, int on_device) {
    if (!h) return NEON_MOE_EINVAL;
    SCU(h, cudaSetDevice(h->cfg.device));
    if (h->last_stream) SCU(h, cudaStreamSynchronize(h->last_stream));
    const size_t px = (size_t)h->cfg.width * h->cfg.height;
    const cudaMemcpyKind kind = on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
    if (colour_a) SCU(h, cudaMemcpy(h->colour_a, colour_a, px * 8, kind)); else SCU(h, cudaMemset(h->colour_a, 0, px * 8));
    if (colour_b) SCU(h, cudaMemcpy(h->colour_b, colour_b, px * 8, kind)); else SCU(h, cudaMemset(h->colour_b, 0, px * 8));
    if (moments) SCU(h, cudaMemcpy(h->data[0], moments, px * 16, kind)); else SCU(h, cudaMemset(h->data[0], 0, px * 16));
    h->ping_pong = ping_pong != 0;
    return NEON_MOE_OK;
}

int neon_svgf_denoise(neon_svgf_handle* h, const float* position, const float* normal, const float* barycentric,
                      const float* motion, uint8_t* image, void* cuda_stream) {
    if (!h) return NEON_MOE_EINVAL;
    if (int rc = check_frame_args(h, position, normal, barycentric, motion, image)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    SCU(h, cudaSetDevice(h->cfg.device));
    const Frame fr{reinterpret_cast<const float4*>(position), reinterpret_cast<const float4*>(normal),
                   reinterpret_cast<const float4*>(barycentric), reinterpret_cast<const float4*>(motion),
                   reinterpret_cast<uchar4*>(image)};
    const int pp = h->ping_pong;
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    bool graphs = h->use_graphs != 0;
    if (graphs && (cudaStreamIsCapturing(st, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone)) {
        cudaGetLastError();
        graphs = false;  // inside the caller's own capture: record the kernels directly
    }
    if (graphs) {
        neon_svgf_handle::Cached* hit = nullptr;
        for (auto& g : h->graphs)
            if (g.ping_pong == pp && !memcmp(&g.fr, &fr, sizeof fr)) { hit = &g; break; }
        if (!hit) {
            if (h->graphs.size() >= 32) drop_graphs(h);
            SCU(h, cudaStreamBeginCapture(h->own_stream, cudaStreamCaptureModeThreadLocal));
            const int n = record_frame(h, fr, pp, h->own_stream);
            cudaGraph_t graph = nullptr;
            cudaError_t ce = cudaStreamEndCapture(h->own_stream, &graph);
            cudaGraphExec_t exec = nullptr;
            if (n >= 0 && ce == cudaSuccess && graph) ce = cudaGraphInstantiate(&exec, graph, 0);
            if (graph) cudaGraphDestroy(graph);
            if (n < 0 || ce != cudaSuccess || !exec) {
                cudaGetLastError();
                h->use_graphs = 0;  // capture is not available here: stay eager
                graphs = false;
            } else {
                h->graphs.push_back({fr, pp, exec});
                hit = &h->graphs.back();
            }
        }
        if (hit) {
            SCU(h, cudaGraphLaunch(hit->exec, st));
            h->launches += h->launches_per_frame;
        }
    }
    if (!graphs) {
        const int n = record_frame(h, fr, pp, st);
        if (n < 0) return sfail(h, NEON_MOE_ECUDA, "kernel launch failed: %s", cudaGetErrorString(cudaGetLastError()));
        h->launches += n;
    }
    h->ping_pong = !pp;
    h->last_stream = st;
    return NEON_MOE_OK;
}

int neon_svgf_denoise_host(neon_svgf_handle* h, const float* position, const float* normal, const float* barycentric,
                           const float* motion, uint8_t* image, void* cuda_stream) {
    if (!h) return NEON_MOE_EINVAL;
    if (int rc = check_frame_args(h, position, normal, barycentric, motion, image)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    SCU(h, cudaSetDevice(h->cfg.device));
    const size_t px = (size_t)h->cfg.width * h->cfg.height;
    if (!h->stage_image) {
        for (auto& p : h->stage) SCU(h, cudaMalloc(&p, px * 16));
        SCU(h, cudaMalloc(&h->stage_image, px * 4));
    }
    const float* src[4] = {position, normal, barycentric, motion};
    for (int i = 0; i < 4; ++i) SCU(h, cudaMemcpyAsync(h->stage[i], src[i], px * 16, cudaMemcpyHostToDevice, st));
    SCU(h, cudaMemcpyAsync(h->stage_image, image, px * 4, cudaMemcpyHostToDevice, st));
    if (int rc = neon_svgf_denoise(h, reinterpret_cast<const float*>(h->stage[0]), reinterpret_cast<const float*>(h->stage[1]),
                                   reinterpret_cast<const float*>(h->stage[2]), reinterpret_cast<const float*>(h->stage[3]),
                                   reinterpret_cast<uint8_t*>(h->stage_image), st))
        return rc;
    SCU(h, cudaMemcpyAsync(image, h->stage_image, px * 4, cudaMemcpyDeviceToHost, st));
    SCU(h, cudaStreamSynchronize(st));
    return NEON_MOE_OK;
}

int neon_svgf_read(neon_svgf_handle* h, const char* name, void* dst, uint64_t bytes) {
    if (!h || !name || !dst) return NEON_MOE_EINVAL;
    SCU(h, cudaSetDevice(h->cfg.device));
    if (h->last_stream) SCU(h, cudaStreamSynchronize(h->last_stream));
    const size_t px = (size_t)h->cfg.width * h->cfg.height;
    const void* src = nullptr;
    size_t need = 0;
    if (!strcmp(name, "colour_a")) { src = h->colour_a; need = px * 8; }
    else if (!strcmp(name, "colour_b")) { src = h->colour_b; need = px * 8; }
    else if (!strcmp(name, "moments")) { src = h->data[0]; need = px * 16; }
    else if (!strcmp(name, "ping_pong")) {
        if (bytes != 4) return sfail(h, NEON_MOE_EINVAL, "ping_pong is 4 bytes");
        const int32_t v = h->ping_pong;
        memcpy(dst, &v, 4);
        return NEON_MOE_OK;
    } else return sfail(h, NEON_MOE_EINVAL, "unknown buffer '%s'", name);
    if (bytes != need) return sfail(h, NEON_MOE_EINVAL, "%s is %zu bytes, not %llu", name, need, (unsigned long long)bytes);
    SCU(h, cudaMemcpy(dst, src, need, cudaMemcpyDeviceToHost));
    return NEON_MOE_OK;
}

int neon_svgf_profile_frame(neon_svgf_handle* h, const float* position, const float* normal, const float* barycentric,
                            const float* motion, uint8_t* image, double* ms2, void* cuda_stream) {
    if (!h || !ms2) return NEON_MOE_EINVAL;
    if (int rc = check_frame_args(h, position, normal, barycentric, motion, image)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    SCU(h, cudaSetDevice(h->cfg.device));
    const Frame fr{reinterpret_cast<const float4*>(position), reinterpret_cast<const float4*>(normal),
                   reinterpret_cast<const float4*>(barycentric), reinterpret_cast<const float4*>(motion),
                   reinterpret_cast<uchar4*>(image)};
    cudaEvent_t ev[3];
    for (auto& e : ev) SCU(h, cudaEventCreate(&e));
    const int n = record_frame(h, fr, h->ping_pong, st, ev);
    int rc = NEON_MOE_OK;
    if (n < 0 || cudaStreamSynchronize(st) != cudaSuccess) rc = sfail(h, NEON_MOE_ECUDA, "profiled frame failed: %s", cudaGetErrorString(cudaGetLastError()));
    else {
        h->launches += n;
        h->ping_pong = !h->ping_pong;
        h->last_stream = st;
        for (int i = 0; i < 2; ++i) {
            float ms = 0.0f;
            cudaEventElapsedTime(&ms, ev[i], ev[i + 1]);
            ms2[i] = ms;
        }
    }
    for (auto& e : ev) cudaEventDestroy(e);
    return rc;
}

int neon_svgf_set_option(neon_svgf_handle* h, const char* name, int64_t value) {
    if (!h || !name) return NEON_MOE_EINVAL;
    if (!strcmp(name, "use_graphs")) {
        h->use_graphs = (int)value;
        if (!value) drop_graphs(h);
    } else return sfail(h, NEON_MOE_EINVAL, "unknown option '%s'", name);
    return NEON_MOE_OK;
}

int64_t neon_svgf_launch_count(const neon_svgf_handle* h) { return h ? h->launches : 0; }

}  // extern "C"
