/*
 * neon_pt.h - C ABI of the path tracer in libneon_moe.so: the reference engine's own ray-traced
 * frame (NeonEngine/shaders/raygen.rgen, closesthit.rchit, miss.rmiss, shadow.rmiss dispatched by
 * vkCmdTraceRaysKHR, NeonEngine/src/raytracing_system.cpp:96-159) as a CUDA kernel over a software
 * bounding-volume hierarchy instead of VK_KHR_acceleration_structure.  No graphics API is involved:
 * the storage image is a plain device buffer.
 *
 * What one frame computes (per pixel, one sample): a jittered pinhole ray from the inverse view and
 * projection matrices (raygen.rgen:55-90, PCG generator :46-51); at every hit the interpolated and
 * face-forwarded normal, emission on the first hit or after glass, at most MAX_DEPTH = 3 bounces
 * (closesthit.rchit:8,307), a roughness-blended diffuse/mirror bounce, next-event estimation towards
 * one of the sphere lights by cone sampling with a shadow ray (:217-256, :371-421), textured (:441-524)
 * and glass (:527-581) materials; a ray that leaves the scene adds 0.1 x throughput (miss.rmiss:21-27).
 * The recursion of the shaders is a tail call and runs as a loop.  The shaders' writes to the ReSTIR
 * reservoir buffer are left out: raygen.rgen never sets the reservoir index (misc.w), so every ray of
 * the reference writes reservoir 0 (closesthit.rchit:302), a race whose result nothing in the frame reads.
 *
 * Conventions Vulkan leaves open and this library fixes (the CPU oracles use the same ones, which is
 * what makes frames comparable bit for bit):
 *   - a triangle (v0, v1, v2) is front-facing for a ray when dot(cross(v1 - v0, v2 - v0), dir) < 0,
 *     i.e. its vertices appear counter-clockwise from the ray origin; rays flagged
 *     gl_RayFlagsCullBackFacingTrianglesEXT skip the others; shadow rays test both faces;
 *   - Moeller-Trumbore intersection in single precision without fused multiply-adds; a hit needs
 *     tmin < t < tmax; of two hits at the same t the lower primitive index wins (so the result does not
 *     depend on the hierarchy or the traversal order);
 *   - normalize(v) = v / sqrt(dot(v, v)) with IEEE division and square root; sin and cos are a fixed
 *     Cody-Waite reduction + polynomial with fused multiply-adds (error < 2e-7); pow(x, 5) is x*x*x*x*x;
 *   - the rgba8 storage image stores nearest-even(clamp(v, 0, 1) * 255), NaN stores 0;
 *   - the texture array is absent from the engine's checkout: a 1 x 1 white texture stands in.
 *
 * All functions return 0 on success or a NEON_PT_E* code; none throws or aborts.
 */
#ifndef NEON_PT_H
#define NEON_PT_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NEON_PT_OK 0
#define NEON_PT_EINVAL 1
#define NEON_PT_ECUDA 2
#define NEON_PT_EDEVICE 4

typedef struct neon_pt_handle neon_pt_handle;

/* = RayTracingVertex, NeonEngine/src/raytracing_system.hpp:42-50 (world-space position and normal) */
typedef struct neon_pt_vertex {
    float pos[4], normal[4], uv[4];
    uint32_t material, pad1, pad2, pad3;
} neon_pt_vertex;

/* = RayTracingMaterial, NeonEngine/src/raytracing_system.hpp:52-57: misc = {roughness, index of
 * refraction, type (0 diffuse/mirror blend, 2 textured, 67 glass), -}; lights come first and carry
 * position = {centre, radius} (raytracing_system.cpp:619-645). */
typedef struct neon_pt_material {
    float emission[4], albedo[4], position[4], misc[4];
} neon_pt_material;

typedef struct neon_pt_config {
    int width, height;  /* 800 x 600 in the engine (raytracing_app.hpp:16-17) */
    int n_lights;       /* GlobalUbo.numLights: materials [0, n_lights) are the sphere lights */
    int device;
} neon_pt_config;

/* Copies the flattened scene (the arrays RayTracingApp::run builds, raytracing_app.cpp:151-176), builds
 * the bounding-volume hierarchy on the host and uploads everything.
 * Follows: RayTracingSystem's constructor building BLAS/TLAS and buffers, raytracing_system.cpp:19-68. */
int neon_pt_create(const neon_pt_config* cfg, const neon_pt_vertex* vertices, int n_vertices, const uint32_t* indices,
                   int n_indices, const neon_pt_material* materials, int n_materials, neon_pt_handle** out);

/* One frame into `image_rgba8` (device memory, width*height*4 bytes), enqueued on `cuda_stream`.
 * inverse_projection / inverse_view: column-major 4x4 as the engine's RayUbo holds them
 * (raytracing_app.cpp:683-692); frame_id: PushData.accum.x (raytracing_system.cpp:132-146).
 * Follows: RayTracingSystem::render recording vkCmdTraceRaysKHR(width, height, 1). */
int neon_pt_render(neon_pt_handle* h, const float* inverse_projection, const float* inverse_view, float frame_id,
                   uint8_t* image_rgba8, void* cuda_stream);

/* The same frame into HOST memory (copies inside, synchronises). */
int neon_pt_render_host(neon_pt_handle* h, const float* inverse_projection, const float* inverse_view, float frame_id,
                        uint8_t* image_rgba8);

/* Rays traced (closest-hit and shadow rays) by all frames since the last call; synchronises. */
int neon_pt_rays(neon_pt_handle* h, uint64_t* rays);

/* Nodes and depth of the hierarchy (for reports). */
int neon_pt_bvh_info(const neon_pt_handle* h, int* n_nodes, int* max_depth);

/* Non-zero when a traversal ran out of stack (never for hierarchies this library builds). */
int neon_pt_status(neon_pt_handle* h, int* device_status_word);

int64_t neon_pt_launch_count(const neon_pt_handle* h);
const char* neon_pt_last_error(const neon_pt_handle* h);
int neon_pt_destroy(neon_pt_handle* h);

#ifdef __cplusplus
}
#endif
#endif /* NEON_PT_H */
