/*
 * neon_svgf.h - C ABI of the reference engine's denoiser as CUDA kernels (same shared library as
 * neon_moe.h): temporal accumulation (NeonEngine/shaders/raytracing_pp.comp) followed by the
 * edge-avoiding a-trous filter (NeonEngine/shaders/raytracing_atrous.comp), one frame per call.
 *
 * What each entry point replaces:
 *   neon_svgf_create ........ the history images RayTracingRast owns: two rgba16f colour images
 *                             and the rgba32f moments image, NeonEngine/src/raytracing_rast.cpp:
 *                             120-160 (cleared to zero here; RayTracingRast::pingPong = false,
 *                             raytracing_rast.hpp:44)
 *   neon_svgf_denoise ....... RayTracingRast::renderCompute + renderAtrous as the frame loop calls
 *                             them, NeonEngine/src/raytracing_app.cpp:735-765 and
 *                             NeonEngine/src/raytracing_rast.cpp:325-428: records the passes of one
 *                             frame into the caller's stream; the G-buffer images and the storage
 *                             image are the caller's, bound per call like the descriptor sets
 *                             (raytracing_app.cpp:437-457)
 *   neon_svgf_read .......... explicit host read-back (NeonEngine/src/water_app.cpp:601-612 style)
 *
 * Results: the bodies of the two shaders (behind the bare `return;` both start with in the
 * reference checkout, which ships the denoiser switched off), in the reference's dispatch order:
 * the temporal pass on the descriptor set the ping-pong flag selects, `atrous_iterations` filter
 * passes alternating between the two sets (so odd passes filter the OLDER history image, as the
 * reference's set order has it), one more pass on the second set when the count is even, then the
 * copy of the storage image into a history image (iteration 98).  The one data race of the
 * shaders - the moments image is read at neighbouring pixels and written in place - is resolved
 * deterministically: every pass reads the moments as the previous pass left them.  With that rule
 * the kernels reproduce the CPU restatement of the shaders bit for bit.
 *
 * Conventions the Vulkan specification leaves open and this library fixes: rgba16f stores round
 * to nearest even; rgba8 stores clamp to [0, 1], scale by 255 and round to nearest even (NaN
 * stores 0); exp2 is a fixed degree-7 polynomial (fused multiply-adds, relative error < 1e-7).
 * All other arithmetic is the shaders' 32-bit float operations in the shaders' order, unfused.
 *
 * Images are row-major [height][width][4]: float for rgba32f, 16-bit patterns for rgba16f,
 * bytes for rgba8.  All functions return 0 or a NEON_MOE_E* code (neon_moe.h).
 */
#ifndef NEON_SVGF_H
#define NEON_SVGF_H

#include <stdint.h>

#include "neon_moe.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct neon_svgf_handle neon_svgf_handle;

typedef struct neon_svgf_config {
    int width, height;      /* 800 x 600 in the reference's window (raytracing_app.hpp:16-17) */
    int atrous_iterations;  /* 3 (raytracing_app.cpp:759)                                      */
    int device;             /* CUDA device ordinal                                             */
} neon_svgf_config;

int neon_svgf_create(const neon_svgf_config* cfg, neon_svgf_handle** out);
int neon_svgf_destroy(neon_svgf_handle* h);
const char* neon_svgf_last_error(const neon_svgf_handle* h);

/* Replaces the state kept between frames (any pointer may be NULL = zeros): colour_a / colour_b
 * rgba16f, moments rgba32f {history length, first moment, second moment, variance}. */
int neon_svgf_set_history(neon_svgf_handle* h, const uint16_t* colour_a, const uint16_t* colour_b, const float* moments,
                          int ping_pong, int on_device);

/* One frame, enqueued on cuda_stream.  Device pointers: position, normal (w = mesh id),
 * barycentric, motion: rgba32f, read only; image: rgba8, the path tracer's output on entry, the
 * denoised frame on return.  The launch sequence of a given argument set is captured into a CUDA
 * graph the first time and replayed afterwards (option use_graphs). */
int neon_svgf_denoise(neon_svgf_handle* h, const float* position, const float* normal, const float* barycentric,
                      const float* motion, uint8_t* image, void* cuda_stream);

/* Same with HOST images: uploads the five images, runs the frame, downloads `image`, waits. */
int neon_svgf_denoise_host(neon_svgf_handle* h, const float* position, const float* normal, const float* barycentric,
                           const float* motion, uint8_t* image, void* cuda_stream);

/* Blocking read-back: "colour_a", "colour_b" (uint16 x 4 per pixel), "moments" (float x 4 per
 * pixel), "ping_pong" (one int32). */
int neon_svgf_read(neon_svgf_handle* h, const char* name, void* dst, uint64_t bytes);

/* Runs ONE frame eagerly with CUDA events between the passes and waits; ms receives the
 * milliseconds of {temporal pass, all a-trous passes (+ copy)}. */
int neon_svgf_profile_frame(neon_svgf_handle* h, const float* position, const float* normal, const float* barycentric,
                            const float* motion, uint8_t* image, double* ms2, void* cuda_stream);

/* Options: "use_graphs" (default 1). */
int neon_svgf_set_option(neon_svgf_handle* h, const char* name, int64_t value);

int64_t neon_svgf_launch_count(const neon_svgf_handle* h);

#ifdef __cplusplus
}
#endif
#endif /* NEON_SVGF_H */
