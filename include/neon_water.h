/*
 * neon_water.h - C ABI of the reference engine's FLIP water step as CUDA kernels (same shared
 * library as neon_moe.h).
 *
 * This is the one path here for which the reference engine has an implementation: the compute
 * shader NeonEngine/shaders/water_grid.comp driven by lve::WaterPhysics
 * (NeonEngine/src/water_physics.{hpp,cpp}).  Each entry point names what it replaces:
 *
 *   neon_water_create .......... WaterPhysics::WaterPhysics, water_physics.cpp:23-123 (owns the
 *                                particle and grid buffers, uploads the start positions) and
 *                                CreateBuffers, water_physics.cpp:449-603
 *   neon_water_step ............ WaterPhysics::RunSimulation / RunAndReadback,
 *                                water_physics.cpp:131, :164-430 (records the passes of one or more
 *                                steps into the caller's stream; nothing is read back)
 *   neon_water_particles_device  the position buffer the render system binds directly
 *                                (partPosBuff, water_physics.hpp)
 *   neon_water_read_* .......... explicit host read-back, NeonEngine/src/water_app.cpp:601-612
 *
 * Results: one step equals the shader's passes 0-8 executed in the dispatch order of
 * water_physics.cpp:164-430 with every pass complete before the next starts.  The shader's data
 * races are resolved deterministically: the particle separation pass (pass 1) reads the
 * positions as they were when the pass started; float accumulations onto the grid (passes 2 and
 * 4) add the contributions of a cell in ascending particle id (a binned gather replaces the
 * shader's compare-and-swap loops).  With these two rules the kernels reproduce the CPU
 * restatement of the shader bit for bit (32-bit floats, no fused multiply-add).
 * Passes 6-8 read the pressure buffer the last Jacobi iteration READ, as the reference does
 * (it never rebinds the descriptor set after the loop).  The shader's debug buffer and particle
 * colours are not produced.
 *
 * All functions return 0 or a NEON_MOE_E* code (neon_moe.h); none throws or aborts.
 */
#ifndef NEON_WATER_H
#define NEON_WATER_H

#include <stdint.h>

#include "neon_moe.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct neon_water_handle neon_water_handle;

/* The fields the shader's uniform block and push constants carry (water_grid.comp:4-43),
 * plus the two loop counts of water_physics.cpp:243 and :321. */
typedef struct neon_water_config {
    int n_particles;         /* 8000                                   */
    int nx, ny, nz;          /* 99 x 37 x 44 cells                     */
    float cell_size;         /* 0.1                                    */
    float over_relaxation;   /* 1.03                                   */
    float rest_density;      /* 1.0                                    */
    float damping;           /* FLIP ratio, 0                          */
    float mass;              /* 20                                     */
    float dt;                /* 1/500                                  */
    float box_min[3], box_max[3], gravity[3];
    int collision_substeps;  /* 4                                      */
    int jacobi_iterations;   /* 50                                     */
    int device;              /* CUDA device ordinal                    */
} neon_water_config;

/* pos4: n_particles x 4 floats (xyz + w), host or device; velocities start at zero. */
int neon_water_create(const neon_water_config* cfg, const float* pos4, int on_device, neon_water_handle** out);
int neon_water_destroy(neon_water_handle* h);
const char* neon_water_last_error(const neon_water_handle* h);

/* Replaces the particle state (vel4 may be NULL = zero). */
int neon_water_set_particles(neon_water_handle* h, const float* pos4, const float* vel4, int on_device);

/* Enqueues n_steps steps on cuda_stream (a cudaStream_t; NULL = default stream).  One step is
 * captured into a CUDA graph on first use and replayed. */
int neon_water_step(neon_water_handle* h, int n_steps, void* cuda_stream);

/* Host-buffer form: uploads pos4/vel4 (n x 4 floats each), runs n_steps, downloads both, waits. */
int neon_water_step_host(neon_water_handle* h, float* pos4, float* vel4, int n_steps, void* cuda_stream);

/* Device addresses of the live particle buffers (n x 4 floats each). */
int neon_water_particles_device(neon_water_handle* h, float** pos4, float** vel4);

/* Blocking read-back of the particle state (either pointer may be NULL). */
int neon_water_read_particles(neon_water_handle* h, float* pos4, float* vel4);

/* Blocking read-back of a grid array of the last step: "u", "v", "w", "pressure" (the buffer
 * passes 6-8 read), "density" (floats, nx*ny*nz) or "flags" (uint32). */
int neon_water_read_grid(neon_water_handle* h, const char* name, void* dst, uint64_t bytes);

/* Runs ONE step eagerly with CUDA events between the pass groups and waits; ms4 receives the
 * milliseconds of {separation (pass 1), particles->grid (passes 0, 2-4), pressure Jacobi
 * (pass 5), pressure apply + grid->particles + integrate (passes 6-8)}. */
int neon_water_profile_step(neon_water_handle* h, double* ms4, void* cuda_stream);

/* Reads (and clears) the device status word: non-zero when the fused Jacobi kernel's bounded
 * grid-barrier wait gave up (the step's result is then invalid).  Synchronises the last stream. */
int neon_water_status(neon_water_handle* h, int* device_status_word);

/* Options: "use_graphs" (default 1); "fused_jacobi" (default 1 where the device supports
 * cooperative launches and the grid has at most 2 cells per resident thread: all pressure
 * iterations in one cooperative kernel with a grid-wide barrier; 0 = one launch per iteration). */
int neon_water_set_option(neon_water_handle* h, const char* name, int64_t value);

int64_t neon_water_launch_count(const neon_water_handle* h);

#ifdef __cplusplus
}
#endif
#endif /* NEON_WATER_H */
