// lve::WaterPhysics - drop-in for the engine's class of the same name with the compute work done
// by libneon_moe.so's CUDA water step (include/neon_water.h) instead of 63 vkCmdDispatch calls of
// shaders/water_grid.comp.  Header-only, C++17.
//
// Kept from the engine's class (NeonEngine/src/water_physics.hpp:52-66): the constructor takes the
// particle count, the start positions and the uniform-block values and owns every simulation
// buffer; RunSimulation(dt, ...) records one step into the caller's stream; the class is not
// copyable; failures are std::runtime_error (NeonEngine/src/water_physics.cpp:617-620).
// Replaced: the 25 per-buffer descriptor getters (water_physics.hpp:68-92) become two device
// pointers (positions, velocities) and explicit read-backs, since there are no Vulkan descriptor
// sets to bind; the Vulkan handles in the signatures (descriptor set layout, LveDevice, the
// game-object map used only for rendering) are dropped.  The step itself uses the constant
// dt = 1/500 the engine pushes to the shader (water_physics.cpp:211), whatever `dt` the caller
// passes, exactly as the engine does.
#pragma once
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "neon_water.h"

namespace lve {

// The fields of the engine's uniform block the simulation reads (water_grid.comp:4-36).
struct WaterPhysUbo {
    int uNumParticles = 0, uNumCells = 0;
    int uGridDim[4] = {0, 0, 0, 1};
    float overRelaxation = 1.03f, uMass = 20.f, uRestDensity = 1.f, uCellSize = 0.1f, uDamping = 0.f;
    float uBoxMin[4] = {0, 0, 0, 1}, uBoxMax[4] = {0, 0, 0, 1}, uGravity[4] = {0, 98.1f, 0, 0};
};

class WaterPhysics {
   public:
    // startPos: particleCount x 4 floats (xyz, w), as the engine's std::vector<glm::vec4>
    WaterPhysics(int particleCount, const float* startPos, const WaterPhysUbo& ubo, int device = 0) {
        neon_water_config c{};
        c.n_particles = particleCount;
        c.nx = ubo.uGridDim[0]; c.ny = ubo.uGridDim[1]; c.nz = ubo.uGridDim[2];
        c.cell_size = ubo.uCellSize; c.over_relaxation = ubo.overRelaxation; c.rest_density = ubo.uRestDensity;
        c.damping = ubo.uDamping; c.mass = ubo.uMass;
        c.dt = 1.0f / 500.f;  // the push constant of every pass, water_physics.cpp:211
        for (int a = 0; a < 3; ++a) { c.box_min[a] = ubo.uBoxMin[a]; c.box_max[a] = ubo.uBoxMax[a]; c.gravity[a] = ubo.uGravity[a]; }
        c.collision_substeps = 4;   // water_physics.cpp:243
        c.jacobi_iterations = 50;   // water_physics.cpp:321
        c.device = device;
        cfg_ = c;
        if (int rc = neon_water_create(&c, startPos, 0, &handle_))
            throw std::runtime_error(std::string("neon_water_create: ") + neon_water_last_error(nullptr) + " (" +
                                     std::to_string(rc) + ")");
    }
    ~WaterPhysics() {
        if (handle_) neon_water_destroy(handle_);
    }
    WaterPhysics(const WaterPhysics&) = delete;
    WaterPhysics& operator=(const WaterPhysics&) = delete;

    // Records one simulation step on `stream` (a cudaStream_t); returns after enqueueing.
    void RunSimulation(float /*dt*/, void* stream) { check(neon_water_step(handle_, 1, stream), "neon_water_step"); }

    // What the render system binds: the live particle buffers on the device (vec4 per particle).
    float* positionsDevice() {
        float* p = nullptr;
        check(neon_water_particles_device(handle_, &p, nullptr), "neon_water_particles_device");
        return p;
    }
    float* velocitiesDevice() {
        float* v = nullptr;
        check(neon_water_particles_device(handle_, nullptr, &v), "neon_water_particles_device");
        return v;
    }

    // Blocking host read-back (the engine's debug read-back path, water_app.cpp:601-612).
    void readPositions(std::vector<float>& outPositions) {
        outPositions.resize((size_t)cfg_.n_particles * 4);
        check(neon_water_read_particles(handle_, outPositions.data(), nullptr), "neon_water_read_particles");
    }
    void readGrid(const char* name, std::vector<float>& out) {
        out.resize((size_t)cfg_.nx * cfg_.ny * cfg_.nz);
        check(neon_water_read_grid(handle_, name, out.data(), out.size() * sizeof(float)), "neon_water_read_grid");
    }
    int deviceStatus() {
        int word = 0;
        neon_water_status(handle_, &word);
        return word;
    }
    const neon_water_config& config() const { return cfg_; }
    neon_water_handle* handle() { return handle_; }

   private:
    void check(int rc, const char* what) {
        if (rc) throw std::runtime_error(std::string(what) + ": " + neon_water_last_error(handle_) + " (" + std::to_string(rc) + ")");
    }
    neon_water_config cfg_{};
    neon_water_handle* handle_ = nullptr;
};

}  // namespace lve
