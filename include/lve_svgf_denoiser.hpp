// lve::SvgfDenoiser - the denoiser half of the engine's RayTracingRast with the compute work done by
// libneon_moe.so's CUDA kernels (include/neon_svgf.h) instead of the vkCmdDispatch calls of
// shaders/raytracing_pp.comp and shaders/raytracing_atrous.comp.  Header-only, C++17.
//
// Kept from the engine's class (NeonEngine/src/raytracing_rast.hpp:30-52, raytracing_rast.cpp:325-428):
// the object owns the two history colour images, the moments image and the ping-pong flag;
// renderCompute + renderAtrous of one frame become render(), which records into the caller's stream;
// the class is not copyable (raytracing_rast.hpp:50-51); failures are std::runtime_error.
// Replaced: descriptor sets become the five device pointers of a frame (G-buffer position, normal,
// barycentric, motion as rgba32f; the rgba8 storage image), bound per call as the sets are
// (NeonEngine/src/raytracing_app.cpp:437-457); the group counts (width + 15) / 16 follow from the
// extent given at construction.
#pragma once
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "neon_svgf.h"

namespace lve {

class SvgfDenoiser {
   public:
    // kAtrousIterations = 3 in the engine's frame loop (raytracing_app.cpp:759)
    SvgfDenoiser(int width, int height, int atrousIterations = 3, int device = 0) {
        cfg_ = neon_svgf_config{width, height, atrousIterations, device};
        if (int rc = neon_svgf_create(&cfg_, &handle_))
            throw std::runtime_error(std::string("neon_svgf_create: ") + neon_svgf_last_error(nullptr) + " (" + std::to_string(rc) + ")");
    }
    ~SvgfDenoiser() {
        if (handle_) neon_svgf_destroy(handle_);
    }
    SvgfDenoiser(const SvgfDenoiser&) = delete;
    SvgfDenoiser& operator=(const SvgfDenoiser&) = delete;

    // Temporal pass + a-trous passes + history copy of one frame on `stream` (a cudaStream_t);
    // `image` holds the path tracer's output on entry and the denoised frame afterwards.
    void render(const float* position, const float* normal, const float* barycentric, const float* motion, uint8_t* image,
                void* stream) {
        check(neon_svgf_denoise(handle_, position, normal, barycentric, motion, image, stream), "neon_svgf_denoise");
    }

    // Blocking read-back of the moments image {history length, first moment, second moment, variance}.
    void readMoments(std::vector<float>& out) {
        out.resize((size_t)cfg_.width * cfg_.height * 4);
        check(neon_svgf_read(handle_, "moments", out.data(), out.size() * sizeof(float)), "neon_svgf_read");
    }
    void resetHistory() { check(neon_svgf_set_history(handle_, nullptr, nullptr, nullptr, 0, 0), "neon_svgf_set_history"); }
    const neon_svgf_config& config() const { return cfg_; }
    neon_svgf_handle* handle() { return handle_; }

   private:
    void check(int rc, const char* what) {
        if (rc) throw std::runtime_error(std::string(what) + ": " + neon_svgf_last_error(handle_) + " (" + std::to_string(rc) + ")");
    }
    neon_svgf_config cfg_{};
    neon_svgf_handle* handle_ = nullptr;
};

}  // namespace lve
