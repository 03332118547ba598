// lve::MoeLayerSystem - engine-style C++ owner of a neon_moe layer (header-only).
//
// Shaped like the engine's compute systems: the constructor creates the GPU object and its
// buffers (NeonEngine/src/water_physics.cpp:23-123), run() records one pass on the caller's
// stream (NeonEngine/src/water_physics.hpp:66, NeonEngine/src/raytracing_system.hpp:79),
// failures become std::runtime_error (NeonEngine/src/water_physics.cpp:617-620), and the
// class is neither copyable nor thread-safe (NeonEngine/src/raytracing_rast.hpp:50-51).
#pragma once
#include <cstdint>
#include <stdexcept>
#include <string>

#include "neon_moe.h"

namespace lve {

class MoeLayerSystem {
   public:
    explicit MoeLayerSystem(const neon_moe_config& cfg) : cfg_(cfg) {
        if (int rc = neon_moe_create(&cfg, &handle_))
            throw std::runtime_error(std::string("neon_moe_create: ") + neon_moe_last_error(nullptr) + " (" +
                                     std::to_string(rc) + ")");
    }
    ~MoeLayerSystem() {
        if (handle_) neon_moe_destroy(handle_);
    }
    MoeLayerSystem(const MoeLayerSystem&) = delete;
    MoeLayerSystem& operator=(const MoeLayerSystem&) = delete;

    void setWeights(const void* routerW, const void* routerB, const uint8_t* gateUpBlocks,
                    const uint8_t* gateUpScales, const void* gateUpBias, const uint8_t* downBlocks,
                    const uint8_t* downScales, const void* downBias, bool onDevice) {
        check(neon_moe_set_weights(handle_, routerW, routerB, gateUpBlocks, gateUpScales, gateUpBias, downBlocks,
                                   downScales, downBias, onDevice ? 1 : 0),
              "neon_moe_set_weights");
    }

    // Records one layer pass on `stream` (a cudaStream_t); all pointers are device memory.
    void run(void* stream, const void* hiddenBf16, int tokens, const float* logitBias, float* outF32,
             int32_t* topkIdx = nullptr, float* topkW = nullptr) {
        check(neon_moe_forward(handle_, hiddenBf16, tokens, logitBias, outF32, topkIdx, topkW, stream),
              "neon_moe_forward");
    }

    // Blocking pass over host memory (copies inside).
    void runHost(const void* hiddenBf16, int tokens, const float* logitBias, float* outF32,
                 int32_t* topkIdx = nullptr, float* topkW = nullptr) {
        check(neon_moe_forward_host(handle_, hiddenBf16, tokens, logitBias, outF32, topkIdx, topkW),
              "neon_moe_forward_host");
    }

    int deviceStatus() {
        int word = 0;
        neon_moe_status(handle_, &word);
        return word;
    }
    const neon_moe_config& config() const { return cfg_; }
    neon_moe_handle* handle() { return handle_; }

   private:
    void check(int rc, const char* what) {
        if (rc) throw std::runtime_error(std::string(what) + ": " + neon_moe_last_error(handle_) + " (" +
                                         std::to_string(rc) + ")");
    }
    neon_moe_config cfg_;
    neon_moe_handle* handle_ = nullptr;
};

}  // namespace lve
