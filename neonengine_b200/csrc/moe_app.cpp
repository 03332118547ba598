// Headless application loop around lve::MoeLayerSystem in the style of the engine's apps
// (NeonEngine/src/raytracing_app.cpp:605-760, NeonEngine/src/water_app.cpp:529-614): the app owns
// the system, runs "frames" in a loop (one frame = one pass of the layer over a batch that lives
// in a device buffer instead of a swapchain image) and reports throughput once per second the
// way the apps put "FPS: %.1f (%.2f ms)" into the window title (raytracing_app.cpp:648-656) -
// here on stdout, as tokens/s.
//
//   moe_app [--weights FILE.nmoe] [--tokens T] [--seconds S] [--hidden H --inter I --experts E --topk K]
//
// Without --weights the layer gets seeded pseudo-random MXFP4 weights.  Exit code 0 when every
// frame ran and the device status word stayed clean.
#include <cuda_runtime.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/lve_moe_layer_system.hpp"

namespace lve {

class MoeApp {
   public:
    struct Options {
        neon_moe_config cfg{2880, 2880, 32, 4, 7.0f, 1.702f, 64, 0, 1, 0};
        std::string weightsFile;
        int tokens = 64;
        double seconds = 3.0;
    };

    explicit MoeApp(const Options& o) : opt(o), moe(withTokens(o)) {
        if (!opt.weightsFile.empty()) {
            if (int rc = neon_moe_load_weights_file(moe.handle(), opt.weightsFile.c_str()))
                throw std::runtime_error(std::string("neon_moe_load_weights_file: ") + neon_moe_last_error(moe.handle()) + " (" +
                                         std::to_string(rc) + ")");
        } else {
            loadRandomWeights();
        }
        const size_t T = opt.tokens, H = opt.cfg.hidden;
        std::vector<uint16_t> hidden(T * H);
        for (auto& v : hidden) v = randomBf16(1.0f);
        cuda(cudaMalloc(&hiddenDev, T * H * 2), "cudaMalloc");
        cuda(cudaMalloc(&outDev, T * H * 4), "cudaMalloc");
        cuda(cudaMemcpy(hiddenDev, hidden.data(), T * H * 2, cudaMemcpyHostToDevice), "cudaMemcpy");
        cuda(cudaStreamCreate(&stream), "cudaStreamCreate");
    }
    ~MoeApp() {
        if (hiddenDev) cudaFree(hiddenDev);
        if (outDev) cudaFree(outDev);
        if (stream) cudaStreamDestroy(stream);
    }

    // The main loop: frames until the time budget is spent; throughput once per second.
    int run() {
        using clock = std::chrono::high_resolution_clock;
        auto currentTime = clock::now();
        const auto start = currentTime;
        float fpsTimer = 0.0f;
        int frameCount = 0;
        long long frames = 0;
        while (std::chrono::duration<double>(clock::now() - start).count() < opt.seconds) {
            moe.run(stream, hiddenDev, opt.tokens, nullptr, outDev);
            cuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize");  // the apps present (and wait) once per frame
            auto newTime = clock::now();
            const float frameTime = std::chrono::duration<float, std::chrono::seconds::period>(newTime - currentTime).count();
            currentTime = newTime;
            fpsTimer += frameTime;
            frameCount++;
            frames++;
            if (fpsTimer >= 1.0f) {
                const float fps = frameCount / fpsTimer;
                std::printf("MoE layer | tokens/s: %.1f (%.3f ms per pass of %d tokens)\n", fps * opt.tokens, 1000.0f / fps, opt.tokens);
                std::fflush(stdout);
                fpsTimer = 0.0f;
                frameCount = 0;
            }
        }
        const int status = moe.deviceStatus();
        std::printf("frames: %lld, device status: %d\n", frames, status);
        return status == 0 && frames > 0 ? 0 : 1;
    }

   private:
    static neon_moe_config withTokens(const Options& o) {
        neon_moe_config c = o.cfg;
        c.max_tokens = o.tokens;
        return c;
    }
    static void cuda(cudaError_t e, const char* what) {
        if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
    }
    uint32_t next() {  // xorshift32
        rng ^= rng << 13; rng ^= rng >> 17; rng ^= rng << 5;
        return rng;
    }
    uint16_t randomBf16(float scale) {  // roughly normal: sum of four uniforms
        float s = 0.f;
        for (int i = 0; i < 4; ++i) s += (next() >> 8) * (1.0f / 16777216.0f) - 0.5f;
        const float v = s * 1.7320508f * scale;
        uint32_t bits;
        std::memcpy(&bits, &v, 4);
        return (uint16_t)((bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16);
    }
    void loadRandomWeights() {
        const size_t H = opt.cfg.hidden, I = opt.cfg.inter, E = opt.cfg.n_experts;
        std::vector<uint16_t> routerW(E * H), routerB(E), guBias(E * 2 * I), dnBias(E * H);
        std::vector<uint8_t> guBlocks(E * 2 * I * H / 2), guScales(E * 2 * I * H / 32), dnBlocks(E * H * I / 2), dnScales(E * H * I / 32);
        for (auto& v : routerW) v = randomBf16(0.02f);
        for (auto& v : routerB) v = randomBf16(0.02f);
        for (auto& v : guBias) v = randomBf16(0.02f);
        for (auto& v : dnBias) v = randomBf16(0.02f);
        for (auto& v : guBlocks) v = (uint8_t)next();
        for (auto& v : dnBlocks) v = (uint8_t)next();
        for (auto& v : guScales) v = (uint8_t)(117 + next() % 7);
        for (auto& v : dnScales) v = (uint8_t)(117 + next() % 7);
        moe.setWeights(routerW.data(), routerB.data(), guBlocks.data(), guScales.data(), guBias.data(), dnBlocks.data(),
                       dnScales.data(), dnBias.data(), false);
    }

    Options opt;
    MoeLayerSystem moe;
    void* hiddenDev = nullptr;
    float* outDev = nullptr;
    cudaStream_t stream = nullptr;
    uint32_t rng = 42u;
};

}  // namespace lve

int main(int argc, char** argv) {
    lve::MoeApp::Options o;
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        auto value = [&]() -> const char* { return i + 1 < argc ? argv[++i] : "0"; };
        if (a == "--weights") o.weightsFile = value();
        else if (a == "--tokens") o.tokens = std::atoi(value());
        else if (a == "--seconds") o.seconds = std::atof(value());
        else if (a == "--hidden") o.cfg.hidden = std::atoi(value());
        else if (a == "--inter") o.cfg.inter = std::atoi(value());
        else if (a == "--experts") o.cfg.n_experts = std::atoi(value());
        else if (a == "--topk") o.cfg.top_k = std::atoi(value());
        else { std::fprintf(stderr, "unknown argument %s\n", a.c_str()); return 2; }
    }
    try {
        lve::MoeApp app{o};
        return app.run();
    } catch (const std::exception& e) {
        std::fprintf(stderr, "%s\n", e.what());
        return 1;
    }
}
