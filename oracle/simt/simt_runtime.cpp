// simt_runtime.cpp -- the host side of the SIMT emulation (see hip/hip_runtime.h in this folder): the kernel registry,
// the module calls the reference's launchers make, and the launch itself. Test infrastructure only.
#include <hip/hip_runtime.h>

#include <map>
#include <string>
#include <thread>
#include <vector>

thread_local simt_ctx simt_self;
simt_dim3 simt_block_dim, simt_grid_dim;

struct simt_function { simt_thunk run; };
struct simt_module { int unused; };

namespace {
std::map<std::string, simt_function>& registry() {
    static std::map<std::string, simt_function> r;
    return r;
}
simt_module g_module;
}  // namespace

void simt_register(const char* name, simt_thunk run_one_thread) { registry()[name] = simt_function{run_one_thread}; }

extern "C" {

// The reference's loader (src/kernel_loader.h): here every registered kernel is "in" every module
hipError_t kernel_module_load(hipModule_t* module, const char* name) {
    (void)name;
    *module = &g_module;
    return hipSuccess;
}

hipError_t hipModuleGetFunction(hipFunction_t* fn, hipModule_t mod, const char* name) {
    (void)mod;
    auto it = registry().find(name);
    if (it == registry().end()) return hipErrorInvalidDeviceFunction;
    *fn = &it->second;
    return hipSuccess;
}

hipError_t hipModuleUnload(hipModule_t mod) { (void)mod; return hipSuccess; }

const char* hipGetErrorString(hipError_t e) { return e == hipSuccess ? "success" : "error"; }

hipError_t hipModuleLaunchKernel(hipFunction_t fn, unsigned gx, unsigned gy, unsigned gz, unsigned bx, unsigned by,
                                 unsigned bz, unsigned shared_bytes, hipStream_t stream, void** args, void** extra) {
    (void)shared_bytes; (void)stream; (void)extra;
    if (!fn || !fn->run || by != 1 || bz != 1 || bx == 0 || bx > 1024) return hipErrorInvalidValue;
    simt_block_dim = {bx, 1, 1};
    simt_grid_dim = {gx, gy, gz};
    const int n_waves = (int)((bx + 31) / 32);
    for (unsigned z = 0; z < gz; ++z)
        for (unsigned y = 0; y < gy; ++y)
            for (unsigned x = 0; x < gx; ++x) {
                std::barrier<> block((std::ptrdiff_t)bx);
                std::vector<std::unique_ptr<simt_wave>> waves;
                for (int w = 0; w < n_waves; ++w)
                    waves.emplace_back(new simt_wave((int)std::min(32u, bx - 32u * (unsigned)w)));
                std::vector<std::thread> threads;
                threads.reserve(bx);
                for (unsigned t = 0; t < bx; ++t)
                    threads.emplace_back([&, t] {
                        simt_self.tid = {t, 0, 0};
                        simt_self.bid = {x, y, z};
                        simt_self.block = &block;
                        simt_self.wave = waves[t / 32].get();
                        simt_self.lane = (int)(t % 32);
                        fn->run(args);
                    });
                for (auto& th : threads) th.join();
            }
    return hipSuccess;
}

}  // extern "C"
