// NVRTC front end.  libnvrtc is opened with dlopen on first use so that the library loads
// (and its host-side logic can be tested) on machines without the CUDA toolkit libraries
// on the loader path.
#include "jit.hpp"

#include <cstring>

#include <dlfcn.h>

#include <cstdlib>
#include <mutex>

namespace cn {

namespace {

typedef struct _nvrtcProgram* nvrtcProgram;
typedef int nvrtcResult;

struct NvrtcApi {
    void* handle = nullptr;
    nvrtcResult (*CreateProgram)(nvrtcProgram*, const char*, const char*, int, const char* const*,
                                 const char* const*) = nullptr;
    nvrtcResult (*DestroyProgram)(nvrtcProgram*) = nullptr;
    nvrtcResult (*CompileProgram)(nvrtcProgram, int, const char* const*) = nullptr;
    nvrtcResult (*GetCUBINSize)(nvrtcProgram, size_t*) = nullptr;
    nvrtcResult (*GetCUBIN)(nvrtcProgram, char*) = nullptr;
    nvrtcResult (*GetProgramLogSize)(nvrtcProgram, size_t*) = nullptr;
    nvrtcResult (*GetProgramLog)(nvrtcProgram, char*) = nullptr;
    const char* (*GetErrorString)(nvrtcResult) = nullptr;
    std::string error;
};

NvrtcApi* load_nvrtc() {
    static NvrtcApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        const char* env = getenv("CN_NVRTC_LIB");
        const char* candidates[] = {env,
                                    "/usr/local/cuda/lib64/libnvrtc.so.12",
                                    "libnvrtc.so.12",
                                    "/usr/local/cuda/lib64/libnvrtc.so",
                                    "libnvrtc.so"};
        for (const char* c : candidates) {
            if (!c || !*c) continue;
            api.handle = dlopen(c, RTLD_NOW | RTLD_LOCAL);
            if (api.handle) break;
        }
        if (!api.handle) {
            api.error = "libnvrtc not found (set CN_NVRTC_LIB to its path)";
            return;
        }
#define CN_SYM(name)                                                            \
    api.name = reinterpret_cast<decltype(api.name)>(dlsym(api.handle, "nvrtc" #name)); \
    if (!api.name) api.error = "libnvrtc lacks nvrtc" #name;
        CN_SYM(CreateProgram)
        CN_SYM(DestroyProgram)
        CN_SYM(CompileProgram)
        CN_SYM(GetCUBINSize)
        CN_SYM(GetCUBIN)
        CN_SYM(GetProgramLogSize)
        CN_SYM(GetProgramLog)
        CN_SYM(GetErrorString)
#undef CN_SYM
    });
    return &api;
}

}  // namespace

long long spill_bytes(const std::string& log) {
    long long total = 0;
    for (const char* what : {" bytes spill stores", " bytes spill loads"}) {
        size_t at = 0;
        while ((at = log.find(what, at)) != std::string::npos) {
            size_t b = at;
            while (b > 0 && log[b - 1] >= '0' && log[b - 1] <= '9') --b;
            if (b < at) total += atoll(log.substr(b, at - b).c_str());
            at += 1;
        }
    }
    return total;
}

uint32_t code_digest(const std::string& source, const TileConfig& tile) {
    uint32_t h = 2166136261u;  // FNV-1a
    auto mix = [&](const char* p, size_t n) {
        for (size_t i = 0; i < n; ++i) {
            h ^= (unsigned char)p[i];
            h *= 16777619u;
        }
    };
    mix(source.data(), source.size());
    mix(kDeviceHeaderText, strlen(kDeviceHeaderText));
    char cfg[160];
    const int n = snprintf(cfg, sizeof(cfg), "tx%d r%d b%d ns%d pf%d sh%d push%d mb%d fu%d tr%d", tile.tx, tile.r, tile.block,
                           tile.ns, tile.prefetch, (int)tile.shfl, (int)tile.push, tile.minb, tile.fill_u, (int)tile.trigger);
    mix(cfg, (size_t)n);
    return h;
}

int nvrtc_compile(const std::string& source, const TileConfig& tile, std::vector<char>* cubin,
                  std::string* log) {
    NvrtcApi* api = load_nvrtc();
    if (!api->handle || !api->error.empty()) {
        if (log) *log = api->error;
        return CN_ERR_COMPILE;
    }
    const char* headers[] = {kDeviceHeaderText, kExpTableText};
    const char* names[] = {"cn_device.cuh", "cn_exp_table.inc"};
    nvrtcProgram prog = nullptr;
    nvrtcResult rc = api->CreateProgram(&prog, source.c_str(), "cn_group.cu", 2, headers, names);
    if (rc != 0) {
        if (log) *log = std::string("nvrtcCreateProgram: ") + api->GetErrorString(rc);
        return CN_ERR_COMPILE;
    }
    std::string d_tx = "-DCN_TX=" + std::to_string(tile.tx);
    std::string d_r = "-DCN_R=" + std::to_string(tile.r);
    std::string d_s0 = "-DCN_S0=" + std::to_string(tile.s0) + "LL";
    std::string d_s1 = "-DCN_S1=" + std::to_string(tile.s1) + "LL";
    std::string d_ns = "-DCN_NS_OVERRIDE=" + std::to_string(tile.ns);
    std::string d_bl = "-DCN_BLOCK=" + std::to_string(tile.block > 0 ? tile.block : 256);
    std::string d_mb = "-DCN_MINB=" + std::to_string(tile.minb > 0 ? tile.minb : 1);
    std::string d_fu = "-DCN_FILL_U=" + std::to_string(tile.fill_u > 0 ? tile.fill_u : 1);
    std::string d_pf = "-DCN_PREFETCH=" + std::to_string(tile.prefetch);
    // --fmad=false: a*b+c stays two roundings, as in the reference's arith.mulf/addf pairs
    // (src/jit.cpp:411-443); division and sqrt stay IEEE-rounded (the defaults, spelled out).
    // --ptxas-options=-v: the log then states registers and spills of the kernel
    const char* opts[] = {"--gpu-architecture=sm_100a", "--fmad=false",    "--prec-div=true",
                          "--ptxas-options=-v",
                          "--prec-sqrt=true",           "--std=c++17",     "-lineinfo",
                          d_tx.c_str(),                 d_r.c_str(),       d_s0.c_str(),
                          d_s1.c_str(),                 d_ns.c_str(),
                          d_bl.c_str(),
                          d_mb.c_str(),                 d_fu.c_str(),
                          d_pf.c_str(),                 tile.shfl ? "-DCN_SHFL=1" : "-DCN_SHFL=0",
                          tile.push ? "-DCN_PUSH=1" : "-DCN_PUSH=0",
                          tile.trigger ? "-DCN_TRIGGER=1" : "-DCN_TRIGGER=0",
                          tile.drop_copies ? "-DCN_DEBUG_DROP_COPIES=1" : "-DCN_DEBUG_DROP_COPIES=0",
                          tile.drop_copies ? "-DCN_WAIT_LIMIT=2000u" : "-DCN_WAIT_LIMIT=2000000u"};
    rc = api->CompileProgram(prog, (int)(sizeof(opts) / sizeof(opts[0])), opts);
    size_t logsz = 0;
    api->GetProgramLogSize(prog, &logsz);
    if (log && logsz > 1) {
        log->resize(logsz);
        api->GetProgramLog(prog, &(*log)[0]);
    }
    if (rc != 0) {
        if (log) *log = std::string("nvrtcCompileProgram: ") + api->GetErrorString(rc) + "\n" + *log;
        api->DestroyProgram(&prog);
        return CN_ERR_COMPILE;
    }
    size_t sz = 0;
    api->GetCUBINSize(prog, &sz);
    cubin->resize(sz);
    api->GetCUBIN(prog, cubin->data());
    api->DestroyProgram(&prog);
    if (sz == 0) {
        if (log) *log += "\nNVRTC produced no cubin";
        return CN_ERR_COMPILE;
    }
    return CN_OK;
}

}  // namespace cn
