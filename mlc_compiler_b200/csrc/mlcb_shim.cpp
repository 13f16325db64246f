// C-ABI shim: NVRTC compile, driver-API module load, stream launches.
//
// libcuda and libnvrtc are opened lazily with dlopen so that the library loads
// (and its symbol table can be checked) on a machine with no GPU driver; the
// first call that needs one of them reports MLCB_ERR_LIBRARY if it is missing.
// cuda.h / nvrtc.h are used for types and enumerators only.

#include "../../include/mlcb.h"

#include <cuda.h>
#include <nvrtc.h>

#include <dlfcn.h>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#define MLCB_STR2(x) #x
#define MLCB_STR(x) MLCB_STR2(x)

namespace {

thread_local std::string g_error;

int fail(int code, const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_error = buf;
    return code;
}

// ---- driver ----------------------------------------------------------------
struct Driver {
    void* lib = nullptr;
    CUresult (*Init)(unsigned) = nullptr;
    CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
    CUresult (*DeviceGet)(CUdevice*, int) = nullptr;
    CUresult (*PrimaryCtxRetain)(CUcontext*, CUdevice) = nullptr;
    CUresult (*PrimaryCtxRelease)(CUdevice) = nullptr;
    CUresult (*CtxPushCurrent)(CUcontext) = nullptr;
    CUresult (*CtxPopCurrent)(CUcontext*) = nullptr;
    CUresult (*CtxGetCurrent)(CUcontext*) = nullptr;
    CUresult (*CtxSetCurrent)(CUcontext) = nullptr;
    CUresult (*ModuleLoadData)(CUmodule*, const void*) = nullptr;
    CUresult (*ModuleUnload)(CUmodule) = nullptr;
    CUresult (*ModuleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
    CUresult (*FuncGetAttribute)(int*, CUfunction_attribute, CUfunction) = nullptr;
    CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned,
                             unsigned, unsigned, CUstream, void**, void**) = nullptr;
    CUresult (*LaunchKernelEx)(const CUlaunchConfig*, CUfunction, void**, void**) = nullptr;
    bool ok = false;
};

Driver g_drv;
std::once_flag g_drv_once;

template <typename F>
bool sym(void* lib, const char* name, F& out) {
    out = reinterpret_cast<F>(dlsym(lib, name));
    return out != nullptr;
}

void load_driver() {
    Driver& d = g_drv;
    d.lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
    if (!d.lib) d.lib = dlopen("libcuda.so", RTLD_NOW | RTLD_GLOBAL);
    if (!d.lib) return;
    bool ok = true;
    ok &= sym(d.lib, MLCB_STR(cuInit), d.Init);
    ok &= sym(d.lib, MLCB_STR(cuGetErrorString), d.GetErrorString);
    ok &= sym(d.lib, MLCB_STR(cuDeviceGet), d.DeviceGet);
    ok &= sym(d.lib, MLCB_STR(cuDevicePrimaryCtxRetain), d.PrimaryCtxRetain);
    ok &= sym(d.lib, MLCB_STR(cuDevicePrimaryCtxRelease), d.PrimaryCtxRelease);
    ok &= sym(d.lib, MLCB_STR(cuCtxPushCurrent), d.CtxPushCurrent);
    ok &= sym(d.lib, MLCB_STR(cuCtxPopCurrent), d.CtxPopCurrent);
    ok &= sym(d.lib, MLCB_STR(cuCtxGetCurrent), d.CtxGetCurrent);
    ok &= sym(d.lib, MLCB_STR(cuCtxSetCurrent), d.CtxSetCurrent);
    ok &= sym(d.lib, MLCB_STR(cuModuleLoadData), d.ModuleLoadData);
    ok &= sym(d.lib, MLCB_STR(cuModuleUnload), d.ModuleUnload);
    ok &= sym(d.lib, MLCB_STR(cuModuleGetFunction), d.ModuleGetFunction);
    ok &= sym(d.lib, MLCB_STR(cuFuncGetAttribute), d.FuncGetAttribute);
    ok &= sym(d.lib, MLCB_STR(cuLaunchKernel), d.LaunchKernel);
    ok &= sym(d.lib, MLCB_STR(cuLaunchKernelEx), d.LaunchKernelEx);
    if (ok && d.Init(0) == CUDA_SUCCESS) d.ok = true;
}

int need_driver() {
    std::call_once(g_drv_once, load_driver);
    if (!g_drv.ok)
        return fail(MLCB_ERR_LIBRARY, "CUDA driver (libcuda.so.1) is not available: %s",
                    g_drv.lib ? "cuInit failed or a symbol is missing" : dlerror());
    return 0;
}

int cu_fail(CUresult r, const char* what) {
    const char* msg = nullptr;
    if (g_drv.GetErrorString) g_drv.GetErrorString(r, &msg);
    return fail((int)r, "%s: %s (CUresult %d)", what, msg ? msg : "unknown error", (int)r);
}

// ---- nvrtc -----------------------------------------------------------------
struct Rtc {
    void* lib = nullptr;
    const char* (*GetErrorString)(nvrtcResult) = nullptr;
    nvrtcResult (*CreateProgram)(nvrtcProgram*, const char*, const char*, int,
                                 const char* const*, const char* const*) = nullptr;
    nvrtcResult (*DestroyProgram)(nvrtcProgram*) = nullptr;
    nvrtcResult (*CompileProgram)(nvrtcProgram, int, const char* const*) = nullptr;
    nvrtcResult (*GetCUBINSize)(nvrtcProgram, size_t*) = nullptr;
    nvrtcResult (*GetCUBIN)(nvrtcProgram, char*) = nullptr;
    nvrtcResult (*GetProgramLogSize)(nvrtcProgram, size_t*) = nullptr;
    nvrtcResult (*GetProgramLog)(nvrtcProgram, char*) = nullptr;
    bool ok = false;
};

Rtc g_rtc;
std::once_flag g_rtc_once;

void load_rtc() {
    Rtc& r = g_rtc;
    const char* names[] = {"libnvrtc.so.12", "libnvrtc.so", "libnvrtc.so.13"};
    for (const char* n : names) {
        r.lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (r.lib) break;
    }
    if (!r.lib) {
        // a toolkit that is installed but not on the loader path
        const char* homes[] = {getenv("CUDA_HOME"), getenv("CUDA_PATH"), "/usr/local/cuda"};
        for (const char* h : homes) {
            if (!h) continue;
            std::string p = std::string(h) + "/lib64/libnvrtc.so";
            r.lib = dlopen(p.c_str(), RTLD_NOW | RTLD_GLOBAL);
            if (r.lib) break;
        }
    }
    if (!r.lib) return;
    bool ok = true;
    ok &= sym(r.lib, "nvrtcGetErrorString", r.GetErrorString);
    ok &= sym(r.lib, "nvrtcCreateProgram", r.CreateProgram);
    ok &= sym(r.lib, "nvrtcDestroyProgram", r.DestroyProgram);
    ok &= sym(r.lib, "nvrtcCompileProgram", r.CompileProgram);
    ok &= sym(r.lib, "nvrtcGetCUBINSize", r.GetCUBINSize);
    ok &= sym(r.lib, "nvrtcGetCUBIN", r.GetCUBIN);
    ok &= sym(r.lib, "nvrtcGetProgramLogSize", r.GetProgramLogSize);
    ok &= sym(r.lib, "nvrtcGetProgramLog", r.GetProgramLog);
    r.ok = ok;
}

int need_rtc() {
    std::call_once(g_rtc_once, load_rtc);
    if (!g_rtc.ok)
        return fail(MLCB_ERR_LIBRARY, "NVRTC (libnvrtc.so.12) is not available");
    return 0;
}

// Makes `want` the calling thread's current context for the guard's lifetime
// when it is not already (a thread that has not touched the runtime yet, or one
// whose current device is another GPU), and restores what was there before.
struct CtxGuard {
    bool pushed = false;
    explicit CtxGuard(CUcontext want) {
        CUcontext cur = nullptr;
        if (g_drv.CtxGetCurrent(&cur) != CUDA_SUCCESS || cur != want)
            pushed = g_drv.CtxPushCurrent(want) == CUDA_SUCCESS;
    }
    ~CtxGuard() {
        if (pushed) {
            CUcontext popped = nullptr;
            g_drv.CtxPopCurrent(&popped);
        }
    }
    CtxGuard(const CtxGuard&) = delete;
    CtxGuard& operator=(const CtxGuard&) = delete;
};

void copy_log(const std::string& s, char* log, size_t cap) {
    if (!log || cap == 0) return;
    size_t n = s.size() < cap - 1 ? s.size() : cap - 1;
    memcpy(log, s.data(), n);
    log[n] = 0;
}

}  // namespace

struct mlcb_module {
    CUmodule mod = nullptr;
    CUcontext ctx = nullptr;
    CUdevice dev = 0;
    std::vector<mlcb_kernel*> kernels;
};

struct mlcb_kernel {
    CUfunction fn = nullptr;
    mlcb_module* owner = nullptr;
    std::string name;
};

extern "C" {

int mlcb_version(void) { return MLCB_ABI_VERSION; }

const char* mlcb_last_error(void) { return g_error.c_str(); }

int mlcb_compile(const char* src, const char* arch, const char* const* opts, int nopts,
                 void** image, size_t* size, char* log, size_t logcap) {
    if (log && logcap) log[0] = 0;
    if (!src || !image || !size) return fail(MLCB_ERR_ARGUMENT, "mlcb_compile: null argument");
    *image = nullptr;
    *size = 0;
    if (int e = need_rtc()) return e;
    Rtc& r = g_rtc;

    nvrtcProgram prog = nullptr;
    nvrtcResult rc = r.CreateProgram(&prog, src, "mlcb_module.cu", 0, nullptr, nullptr);
    if (rc != NVRTC_SUCCESS)
        return fail(MLCB_NVRTC_BASE + (int)rc, "nvrtcCreateProgram: %s", r.GetErrorString(rc));

    std::vector<std::string> owned;
    owned.push_back(std::string("--gpu-architecture=") + (arch && *arch ? arch : "sm_100a"));
    for (int i = 0; i < nopts; ++i)
        if (opts && opts[i]) owned.push_back(opts[i]);
    std::vector<const char*> argv;
    for (auto& s : owned) argv.push_back(s.c_str());

    rc = r.CompileProgram(prog, (int)argv.size(), argv.data());
    size_t ln = 0;
    std::string text;
    if (r.GetProgramLogSize(prog, &ln) == NVRTC_SUCCESS && ln > 1) {
        text.resize(ln);
        r.GetProgramLog(prog, &text[0]);
        while (!text.empty() && text.back() == 0) text.pop_back();
    }
    copy_log(text, log, logcap);
    if (rc != NVRTC_SUCCESS) {
        r.DestroyProgram(&prog);
        return fail(MLCB_NVRTC_BASE + (int)rc, "nvrtcCompileProgram: %s\n%.700s",
                    r.GetErrorString(rc), text.c_str());
    }
    size_t n = 0;
    rc = r.GetCUBINSize(prog, &n);
    if (rc != NVRTC_SUCCESS || n == 0) {
        r.DestroyProgram(&prog);
        return fail(MLCB_NVRTC_BASE + (int)rc, "nvrtcGetCUBINSize: %s (is arch a real sm_ target?)",
                    r.GetErrorString(rc));
    }
    char* buf = (char*)malloc(n);
    if (!buf) {
        r.DestroyProgram(&prog);
        return fail(MLCB_ERR_ARGUMENT, "mlcb_compile: out of host memory");
    }
    rc = r.GetCUBIN(prog, buf);
    r.DestroyProgram(&prog);
    if (rc != NVRTC_SUCCESS) {
        free(buf);
        return fail(MLCB_NVRTC_BASE + (int)rc, "nvrtcGetCUBIN: %s", r.GetErrorString(rc));
    }
    *image = buf;
    *size = n;
    return 0;
}

void mlcb_free_image(void* image) { free(image); }

int mlcb_module_load(const void* image, size_t size, int device, mlcb_module** out) {
    if (!image || !size || !out) return fail(MLCB_ERR_ARGUMENT, "mlcb_module_load: null argument");
    *out = nullptr;
    if (int e = need_driver()) return e;
    Driver& d = g_drv;
    CUdevice dev;
    CUresult r = d.DeviceGet(&dev, device);
    if (r != CUDA_SUCCESS) return cu_fail(r, "cuDeviceGet");
    CUcontext ctx = nullptr;
    r = d.PrimaryCtxRetain(&ctx, dev);
    if (r != CUDA_SUCCESS) return cu_fail(r, "cuDevicePrimaryCtxRetain");
    r = d.CtxPushCurrent(ctx);
    if (r != CUDA_SUCCESS) {
        d.PrimaryCtxRelease(dev);
        return cu_fail(r, "cuCtxPushCurrent");
    }
    CUmodule mod = nullptr;
    r = d.ModuleLoadData(&mod, image);
    CUcontext popped = nullptr;
    d.CtxPopCurrent(&popped);
    if (r != CUDA_SUCCESS) {
        d.PrimaryCtxRelease(dev);
        return cu_fail(r, "cuModuleLoadData");
    }
    mlcb_module* m = new mlcb_module();
    m->mod = mod;
    m->ctx = ctx;
    m->dev = dev;
    *out = m;
    return 0;
}

int mlcb_module_unload(mlcb_module* m) {
    if (!m) return 0;
    int rc = 0;
    if (g_drv.ok && m->mod) {
        g_drv.CtxPushCurrent(m->ctx);
        CUresult r = g_drv.ModuleUnload(m->mod);
        CUcontext popped = nullptr;
        g_drv.CtxPopCurrent(&popped);
        g_drv.PrimaryCtxRelease(m->dev);
        if (r != CUDA_SUCCESS) rc = cu_fail(r, "cuModuleUnload");
    }
    for (mlcb_kernel* k : m->kernels) delete k;
    delete m;
    return rc;
}

int mlcb_get_kernel(mlcb_module* m, const char* name, mlcb_kernel** out) {
    if (!m || !name || !out) return fail(MLCB_ERR_ARGUMENT, "mlcb_get_kernel: null argument");
    *out = nullptr;
    if (int e = need_driver()) return e;
    CUfunction fn = nullptr;
    CtxGuard in_module_context(m->ctx);
    CUresult r = g_drv.ModuleGetFunction(&fn, m->mod, name);
    if (r != CUDA_SUCCESS) {
        char what[256];
        snprintf(what, sizeof what, "cuModuleGetFunction(%s)", name);
        return cu_fail(r, what);
    }
    mlcb_kernel* k = new mlcb_kernel();
    k->fn = fn;
    k->owner = m;
    k->name = name;
    m->kernels.push_back(k);
    *out = k;
    return 0;
}

int mlcb_kernel_info(mlcb_kernel* k, int* regs, int* static_smem, int* max_threads) {
    if (!k) return fail(MLCB_ERR_ARGUMENT, "mlcb_kernel_info: null kernel");
    if (int e = need_driver()) return e;
    CtxGuard in_module_context(k->owner->ctx);
    CUresult r;
    if (regs && (r = g_drv.FuncGetAttribute(regs, CU_FUNC_ATTRIBUTE_NUM_REGS, k->fn)) != CUDA_SUCCESS)
        return cu_fail(r, "cuFuncGetAttribute(NUM_REGS)");
    if (static_smem &&
        (r = g_drv.FuncGetAttribute(static_smem, CU_FUNC_ATTRIBUTE_SHARED_SIZE_BYTES, k->fn)) != CUDA_SUCCESS)
        return cu_fail(r, "cuFuncGetAttribute(SHARED_SIZE_BYTES)");
    if (max_threads &&
        (r = g_drv.FuncGetAttribute(max_threads, CU_FUNC_ATTRIBUTE_MAX_THREADS_PER_BLOCK, k->fn)) != CUDA_SUCCESS)
        return cu_fail(r, "cuFuncGetAttribute(MAX_THREADS_PER_BLOCK)");
    return 0;
}

static int launch_one(mlcb_kernel* k, uint32_t grid_x, uint32_t block_x, uint32_t smem_bytes,
                      const uint64_t* device_ptrs, int nptrs, uint64_t stream, uint32_t flags) {
    enum { MAX_PTRS = 64 };
    if (!k || nptrs < 0 || nptrs > MAX_PTRS || (nptrs && !device_ptrs) || !grid_x || !block_x)
        return fail(MLCB_ERR_ARGUMENT, "mlcb_launch: bad argument (kernel=%p nptrs=%d grid=%u block=%u)",
                    (void*)k, nptrs, grid_x, block_x);
    // every kernel parameter is a pointer; the driver copies the values now
    uint64_t vals[MAX_PTRS];
    void* args[MAX_PTRS];
    for (int i = 0; i < nptrs; ++i) {
        vals[i] = device_ptrs[i];
        args[i] = &vals[i];
    }
    Driver& d = g_drv;
    CUresult r;
    // the launch happens in the context the module was loaded into, whatever the
    // calling thread had current; `stream` must belong to that context
    CtxGuard in_module_context(k->owner->ctx);
    {
        if (flags & MLCB_LAUNCH_DEPENDENT) {
            CUlaunchAttribute attr;
            memset(&attr, 0, sizeof attr);
            attr.id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
            attr.value.programmaticStreamSerializationAllowed = 1;
            CUlaunchConfig cfg;
            memset(&cfg, 0, sizeof cfg);
            cfg.gridDimX = grid_x;
            cfg.gridDimY = cfg.gridDimZ = 1;
            cfg.blockDimX = block_x;
            cfg.blockDimY = cfg.blockDimZ = 1;
            cfg.sharedMemBytes = smem_bytes;
            cfg.hStream = (CUstream)(uintptr_t)stream;
            cfg.attrs = &attr;
            cfg.numAttrs = 1;
            r = d.LaunchKernelEx(&cfg, k->fn, args, nullptr);
        } else {
            r = d.LaunchKernel(k->fn, grid_x, 1, 1, block_x, 1, 1, smem_bytes,
                               (CUstream)(uintptr_t)stream, args, nullptr);
        }
    }
    if (r != CUDA_SUCCESS) {
        char what[256];
        snprintf(what, sizeof what, "launch of %s <<<%u, %u>>>", k->name.c_str(), grid_x, block_x);
        return cu_fail(r, what);
    }
    return 0;
}

int mlcb_launch(mlcb_kernel* k, uint32_t grid_x, uint32_t block_x, uint32_t smem_bytes,
                const uint64_t* device_ptrs, int nptrs, uint64_t stream, uint32_t flags) {
    if (!g_drv.ok)
        if (int e = need_driver()) return e;
    return launch_one(k, grid_x, block_x, smem_bytes, device_ptrs, nptrs, stream, flags);
}

int mlcb_launch_many(const mlcb_launch_desc* descs, int n, uint64_t stream, int* failed_at) {
    if (failed_at) *failed_at = -1;
    if (n < 0 || (n && !descs)) return fail(MLCB_ERR_ARGUMENT, "mlcb_launch_many: bad argument");
    if (!g_drv.ok)
        if (int e = need_driver()) return e;
    for (int i = 0; i < n; ++i) {
        const mlcb_launch_desc& d = descs[i];
        int e = launch_one(d.kernel, d.grid_x, d.block_x, d.smem_bytes, d.device_ptrs, d.nptrs,
                           stream, d.flags);
        if (e) {
            if (failed_at) *failed_at = i;
            return e;
        }
    }
    return 0;
}

}  // extern "C"
