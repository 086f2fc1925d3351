// Status reporting, device probing and the per-device default workspace.
#include <stdarg.h>

#include <atomic>
#include <mutex>

#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "tma.cuh"

namespace b200k {

static thread_local char g_err[512] = "";

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int launch_status(const char *what) {
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return 0;
    snprintf(g_err, sizeof(g_err), "%s: %s", what, cudaGetErrorString(e));
    return (int)e;
}

static const int kMaxDev = 16;
static std::mutex g_mu;
static void *g_ws[kMaxDev];
static size_t g_ws_bytes[kMaxDev];
static bool g_ws_owned[kMaxDev];
static std::atomic<int> g_sms[kMaxDev];

// Environment overrides are read once per process and kept: at most 32 distinct names, looked up under a mutex
// the first time and lock-free afterwards (entries are published with release stores and never change).
namespace {
struct EnvEntry {
    std::atomic<const char *> name{nullptr};
    int value = 0;
    int first_char = 0;
    bool set = false;
};
EnvEntry g_env[32];
std::mutex g_env_mu;
const EnvEntry *env_lookup(const char *name) {
    for (auto &e : g_env) {
        const char *n = e.name.load(std::memory_order_acquire);
        if (!n) break;
        if (n == name || !strcmp(n, name)) return &e;
    }
    std::lock_guard<std::mutex> lk(g_env_mu);
    for (auto &e : g_env) {
        const char *n = e.name.load(std::memory_order_relaxed);
        if (n && !strcmp(n, name)) return &e;
        if (!n) {
            const char *v = getenv(name);
            e.set = v && v[0];
            e.value = e.set ? atoi(v) : 0;
            e.first_char = e.set ? (unsigned char)v[0] : 0;
            e.name.store(name, std::memory_order_release);   // callers pass string literals
            return &e;
        }
    }
    return nullptr;   // table full: treated as unset
}
}  // namespace

int env_int(const char *name, int dflt) {
    const EnvEntry *e = env_lookup(name);
    return e && e->set ? e->value : dflt;
}
int env_char(const char *name) {
    const EnvEntry *e = env_lookup(name);
    return e && e->set ? e->first_char : 0;
}

bool pdl_enabled() { return env_char("B200K_PDL") != '0'; }

int sm_count() {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= kMaxDev) return 148;
    int n = g_sms[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        n = n > 0 ? n : 148;
        g_sms[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

int default_workspace(void **ptr, size_t *bytes) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDev)
        return fail(B200K_E_DEVICE, "default workspace: no usable current device");
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_ws[dev]) {
        void *p = nullptr;
        e = cudaMalloc(&p, B200K_DEFAULT_WORKSPACE_BYTES);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fail(B200K_E_WORKSPACE, "default workspace: cudaMalloc of %zu bytes failed: %s",
                        (size_t)B200K_DEFAULT_WORKSPACE_BYTES, cudaGetErrorString(e));
        }
        // Counters inside the workspace must start at zero; kernels leave them at zero.
        cudaMemset(p, 0, B200K_DEFAULT_WORKSPACE_BYTES);
        g_ws[dev] = p;
        g_ws_bytes[dev] = B200K_DEFAULT_WORKSPACE_BYTES;
        g_ws_owned[dev] = true;
    }
    *ptr = g_ws[dev];
    *bytes = g_ws_bytes[dev];
    return 0;
}

int *status_word() {
    void *ws = nullptr;
    size_t bytes = 0;
    return default_workspace(&ws, &bytes) == 0 ? (int *)ws : nullptr;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int make_tensor_map(CUtensorMap *map, CUtensorMapDataType dtype, int rank, const void *base, const uint64_t *dims,
                    const uint64_t *strides_bytes, const uint32_t *box, CUtensorMapSwizzle swizzle) {
    static std::atomic<EncodeTiledFn> encode_fn{nullptr};
    EncodeTiledFn encode = encode_fn.load(std::memory_order_acquire);
    if (!encode) {   // several threads may look it up at once: they all store the same pointer
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) {
            cudaGetLastError();
            return fail(B200K_E_DEVICE, "cuTensorMapEncodeTiled is not available from the driver");
        }
        encode = (EncodeTiledFn)fn;
        encode_fn.store(encode, std::memory_order_release);
    }
    cuuint64_t gdim[5], gstr[4];
    cuuint32_t bdim[5], estr[5];
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        bdim[i] = box[i];
        estr[i] = 1;
        if (i > 0) gstr[i - 1] = strides_bytes[i - 1];
    }
    CUresult r = encode(map, dtype, (cuuint32_t)rank, const_cast<void *>(base), gdim, gstr, bdim, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B200K_E_ALIGN, "tensor map rejected by the driver (CUresult %d)", (int)r);
    return 0;
}

}  // namespace b200k

using namespace b200k;

extern "C" const char *b200k_last_error(void) { return g_err; }
extern "C" const char *b200k_version(void) { return "b200_kernels 0.1 (sm_100a)"; }

extern "C" int b200k_device_check(void) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(B200K_E_DEVICE, "no CUDA device: %s", cudaGetErrorString(e));
    }
    int major = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (major != 10) return fail(B200K_E_DEVICE, "device %d has compute capability %d.x, need 10.x", dev, major);
    return 0;
}

extern "C" int b200k_set_workspace(void *workspace, size_t bytes) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev)
        return fail(B200K_E_DEVICE, "set_workspace: no usable current device");
    B200K_REQUIRE(workspace != nullptr, B200K_E_NULL, "set_workspace: workspace is NULL");
    B200K_REQUIRE(aligned16(workspace) && bytes >= (1u << 20), B200K_E_WORKSPACE,
                  "set_workspace: need a 16-byte aligned buffer of at least 1 MiB");
    // status word and arrival counters (first 128 KiB) start at zero; kernels leave them at zero
    if (cudaMemset(workspace, 0, 128 * 1024) != cudaSuccess) {
        cudaGetLastError();
        return fail(B200K_E_WORKSPACE, "set_workspace: cannot clear the buffer (is it device memory?)");
    }
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_ws[dev] && g_ws_owned[dev]) cudaFree(g_ws[dev]);
    g_ws[dev] = workspace;
    g_ws_bytes[dev] = bytes;
    g_ws_owned[dev] = false;
    return 0;
}

extern "C" int b200k_workspace_status(const void *workspace, int *host_status_out, b200k_stream stream) {
    B200K_REQUIRE(workspace && host_status_out, B200K_E_NULL, "b200k_workspace_status: NULL pointer");
    cudaError_t e = cudaMemcpyAsync(host_status_out, workspace, sizeof(int), cudaMemcpyDeviceToHost, to_stream(stream));
    if (e == cudaSuccess) e = cudaStreamSynchronize(to_stream(stream));
    if (e != cudaSuccess) return fail((int)e, "b200k_workspace_status: %s", cudaGetErrorString(e));
    return 0;
}

extern "C" int b200k_workspace_clear_status(void *workspace, b200k_stream stream) {
    B200K_REQUIRE(workspace, B200K_E_NULL, "b200k_workspace_clear_status: NULL pointer");
    cudaError_t e = cudaMemsetAsync(workspace, 0, sizeof(int), to_stream(stream));
    if (e != cudaSuccess) return fail((int)e, "b200k_workspace_clear_status: %s", cudaGetErrorString(e));
    return 0;
}
