// Status reporting, device probing and the per-device default workspace.
#include <stdarg.h>

#include <mutex>

#include <stdlib.h>

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
static int g_sms[kMaxDev];

bool pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char *e = getenv("B200K_PDL");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

int sm_count() {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= kMaxDev) return 148;
    if (g_sms[dev] == 0) {
        int n = 0;
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        g_sms[dev] = n > 0 ? n : 148;
    }
    return g_sms[dev];
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

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int make_tensor_map(CUtensorMap *map, CUtensorMapDataType dtype, int rank, const void *base, const uint64_t *dims,
                    const uint64_t *strides_bytes, const uint32_t *box, CUtensorMapSwizzle swizzle) {
    static EncodeTiledFn encode = nullptr;
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) {
            cudaGetLastError();
            return fail(B200K_E_DEVICE, "cuTensorMapEncodeTiled is not available from the driver");
        }
        encode = (EncodeTiledFn)fn;
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
