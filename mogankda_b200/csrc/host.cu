// Error reporting and ABI self-description.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/mkda.h"
#include "host.h"

namespace mkda {

static thread_local char g_err[512] = "";

int set_error(int code, const char* msg) {
    snprintf(g_err, sizeof(g_err), "%s", msg);
    return code;
}

int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        snprintf(g_err, sizeof(g_err), "%s: %s", what, cudaGetErrorString(e));
        return MKDA_ERR_LAUNCH;
    }
    return MKDA_OK;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!cached[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

int ensure_smem(const void* func, int bytes, const char* what) {
    // (function, device) pairs whose limit is already raised; a launcher asks before every launch
    struct Done { const void* func; int dev; int bytes; };
    static Done done[256];
    static int ndone = 0;
    int dev = 0;
    (void)cudaGetDevice(&dev);
    for (int i = 0; i < ndone; ++i)
        if (done[i].func == func && done[i].dev == dev && done[i].bytes >= bytes) return MKDA_OK;
    cudaError_t e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) {
        snprintf(g_err, sizeof(g_err), "%s: cannot reserve %d bytes of shared memory: %s", what, bytes, cudaGetErrorString(e));
        (void)cudaGetLastError();
        return MKDA_ERR_LAUNCH;
    }
    if (ndone < 256) done[ndone++] = Done{func, dev, bytes};      // single-threaded host, as the reference assumes
    return MKDA_OK;
}

}  // namespace mkda

namespace mkda {
int selftest_status(unsigned int* out);
int selftest_status_clear();
}
extern "C" int mkda_device_status(void) {
    unsigned int f = 0, any = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (mkda::selftest_status(&f) == 0) any |= f;
    if (mkda::tc_chunk_status(&f) == 0) any |= f;
    if (mkda::tc_recur_status(&f) == 0) any |= f;
    if (mkda::tc_intra_status(&f) == 0) any |= f;
    return (int)any;
}
extern "C" int mkda_device_status_clear(void) {
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    int rc = 0;
    rc |= mkda::selftest_status_clear();
    rc |= mkda::tc_chunk_status_clear();
    rc |= mkda::tc_recur_status_clear();
    rc |= mkda::tc_intra_status_clear();
    return rc;
}
extern "C" const char* mkda_last_error(void) { return mkda::g_err; }
extern "C" int mkda_abi_version(void) { return 3; }
extern "C" int mkda_struct_sizes(int* out, int n) {
    const int sizes[] = {
        (int)sizeof(MkdaLayout),   (int)sizeof(MkdaGateFwd),  (int)sizeof(MkdaGateBwd),     (int)sizeof(MkdaReduce),
        (int)sizeof(MkdaL2Norm),   (int)sizeof(MkdaIntraFwd), (int)sizeof(MkdaRecurFwd),    (int)sizeof(MkdaOutFwd),
        (int)sizeof(MkdaEpilogueBwd), (int)sizeof(MkdaEpilogueBwdTiles), (int)sizeof(MkdaEpilogueBwdNoAlloc), (int)sizeof(MkdaBwdDh), (int)sizeof(MkdaBwdChunk),
        (int)sizeof(MkdaQkGrad),   (int)sizeof(MkdaCombine), (int)sizeof(MkdaSelfTest), (int)sizeof(MkdaSelfTestWait)};
    const int cnt = (int)(sizeof(sizes) / sizeof(sizes[0]));
    for (int i = 0; i < n && i < cnt; ++i) out[i] = sizes[i];
    return cnt;
}
