// Error reporting and ABI self-description.
#include <stdint.h>
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

int make_rows_map(CUtensorMap* out, const void* base, int elem_bytes, unsigned long long rows, unsigned long long row_elems, const char* what) {
    typedef CUresult (*Encode)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                               const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static Encode encode = nullptr;                    // resolved through the runtime: the library does not link against the driver
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
            (void)cudaGetLastError();
            snprintf(g_err, sizeof(g_err), "%s: the driver does not provide cuTensorMapEncodeTiled", what);
            return MKDA_ERR_LAUNCH;
        }
        encode = reinterpret_cast<Encode>(fn);
    }
    const unsigned long long pitch = row_elems * (unsigned long long)elem_bytes;
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (pitch & 15) || row_elems < 128 || rows == 0) {
        snprintf(g_err, sizeof(g_err), "%s: tensor not 16-byte aligned for tiled copies", what);
        return MKDA_ERR_ARG;
    }
    const cuuint64_t gdim[2] = {row_elems, rows};
    const cuuint64_t gstride[1] = {pitch};
    const cuuint32_t box[2] = {128, 64}, estr[2] = {1, 1};
    const CUresult r = encode(out, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base), gdim,
                              gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(g_err, sizeof(g_err), "%s: cuTensorMapEncodeTiled failed (%d)", what, (int)r);
        return MKDA_ERR_LAUNCH;
    }
    return MKDA_OK;
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
extern "C" int mkda_abi_version(void) { return 4; }
extern "C" int mkda_struct_sizes(int* out, int n) {
    const int sizes[] = {
        (int)sizeof(MkdaLayout),   (int)sizeof(MkdaGateFwd),  (int)sizeof(MkdaGateBwd),     (int)sizeof(MkdaReduce),
        (int)sizeof(MkdaL2Norm),   (int)sizeof(MkdaIntraFwd), (int)sizeof(MkdaRecurFwd),    (int)sizeof(MkdaOutFwd),
        (int)sizeof(MkdaEpilogueBwd), (int)sizeof(MkdaEpilogueBwdTiles), (int)sizeof(MkdaEpilogueBwdNoAlloc), (int)sizeof(MkdaBwdDh), (int)sizeof(MkdaBwdChunk),
        (int)sizeof(MkdaQkGrad),   (int)sizeof(MkdaCombine), (int)sizeof(MkdaWarmup), (int)sizeof(MkdaSelfTest), (int)sizeof(MkdaSelfTestWait)};
    const int cnt = (int)(sizeof(sizes) / sizeof(sizes[0]));
    for (int i = 0; i < n && i < cnt; ++i) out[i] = sizes[i];
    return cnt;
}
