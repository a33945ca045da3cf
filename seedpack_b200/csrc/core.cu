// Library-wide state: status word, error text, type table.
#include <cstring>
#include <mutex>
#include <string>

#include "api_util.h"

namespace sg {

__device__ int g_status = 0;

static thread_local std::string t_cuda_error;
static std::mutex g_mu;
static constexpr int MAX_DEV = 64;
static int* g_status_ptr[MAX_DEV] = {nullptr};

int cuda_ok(cudaError_t e) {
    if (e == cudaSuccess) return SG_OK;
    t_cuda_error = std::string(cudaGetErrorName(e)) + ": " + cudaGetErrorString(e);
    return SG_ERR_CUDA;
}

int use_device(int device) {
    if (device < 0 || device >= MAX_DEV) return SG_ERR_ARG;
    return cuda_ok(cudaSetDevice(device));
}

int* status_word(int device) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_status_ptr[device]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_status) != cudaSuccess) return nullptr;
        g_status_ptr[device] = (int*)p;
    }
    return g_status_ptr[device];
}

struct TypeInfo { int type, qk, bs, needs_imx; };
static const TypeInfo TYPES[] = {
    {SG_Q4_0, 32, 18, 0}, {SG_Q4_1, 32, 20, 0}, {SG_Q5_0, 32, 22, 0}, {SG_Q5_1, 32, 24, 0}, {SG_Q8_0, 32, 34, 0},
    {SG_Q2_K, 256, 84, 0}, {SG_Q3_K, 256, 110, 0}, {SG_Q4_K, 256, 144, 0}, {SG_Q5_K, 256, 176, 0}, {SG_Q6_K, 256, 210, 0},
    {SG_IQ2_XXS, 256, 66, 1}, {SG_IQ2_XS, 256, 74, 1}, {SG_IQ3_XXS, 256, 98, 0}, {SG_IQ1_S, 256, 50, 1},
    {SG_IQ4_NL, 32, 18, 0}, {SG_IQ3_S, 256, 110, 0}, {SG_IQ2_S, 256, 82, 0}, {SG_IQ4_XS, 256, 136, 0},
    {SG_IQ1_M, 256, 56, 0}, {SG_Q2_0, 64, 18, 0},
    {SG_TQ1_0, 256, 54, 0}, {SG_TQ2_0, 256, 66, 0}, {SG_MXFP4, 32, 17, 0}, {SG_NVFP4, 64, 36, 0}, {SG_Q1_0, 128, 18, 0},
};

}  // namespace sg

using namespace sg;

extern "C" int sg_version(void) { return 100; }

extern "C" const char* sg_status_string(int s) {
    switch (s) {
        case SG_OK: return "ok";
        case SG_ERR_ARG: return "bad argument";
        case SG_ERR_TYPE: return "unsupported ggml type or variant";
        case SG_ERR_SHAPE: return "row length is not a multiple of the block size";
        case SG_ERR_ALIGN: return "offset or pointer not aligned for vector access";
        case SG_ERR_IMATRIX: return "this type needs an importance matrix";
        case SG_ERR_SCRATCH: return "scratch buffer missing or too small";
        case SG_ERR_TABLES: return "IQ tables are not installed on this device";
        case SG_ERR_CUDA: return "CUDA runtime error";
        case SG_ERR_OVERFLOW: return "output slot too small";
        case SG_ERR_CORRUPT: return "coded stream is corrupt";
        case SG_ERR_LIMIT: return "size beyond a fixed maximum";
        default: return "unknown status";
    }
}

extern "C" const char* sg_last_cuda_error(void) { return t_cuda_error.c_str(); }

extern "C" int sg_type_info(int type, int* qk, int* bs) {
    for (const TypeInfo& t : TYPES)
        if (t.type == type) {
            if (qk) *qk = t.qk;
            if (bs) *bs = t.bs;
            return SG_OK;
        }
    return SG_ERR_TYPE;
}

extern "C" int sg_type_needs_imatrix(int type) {
    for (const TypeInfo& t : TYPES) if (t.type == type) return t.needs_imx;
    return 0;
}

extern "C" int sg_status_fetch(int device, void* stream, int* h_bits) {
    if (!h_bits) return SG_ERR_ARG;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    int* p = status_word(device);
    if (!p) return SG_ERR_CUDA;
    cudaStream_t st = (cudaStream_t)stream;
    rc = cuda_ok(cudaMemcpyAsync(h_bits, p, sizeof(int), cudaMemcpyDeviceToHost, st));
    if (rc != SG_OK) return rc;
    rc = cuda_ok(cudaMemsetAsync(p, 0, sizeof(int), st));
    if (rc != SG_OK) return rc;
    return cuda_ok(cudaStreamSynchronize(st));
}
