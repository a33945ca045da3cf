// C-ABI entry points of the re-quantisers and their launch logic.
#include <cstdio>
#include <cstring>
#include <mutex>

#include "api_util.h"
#include "quant_iq.cuh"
#include "quant_extra.cuh"
#include "quant_legacy.cuh"

namespace sg {

template <class T, int DT, bool IMX>
__global__ void __launch_bounds__(128) k_quant(const __grid_constant__ Job job) {
    constexpr int LANES = T::LANES;
    const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long s = g / LANES;
    const int sub = (int)(g - s * LANES);
    const bool valid = s < job.nslabs;
    if (!valid) s = job.nslabs - 1;          // keep the lane alive for the group's shuffles
    const Slab sl = locate<T::SLAB>(job, s);
    T::template run<DT, IMX>(job, sl, sub, valid);
}

template <class T, bool IMX>
static int launch(const Job& job, int dt, cudaStream_t st) {
    const long long threads = job.nslabs * T::LANES;
    const unsigned grid = (unsigned)((threads + 127) / 128);
    if (grid == 0) return SG_OK;
    switch (dt) {
        case SG_DT_BF16: k_quant<T, SG_DT_BF16, IMX><<<grid, 128, 0, st>>>(job); break;
        case SG_DT_F16:  k_quant<T, SG_DT_F16, IMX><<<grid, 128, 0, st>>>(job); break;
        case SG_DT_F32:  k_quant<T, SG_DT_F32, IMX><<<grid, 128, 0, st>>>(job); break;
        default: return SG_ERR_ARG;
    }
    return cuda_ok(cudaGetLastError());
}

template <int TYPE>
static int launch_legacy_ref(const Job& job, int dt, cudaStream_t st) {
    const long long threads = job.nslabs * (256 / LegacyRef<TYPE>::QK);
    const unsigned grid = (unsigned)((threads + 127) / 128);
    if (grid == 0) return SG_OK;
    switch (dt) {
        case SG_DT_BF16: k_quant_legacy_ref<TYPE, SG_DT_BF16><<<grid, 128, 0, st>>>(job); break;
        case SG_DT_F16:  k_quant_legacy_ref<TYPE, SG_DT_F16><<<grid, 128, 0, st>>>(job); break;
        case SG_DT_F32:  k_quant_legacy_ref<TYPE, SG_DT_F32><<<grid, 128, 0, st>>>(job); break;
        default: return SG_ERR_ARG;
    }
    return cuda_ok(cudaGetLastError());
}

static int launch_meansq(const Job& job, long long nrows, int dt, cudaStream_t st) {
    const unsigned grid = (unsigned)((nrows + 3) / 4);
    switch (dt) {
        case SG_DT_BF16: k_row_meansq<SG_DT_BF16><<<grid, 128, 0, st>>>(job, nrows); break;
        case SG_DT_F16:  k_row_meansq<SG_DT_F16><<<grid, 128, 0, st>>>(job, nrows); break;
        case SG_DT_F32:  k_row_meansq<SG_DT_F32><<<grid, 128, 0, st>>>(job, nrows); break;
        default: return SG_ERR_ARG;
    }
    return cuda_ok(cudaGetLastError());
}

static bool legacy_imx_type(int t) { return t == SG_Q4_0 || t == SG_Q4_1 || t == SG_Q5_0 || t == SG_Q5_1; }

// types whose quantize_<t> does the same with and without quant_weights
static bool ignores_imatrix(int type) {
    return type == SG_Q8_0 || type == SG_Q2_0 || type == SG_Q1_0 || type == SG_TQ1_0 || type == SG_TQ2_0 || type == SG_MXFP4 || type == SG_NVFP4;
}

static int dispatch(int type, int variant, bool imx, int device, const Job& job, int dt, cudaStream_t st) {
    switch (type) {
        case SG_Q4_0: return imx ? launch<LegacyImx<SG_Q4_0>, true>(job, dt, st) : launch_legacy_ref<SG_Q4_0>(job, dt, st);
        case SG_Q4_1: return imx ? launch<LegacyImx<SG_Q4_1>, true>(job, dt, st) : launch_legacy_ref<SG_Q4_1>(job, dt, st);
        case SG_Q5_0: return imx ? launch<LegacyImx<SG_Q5_0>, true>(job, dt, st) : launch_legacy_ref<SG_Q5_0>(job, dt, st);
        case SG_Q5_1: return imx ? launch<LegacyImx<SG_Q5_1>, true>(job, dt, st) : launch_legacy_ref<SG_Q5_1>(job, dt, st);
        case SG_Q8_0: return launch_legacy_ref<SG_Q8_0>(job, dt, st);
        case SG_Q2_0: return launch_legacy_ref<SG_Q2_0>(job, dt, st);
        case SG_Q1_0: return launch_extra<SG_Q1_0>(job, dt, st);
        case SG_TQ1_0: return launch_extra<SG_TQ1_0>(job, dt, st);
        case SG_TQ2_0: return launch_extra<SG_TQ2_0>(job, dt, st);
        case SG_MXFP4: return launch_extra<SG_MXFP4>(job, dt, st);
        case SG_NVFP4: return launch_extra<SG_NVFP4>(job, dt, st);
        case SG_Q2_K: return imx ? launch<Q2K, true>(job, dt, st) : launch<Q2K, false>(job, dt, st);
        case SG_Q3_K: return imx ? launch<Q3K, true>(job, dt, st) : launch<Q3K, false>(job, dt, st);
        case SG_Q4_K: return imx ? launch<Q45K<4>, true>(job, dt, st) : launch<Q45K<4>, false>(job, dt, st);
        case SG_Q5_K: return imx ? launch<Q45K<5>, true>(job, dt, st) : launch<Q45K<5>, false>(job, dt, st);
        case SG_Q6_K: return imx ? launch<Q6K, true>(job, dt, st) : launch<Q6K, false>(job, dt, st);
        default: return dispatch_iq(type, variant, imx, device, job, dt, st);
    }
}

}  // namespace sg

using namespace sg;

extern "C" size_t sg_quantize_scratch_bytes(int type, const sg_tensor* h, int n) {
    if (!legacy_imx_type(type) || !h || n <= 0) return 0;
    long long rows = 0;
    for (int i = 0; i < n; ++i) if (h[i].w_off >= 0) rows += h[i].n_rows;
    return rows > 0 ? (size_t)((rows * 4 + 255) / 256 * 256) : 0;
}

extern "C" int sg_quantize_tensors(int device, void* stream, int type, int variant, const void* x, int x_dtype,
                                   void* y, const float* w, const sg_tensor* h, int n,
                                   void* scratch, size_t scratch_bytes) {
    int qk, bs;
    if (sg_type_info(type, &qk, &bs) != SG_OK) return SG_ERR_TYPE;
    if (variant != 0 && !(type == SG_IQ1_M && variant == 1)) return SG_ERR_TYPE;
    if (n < 0 || (n > 0 && (!h || !x || !y))) return SG_ERR_ARG;
    if (x_dtype != SG_DT_BF16 && x_dtype != SG_DT_F16 && x_dtype != SG_DT_F32) return SG_ERR_ARG;
    if (n == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const int yal = bs % 16 == 0 ? 16 : bs % 8 == 0 ? 8 : bs % 4 == 0 ? 4 : 2;
    const int xal = x_dtype == SG_DT_F32 ? 4 : 8;
    // validate every tensor first, then launch in groups of SG_MAX_TENSORS with one importance setting per launch
    for (int i = 0; i < n; ++i) {
        const sg_tensor& t = h[i];
        if (t.n_rows < 0 || t.n_per_row <= 0 || t.x_off < 0 || t.y_off < 0) return SG_ERR_ARG;
        if (t.n_per_row % qk) return SG_ERR_SHAPE;
        if (t.n_per_row > 0x7fffff00LL) return SG_ERR_LIMIT;
        if (t.x_off % xal || t.y_off % yal || (t.w_off >= 0 && t.w_off % 4)) return SG_ERR_ALIGN;
        if (t.w_off >= 0 && !w) return SG_ERR_ARG;
        if (t.w_off < 0 && sg_type_needs_imatrix(type)) return SG_ERR_IMATRIX;
    }
    if ((uintptr_t)x % 16 || (uintptr_t)y % 16 || (w && (uintptr_t)w % 16)) return SG_ERR_ALIGN;
    const size_t need = sg_quantize_scratch_bytes(type, h, n);
    if (need && (!scratch || scratch_bytes < need)) return SG_ERR_SCRATCH;

    long long scratch_row = 0;
    int i = 0;
    while (i < n) {
        Job job;
        memset(&job, 0, sizeof(job));
        job.x = x; job.y = (uint8_t*)y; job.w = w; job.status = status_word(device);
        const bool imx = h[i].w_off >= 0 && !ignores_imatrix(type);
        long long slabs = 0, rows = 0;
        int k = 0;
        while (i < n && k < SG_MAX_TENSORS) {
            const bool imx_i = h[i].w_off >= 0 && !ignores_imatrix(type);
            if (imx_i != imx) break;
            Tensor& t = job.t[k];
            t.xoff = h[i].x_off; t.yoff = h[i].y_off; t.woff = imx ? h[i].w_off : -1;
            t.nrows = (int)h[i].n_rows; t.npr = (int)h[i].n_per_row;
            t.spr = (t.npr + 255) / 256;
            t.slab0 = slabs; t.row0 = rows;
            if (h[i].n_rows > 0x7fffffffLL) return SG_ERR_LIMIT;
            slabs += (long long)t.nrows * t.spr;
            rows += t.nrows;
            ++k; ++i;
        }
        job.ntens = k; job.nslabs = slabs;
        if (slabs == 0) continue;
        if (slabs * 16 / 128 > 0x7fffffffLL) return SG_ERR_LIMIT;
        if (imx && legacy_imx_type(type)) {
            job.rowstat = (float*)scratch + scratch_row;
            scratch_row += rows;
            rc = launch_meansq(job, rows, x_dtype, st);
            if (rc != SG_OK) return rc;
        }
        rc = dispatch(type, variant, imx, device, job, x_dtype, st);
        if (rc != SG_OK) return rc;
    }
    return SG_OK;
}

// ---------------------------------------------------------------------------------------------------
// Allocation-free variant of the importance-weighted legacy quantisers.
//
// Some hosts must not see a device allocation from this library once they are running: an archiver that has
// measured free device memory and carved it into fixed windows (a hidden cudaMalloc can fail, or take the
// block the next window was counting on), or a pipelined service in which cudaMalloc's implicit
// device-wide synchronisation would stall every other stream.  Such callers cannot provide the per-row
// scratch of sg_quantize_tensors from a pool either, so the scratch lives here, in a fixed array that
// every GPU loading the library holds until the process exits.
constexpr long long SG_STATIC_ROWS = 65536;                          // rows per call: 256 KiB of device memory
static __device__ __align__(256) float g_static_rowstat[SG_STATIC_ROWS];

static std::mutex g_static_mu;
static float* g_static_ptr[64] = {nullptr};

// Device address of the array for `device`, which must be current.  The array's name is only a host-side
// handle; the address a kernel can use comes from cudaGetSymbolAddress, once per device.
static int static_rowstat(int device, float** out) {
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (!g_static_ptr[device]) {
        float* p = nullptr;
        const int rc = cuda_ok(cudaGetSymbolAddress((void**)&p, g_static_rowstat));
        if (rc != SG_OK) return rc;
        if (!p) return SG_ERR_CUDA;
        g_static_ptr[device] = p;
    }
    *out = g_static_ptr[device];
    return SG_OK;
}

extern "C" int sg_quantize_legacy_imx_static(int device, void* stream, int type, const void* x, int x_dtype, void* y,
                                             const float* w, const sg_tensor* h, int n) {
    if (!legacy_imx_type(type)) return SG_ERR_TYPE;
    if (n < 0 || (n > 0 && (!h || !x || !y || !w))) return SG_ERR_ARG;
    long long rows = 0;
    for (int i = 0; i < n; ++i) {
        if (h[i].w_off < 0) return SG_ERR_IMATRIX;           // the matrix-free routines need no scratch: use sg_quantize_tensors
        if (h[i].n_rows < 0) return SG_ERR_ARG;
        rows += h[i].n_rows;
        if (rows > SG_STATIC_ROWS) return SG_ERR_LIMIT;
    }
    if (n == 0) return SG_OK;
    int rc = use_device(device);
    if (rc != SG_OK) return rc;
    float* scratch = nullptr;
    rc = static_rowstat(device, &scratch);
    if (rc != SG_OK) return rc;
    return sg_quantize_tensors(device, stream, type, 0, x, x_dtype, y, w, h, n, scratch, (size_t)SG_STATIC_ROWS * sizeof(float));
}
