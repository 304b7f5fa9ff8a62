// Error plumbing, argument validation and the dequantisation kernels.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include "rwkvq_common.cuh"

namespace rwkvq {

static thread_local char g_detail[512] = "";

void set_error_detail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_detail, sizeof(g_detail), fmt, ap);
    va_end(ap);
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_detail, sizeof(g_detail), fmt, ap);
    va_end(ap);
    return code;
}

bool pdl_enabled() {
    static const bool on = [] {
        const char* e = getenv("RWKVQ_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}

int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
    return RWKVQ_OK;
}

int validate_qtensor(const rwkvq_qtensor* t, const char* who) {
    RWKVQ_REQUIRE(t != nullptr, RWKVQ_E_NULL, "%s: tensor descriptor is null", who);
    RWKVQ_REQUIRE(t->rows > 0 && t->cols > 0, RWKVQ_E_SHAPE, "%s: empty shape [%d, %d]", who,
                  t->rows, t->cols);
    RWKVQ_REQUIRE(t->codes != nullptr, RWKVQ_E_NULL, "%s: codes pointer is null", who);
    switch (t->kind) {
        case RWKVQ_KIND_SB6:
            RWKVQ_REQUIRE(t->bits >= 4 && t->bits <= 6, RWKVQ_E_DTYPE, "%s: sb6 at %d bits", who, t->bits);
            RWKVQ_REQUIRE(t->gs == 32 && t->sb == 8, RWKVQ_E_DTYPE,
                          "%s: sb6 needs block 32 / super-block 8, got %d / %d", who, t->gs, t->sb);
            RWKVQ_REQUIRE(t->cols % 256 == 0, RWKVQ_E_SHAPE, "%s: sb6 needs IN %% 256 == 0, IN=%d", who, t->cols);
            RWKVQ_REQUIRE(t->qsqm && t->d && t->dm, RWKVQ_E_NULL, "%s: sb6 scale buffers missing", who);
            RWKVQ_REQUIRE((t->bits >= 5) == (t->qh != nullptr) && (t->bits >= 6) == (t->qh2 != nullptr),
                          RWKVQ_E_DTYPE, "%s: sb6 bit-planes do not match bits=%d", who, t->bits);
            RWKVQ_REQUIRE(aligned(t->codes, 16) && aligned(t->qsqm, 4) && aligned(t->d, 2) &&
                              aligned(t->dm, 2) && aligned(t->qh, 4) && aligned(t->qh2, 4),
                          RWKVQ_E_ALIGN, "%s: sb6 buffers need 16-byte codes, 4-byte planes/meta", who);
            break;
        case RWKVQ_KIND_SYM:
            RWKVQ_REQUIRE(t->bits == 6 || t->bits == 8, RWKVQ_E_DTYPE, "%s: sym at %d bits", who, t->bits);
            RWKVQ_REQUIRE(t->gs == 16 && t->sb == 16, RWKVQ_E_DTYPE,
                          "%s: sym needs block 16 / super-block 16, got %d / %d", who, t->gs, t->sb);
            RWKVQ_REQUIRE(t->cols % 256 == 0, RWKVQ_E_SHAPE, "%s: sym needs IN %% 256 == 0, IN=%d", who, t->cols);
            RWKVQ_REQUIRE(t->qs && t->d, RWKVQ_E_NULL, "%s: sym scale buffers missing", who);
            RWKVQ_REQUIRE((t->bits == 6) == (t->qh != nullptr) && (t->bits == 6) == (t->qh2 != nullptr),
                          RWKVQ_E_DTYPE, "%s: sym bit-planes do not match bits=%d", who, t->bits);
            RWKVQ_REQUIRE(aligned(t->codes, 16) && aligned(t->qs, 2) && aligned(t->d, 2) &&
                              aligned(t->qh, 4) && aligned(t->qh2, 4),
                          RWKVQ_E_ALIGN, "%s: sym buffers need 16-byte codes, 4-byte planes", who);
            break;
        case RWKVQ_KIND_ASYM:
            RWKVQ_REQUIRE(t->gs > 0, RWKVQ_E_SHAPE, "%s: asym block size %d", who, t->gs);
            RWKVQ_REQUIRE(t->scale && t->mn, RWKVQ_E_NULL, "%s: asym scale/min missing", who);
            break;
        case RWKVQ_KIND_RTN:
            RWKVQ_REQUIRE(t->bits >= 2 && t->bits <= 8, RWKVQ_E_DTYPE, "%s: rtn at %d bits", who, t->bits);
            RWKVQ_REQUIRE(t->scale != nullptr, RWKVQ_E_NULL, "%s: rtn scale missing", who);
            break;
        case RWKVQ_KIND_DENSE:
            break;
        default:
            return fail(RWKVQ_E_DTYPE, "%s: unknown tensor kind %d", who, t->kind);
    }
    return RWKVQ_OK;
}

// ------------------------------------------------------------------ dequant
template <typename OutT>
__device__ __forceinline__ OutT cast_out(float v);
template <>
__device__ __forceinline__ float cast_out<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half cast_out<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 cast_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// One thread per element, consecutive threads on consecutive columns: reads of
// the packed bytes are broadcast within a warp, writes are fully coalesced.
template <typename OutT>
__global__ void __launch_bounds__(256) dequant_kernel(QView t, OutT* __restrict__ out, int round_bf16) {
    const size_t total = static_cast<size_t>(t.rows) * t.cols;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int r = static_cast<int>(i / t.cols), c = static_cast<int>(i % t.cols);
        float v = decode_element(t, r, c);
        if (round_bf16) v = bf16_roundtrip(v);
        out[i] = cast_out<OutT>(v);
    }
}

}  // namespace rwkvq

using namespace rwkvq;

extern "C" {

const char* rwkvq_strerror(int code) {
    switch (code) {
        case RWKVQ_OK: return "ok";
        case RWKVQ_E_SHAPE: return "shape violates a layout rule";
        case RWKVQ_E_ALIGN: return "misaligned pointer";
        case RWKVQ_E_DTYPE: return "unsupported dtype / layout / bit width";
        case RWKVQ_E_ARCH: return "device is not sm_100";
        case RWKVQ_E_LAUNCH: return "CUDA launch failed";
        case RWKVQ_E_TIMEOUT: return "bounded device-side wait ran out";
        case RWKVQ_E_NULL: return "required pointer is null";
        case RWKVQ_E_LIMIT: return "size exceeds a documented maximum";
        case RWKVQ_E_FORMAT: return "not a readable .rwkvq container";
        default: return "unknown error";
    }
}

const char* rwkvq_last_error_detail(void) { return g_detail; }

int rwkvq_abi_version(void) { return 1; }

int rwkvq_check_device(void) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(RWKVQ_E_ARCH, "cudaGetDevice: %s", cudaGetErrorString(e));
    int major = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return fail(RWKVQ_E_ARCH, "cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
    if (major != 10) return fail(RWKVQ_E_ARCH, "device %d has compute capability %d.x, need 10.x", dev, major);
    return RWKVQ_OK;
}

int rwkvq_dequant(const rwkvq_qtensor* t, void* out, int out_dtype, int round_bf16, void* stream) {
    int rc = validate_qtensor(t, "rwkvq_dequant");
    if (rc) return rc;
    RWKVQ_REQUIRE(out != nullptr, RWKVQ_E_NULL, "rwkvq_dequant: out is null");
    const QView v = make_view(*t);
    const size_t total = static_cast<size_t>(t->rows) * t->cols;
    const int threads = 256;
    size_t want = (total + threads - 1) / threads;
    const int blocks = static_cast<int>(want < 148 * 32 ? want : 148 * 32);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (out_dtype) {
        case RWKVQ_F32:
            dequant_kernel<float><<<blocks, threads, 0, s>>>(v, static_cast<float*>(out), round_bf16);
            break;
        case RWKVQ_F16:
            dequant_kernel<__half><<<blocks, threads, 0, s>>>(v, static_cast<__half*>(out), round_bf16);
            break;
        case RWKVQ_BF16:
            dequant_kernel<__nv_bfloat16><<<blocks, threads, 0, s>>>(v, static_cast<__nv_bfloat16*>(out), round_bf16);
            break;
        default:
            return fail(RWKVQ_E_DTYPE, "rwkvq_dequant: out_dtype %d", out_dtype);
    }
    return check_launch("rwkvq_dequant");
}

}  // extern "C"
