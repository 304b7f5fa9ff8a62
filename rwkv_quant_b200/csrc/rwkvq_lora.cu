// x^T W products against tensors stored [in, out] (world-naming LoRA matrices):
// y[n, o] = act(sum_i x[n, i] * Wt[i, o]).  The stored orientation makes every
// weight load coalesced with a lane per group of 4 output columns, and the
// per-row (rtn) or per-(row, 64-column block) (asym) scales are indexed by the
// loop variable, so the file bytes are consumed as they lie.
#include "rwkvq_common.cuh"

namespace rwkvq {

constexpr int kLoraWarps = 8;
constexpr int kLoraColsPerCta = 128;   // 32 lanes x 4 columns
constexpr int kLoraMaxN = 8;

struct LoraArgs {
    QView t;
    const float* x;
    long long ldx;
    float* y;
    long long ldy;
    int n_cols;
    int act;
    int round_w;
};

__device__ __forceinline__ float lora_act(float v, int act) {
    if (act == 1) return tanhf(v);
    if (act == 2) return 1.f / (1.f + __expf(-v));
    return v;
}

// 4 consecutive weights of stored row i starting at column c (c % 4 == 0)
__device__ __forceinline__ void lora_load4(const QView& t, int i, int c, int round_w, float (&w)[4]) {
    const size_t I = static_cast<size_t>(i);
    if (t.kind == RWKVQ_KIND_ASYM && (t.cols & 3) == 0) {
        const uint32_t q = ld_stream_u32(t.codes + I * t.cols + c);
        const int nb = (t.cols + t.gs - 1) / t.gs;
        const float s = static_cast<const float*>(t.scale)[I * nb + c / t.gs];
        const float m = t.mn[I * nb + c / t.gs];
#pragma unroll
        for (int k = 0; k < 4; ++k) w[k] = __fadd_rn(__fmul_rn(static_cast<float>((q >> (8 * k)) & 0xFFu), s), m);
    } else if (t.kind == RWKVQ_KIND_RTN && t.bits > 4 && (t.cols & 3) == 0) {
        const uint32_t q = ld_stream_u32(t.codes + I * t.cols + c);
        const float s = __half2float(static_cast<const __half*>(t.scale)[I]);
#pragma unroll
        for (int k = 0; k < 4; ++k) w[k] = __fmul_rn(static_cast<float>(static_cast<int8_t>((q >> (8 * k)) & 0xFFu)), s);
    } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) w[k] = (c + k < t.cols) ? decode_element(t, i, c + k) : 0.f;
    }
    if (round_w) {
#pragma unroll
        for (int k = 0; k < 4; ++k) w[k] = dense_param_rounding(w[k]);
    }
}

__global__ void __launch_bounds__(kLoraWarps * 32) gemv_t_kernel(const LoraArgs a) {
    __shared__ float red[kLoraWarps][kLoraMaxN][kLoraColsPerCta];
    const QView& t = a.t;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = blockIdx.x * kLoraColsPerCta + lane * 4;
    float acc[kLoraMaxN][4];
#pragma unroll
    for (int n = 0; n < kLoraMaxN; ++n)
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[n][k] = 0.f;
    if (c < t.cols) {
        for (int i = warp; i < t.rows; i += kLoraWarps) {
            float w[4];
            lora_load4(t, i, c, a.round_w, w);
#pragma unroll
            for (int n = 0; n < kLoraMaxN; ++n) {
                if (n >= a.n_cols) break;
                const float xv = __ldcg(a.x + n * a.ldx + i);
#pragma unroll
                for (int k = 0; k < 4; ++k) acc[n][k] = fmaf(xv, w[k], acc[n][k]);
            }
        }
    }
#pragma unroll
    for (int n = 0; n < kLoraMaxN; ++n) {
        if (n >= a.n_cols) break;
#pragma unroll
        for (int k = 0; k < 4; ++k) red[warp][n][lane * 4 + k] = acc[n][k];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < a.n_cols * kLoraColsPerCta; idx += blockDim.x) {
        const int n = idx / kLoraColsPerCta, cc = idx % kLoraColsPerCta;
        const int col = blockIdx.x * kLoraColsPerCta + cc;
        if (col >= t.cols) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kLoraWarps; ++w) v += red[w][n][cc];
        a.y[n * a.ldy + col] = lora_act(v, a.act);
    }
}

}  // namespace rwkvq

using namespace rwkvq;

extern "C" int rwkvq_gemv_t(const rwkvq_qtensor* t, const float* x, int N, int64_t ldx, float* y,
                            int64_t ldy, int act, int round_w, void* stream) {
    int rc = validate_qtensor(t, "rwkvq_gemv_t");
    if (rc) return rc;
    RWKVQ_REQUIRE(x && y, RWKVQ_E_NULL, "rwkvq_gemv_t: x or y is null");
    RWKVQ_REQUIRE(N >= 1, RWKVQ_E_SHAPE, "rwkvq_gemv_t: N=%d", N);
    RWKVQ_REQUIRE(ldx >= t->rows && ldy >= t->cols, RWKVQ_E_SHAPE, "rwkvq_gemv_t: ldx=%lld ldy=%lld too small",
                  (long long)ldx, (long long)ldy);
    RWKVQ_REQUIRE(act >= 0 && act <= 2, RWKVQ_E_DTYPE, "rwkvq_gemv_t: act %d", act);
    RWKVQ_REQUIRE(aligned(t->codes, 4), RWKVQ_E_ALIGN, "rwkvq_gemv_t: codes need 4-byte alignment");
    LoraArgs a{};
    a.t = make_view(*t);
    a.ldx = ldx; a.ldy = ldy; a.act = act; a.round_w = round_w;
    const int grid = (t->cols + kLoraColsPerCta - 1) / kLoraColsPerCta;
    for (int n0 = 0; n0 < N; n0 += kLoraMaxN) {
        a.x = x + static_cast<size_t>(n0) * ldx;
        a.y = y + static_cast<size_t>(n0) * ldy;
        a.n_cols = (N - n0 < kLoraMaxN) ? (N - n0) : kLoraMaxN;
        gemv_t_kernel<<<grid, kLoraWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(a);
    }
    return check_launch("rwkvq_gemv_t");
}
