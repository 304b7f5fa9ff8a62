// Small device functions shared by the kernels of the decode step.
#pragma once
#include "rwkvq_common.cuh"

namespace rwkvq {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) s += red[w];
    return s;
}

// 4 consecutive weights of stored row i at column c, in the loader's precision.
// MODE 0: asym, cols % 4 == 0;  1: per-row int8, cols % 4 == 0;  2: anything (slow).
template <int MODE>
__device__ __forceinline__ void lora_w4(const QView& t, int i, int c, int nb, int blk, float (&w)[4]) {
    const size_t I = static_cast<size_t>(i);
    if (MODE == 0) {
        const uint32_t q = ld_stream_u32(t.codes + I * t.cols + c);
        const float s = __ldg(static_cast<const float*>(t.scale) + I * nb + blk), m = __ldg(t.mn + I * nb + blk);
#pragma unroll
        for (int k = 0; k < 4; ++k) w[k] = __fadd_rn(__fmul_rn(static_cast<float>((q >> (8 * k)) & 0xFFu), s), m);
    } else if (MODE == 1) {
        const uint32_t q = ld_stream_u32(t.codes + I * t.cols + c);
        const float s = __half2float(__ldg(static_cast<const __half*>(t.scale) + I));
#pragma unroll
        for (int k = 0; k < 4; ++k) w[k] = __fmul_rn(static_cast<float>(static_cast<int8_t>((q >> (8 * k)) & 0xFFu)), s);
    } else {
        for (int k = 0; k < 4; ++k) w[k] = (c + k < t.cols) ? decode_element(t, i, c + k) : 0.f;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) w[k] = dense_param_rounding(w[k]);
}

__device__ __forceinline__ int lora_mode(const QView& t) {
    if (t.kind == RWKVQ_KIND_ASYM && (t.cols & 3) == 0) return 0;
    if (t.kind == RWKVQ_KIND_RTN && t.bits > 4 && (t.cols & 3) == 0) return 1;
    return 2;
}

// greedy argmax: lowest index wins ties
__device__ __forceinline__ void argmax_combine(float& best, int& idx, float ov, int oi) {
    if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
}
}  // namespace rwkvq
