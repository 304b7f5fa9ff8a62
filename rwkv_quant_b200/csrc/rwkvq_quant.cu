// Block quantizers for the sb6 and sym layouts on the device.  sb6: the search the reference runs in torch on the
// host (rwkv_quant/calibration/groupwise.py:207-300, `_gw_one` with 8 blocks of 32 per super-block).
//
// One warp owns one (row, super-block) = 256 weights: lane l holds element l of each of the 8
// blocks, so every per-block reduction (min, max, the weighted means, covariance, variance, squared
// error) is a 5-step shuffle tree and nothing touches shared memory.
//   per block      s0 = max((max - min) / qmax, 1e-8); with search, for each factor f of
//                  {0.7 .. 1.05}: q = clamp(rint((w - min) / (f s0))), the closed-form least-squares
//                  (s, m) for those codes (weights E[x^2] of the input channel when given), the codes
//                  again with (s, m), their squared error; the (s, m) with the smallest error wins,
//                  the first factor on ties
//   per super-block  d = fp16(max s / 63), qs = clamp(rint(s / d), 1, 63), dm = fp16(max|m| / 31),
//                  qm = clamp(rint(m / dm), -31, 31); s' = max(fp16(qs d), 1e-8), m' = fp16(qm dm)
//   per weight     q = clamp(rint((w - m') / s'), 0, qmax)
// All in fp32 with IEEE division and round-half-to-even, like the torch code.  The sums run as
// shuffle trees, torch's in its own order: (s, m) agree to their last bits, so a code can differ
// where a quotient sits within an ulp of a rounding boundary or two factors tie (measured: 3 codes
// per million against tensors packed by the reference).
#include <cuda_fp16.h>

#include "rwkvq_common.cuh"

namespace rwkvq {

namespace {

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}
__device__ __forceinline__ float wmax(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}
__device__ __forceinline__ float wmin(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}
__device__ __forceinline__ float hrt(float x) { return __half2float(__float2half_rn(x)); }
__device__ __forceinline__ float clampf(float v, float lo, float hi) { return fminf(fmaxf(v, lo), hi); }

__global__ void __launch_bounds__(256) quant_sb6_kernel(const float* __restrict__ w, long long ldw, int rows, int nsb, int bits,
                                                         int search, const float* __restrict__ ex2, uint8_t* __restrict__ q,
                                                         uint8_t* __restrict__ qs_out, int8_t* __restrict__ qm_out,
                                                         __half* __restrict__ d_out, __half* __restrict__ dm_out) {
    const int lane = threadIdx.x & 31;
    const long long unit = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (unit >= static_cast<long long>(rows) * nsb) return;          // whole warps leave together
    const int row = static_cast<int>(unit / nsb), sbk = static_cast<int>(unit % nsb);
    const float* wp = w + static_cast<size_t>(row) * ldw + sbk * 256 + lane;
    const float qmax = static_cast<float>((1 << bits) - 1);
    float wv[8], ev[8];
#pragma unroll
    for (int b = 0; b < 8; ++b) {
        wv[b] = wp[b * 32];
        ev[b] = ex2 ? fmaxf(ex2[sbk * 256 + b * 32 + lane], 1e-12f) : 1.f;
    }
    float my_s = 0.f, my_m = 0.f;          // lane b keeps the pair of block b
#pragma unroll
    for (int b = 0; b < 8; ++b) {
        const float x = wv[b];
        float mn = wmin(x);
        const float mx = wmax(x);
        float scale = fmaxf(__fdiv_rn(mx - mn, qmax), 1e-8f);
        if (search) {
            const float e = ev[b];
            const float es = ex2 ? wsum(e) : 32.f;
            const float wm = __fdiv_rn(ex2 ? wsum(e * x) : wsum(x), es);
            float best_s = 0.f, best_m = 0.f, best_e = 0.f;
            const float factors[8] = {0.7f, 0.75f, 0.8f, 0.85f, 0.9f, 0.95f, 1.0f, 1.05f};
#pragma unroll
            for (int fi = 0; fi < 8; ++fi) {
                const float sc = scale * factors[fi];
                const float qq = clampf(rintf(__fdiv_rn(x - mn, sc)), 0.f, qmax);
                const float qm_ = __fdiv_rn(ex2 ? wsum(e * qq) : wsum(qq), es);
                const float dq = qq - qm_;
                const float cov = wsum(ex2 ? e * dq * (x - wm) : dq * (x - wm));
                const float var = fmaxf(wsum(ex2 ? e * dq * dq : dq * dq), 1e-12f);
                float s_ls = __fdiv_rn(cov, var);
                const float m_ls = __fsub_rn(wm, __fmul_rn(s_ls, qm_));       // separate multiply and subtract, as in torch
                s_ls = s_ls > 1e-8f ? s_ls : sc;
                const float q2 = clampf(rintf(__fdiv_rn(x - m_ls, s_ls)), 0.f, qmax);
                const float r = __fadd_rn(__fmul_rn(q2, s_ls), m_ls) - x;        // (q2 * s + m) - w, no contraction
                const float err = wsum(ex2 ? e * (r * r) : r * r);
                if (fi == 0 || err < best_e) { best_s = s_ls; best_m = m_ls; best_e = err; }
            }
            scale = fmaxf(best_s, 1e-8f);
            mn = best_m;
        }
        if (lane == b) { my_s = scale; my_m = mn; }
    }
    // super-block: lanes 0-7 hold (s, m) of the 8 blocks
    const bool holder = lane < 8;
    const float smax_v = wmax(holder ? my_s : 0.f);
    const float mabs = wmax(holder ? fabsf(my_m) : 0.f);
    const float d = hrt(fmaxf(__fdiv_rn(smax_v, 63.f), 1e-12f));
    const float dm = hrt(fmaxf(__fdiv_rn(mabs, 31.f), 1e-12f));
    const float qsv = clampf(rintf(__fdiv_rn(my_s, d)), 1.f, 63.f);
    // an all-zero super-block has dm = fp16(1e-12) = 0: min code 0 (the reference's 0 / 0 leaves NaN there)
    const float qmv = (dm > 0.f || my_m != 0.f) ? clampf(rintf(__fdiv_rn(my_m, dm)), -31.f, 31.f) : 0.f;
    const float s2 = fmaxf(hrt(__fmul_rn(qsv, d)), 1e-8f);
    const float m2 = hrt(__fmul_rn(qmv, dm));
    const size_t nb = static_cast<size_t>(nsb) * 8;
    if (holder) {
        qs_out[static_cast<size_t>(row) * nb + sbk * 8 + lane] = static_cast<uint8_t>(qsv);
        qm_out[static_cast<size_t>(row) * nb + sbk * 8 + lane] = static_cast<int8_t>(qmv);
    }
    if (lane == 0) {
        d_out[static_cast<size_t>(row) * nsb + sbk] = __float2half_rn(d);
        dm_out[static_cast<size_t>(row) * nsb + sbk] = __float2half_rn(dm);
    }
    uint8_t* qp = q + static_cast<size_t>(row) * (static_cast<size_t>(nsb) * 256) + sbk * 256 + lane;
#pragma unroll
    for (int b = 0; b < 8; ++b) {
        const float sb_ = __shfl_sync(0xFFFFFFFFu, s2, b), mb_ = __shfl_sync(0xFFFFFFFFu, m2, b);
        qp[b * 32] = static_cast<uint8_t>(clampf(rintf(__fdiv_rn(wv[b] - mb_, sb_)), 0.f, qmax));
    }
}


// The symmetric layout (blocks of 16, int8 block-scale codes against one fp16 per 256 weights;
// calibration/groupwise.py:358-473 `_sym_one`): a warp owns a super-block, a half-warp a block, two
// blocks per round.  Per block s0 = max(max|w|, 1e-12) / qmax and, over the caller's factors (the
// reference's 19 float32 nodes of linspace(0.7, 1.15), or 1.0 alone), the s = f s0 with the
// smallest (weighted) squared error of w - clamp(rint(w / s)) s, the first on ties; then
// d = fp16(max s / 127), qs = clamp(rint(s / d), -128, 127), s' = fp16(qs d) and
// q = clamp(rint(w / s')) (0 where s' is 0).
__device__ __forceinline__ float hsum16(float v) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}
__device__ __forceinline__ float hmax16(float v) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}

__global__ void __launch_bounds__(256) quant_sym_kernel(const float* __restrict__ w, long long ldw, int rows, int nsb, int bits,
                                                         const float* __restrict__ factors, int n_factors,
                                                         const float* __restrict__ ex2, int8_t* __restrict__ q,
                                                         int8_t* __restrict__ qs_out, __half* __restrict__ d_out) {
    const int lane = threadIdx.x & 31, hl = lane & 15, hw = lane >> 4;
    const long long unit = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (unit >= static_cast<long long>(rows) * nsb) return;
    const int row = static_cast<int>(unit / nsb), sbk = static_cast<int>(unit % nsb);
    const float* wp = w + static_cast<size_t>(row) * ldw + sbk * 256;
    const float qmax = static_cast<float>((1 << (bits - 1)) - 1), qmin = -qmax - 1.f;
    float wv[8];
    float my_s = 0.f;                       // lane b (< 16) keeps the scale of block b
#pragma unroll
    for (int r = 0; r < 8; ++r) {           // round r: blocks 2r (lanes 0-15) and 2r + 1 (lanes 16-31)
        const int col = (2 * r + hw) * 16 + hl;
        const float x = wp[col];
        wv[r] = x;
        const float e = ex2 ? fmaxf(ex2[sbk * 256 + col], 1e-12f) : 1.f;
        const float base = __fdiv_rn(fmaxf(hmax16(fabsf(x)), 1e-12f), qmax);
        float best_s = base, best_e = 0.f;
        for (int fi = 0; fi < n_factors; ++fi) {
            const float s = __fmul_rn(base, factors[fi]);
            const float qv = clampf(rintf(__fdiv_rn(x, s)), qmin, qmax);
            const float dlt = __fsub_rn(x, __fmul_rn(qv, s));
            const float err = hsum16(ex2 ? e * (dlt * dlt) : dlt * dlt);
            if (fi == 0 || err < best_e) { best_s = s; best_e = err; }
        }
        // both half-warps hand their block's scale to the lane with the block's number
        const float s_even = __shfl_sync(0xFFFFFFFFu, best_s, 0), s_odd = __shfl_sync(0xFFFFFFFFu, best_s, 16);
        if (lane == 2 * r) my_s = s_even;
        if (lane == 2 * r + 1) my_s = s_odd;
    }
    const bool holder = lane < 16;
    const float d = hrt(fmaxf(__fdiv_rn(wmax(holder ? my_s : 0.f), 127.f), 1e-12f));
    float qsv = clampf(rintf(__fdiv_rn(my_s, d)), -128.f, 127.f);
    if (!(qsv == qsv)) qsv = 0.f;           // 0 / 0: code 0, as the reference writes
    const float s2 = hrt(__fmul_rn(qsv, d));
    const size_t nb = static_cast<size_t>(nsb) * 16;
    if (holder) qs_out[static_cast<size_t>(row) * nb + sbk * 16 + lane] = static_cast<int8_t>(qsv);
    if (lane == 0) d_out[static_cast<size_t>(row) * nsb + sbk] = __float2half_rn(d);
    int8_t* qp = q + static_cast<size_t>(row) * (static_cast<size_t>(nsb) * 256) + sbk * 256;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        const float sb_ = __shfl_sync(0xFFFFFFFFu, s2, 2 * r + hw);
        const float qv = fabsf(sb_) > 0.f ? clampf(rintf(__fdiv_rn(wv[r], sb_)), qmin, qmax) : 0.f;
        qp[(2 * r + hw) * 16 + hl] = static_cast<int8_t>(qv);
    }
}

}  // namespace
}  // namespace rwkvq

using namespace rwkvq;

extern "C" int rwkvq_quantize_sb6(const float* w, int64_t ldw, int rows, int cols, int bits, int search, const float* ex2,
                                  uint8_t* q, uint8_t* qs, int8_t* qm, void* d, void* dm, void* stream) {
    RWKVQ_REQUIRE(w && q && qs && qm && d && dm, RWKVQ_E_NULL, "rwkvq_quantize_sb6: null pointer");
    RWKVQ_REQUIRE(rows >= 1 && cols >= 256 && cols % 256 == 0 && ldw >= cols, RWKVQ_E_SHAPE,
                  "rwkvq_quantize_sb6: [%d, %d] (columns in multiples of 256), ldw %lld", rows, cols, (long long)ldw);
    RWKVQ_REQUIRE(bits >= 4 && bits <= 6, RWKVQ_E_DTYPE, "rwkvq_quantize_sb6: %d bits (4, 5 or 6)", bits);
    const int nsb = cols / 256;
    const long long units = static_cast<long long>(rows) * nsb;
    RWKVQ_REQUIRE((units + 7) / 8 <= 0x7FFFFFFFLL, RWKVQ_E_LIMIT, "rwkvq_quantize_sb6: tensor too large for one launch");
    quant_sb6_kernel<<<static_cast<unsigned int>((units + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        w, static_cast<long long>(ldw), rows, nsb, bits, search, ex2, q, qs, qm, static_cast<__half*>(d), static_cast<__half*>(dm));
    return check_launch("rwkvq_quantize_sb6");
}

extern "C" int rwkvq_quantize_sym(const float* w, int64_t ldw, int rows, int cols, int bits, const float* factors, int n_factors,
                                  const float* ex2, int8_t* q, int8_t* qs, void* d, void* stream) {
    RWKVQ_REQUIRE(w && q && qs && d && factors, RWKVQ_E_NULL, "rwkvq_quantize_sym: null pointer");
    RWKVQ_REQUIRE(rows >= 1 && cols >= 256 && cols % 256 == 0 && ldw >= cols, RWKVQ_E_SHAPE,
                  "rwkvq_quantize_sym: [%d, %d] (columns in multiples of 256), ldw %lld", rows, cols, (long long)ldw);
    RWKVQ_REQUIRE(bits == 6 || bits == 8, RWKVQ_E_DTYPE, "rwkvq_quantize_sym: %d bits (6 or 8)", bits);
    RWKVQ_REQUIRE(n_factors >= 1 && n_factors <= 64, RWKVQ_E_LIMIT, "rwkvq_quantize_sym: %d factors", n_factors);
    const int nsb = cols / 256;
    const long long units = static_cast<long long>(rows) * nsb;
    RWKVQ_REQUIRE((units + 7) / 8 <= 0x7FFFFFFFLL, RWKVQ_E_LIMIT, "rwkvq_quantize_sym: tensor too large for one launch");
    quant_sym_kernel<<<static_cast<unsigned int>((units + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        w, static_cast<long long>(ldw), rows, nsb, bits, factors, n_factors, ex2, q, qs, static_cast<__half*>(d));
    return check_launch("rwkvq_quantize_sym");
}
