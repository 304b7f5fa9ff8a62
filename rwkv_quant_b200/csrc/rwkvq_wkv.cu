// WKV-7 recurrence and the time-mix tail.
//
// State S[dv][dk] (64 x 64 fp32 per batch element and head).  Per step
//     sa = S a;   S = S diag(w) + sa b^T + v k^T;   y = S r
// (call site backends/metal/quant_model.py:118-125, math models/rwkv7_ref.py:244-254,
// prototype kernel tests/bench_wkv_shared.py:64-97).  The 64 state rows are
// independent, so a CTA of 256 threads owns one (batch, head): thread (dv, part)
// keeps 16 columns of row dv in registers for the whole scan, and the two dot
// products per step are finished with two quad shuffles.  The r/w/k/v/a/b rows of
// following steps are fetched while step t is computed (double-buffered shared memory, one
// barrier per step).
#include "rwkvq_common.cuh"

namespace rwkvq {

constexpr int kS = 64;             // head size

struct WkvArgs {
    const float *r, *w, *k, *v, *a, *b;   // [B, T, H, 64]
    const float* h_in;                     // [B, H, 64, 64] or null (zeros)
    float* out;                            // [B, T, H, 64]
    float* h_out;                          // [B, H, 64, 64] (may alias h_in)
    int B, T, H;
};

// Shared-memory rows of a, w, k, b, r: the 16 values of column quarter `part` start at float
// part * 20 (4 floats of padding per quarter), so that the four quarters a warp reads with one
// 128-bit load fall into different bank groups: one wavefront per load instead of 2 x 4.
constexpr int kRowPad = 80;
__device__ __forceinline__ int padded(int c) { return (c >> 4) * 20 + (c & 15); }

// DEEP: the rows of step t+2 are requested while step t is computed (two register sets with fixed
// roles); used when the grid leaves the SMs mostly empty and a step is shorter than a load from L2.
// Otherwise one step ahead and 4 CTAs per SM.
template <bool DEEP>
__global__ void __launch_bounds__(256, DEEP ? 2 : 4) wkv7_kernel(const WkvArgs p) {
    __shared__ __align__(16) float sh[2][5][kRowPad];
    __shared__ float shv[2][kS];
    const int bh = blockIdx.x, bi = bh / p.H, hi = bh % p.H;
    const int tid = threadIdx.x, dv = tid >> 2, part = tid & 3;
    float h[16];
    const size_t hbase = (static_cast<size_t>(bh) * kS + dv) * kS + part * 16;
    if (p.h_in) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 v4 = *reinterpret_cast<const float4*>(p.h_in + hbase + 4 * i);
            h[4 * i] = v4.x; h[4 * i + 1] = v4.y; h[4 * i + 2] = v4.z; h[4 * i + 3] = v4.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) h[i] = 0.f;
    }
    const float* src[6] = {p.a, p.w, p.k, p.b, p.r, p.v};
    // thread `tid` stages value tid (and tid+256 for tid < 128) of the 6 x 64 row set
    auto fetch = [&](int t, float& x0, float& x1) {
        const size_t base = ((static_cast<size_t>(bi) * p.T + t) * p.H + hi) * kS;
        x0 = src[tid >> 6][base + (tid & 63)];
        x1 = 0.f;
        if (tid < 128) x1 = src[4 + (tid >> 6)][base + (tid & 63)];
    };
    auto stash = [&](int buf, float x0, float x1) {
        sh[buf][tid >> 6][padded(tid & 63)] = x0;
        if (tid < 64) sh[buf][4][padded(tid)] = x1;
        else if (tid < 128) shv[buf][tid & 63] = x1;
    };
    // one step of the recurrence on the rows staged in buffer `cur`
    auto step = [&](int t, int cur) {
        const float4* A = reinterpret_cast<const float4*>(sh[cur][0] + part * 20);
        const float4* W = reinterpret_cast<const float4*>(sh[cur][1] + part * 20);
        const float4* K = reinterpret_cast<const float4*>(sh[cur][2] + part * 20);
        const float4* Bv = reinterpret_cast<const float4*>(sh[cur][3] + part * 20);
        const float4* R = reinterpret_cast<const float4*>(sh[cur][4] + part * 20);
        const float vv = shv[cur][dv];
        // four independent partial sums per dot product (a chain of 16 dependent FMAs is the
        // longest link of a step otherwise), combined pairwise
        float ps[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 a4 = A[i];
            ps[i] = h[4 * i] * a4.x;
            ps[i] = fmaf(h[4 * i + 1], a4.y, ps[i]);
            ps[i] = fmaf(h[4 * i + 2], a4.z, ps[i]);
            ps[i] = fmaf(h[4 * i + 3], a4.w, ps[i]);
        }
        float sa = (ps[0] + ps[1]) + (ps[2] + ps[3]);
        sa += __shfl_xor_sync(0xFFFFFFFFu, sa, 1);
        sa += __shfl_xor_sync(0xFFFFFFFFu, sa, 2);
        float py[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 w4 = W[i], k4 = K[i], b4 = Bv[i], r4 = R[i];
            h[4 * i] = fmaf(w4.x, h[4 * i], fmaf(vv, k4.x, sa * b4.x));             py[i] = h[4 * i] * r4.x;
            h[4 * i + 1] = fmaf(w4.y, h[4 * i + 1], fmaf(vv, k4.y, sa * b4.y));     py[i] = fmaf(h[4 * i + 1], r4.y, py[i]);
            h[4 * i + 2] = fmaf(w4.z, h[4 * i + 2], fmaf(vv, k4.z, sa * b4.z));     py[i] = fmaf(h[4 * i + 2], r4.z, py[i]);
            h[4 * i + 3] = fmaf(w4.w, h[4 * i + 3], fmaf(vv, k4.w, sa * b4.w));     py[i] = fmaf(h[4 * i + 3], r4.w, py[i]);
        }
        float y = (py[0] + py[1]) + (py[2] + py[3]);
        y += __shfl_xor_sync(0xFFFFFFFFu, y, 1);
        y += __shfl_xor_sync(0xFFFFFFFFu, y, 2);
        if (part == 0) p.out[((static_cast<size_t>(bi) * p.T + t) * p.H + hi) * kS + dv] = y;
    };
    if (DEEP) {
        float e0, e1, o0 = 0.f, o1 = 0.f;
        fetch(0, e0, e1);
        stash(0, e0, e1);
        if (p.T > 1) fetch(1, o0, o1);
        __syncthreads();
        for (int t = 0; t < p.T; t += 2) {
            if (t + 2 < p.T) fetch(t + 2, e0, e1);
            step(t, 0);
            if (t + 1 < p.T) stash(1, o0, o1);
            __syncthreads();
            if (t + 1 >= p.T) break;
            if (t + 3 < p.T) fetch(t + 3, o0, o1);
            step(t + 1, 1);
            if (t + 2 < p.T) stash(0, e0, e1);
            __syncthreads();
        }
    } else {
        float x0, x1;
        fetch(0, x0, x1);
        stash(0, x0, x1);
        __syncthreads();
        for (int t = 0; t < p.T; ++t) {
            const int cur = t & 1;
            if (t + 1 < p.T) fetch(t + 1, x0, x1);
            step(t, cur);
            if (t + 1 < p.T) stash(cur ^ 1, x0, x1);
            __syncthreads();
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
        *reinterpret_cast<float4*>(p.h_out + hbase + 4 * i) = make_float4(h[4 * i], h[4 * i + 1], h[4 * i + 2], h[4 * i + 3]);
}

// (group_norm(wkv) * ln_w + ln_b + (sum r*k*r_k) * v) * g per (row, head); a warp per
// pair, two-pass variance as in backends/metal/fused_tail.py:43-76.
__global__ void __launch_bounds__(128) wkv_tail_kernel(const float* wkv, const float* r, const float* k,
                                                       const float* v, const float* r_k, const float* ln_w,
                                                       const float* ln_b, const float* g, float* out,
                                                       int n_pairs, int H, float eps) {
    const int pair = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (pair >= n_pairs) return;
    const int hd = pair % H;
    const size_t base = static_cast<size_t>(pair) * kS;
    const int hb = hd * kS;
    const float x0 = wkv[base + lane], x1 = wkv[base + lane + 32];
    float s = x0 + x1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
    const float mean = s / kS;
    const float d0 = x0 - mean, d1 = x1 - mean;
    float s2 = d0 * d0 + d1 * d1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s2 += __shfl_xor_sync(0xFFFFFFFFu, s2, o);
    const float inv = 1.0f / sqrtf(s2 / kS + eps);
    float dp = r[base + lane] * k[base + lane] * r_k[hb + lane] +
               r[base + lane + 32] * k[base + lane + 32] * r_k[hb + lane + 32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dp += __shfl_xor_sync(0xFFFFFFFFu, dp, o);
    out[base + lane] = (d0 * inv * ln_w[hb + lane] + ln_b[hb + lane] + dp * v[base + lane]) * g[base + lane];
    out[base + lane + 32] =
        (d1 * inv * ln_w[hb + lane + 32] + ln_b[hb + lane + 32] + dp * v[base + lane + 32]) * g[base + lane + 32];
}

}  // namespace rwkvq

using namespace rwkvq;

extern "C" {

int rwkvq_wkv7(const float* r, const float* w, const float* k, const float* v, const float* a,
               const float* b, const float* h_in, float* out, float* h_out, int B, int T, int H,
               int head_size, void* stream) {
    RWKVQ_REQUIRE(r && w && k && v && a && b && out && h_out, RWKVQ_E_NULL, "rwkvq_wkv7: null pointer");
    RWKVQ_REQUIRE(head_size == kS, RWKVQ_E_SHAPE, "rwkvq_wkv7: head size %d, only 64 is built", head_size);
    RWKVQ_REQUIRE(B >= 1 && T >= 1 && H >= 1, RWKVQ_E_SHAPE, "rwkvq_wkv7: B=%d T=%d H=%d", B, T, H);
    RWKVQ_REQUIRE(aligned(h_out, 16) && aligned(h_in, 16), RWKVQ_E_ALIGN, "rwkvq_wkv7: state must be 16-byte aligned");
    WkvArgs p{r, w, k, v, a, b, h_in, out, h_out, B, T, H};
    if (B * H <= 2 * 148 && T > 2) wkv7_kernel<true><<<B * H, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
    else wkv7_kernel<false><<<B * H, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
    return check_launch("rwkvq_wkv7");
}

int rwkvq_wkv_tail(const float* wkv, const float* r, const float* k, const float* v, const float* r_k,
                   const float* ln_w, const float* ln_b, const float* g, float* out, int N, int H,
                   int head_size, float eps, void* stream) {
    RWKVQ_REQUIRE(wkv && r && k && v && r_k && ln_w && ln_b && g && out, RWKVQ_E_NULL, "rwkvq_wkv_tail: null pointer");
    RWKVQ_REQUIRE(head_size == kS, RWKVQ_E_SHAPE, "rwkvq_wkv_tail: head size %d, only 64 is built", head_size);
    RWKVQ_REQUIRE(N >= 1 && H >= 1, RWKVQ_E_SHAPE, "rwkvq_wkv_tail: N=%d H=%d", N, H);
    const int pairs = N * H;
    wkv_tail_kernel<<<(pairs + 3) / 4, 128, 0, static_cast<cudaStream_t>(stream)>>>(wkv, r, k, v, r_k, ln_w, ln_b, g,
                                                                                  out, pairs, H, eps);
    return check_launch("rwkvq_wkv_tail");
}

}  // extern "C"
