// Glue kernels of the sequence (prefill) path, T > 1: what the decode step does inside
// ln_shift_mix_kernel / tmix_core_kernel for one token, for all B*T tokens of a call.
//
//   seq_ln_shift_mix   xn = LN(x[b,t]);  prev = xn[b,t-1] (t = 0: the carried shift state, zeros
//                      for a fresh stream);  out[m][b,t] = xn + (prev - xn) * mix[m];
//                      new shift state = xn[b,T-1]            (quant_model.py:281-301, 648-651)
//   seq_tmix_pre       decay w = exp(-0.606531 sigmoid(yw + w0)), gate a = sigmoid(ya + a0),
//                      kk = l2norm_head(k * k_k), k' = k (1 + (a - 1) k_a),
//                      v' = v + (v_first - v) sigmoid(yv + v0) (layers > 0); emits w, k', v',
//                      -kk and kk*a, the operands of the WKV-7 scan       (quant_model.py:700-712)
#include "rwkvq_decode_parts.cuh"

namespace rwkvq {

constexpr int kSeqThreads = 256;
constexpr int kSeqPer = 16;          // D <= 4096

// One CTA per token.  The previous token's normalised row is recomputed here (same code,
// same bits as the CTA that owns it), so tokens do not depend on one another.
template <int NMIX>
__global__ void __launch_bounds__(kSeqThreads) seq_ln_shift_mix_kernel(const float* __restrict__ x,
                                                                       const float* __restrict__ ln_w,
                                                                       const float* __restrict__ ln_b,
                                                                       const float* __restrict__ shift_in,
                                                                       const float* __restrict__ mix,
                                                                       float* __restrict__ out,
                                                                       float* __restrict__ shift_out, int T, int D,
                                                                       long long n_tokens) {
    __shared__ float red[kSeqThreads / 32];
    const long long tok = blockIdx.x;
    const int b = static_cast<int>(tok / T), t = static_cast<int>(tok % T);
    const float* row = x + tok * D;
    float v[kSeqPer], pv[kSeqPer], lw[kSeqPer], lb[kSeqPer];
#pragma unroll
    for (int i = 0; i < kSeqPer; ++i) {
        const int d = threadIdx.x + i * kSeqThreads;
        const bool ok = d < D;
        v[i] = ok ? row[d] : 0.f;
        pv[i] = !ok ? 0.f : (t > 0 ? row[d - D] : (shift_in ? shift_in[static_cast<size_t>(b) * D + d] : 0.f));
        lw[i] = ok ? ln_w[d] : 0.f;
        lb[i] = ok ? ln_b[d] : 0.f;
    }
    auto normalise = [&](float (&y)[kSeqPer]) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < kSeqPer; ++i) s += y[i];
        const float mean = block_sum(s, red) / D;
        float s2 = 0.f;
#pragma unroll
        for (int i = 0; i < kSeqPer; ++i) {
            const float c = (threadIdx.x + i * kSeqThreads < D) ? y[i] - mean : 0.f;
            s2 += c * c;
        }
        const float inv = 1.0f / sqrtf(block_sum(s2, red) / D + 1e-5f);
#pragma unroll
        for (int i = 0; i < kSeqPer; ++i) y[i] = (y[i] - mean) * inv * lw[i] + lb[i];
    };
    normalise(v);
    if (t > 0) normalise(pv);               // t == 0: pv already is a normalised row (or zeros)
#pragma unroll
    for (int i = 0; i < kSeqPer; ++i) {
        const int d = threadIdx.x + i * kSeqThreads;
        if (d >= D) continue;
        const float xx = pv[i] - v[i];
        if (t == T - 1) shift_out[static_cast<size_t>(b) * D + d] = v[i];
#pragma unroll
        for (int m = 0; m < NMIX; ++m)
            out[(static_cast<size_t>(m) * n_tokens + tok) * D + d] = v[i] + xx * __ldg(mix + m * D + d);
    }
}

// ---- the same, emitting what the consumers of each mix read ---------------------------------
// A mix row feeds either the dequant-fused GEMM (which reads a per-token power-of-two-scaled
// fp16 copy, pitch D + 64 halves, plus the scale) or the LoRA GEMM (which reads the fp16 hi/lo
// split [hi | lo]), or both; writing those forms here saves the fp32 round trip through HBM and
// one launch per consumer.  The conversions are those of the GEMM's own pre-pass (scale =
// 2^(14 - exponent of the row maximum)) and of split_fp16_kernel.
constexpr int kPrepScaled = 1, kPrepSplit = 2, kPrepF32 = 4;
struct SeqPrepArgs {
    const float *x, *ln_w, *ln_b, *shift_in, *mix;
    float* shift_out;
    __half* x16[6];        // [N, D + 64]
    float* scale[6];       // [N]
    __half* split[6];      // [N, 2 D]
    float* f32[6];         // [N, D]
    int mode[6];
    int T, D, n_mix;
};

__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float m = red[0];
    for (int w = 1; w < (blockDim.x >> 5); ++w) m = fmaxf(m, red[w]);
    return m;
}

// One CTA per token; thread t owns the column pairs 2 (t + 256 i), i < 8 (D <= 4096, D even).
__global__ void __launch_bounds__(kSeqThreads, 3) seq_ln_shift_mix_prep_kernel(const SeqPrepArgs a) {
    __shared__ float red[kSeqThreads / 32];
    constexpr int kPairs = kSeqPer / 2;
    const long long tok = blockIdx.x;
    const int D = a.D, b = static_cast<int>(tok / a.T), t = static_cast<int>(tok % a.T);
    const float* row = a.x + tok * D;
    float2 v[kPairs], pv[kPairs];
    const float2 zero = make_float2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < kPairs; ++i) {
        const int d = 2 * (threadIdx.x + i * kSeqThreads);
        const bool ok = d < D;
        v[i] = ok ? *reinterpret_cast<const float2*>(row + d) : zero;
        pv[i] = !ok ? zero
                    : (t > 0 ? *reinterpret_cast<const float2*>(row + d - D)
                             : (a.shift_in ? *reinterpret_cast<const float2*>(a.shift_in + static_cast<size_t>(b) * D + d) : zero));
    }
    // LayerNorm of the token's row and of its predecessor's at once: the two means, then the two
    // variances, each pair in one block reduction (one barrier each)
    __shared__ float2 red_mean[kSeqThreads / 32], red_var[kSeqThreads / 32];
    auto block_sum2 = [&](float2 q, float2* buf) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            q.x += __shfl_xor_sync(0xFFFFFFFFu, q.x, o);
            q.y += __shfl_xor_sync(0xFFFFFFFFu, q.y, o);
        }
        if ((threadIdx.x & 31) == 0) buf[threadIdx.x >> 5] = q;
        __syncthreads();
        float2 tot = buf[0];
#pragma unroll
        for (int w = 1; w < kSeqThreads / 32; ++w) { tot.x += buf[w].x; tot.y += buf[w].y; }
        return tot;
    };
    float2 sum = zero;
#pragma unroll
    for (int i = 0; i < kPairs; ++i) { sum.x += v[i].x + v[i].y; sum.y += pv[i].x + pv[i].y; }
    sum = block_sum2(sum, red_mean);
    const float mean = sum.x / D, pmean = sum.y / D;
    float2 sq = zero;
#pragma unroll
    for (int i = 0; i < kPairs; ++i) {
        if (2 * (threadIdx.x + i * kSeqThreads) < D) {
            const float c0 = v[i].x - mean, c1 = v[i].y - mean, p0 = pv[i].x - pmean, p1 = pv[i].y - pmean;
            sq.x += c0 * c0 + c1 * c1;
            sq.y += p0 * p0 + p1 * p1;
        }
    }
    sq = block_sum2(sq, red_var);
    const float inv = 1.0f / sqrtf(sq.x / D + 1e-5f), pinv = 1.0f / sqrtf(sq.y / D + 1e-5f);
#pragma unroll
    for (int i = 0; i < kPairs; ++i) {
        const int d = 2 * (threadIdx.x + i * kSeqThreads);
        if (d >= D) continue;
        const float2 lw = __ldg(reinterpret_cast<const float2*>(a.ln_w + d)), lb = __ldg(reinterpret_cast<const float2*>(a.ln_b + d));
        v[i].x = (v[i].x - mean) * inv * lw.x + lb.x;
        v[i].y = (v[i].y - mean) * inv * lw.y + lb.y;
        if (t > 0) {                    // t == 0: pv already is a normalised row (or zeros)
            pv[i].x = (pv[i].x - pmean) * pinv * lw.x + lb.x;
            pv[i].y = (pv[i].y - pmean) * pinv * lw.y + lb.y;
        }
    }
#pragma unroll
    for (int i = 0; i < kPairs; ++i) {
        const int d = 2 * (threadIdx.x + i * kSeqThreads);
        if (d < D && t == a.T - 1) *reinterpret_cast<float2*>(a.shift_out + static_cast<size_t>(b) * D + d) = v[i];
        pv[i].x -= v[i].x;                     // xx = prev - cur
        pv[i].y -= v[i].y;
    }
    for (int m = 0; m < a.n_mix; ++m) {
        float2 val[kPairs];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < kPairs; ++i) {
            const int d = 2 * (threadIdx.x + i * kSeqThreads);
            val[i] = zero;
            if (d < D) {
                const float2 mx = __ldg(reinterpret_cast<const float2*>(a.mix + static_cast<size_t>(m) * D + d));
                val[i].x = v[i].x + pv[i].x * mx.x;
                val[i].y = v[i].y + pv[i].y * mx.y;
                amax = fmaxf(amax, fmaxf(fabsf(val[i].x), fabsf(val[i].y)));
            }
        }
        const int mode = a.mode[m];
        float sc = 1.f;
        if (mode & kPrepScaled) {
            amax = block_max(amax, red);
            int e = 0;
            if (amax > 0.f && amax < INFINITY) frexpf(amax, &e);
            sc = ldexpf(1.f, 14 - e);
            if (threadIdx.x == 0) a.scale[m][tok] = sc;
        }
#pragma unroll
        for (int i = 0; i < kPairs; ++i) {
            const int d = 2 * (threadIdx.x + i * kSeqThreads);
            if (d >= D) continue;
            if (mode & kPrepScaled)
                *reinterpret_cast<__half2*>(a.x16[m] + tok * (D + 64) + d) = __floats2half2_rn(val[i].x * sc, val[i].y * sc);
            if (mode & kPrepSplit) {
                const __half2 hi = __floats2half2_rn(val[i].x, val[i].y);
                const float2 hf = __half22float2(hi);
                __half* o = a.split[m] + tok * 2 * D + d;
                *reinterpret_cast<__half2*>(o) = hi;
                *reinterpret_cast<__half2*>(o + D) = __floats2half2_rn(val[i].x - hf.x, val[i].y - hf.y);
            }
            if (mode & kPrepF32) *reinterpret_cast<float2*>(a.f32[m] + tok * D + d) = val[i];
        }
    }
}

struct TmixPreArgs {
    const float *k, *v, *yw, *ya, *yv, *v_first;     // [N, D]; yv / v_first null on layer 0
    const float *w0, *a0, *v0, *k_k, *k_a;           // [D]
    float *w, *k2, *v2, *na, *nb;                     // [N, D]: decay, k', v', -kk, kk * a
    long long n_pairs;                                // N * H
    int H;
};

// One warp per (token, head): lane owns the channel pair 2 lane, 2 lane + 1 of the head (64-bit
// loads and stores).
__global__ void __launch_bounds__(256) seq_tmix_pre_kernel(const TmixPreArgs p) {
    const long long pair = blockIdx.x * 8ll + (threadIdx.x >> 5);
    if (pair >= p.n_pairs) return;
    const int lane = threadIdx.x & 31, hd = static_cast<int>(pair % p.H);
    const size_t i = static_cast<size_t>(pair) * 64 + 2 * lane;
    const int c = hd * 64 + 2 * lane;
    auto ld2 = [](const float* q, size_t at) { return *reinterpret_cast<const float2*>(q + at); };
    auto st2 = [](float* q, size_t at, float x, float y) { *reinterpret_cast<float2*>(q + at) = make_float2(x, y); };
    const float2 k = ld2(p.k, i), yw = ld2(p.yw, i), ya = ld2(p.ya, i);
    float2 v = ld2(p.v, i);
    const float2 w0 = ld2(p.w0, c), a0 = ld2(p.a0, c), kk_w = ld2(p.k_k, c), ka_w = ld2(p.k_a, c);
    if (p.yv) {
        const float2 yv = ld2(p.yv, i), vf = ld2(p.v_first, i), v0 = ld2(p.v0, c);
        v.x = v.x + (vf.x - v.x) * sigmoidf_(yv.x + v0.x);
        v.y = v.y + (vf.y - v.y) * sigmoidf_(yv.y + v0.y);
    }
    st2(p.w, i, expf(-0.606531f * sigmoidf_(yw.x + w0.x)), expf(-0.606531f * sigmoidf_(yw.y + w0.y)));
    const float ax = sigmoidf_(ya.x + a0.x), ay = sigmoidf_(ya.y + a0.y);
    const float kx = k.x * kk_w.x, ky = k.y * kk_w.y;
    float n2 = kx * kx + ky * ky;
    st2(p.k2, i, k.x * (1.0f + (ax - 1.0f) * ka_w.x), k.y * (1.0f + (ay - 1.0f) * ka_w.y));
    st2(p.v2, i, v.x, v.y);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) n2 += __shfl_xor_sync(0xFFFFFFFFu, n2, o);
    const float inv = 1.0f / sqrtf(n2 + 1e-12f);
    st2(p.na, i, -(kx * inv), -(ky * inv));
    st2(p.nb, i, kx * inv * ax, ky * inv * ay);
}

// x fp32 [rows, cols] -> out fp16 [rows, 2 * cols] = [hi | lo] with hi = fp16(x), lo = fp16(x - hi):
// a product of [hi | lo] with a matrix stacked twice equals x @ W to ~2^-22 relative while running
// on the fp16 tensor cores.  One pass over x.
__global__ void __launch_bounds__(256) split_fp16_kernel(const float* __restrict__ x, __half* __restrict__ out,
                                                         long long n_pairs, int cols) {
    const int half_cols = cols >> 1;
    for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n_pairs; i += gridDim.x * 256ll) {
        const long long r = i / half_cols;
        const int c = static_cast<int>(i % half_cols) * 2;
        const float2 v = *reinterpret_cast<const float2*>(x + r * cols + c);
        const __half2 hi = __floats2half2_rn(v.x, v.y);
        const float2 hf = __half22float2(hi);
        const __half2 lo = __floats2half2_rn(v.x - hf.x, v.y - hf.y);
        __half* o = out + r * 2 * cols + c;
        *reinterpret_cast<__half2*>(o) = hi;
        *reinterpret_cast<__half2*>(o + cols) = lo;
    }
}

}  // namespace rwkvq

using namespace rwkvq;

extern "C" {

int rwkvq_seq_ln_shift_mix(const float* x, const float* ln_w, const float* ln_b, const float* shift_in,
                           const float* mix, int n_mix, float* out, float* shift_out, int B, int T, int D,
                           void* stream) {
    RWKVQ_REQUIRE(x && ln_w && ln_b && out && shift_out, RWKVQ_E_NULL, "rwkvq_seq_ln_shift_mix: null pointer");
    RWKVQ_REQUIRE(B >= 1 && T >= 1 && D >= 1 && D <= kSeqThreads * kSeqPer, RWKVQ_E_LIMIT,
                  "rwkvq_seq_ln_shift_mix: B=%d T=%d D=%d (D at most %d)", B, T, D, kSeqThreads * kSeqPer);
    RWKVQ_REQUIRE((n_mix == 1 || n_mix == 6) && mix, RWKVQ_E_SHAPE, "rwkvq_seq_ln_shift_mix: n_mix %d (1 or 6)", n_mix);
    const long long n = static_cast<long long>(B) * T;
    RWKVQ_REQUIRE(n < (1ll << 31), RWKVQ_E_LIMIT, "rwkvq_seq_ln_shift_mix: %lld tokens", n);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (n_mix == 6)
        seq_ln_shift_mix_kernel<6><<<static_cast<unsigned>(n), kSeqThreads, 0, s>>>(x, ln_w, ln_b, shift_in, mix, out, shift_out, T, D, n);
    else
        seq_ln_shift_mix_kernel<1><<<static_cast<unsigned>(n), kSeqThreads, 0, s>>>(x, ln_w, ln_b, shift_in, mix, out, shift_out, T, D, n);
    return check_launch("rwkvq_seq_ln_shift_mix");
}

int rwkvq_seq_ln_shift_mix_prep(const float* x, const float* ln_w, const float* ln_b, const float* shift_in,
                                const float* mix, int n_mix, const int* modes, void* const* out_x16,
                                float* const* out_scale, void* const* out_split, float* const* out_f32,
                                float* shift_out, int B, int T, int D, void* stream) {
    RWKVQ_REQUIRE(x && ln_w && ln_b && mix && modes && shift_out, RWKVQ_E_NULL, "rwkvq_seq_ln_shift_mix_prep: null pointer");
    RWKVQ_REQUIRE(B >= 1 && T >= 1 && D >= 2 && D % 2 == 0 && D <= kSeqThreads * kSeqPer, RWKVQ_E_LIMIT,
                  "rwkvq_seq_ln_shift_mix_prep: B=%d T=%d D=%d (even, at most %d)", B, T, D, kSeqThreads * kSeqPer);
    RWKVQ_REQUIRE(n_mix >= 1 && n_mix <= 6, RWKVQ_E_SHAPE, "rwkvq_seq_ln_shift_mix_prep: n_mix %d (1..6)", n_mix);
    const long long n = static_cast<long long>(B) * T;
    RWKVQ_REQUIRE(n < (1ll << 31), RWKVQ_E_LIMIT, "rwkvq_seq_ln_shift_mix_prep: %lld tokens", n);
    RWKVQ_REQUIRE(aligned(x, 8) && aligned(ln_w, 8) && aligned(ln_b, 8) && aligned(mix, 8) && aligned(shift_in, 8) &&
                      aligned(shift_out, 8), RWKVQ_E_ALIGN, "rwkvq_seq_ln_shift_mix_prep: 8-byte aligned rows required");
    SeqPrepArgs a{};
    a.x = x; a.ln_w = ln_w; a.ln_b = ln_b; a.shift_in = shift_in; a.mix = mix; a.shift_out = shift_out;
    a.T = T; a.D = D; a.n_mix = n_mix;
    for (int m = 0; m < n_mix; ++m) {
        const int mode = modes[m];
        RWKVQ_REQUIRE(mode >= 1 && mode <= 7, RWKVQ_E_DTYPE, "rwkvq_seq_ln_shift_mix_prep: mode[%d] = %d", m, mode);
        a.mode[m] = mode;
        if (mode & kPrepScaled) {
            RWKVQ_REQUIRE(out_x16 && out_scale && out_x16[m] && out_scale[m] && aligned(out_x16[m], 16), RWKVQ_E_NULL,
                          "rwkvq_seq_ln_shift_mix_prep: scaled output %d missing or unaligned", m);
            a.x16[m] = static_cast<__half*>(out_x16[m]);
            a.scale[m] = out_scale[m];
        }
        if (mode & kPrepSplit) {
            RWKVQ_REQUIRE(out_split && out_split[m] && aligned(out_split[m], 4), RWKVQ_E_NULL,
                          "rwkvq_seq_ln_shift_mix_prep: split output %d missing or unaligned", m);
            a.split[m] = static_cast<__half*>(out_split[m]);
        }
        if (mode & kPrepF32) {
            RWKVQ_REQUIRE(out_f32 && out_f32[m] && aligned(out_f32[m], 8), RWKVQ_E_NULL,
                          "rwkvq_seq_ln_shift_mix_prep: fp32 output %d missing or unaligned", m);
            a.f32[m] = out_f32[m];
        }
    }
    seq_ln_shift_mix_prep_kernel<<<static_cast<unsigned>(n), kSeqThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
    return check_launch("rwkvq_seq_ln_shift_mix_prep");
}

int rwkvq_seq_tmix_pre(const float* k, const float* v, const float* yw, const float* ya, const float* yv,
                       const float* v_first, const float* w0, const float* a0, const float* v0, const float* k_k,
                       const float* k_a, float* w, float* k2, float* v2, float* neg_kk, float* kk_a, int64_t n_tokens,
                       int H, void* stream) {
    RWKVQ_REQUIRE(k && v && yw && ya && w0 && a0 && k_k && k_a && w && k2 && v2 && neg_kk && kk_a, RWKVQ_E_NULL,
                  "rwkvq_seq_tmix_pre: null pointer");
    RWKVQ_REQUIRE((yv == nullptr) == (v_first == nullptr) && (yv == nullptr || v0 != nullptr), RWKVQ_E_NULL,
                  "rwkvq_seq_tmix_pre: yv, v_first and v0 go together");
    RWKVQ_REQUIRE(n_tokens >= 1 && H >= 1, RWKVQ_E_SHAPE, "rwkvq_seq_tmix_pre: n_tokens=%lld H=%d", (long long)n_tokens, H);
    for (const void* q : {(const void*)k, (const void*)v, (const void*)yw, (const void*)ya, (const void*)yv, (const void*)v_first,
                          (const void*)w0, (const void*)a0, (const void*)v0, (const void*)k_k, (const void*)k_a, (const void*)w,
                          (const void*)k2, (const void*)v2, (const void*)neg_kk, (const void*)kk_a})
        RWKVQ_REQUIRE(aligned(q, 8), RWKVQ_E_ALIGN, "rwkvq_seq_tmix_pre: 8-byte aligned arrays required");
    TmixPreArgs p{k, v, yw, ya, yv, v_first, w0, a0, v0, k_k, k_a, w, k2, v2, neg_kk, kk_a, n_tokens * H, H};
    const long long blocks = (p.n_pairs + 7) / 8;
    RWKVQ_REQUIRE(blocks < (1ll << 31), RWKVQ_E_LIMIT, "rwkvq_seq_tmix_pre: too many tokens");
    seq_tmix_pre_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
    return check_launch("rwkvq_seq_tmix_pre");
}

int rwkvq_split_fp16(const float* x, void* out_fp16, int64_t rows, int cols, void* stream) {
    RWKVQ_REQUIRE(x && out_fp16, RWKVQ_E_NULL, "rwkvq_split_fp16: null pointer");
    RWKVQ_REQUIRE(rows >= 1 && cols >= 2 && cols % 2 == 0, RWKVQ_E_SHAPE, "rwkvq_split_fp16: rows=%lld cols=%d (even)",
                  (long long)rows, cols);
    RWKVQ_REQUIRE(aligned(x, 8) && aligned(out_fp16, 4), RWKVQ_E_ALIGN, "rwkvq_split_fp16: x needs 8-byte, out 4-byte alignment");
    const long long n_pairs = rows * (cols / 2);
    long long blocks = (n_pairs + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    split_fp16_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        x, static_cast<__half*>(out_fp16), n_pairs, cols);
    return check_launch("rwkvq_split_fp16");
}

}  // extern "C"
