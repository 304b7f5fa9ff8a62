// Single-token decode step of a quantized RWKV-7 model: the glue kernels between
// the GEMVs and the host-side launch sequence (rwkvq_decode_step).
//
// Per layer (backends/metal/quant_model.py:638-728, 803-836):
//   ln_shift_mix   LN1 + token shift + the six lerps           -> xs[6][B][D]
//   gemv x3        r, k, v projections (one fused launch)
//   lora_multi     the LoRA down projections w1, a1, v1, g1 (tanh / - / - / sigmoid)
//   lora_multi     the LoRA up projections w2, a2, v2, g2
//   tmix_core      decay, gates, kk, k and v updates, WKV-7 step on the 64x64 state,
//                  group norm, bonus, gate                      -> og[B][D]
//   gemv + add     output projection and residual
//   ln_shift_mix   LN2 + token shift + lerp                     -> xk[B][D]
//   gemv + relu^2  ffn key;  gemv + add  ffn value and residual
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

// LayerNorm of row b held as `per` values per thread (two-pass variance, eps 1e-5).
template <int PER>
__device__ __forceinline__ void layer_norm_row(float (&x)[PER], int D, const float* w, const float* b,
                                               float* red) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) s += x[i];
    const float mean = block_sum(s, red) / D;
    float s2 = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int d = threadIdx.x + i * blockDim.x;
        const float c = (d < D) ? x[i] - mean : 0.f;
        s2 += c * c;
    }
    const float inv = 1.0f / sqrtf(block_sum(s2, red) / D + 1e-5f);
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int d = threadIdx.x + i * blockDim.x;
        if (d < D) x[i] = (x[i] - mean) * inv * w[d] + b[d];
    }
}

constexpr int kRowThreads = 256;
constexpr int kRowPer = 16;      // D <= 4096

// x[b] = LN0(fp16(bf16(dequant(emb[token[b]])))): one embedding row is decoded from the
// packed table (quant_model.py:853, 975-976; rounding policy :128-154).
__global__ void __launch_bounds__(kRowThreads) embed_ln0_kernel(QView emb, const long long* tokens,
                                                               const float* ln_w, const float* ln_b,
                                                               float* x, int D) {
    __shared__ float red[kRowThreads / 32];
    const int b = blockIdx.x;
    long long tok = tokens[b];
    tok = tok < 0 ? 0 : (tok >= emb.rows ? emb.rows - 1 : tok);
    float v[kRowPer];
#pragma unroll
    for (int i = 0; i < kRowPer; ++i) {
        const int d = threadIdx.x + i * kRowThreads;
        v[i] = (d < D) ? dense_param_rounding(decode_element(emb, static_cast<int>(tok), d)) : 0.f;
    }
    layer_norm_row<kRowPer>(v, D, ln_w, ln_b, red);
#pragma unroll
    for (int i = 0; i < kRowPer; ++i) {
        const int d = threadIdx.x + i * kRowThreads;
        if (d < D) x[static_cast<size_t>(b) * D + d] = v[i];
    }
}

// xn = LN(x[b]); prev = shift[b] (zeros for a fresh stream); shift[b] = xn;
// out[m][b] = xn + (prev - xn) * mix[m]   for m < n_mix   (n_mix = 0: out[0][b] = xn)
__global__ void __launch_bounds__(kRowThreads) ln_shift_mix_kernel(const float* x, const float* ln_w,
                                                                  const float* ln_b, float* shift,
                                                                  const float* mix, int n_mix, float* out,
                                                                  int B, int D) {
    __shared__ float red[kRowThreads / 32];
    const int b = blockIdx.x;
    float v[kRowPer];
#pragma unroll
    for (int i = 0; i < kRowPer; ++i) {
        const int d = threadIdx.x + i * kRowThreads;
        v[i] = (d < D) ? x[static_cast<size_t>(b) * D + d] : 0.f;
    }
    layer_norm_row<kRowPer>(v, D, ln_w, ln_b, red);
#pragma unroll
    for (int i = 0; i < kRowPer; ++i) {
        const int d = threadIdx.x + i * kRowThreads;
        if (d >= D) continue;
        const size_t bd = static_cast<size_t>(b) * D + d;
        if (n_mix == 0) { out[bd] = v[i]; continue; }
        const float xx = shift[bd] - v[i];
        shift[bd] = v[i];
        for (int m = 0; m < n_mix; ++m) out[(static_cast<size_t>(m) * B) * D + bd] = v[i] + xx * mix[m * D + d];
    }
}

// ---- batched LoRA products: up to 4 branches, each y = act(x @ Wt) with Wt stored [in, out]
constexpr int kLmWarps = 8, kLmCols = 128, kLmMaxN = 8;
struct LoraMultiArgs {
    QView t[4];
    const float* x[4];
    float* y[4];
    int act[4];
    long long ldx, ldy;
    int n_cols;     // right-hand sides (<= kLmMaxN)
};

__device__ __forceinline__ void lora_w4(const QView& t, int i, int c, float (&w)[4]) {
    const size_t I = static_cast<size_t>(i);
    if (t.kind == RWKVQ_KIND_ASYM && (t.cols & 3) == 0) {
        const uint32_t q = ld_stream_u32(t.codes + I * t.cols + c);
        const int nb = (t.cols + t.gs - 1) / t.gs;
        const float s = static_cast<const float*>(t.scale)[I * nb + c / t.gs], m = t.mn[I * nb + c / t.gs];
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
#pragma unroll
    for (int k = 0; k < 4; ++k) w[k] = dense_param_rounding(w[k]);
}

__global__ void __launch_bounds__(kLmWarps * 32) lora_multi_kernel(const LoraMultiArgs a) {
    __shared__ float red[kLmWarps][kLmMaxN][kLmCols];
    const int br = blockIdx.y;
    const QView& t = a.t[br];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = blockIdx.x * kLmCols + lane * 4;
    if (blockIdx.x * kLmCols >= t.cols) return;
    float acc[kLmMaxN][4];
#pragma unroll
    for (int n = 0; n < kLmMaxN; ++n)
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[n][k] = 0.f;
    if (c < t.cols) {
        for (int i = warp; i < t.rows; i += kLmWarps) {
            float w[4];
            lora_w4(t, i, c, w);
#pragma unroll
            for (int n = 0; n < kLmMaxN; ++n) {
                if (n >= a.n_cols) break;
                const float xv = __ldg(a.x[br] + n * a.ldx + i);
#pragma unroll
                for (int k = 0; k < 4; ++k) acc[n][k] = fmaf(xv, w[k], acc[n][k]);
            }
        }
    }
#pragma unroll
    for (int n = 0; n < kLmMaxN; ++n) {
        if (n >= a.n_cols) break;
#pragma unroll
        for (int k = 0; k < 4; ++k) red[warp][n][lane * 4 + k] = acc[n][k];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < a.n_cols * kLmCols; idx += blockDim.x) {
        const int n = idx / kLmCols, cc = idx % kLmCols;
        const int col = blockIdx.x * kLmCols + cc;
        if (col >= t.cols) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kLmWarps; ++w) v += red[w][n][cc];
        if (a.act[br] == 1) v = tanhf(v);
        else if (a.act[br] == 2) v = sigmoidf_(v);
        a.y[br][n * a.ldy + col] = v;
    }
}

// ---- time-mix core for one token: grid (H, B), 256 threads = (state row dv, quarter)
struct TmixCoreArgs {
    const float *r, *k, *v;            // [B, D] projections
    const float *yw, *ya, *yv, *g;     // [B, D] LoRA outputs (yv null on layer 0)
    const float *w0, *a0, *v0;         // [D]
    const float *k_k, *k_a, *r_k, *lnx_w, *lnx_b;
    float* v_first;                    // [B, D] written by layer 0, read by the others
    float* state;                      // [B, H, 64, 64] in place
    float* og;                         // [B, D]
    int D, H, layer0;
};

__global__ void __launch_bounds__(256) tmix_core_kernel(const TmixCoreArgs p) {
    __shared__ float sA[64], sW[64], sK[64], sB[64], sR[64], sV[64], sY[64], sG[64];
    __shared__ float red[8];
    const int hi = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
    const size_t row = static_cast<size_t>(b) * p.D + hi * 64;
    float kk = 0.f, av = 0.f;
    if (tid < 64) {
        const int c = hi * 64 + tid;
        const float r = p.r[row + tid], k = p.k[row + tid];
        float v = p.v[row + tid];
        const float w = expf(-0.606531f * sigmoidf_(p.yw[row + tid] + p.w0[c]));
        av = sigmoidf_(p.ya[row + tid] + p.a0[c]);
        kk = k * p.k_k[c];
        const float k2 = k * (1.0f + (av - 1.0f) * p.k_a[c]);
        if (p.layer0) p.v_first[row + tid] = v;
        else v = v + (p.v_first[row + tid] - v) * sigmoidf_(p.yv[row + tid] + p.v0[c]);
        sW[tid] = w; sK[tid] = k2; sR[tid] = r; sV[tid] = v; sG[tid] = p.g[row + tid];
    }
    const float n2 = block_sum(tid < 64 ? kk * kk : 0.f, red);
    if (tid < 64) {
        const float kn = kk / sqrtf(n2 + 1e-12f);
        sA[tid] = -kn;
        sB[tid] = kn * av;
    }
    __syncthreads();
    // one WKV-7 step on the thread's 16 state columns
    const int dv = tid >> 2, part = tid & 3;
    float* hp = p.state + ((static_cast<size_t>(b) * p.H + hi) * 64 + dv) * 64 + part * 16;
    float h[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 v4 = *reinterpret_cast<const float4*>(hp + 4 * i);
        h[4 * i] = v4.x; h[4 * i + 1] = v4.y; h[4 * i + 2] = v4.z; h[4 * i + 3] = v4.w;
    }
    float sa = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) sa = fmaf(h[i], sA[part * 16 + i], sa);
    sa += __shfl_xor_sync(0xFFFFFFFFu, sa, 1);
    sa += __shfl_xor_sync(0xFFFFFFFFu, sa, 2);
    const float vv = sV[dv];
    float y = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int dk = part * 16 + i;
        h[i] = fmaf(sW[dk], h[i], fmaf(vv, sK[dk], sa * sB[dk]));
        y = fmaf(h[i], sR[dk], y);
    }
    y += __shfl_xor_sync(0xFFFFFFFFu, y, 1);
    y += __shfl_xor_sync(0xFFFFFFFFu, y, 2);
#pragma unroll
    for (int i = 0; i < 4; ++i)
        *reinterpret_cast<float4*>(hp + 4 * i) = make_float4(h[4 * i], h[4 * i + 1], h[4 * i + 2], h[4 * i + 3]);
    if (part == 0) sY[dv] = y;
    __syncthreads();
    // group norm over the head (two-pass), bonus, gate
    const float yv_ = tid < 64 ? sY[tid] : 0.f;
    const float mean = block_sum(yv_, red) / 64.f;
    const float dc = tid < 64 ? yv_ - mean : 0.f;
    const float var = block_sum(dc * dc, red) / 64.f;
    const float dp = block_sum(tid < 64 ? sR[tid] * sK[tid] * p.r_k[hi * 64 + tid] : 0.f, red);
    if (tid < 64) {
        const int c = hi * 64 + tid;
        const float nrm = dc * (1.0f / sqrtf(var + 64e-5f));
        p.og[row + tid] = (nrm * p.lnx_w[c] + p.lnx_b[c] + dp * sV[tid]) * sG[tid];
    }
}

__global__ void __launch_bounds__(256) argmax_kernel(const float* logits, long long* out, int V) {
    __shared__ float bv[8];
    __shared__ int bi[8];
    const float* row = logits + static_cast<size_t>(blockIdx.x) * V;
    float best = -INFINITY;
    int idx = 0;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = row[i];
        if (v > best) { best = v; idx = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        const int oi = __shfl_xor_sync(0xFFFFFFFFu, idx, o);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
    }
    if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w)
            if (bv[w] > best || (bv[w] == best && bi[w] < idx)) { best = bv[w]; idx = bi[w]; }
        out[blockIdx.x] = idx;
    }
}

}  // namespace rwkvq

using namespace rwkvq;

namespace {

struct Workspace {
    float *x, *xs, *rkv, *hid, *yl, *og, *xk, *hffn, *xo, *v_first, *logits;
    size_t bytes;
};

Workspace carve(const rwkvq_model& m, int B, void* base) {
    const size_t D = m.n_embd, F = m.ffn_dim, R = m.max_rank, V = m.vocab_size, b = B;
    Workspace w{};
    size_t off = 0;
    auto take = [&](size_t n) {
        float* p = base ? reinterpret_cast<float*>(static_cast<char*>(base) + off) : nullptr;
        off += ((n * sizeof(float) + 255) / 256) * 256;
        return p;
    };
    w.x = take(b * D); w.xs = take(6 * b * D); w.rkv = take(3 * b * D); w.hid = take(4 * b * R);
    w.yl = take(4 * b * D); w.og = take(b * D); w.xk = take(b * D); w.hffn = take(b * F);
    w.xo = take(b * D); w.v_first = take(b * D); w.logits = take(b * V);
    w.bytes = off;
    return w;
}

int lora_multi(const rwkvq_qtensor* const* ts, const float* const* xs, float* const* ys, const int* acts,
               int n_br, int B, long long ldx, long long ldy, cudaStream_t s) {
    int max_cols = 0;
    LoraMultiArgs a{};
    for (int i = 0; i < n_br; ++i) {
        int rc = validate_qtensor(ts[i], "rwkvq_decode_step(lora)");
        if (rc) return rc;
        a.t[i] = make_view(*ts[i]);
        a.x[i] = xs[i]; a.y[i] = ys[i]; a.act[i] = acts[i];
        if (ts[i]->cols > max_cols) max_cols = ts[i]->cols;
    }
    a.ldx = ldx; a.ldy = ldy;
    for (int n0 = 0; n0 < B; n0 += kLmMaxN) {
        LoraMultiArgs c = a;
        c.n_cols = B - n0 < kLmMaxN ? B - n0 : kLmMaxN;
        for (int i = 0; i < n_br; ++i) { c.x[i] = a.x[i] + n0 * ldx; c.y[i] = a.y[i] + n0 * ldy; }
        lora_multi_kernel<<<dim3((max_cols + kLmCols - 1) / kLmCols, n_br), kLmWarps * 32, 0, s>>>(c);
    }
    return RWKVQ_OK;
}

}  // namespace

extern "C" {

size_t rwkvq_decode_workspace_bytes(const rwkvq_model* m, int B) {
    if (!m || B < 1) return 0;
    return carve(*m, B, nullptr).bytes;
}

int rwkvq_decode_step(const rwkvq_model* m, int B, const int64_t* tokens, float* const* wkv,
                      float* const* tshift, float* const* cshift, void* workspace, size_t workspace_bytes,
                      float* logits, int64_t* next_tokens, void* stream) {
    RWKVQ_REQUIRE(m && m->layers && tokens && wkv && tshift && cshift && workspace, RWKVQ_E_NULL,
                  "rwkvq_decode_step: null pointer");
    RWKVQ_REQUIRE(B >= 1, RWKVQ_E_SHAPE, "rwkvq_decode_step: B=%d", B);
    RWKVQ_REQUIRE(m->head_size == 64, RWKVQ_E_SHAPE, "rwkvq_decode_step: head size %d, only 64 is built", m->head_size);
    RWKVQ_REQUIRE(m->n_embd % 64 == 0 && m->n_embd <= kRowThreads * kRowPer, RWKVQ_E_LIMIT,
                  "rwkvq_decode_step: n_embd %d (multiple of 64, at most %d)", m->n_embd, kRowThreads * kRowPer);
    const Workspace w = carve(*m, B, workspace);
    RWKVQ_REQUIRE(workspace_bytes >= w.bytes, RWKVQ_E_LIMIT, "rwkvq_decode_step: workspace %zu < %zu bytes",
                  workspace_bytes, w.bytes);
    RWKVQ_REQUIRE(aligned(workspace, 256), RWKVQ_E_ALIGN, "rwkvq_decode_step: workspace must be 256-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int D = m->n_embd, H = D / 64, F = m->ffn_dim, V = m->vocab_size;
    const size_t BD = static_cast<size_t>(B) * D;
    int rc = validate_qtensor(&m->emb, "rwkvq_decode_step(emb)");
    if (rc) return rc;
    float* lg = logits ? logits : w.logits;

    embed_ln0_kernel<<<B, kRowThreads, 0, s>>>(make_view(m->emb), reinterpret_cast<const long long*>(tokens),
                                              m->ln0_w, m->ln0_b, w.x, D);
    for (int l = 0; l < m->n_layer; ++l) {
        const rwkvq_layer& L = m->layers[l];
        const bool layer0 = l == 0;
        // ---- time mix
        ln_shift_mix_kernel<<<B, kRowThreads, 0, s>>>(w.x, L.ln1_w, L.ln1_b, tshift[l], L.x_mix, 6, w.xs, B, D);
        float *xr = w.xs, *xw = w.xs + BD, *xk = w.xs + 2 * BD, *xv = w.xs + 3 * BD, *xa = w.xs + 4 * BD,
              *xg = w.xs + 5 * BD;
        float *r = w.rkv, *k = w.rkv + BD, *v = w.rkv + 2 * BD;
        rc = rwkvq_gemv(&L.Wr, xr, RWKVQ_F32, B, D, r, D, RWKVQ_EPI_NONE, nullptr, stream);
        if (rc) return rc;
        rc = rwkvq_gemv(&L.Wk, xk, RWKVQ_F32, B, D, k, D, RWKVQ_EPI_NONE, nullptr, stream);
        if (rc) return rc;
        rc = rwkvq_gemv(&L.Wv, xv, RWKVQ_F32, B, D, v, D, RWKVQ_EPI_NONE, nullptr, stream);
        if (rc) return rc;
        const size_t BR = static_cast<size_t>(B) * m->max_rank;
        float *hw = w.hid, *ha = w.hid + BR, *hv = w.hid + 2 * BR, *hg = w.hid + 3 * BR;
        float *yw = w.yl, *ya = w.yl + BD, *yv = w.yl + 2 * BD, *yg = w.yl + 3 * BD;
        {
            const rwkvq_qtensor* t1[4] = {&L.w1, &L.a1, &L.g1, &L.v1};
            const float* x1[4] = {xw, xa, xg, xv};
            float* y1[4] = {hw, ha, hg, hv};
            const int act1[4] = {1, 0, 2, 0};
            rc = lora_multi(t1, x1, y1, act1, layer0 ? 3 : 4, B, D, m->max_rank, s);
            if (rc) return rc;
            const rwkvq_qtensor* t2[4] = {&L.w2, &L.a2, &L.g2, &L.v2};
            const float* x2[4] = {hw, ha, hg, hv};
            float* y2[4] = {yw, ya, yg, yv};
            const int act2[4] = {0, 0, 0, 0};
            rc = lora_multi(t2, x2, y2, act2, layer0 ? 3 : 4, B, m->max_rank, D, s);
            if (rc) return rc;
        }
        TmixCoreArgs tc{r, k, v, yw, ya, layer0 ? nullptr : yv, yg, L.w0, L.a0, L.v0, L.k_k, L.k_a, L.r_k,
                        L.lnx_w, L.lnx_b, w.v_first, wkv[l], w.og, D, H, layer0 ? 1 : 0};
        tmix_core_kernel<<<dim3(H, B), 256, 0, s>>>(tc);
        rc = rwkvq_gemv(&L.Wo, w.og, RWKVQ_F32, B, D, w.x, D, RWKVQ_EPI_ADD, w.x, stream);
        if (rc) return rc;
        // ---- channel mix
        ln_shift_mix_kernel<<<B, kRowThreads, 0, s>>>(w.x, L.ln2_w, L.ln2_b, cshift[l], L.ffn_x_k, 1, w.xk, B, D);
        rc = rwkvq_gemv(&L.Wfk, w.xk, RWKVQ_F32, B, D, w.hffn, F, RWKVQ_EPI_RELU2, nullptr, stream);
        if (rc) return rc;
        rc = rwkvq_gemv(&L.Wfv, w.hffn, RWKVQ_F32, B, F, w.x, D, RWKVQ_EPI_ADD, w.x, stream);
        if (rc) return rc;
    }
    ln_shift_mix_kernel<<<B, kRowThreads, 0, s>>>(w.x, m->lnout_w, m->lnout_b, nullptr, nullptr, 0, w.xo, B, D);
    rc = rwkvq_gemv(&m->head, w.xo, RWKVQ_F32, B, D, lg, V, RWKVQ_EPI_NONE, nullptr, stream);
    if (rc) return rc;
    if (next_tokens) argmax_kernel<<<B, 256, 0, s>>>(lg, reinterpret_cast<long long*>(next_tokens), V);
    return check_launch("rwkvq_decode_step");
}

}  // extern "C"
